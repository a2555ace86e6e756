"""csa_validate_sa (the device form of the reference's is_correct_SA) against the oracle's verdict: it accepts every golden
suffix array and rejects corrupted ones exactly where the oracle does."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from cascade_b200 import api
    c = api.Context(0)
    yield c
    c.close()


def _pack40(sa):
    sa = np.asarray(sa, np.uint64)
    out = np.zeros(5 * len(sa) + 128, np.uint8)
    b = out[:5 * len(sa)].reshape(len(sa), 5)
    for k in range(5):
        b[:, k] = ((sa >> np.uint64(8 * k)) & np.uint64(0xFF)).astype(np.uint8)
    return out


def _validate(ctx, T, sa40):
    from cascade_b200 import api
    n = len(T)
    Tp = np.concatenate([np.ascontiguousarray(T, np.uint16), np.zeros(api.TEXT_PAD, np.uint16)])
    td = torch.from_numpy(Tp.view(np.int16)).cuda().view(torch.uint16)
    sd = torch.from_numpy(np.ascontiguousarray(sa40)).cuda()
    return api.validate_sa(ctx, td, n, sd)


def test_golden_arrays_pass_and_corrupted_ones_fail_like_the_oracle(ctx, oracle):
    g = np.load(os.path.join(GOLDEN, "sa_fixtures.npz"))
    rng = np.random.default_rng(11)
    checked = 0
    for name in [k[2:] for k in g.files if k.startswith("T_")]:
        T, sa = g["T_" + name], g["SA_" + name].astype(np.uint64)
        n = len(T)
        good = _pack40(sa)
        r = _validate(ctx, T, good)
        assert r["ok"] and oracle.is_correct(T, good), name
        if n < 4:
            continue
        # a swap of two neighbours, a swap of two far entries, a duplicate, an entry out of range
        cases = []
        i = int(rng.integers(0, n - 1))
        s = sa.copy(); s[i], s[i + 1] = s[i + 1], s[i]; cases.append(("swap", s))
        a, b = int(rng.integers(0, n // 2)), int(rng.integers(n // 2, n))
        s = sa.copy(); s[a], s[b] = s[b], s[a]; cases.append(("far", s))
        s = sa.copy(); s[b] = s[a]; cases.append(("dup", s))
        s = sa.copy(); s[a] = np.uint64(n + 5); cases.append(("range", s))
        for kind, s in cases:
            bad = _pack40(s)
            want = oracle.is_correct(T, bad)
            got = _validate(ctx, T, bad)
            assert got["ok"] == want, (name, kind, got)
            if kind == "dup":
                assert got["duplicates"] >= 1
            if kind == "range":
                assert got["out_of_range"] == 1
            checked += 1
    assert checked > 100


def test_a_built_array_validates_and_one_wrong_generation_would_not(ctx, oracle):
    """A 2^22-token build passes; the same array with two suffixes that share a long prefix exchanged does not (their first
    symbols agree, so only the rank comparison can tell)."""
    from cascade_b200 import api
    n = 1 << 22
    T = api.gen_repeat_corpus_host(n, seed=3, base_docs=8, mean_doc=4096, mutate=0.001)
    Tp = torch.from_numpy(np.concatenate([T[:n], np.zeros(api.TEXT_PAD, np.uint16)]).view(np.int16)).cuda().view(torch.uint16)
    sa, st = api.build_sa(ctx, Tp, n, 16)
    r = api.validate_sa(ctx, Tp, n, sa)
    assert r["ok"], r
    h = sa.cpu().numpy()
    e = h[:5 * n].reshape(n, 5)
    # find neighbours whose suffixes share at least 64 symbols and exchange them
    from conftest import sa40_to_u64
    v = sa40_to_u64(h, n)
    k = None
    for i in range(n // 2, n - 1):
        x, y = int(v[i]), int(v[i + 1])
        if x + 64 < n and y + 64 < n and np.array_equal(T[x:x + 64], T[y:y + 64]):
            k = i
            break
    assert k is not None
    e[[k, k + 1]] = e[[k + 1, k]]
    bad = torch.from_numpy(h).cuda()
    r = api.validate_sa(ctx, Tp, n, bad)
    assert not r["ok"] and r["out_of_order"] >= 1 and r["first_bad_rank"] in (k, k + 1, k + 2), r
