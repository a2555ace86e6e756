"""The suffix-array build on the GPU (through the C ABI) against the CPU oracle and the golden fixtures made by the
reference's own code: byte-for-byte equal sa40 arrays."""
import os

import numpy as np
import pytest
import torch

from conftest import GOLDEN, sa40_to_u64

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from cascade_b200 import api
    c = api.Context(0)
    yield c
    c.close()


def _build(ctx, T, p):
    from cascade_b200 import api
    n = len(T)
    Tp = np.concatenate([np.ascontiguousarray(T, np.uint16), np.zeros(api.TEXT_PAD, np.uint16)])
    td = torch.from_numpy(Tp.view(np.int16)).cuda().view(torch.uint16)
    sa, st = api.build_sa(ctx, td, n, p)
    return sa.cpu().numpy(), st


@pytest.mark.parametrize("p", [1, 3, 64])
def test_golden_sa_fixtures(ctx, p):
    g = np.load(os.path.join(GOLDEN, "sa_fixtures.npz"))
    for name in [k[2:] for k in g.files if k.startswith("T_")]:
        T, want = g["T_" + name], g["SA_" + name]
        sa, st = _build(ctx, T, p)
        got = sa40_to_u64(sa, len(T)).astype(np.uint32)
        assert np.array_equal(got, want), (name, p)
        assert np.all(sa[5 * len(T):] == 0), "bytes past the array must stay untouched"


def test_corner_case_prefix(ctx):
    # dataset/make-corner-case.py of the reference: with l trailing zeros, SA[0, l) = n-1, n-2, ..., n-l.
    rng = np.random.default_rng(0)
    T = np.concatenate([rng.integers(1, 4, 2000), np.zeros(16, np.int64)]).astype(np.uint16)
    sa, _ = _build(ctx, T, 4)
    got = sa40_to_u64(sa, len(T))
    assert list(got[:16]) == [len(T) - 1 - i for i in range(16)]


@pytest.mark.parametrize("n,sigma,p", [(100000, 2, 1), (100000, 2, 16), (300000, 4, 8), (1 << 20, 50000, 64), (777777, 3, 5)])
def test_random_texts_against_oracle(ctx, oracle, n, sigma, p):
    rng = np.random.default_rng(n + sigma)
    T = rng.integers(0, sigma, n).astype(np.uint16)
    T[rng.integers(0, 300, n) == 0] = 0xFFFF
    sa, st = _build(ctx, T, p)
    want = oracle.build_sa40(T)
    assert np.array_equal(sa[:5 * n], want[:5 * n])
    assert st.partitions >= 1 and st.n == n


def test_zipf_corpus_against_oracle_and_host_generator(ctx, oracle):
    from cascade_b200 import api
    n = 1 << 21
    cdf = api.zipf_cdf()
    Th = api.gen_corpus_host(n, 0, 512, cdf)
    Td = api.gen_corpus_device(ctx, n, 0, 512, cdf)
    assert np.array_equal(Td.cpu().view(torch.int16).numpy().view(np.uint16), Th), "host and device generators differ"
    sa, st = api.build_sa(ctx, Td, n, 16)
    want = oracle.build_sa40(Th[:n])
    assert np.array_equal(sa.cpu().numpy()[:5 * n], want[:5 * n])
    # the host-buffer entry point gives the same bytes
    sa_h, _ = api.build_sa_host(ctx, Th, n, 16)
    assert np.array_equal(sa_h[:5 * n], want[:5 * n])


def test_repetitive_corpus_against_oracle(ctx, oracle):
    from cascade_b200 import api
    n = 600000
    T = api.gen_repeat_corpus_host(n, seed=0, base_docs=16, mean_doc=2048, mutate=0.001)
    sa, st = _build(ctx, T[:n], 8)
    assert st.generations >= 6, "long shared suffixes need many doubling generations"
    assert oracle.is_correct(T[:n], sa)
    want = oracle.build_sa40(T[:n])
    assert np.array_equal(sa[:5 * n], want[:5 * n])


def test_config1_16m_tokens_single_partition(ctx, oracle):
    """BASELINE config 1: 16 Mi tokens, Zipf(1.1), documents of mean length 512, one partition, byte-for-byte."""
    from cascade_b200 import api
    n = 1 << 24
    Td = api.gen_corpus_device(ctx, n, 0, 512)
    sa, st = api.build_sa(ctx, Td, n, 1)
    Th = Td.cpu().view(torch.int16).numpy().view(np.uint16)
    sa_h = sa.cpu().numpy()
    assert oracle.is_correct(Th[:n], sa_h)
    want = oracle.build_sa40(Th[:n])
    assert np.array_equal(sa_h[:5 * n], want[:5 * n])


def test_just_above_16m_tokens_ranks_reach_the_inverse_array_through_buckets(ctx, oracle):
    """Above 2^24 positions the rank updates are bucketed by the top 8 position bits before they are applied (generation 0 by
    the counting-free bucket kernel, later generations by a digit pass); the last bucket is ragged here."""
    from cascade_b200 import api
    n = (1 << 24) + (1 << 20) + 13
    Td = api.gen_corpus_device(ctx, n, 7, 256)
    sa, st = api.build_sa(ctx, Td, n, 16)
    assert st.generations >= 1
    Th = Td.cpu().view(torch.int16).numpy().view(np.uint16)
    want = oracle.build_sa40(Th[:n])
    assert np.array_equal(sa.cpu().numpy()[:5 * n], want[:5 * n])


def test_partition_count_does_not_change_the_result(ctx):
    from cascade_b200 import api
    n = 3_000_000
    Td = api.gen_corpus_device(ctx, n, 5, 1024)
    ref, _ = api.build_sa(ctx, Td, n, 1)
    for p in (2, 7, 64, 300, 4096):
        sa, st = api.build_sa(ctx, Td, n, p, seed=p)
        assert torch.equal(sa, ref), p


def test_bad_arguments_are_refused(ctx):
    from cascade_b200 import api
    T = torch.zeros(1000 + api.TEXT_PAD, dtype=torch.uint16, device="cuda")
    out = torch.zeros(5 * 1000 + 128, dtype=torch.uint8, device="cuda")
    with pytest.raises(api.CascadeError):
        api.build_sa(ctx, T, 0, 1, out=out)
    with pytest.raises(api.CascadeError):
        api.build_sa(ctx, T, 1000, 0, out=out)
    with pytest.raises(api.CascadeError):
        api.build_sa(ctx, T, 1000, 5000, out=out)
