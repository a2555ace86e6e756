"""The batched count / locate engine on the GPU (through the C ABI) against the oracle's intervals and positions and
against the golden intervals made by the reference's host search."""
import json
import os

import numpy as np
import pytest
import torch

import conftest
from conftest import GOLDEN, sa40_to_u64

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from cascade_b200 import api
    c = api.Context(0)
    yield c
    c.close()


def _index(ctx, T, sa40, stride):
    from cascade_b200 import api
    n = len(T)
    Tp = np.concatenate([np.ascontiguousarray(T, np.uint16), np.zeros(api.TEXT_PAD, np.uint16)])
    td = torch.from_numpy(Tp.view(np.int16)).cuda().view(torch.uint16)
    sd = torch.from_numpy(np.ascontiguousarray(sa40)).cuda()
    return api.SuffixIndex(ctx, td, sd, n, stride)


def _dev(off, sym):
    o = torch.from_numpy(off.view(np.int64)).cuda()
    s = torch.from_numpy(np.concatenate([sym, np.zeros(8, np.uint16)]).view(np.int16)).cuda()
    return o, s


def test_known_answer_table(ctx, oracle):
    with open(os.path.join(GOLDEN, "known_answers.json")) as f:
        cases = json.load(f)
    for stride in (1, 2, 32):
        for c in cases:
            T, P = np.array(c["text"], np.uint16), np.array(c["pattern"], np.uint16)
            sa = oracle.build_sa40(T)
            idx = _index(ctx, T, sa, stride)
            off = np.array([0, len(P)], np.uint64)
            o, s = _dev(off, P)
            itv = idx.find(o, s, 1).cpu().numpy().view(np.uint64)
            assert (int(itv[0]), int(itv[1])) == (c["lo"], c["hi"]), (c, stride)


@pytest.mark.parametrize("stride", [1, 2, 3, 16, 64, 100000])
def test_golden_query_fixtures(ctx, oracle, stride):
    g = np.load(os.path.join(GOLDEN, "query_fixtures.npz"))
    s = np.load(os.path.join(GOLDEN, "sa_fixtures.npz"))
    for name in [k[4:] for k in g.files if k.startswith("off_")]:
        T = s["T_" + name]
        sa = oracle.build_sa40(T)
        idx = _index(ctx, T, sa, stride)
        off, sym, want = g["off_" + name], g["sym_" + name], g["itv_" + name]
        q = len(off) - 1
        o, sy = _dev(off, sym)
        itv = idx.find(o, sy, q)
        got = itv.cpu().numpy().view(np.uint64)
        bad = np.flatnonzero(got != want)
        assert bad.size == 0, (name, stride, bad[:4] // 2, got[bad[:4]], want[bad[:4]])
        fails, first = idx.certify(o, sy, q, itv)
        assert fails == 0
        pos, cnt = idx.locate(itv, q, 100)
        wp, wc = oracle.locate_batch(sa, got, 100)
        assert np.array_equal(cnt.cpu().numpy().view(np.uint32), wc)
        pn = pos.cpu().numpy().view(np.uint64)
        for i in range(q):
            assert np.array_equal(pn[i, :wc[i]], wp[i, :wc[i]]), (name, i)


def test_certificate_rejects_wrong_intervals(ctx, oracle):
    rng = np.random.default_rng(1)
    T = rng.integers(0, 3, 5000).astype(np.uint16)
    sa = oracle.build_sa40(T)
    idx = _index(ctx, T, sa, 8)
    off, sym, _ = conftest.fixture_queries(T, rng, 64)
    o, s = _dev(off, sym)
    itv = idx.find(o, s, 64)
    assert idx.certify(o, s, 64, itv) == (0, 2**64 - 1)
    bad = itv.clone()
    k = next(i for i in range(64) if int(bad[2 * i + 1]) - int(bad[2 * i]) >= 2)
    bad[2 * k] += 1
    fails, first = idx.certify(o, s, 64, bad)
    assert fails == 1 and first == k


def test_zipf_index_batch_and_host_entry_point(ctx, oracle):
    """A 2 Mi-token Zipf corpus built on the GPU, queried with the two halves of BASELINE config 5 (substrings and random
    strings of 1-16 tokens): intervals, counts hash and positions equal the oracle's; the host-buffer entry point agrees."""
    from cascade_b200 import api
    n = 1 << 21
    Td = api.gen_corpus_device(ctx, n, 0, 1024)
    sa, _ = api.build_sa(ctx, Td, n, 8)
    Th = Td.cpu().view(torch.int16).numpy().view(np.uint16)
    sa_h = sa.cpu().numpy()
    idx = api.SuffixIndex(ctx, Td, sa, n, 32)
    oa, sa_ = api.gen_queries("substring", Th, n, 20000, seed=1)
    ob, sb = api.gen_queries("random", None, 0, 20000, seed=2)
    off = np.concatenate([oa, ob[1:] + oa[-1]])
    sym = np.concatenate([sa_, sb])
    q = len(off) - 1
    o, s = _dev(off, sym)
    itv = idx.find(o, s, q)
    got = itv.cpu().numpy().view(np.uint64)
    want = oracle.find_batch(Th[:n], sa_h, off, sym)
    assert np.array_equal(got, want)
    assert api.counts_hash(got) == oracle.counts_hash(want)
    assert idx.certify(o, s, q, itv)[0] == 0
    itv_h, cnt_h, poff_h, pos_h, total = idx.query_host(off, sym, 100)
    assert np.array_equal(itv_h, want)
    wp, wc = oracle.locate_batch(sa_h, want, 100)
    assert np.array_equal(cnt_h, wc) and total == int(wc.sum()) and int(poff_h[-1]) == total
    for i in list(range(0, q, 997)) + [q - 1]:
        assert np.array_equal(pos_h[int(poff_h[i]):int(poff_h[i + 1])], wp[i, :wc[i]])


def test_suffix_array_in_pinned_host_memory(ctx, oracle):
    """The index with its suffix array in pinned host memory (read by the device over PCIe) gives the same intervals and positions."""
    from cascade_b200 import api
    rng = np.random.default_rng(4)
    n = 200000
    T = rng.integers(0, 50, n).astype(np.uint16)
    sa = oracle.build_sa40(T)
    Tp = np.concatenate([T, np.zeros(api.TEXT_PAD, np.uint16)])
    td = torch.from_numpy(Tp.view(np.int16)).cuda().view(torch.uint16)
    sa_pinned = torch.from_numpy(np.ascontiguousarray(sa)).pin_memory()
    idx = api.SuffixIndex(ctx, td, sa_pinned, n, 32)
    off, sym, _ = conftest.fixture_queries(T, rng, 500)
    o, s_ = _dev(off, sym)
    itv = idx.find(o, s_, 500)
    want = oracle.find_batch(T, sa, off, sym)
    assert np.array_equal(itv.cpu().numpy().view(np.uint64), want)
    # a text with long runs: patterns longer than the table's K symbols whose K-gram is frequent get brackets wider than a
    # gathered window and are searched in place
    T2 = np.zeros(30000, np.uint16)
    T2[rng.integers(0, 30000, 300)] = 1
    sa2 = oracle.build_sa40(T2)
    td2 = torch.from_numpy(np.concatenate([T2, np.zeros(api.TEXT_PAD, np.uint16)]).view(np.int16)).cuda().view(torch.uint16)
    idx2 = api.SuffixIndex(ctx, td2, torch.from_numpy(np.ascontiguousarray(sa2)).pin_memory(), 30000, 16)
    off2, sym2, _ = conftest.fixture_queries(T2, rng, 300)
    o2, s2 = _dev(off2, sym2)
    assert np.array_equal(idx2.find(o2, s2, 300).cpu().numpy().view(np.uint64), oracle.find_batch(T2, sa2, off2, sym2))
    pos, cnt = idx.locate(itv, 500, 100)
    wp, wc = oracle.locate_batch(sa, want, 100)
    assert np.array_equal(cnt.cpu().numpy().view(np.uint32), wc)
    pn = pos.cpu().numpy().view(np.uint64)
    for i in range(0, 500, 7):
        assert np.array_equal(pn[i, :wc[i]], wp[i, :wc[i]])


def test_index_sharded_by_suffix_array_range(ctx, oracle):
    """Three slices of one suffix array, each with its own sample table: the per-slice counts add up to the oracle's interval
    and the slices' position windows add up to the oracle's positions."""
    from cascade_b200 import api, multi
    rng = np.random.default_rng(9)
    n = 150000
    T = rng.integers(0, 30, n).astype(np.uint16)
    T[rng.integers(0, 100, n) == 0] = 0xFFFF
    sa = oracle.build_sa40(T)
    Tp = np.concatenate([T, np.zeros(api.TEXT_PAD, np.uint16)])
    td = torch.from_numpy(Tp.view(np.int16)).cuda().view(torch.uint16)
    cuts = [0, 40000, 40064, 100032, n]          # slice starts are multiples of 4 entries (4-byte aligned bytes); one tiny slice
    off, sym, _ = conftest.fixture_queries(T, rng, 600)
    o, s_ = _dev(off, sym)
    want = oracle.find_batch(T, sa, off, sym)
    total = torch.zeros(1200, dtype=torch.int64, device="cuda")
    shards = []
    for a, b in zip(cuts[:-1], cuts[1:]):
        sl = np.concatenate([sa[5 * a:5 * b], np.zeros(128, np.uint8)])
        sh = multi.ShardedIndex(ctx, td, torch.from_numpy(sl).cuda(), n, a, b - a, stride=32)
        shards.append(sh)
        total += sh.find(o, s_, 600, reduce=False)
    assert np.array_equal(total.cpu().numpy().view(np.uint64), want)
    # the packed form: every shard adds its entries to one packed array (here one after another into the same array)
    packed = None
    for sh in shards:
        pos, poff, cnt = sh.locate_packed(total, 600, 100, reduce=False)
        packed = pos.clone() if packed is None else packed + pos
    wp0, wc0 = oracle.locate_batch(sa, want, 100)
    pk, po = packed.cpu().numpy().view(np.uint64), poff.cpu().numpy()
    assert np.array_equal(cnt.cpu().numpy().view(np.uint32), wc0) and int(po[-1]) == int(wc0.sum())
    for i in range(600):
        assert np.array_equal(pk[int(po[i]):int(po[i + 1])], wp0[i, :wc0[i]]), i
    rows = torch.zeros(600 * 100, dtype=torch.int64, device="cuda")
    for sh in shards:
        sh.local.locate_window(total, 600, 100, rows)
    wp, wc = oracle.locate_batch(sa, want, 100)
    rn = rows.view(600, 100).cpu().numpy().view(np.uint64)
    for i in range(600):
        assert np.array_equal(rn[i, :wc[i]], wp[i, :wc[i]]), i


def test_host_batches_of_several_chunks_over_the_lanes(ctx, oracle):
    """A host batch larger than one chunk (2^18 queries) runs as a pipeline of chunks over three streams; its intervals,
    counts, offsets and packed positions must be those of the device path and of the oracle. The same with the suffix array
    in pinned host memory (one lane), and with a positions buffer that is too small."""
    from cascade_b200 import api
    n = 1 << 20
    Td = api.gen_corpus_device(ctx, n, 2, 256)
    sa, _ = api.build_sa(ctx, Td, n, 4)
    Th = Td.cpu().view(torch.int16).numpy().view(np.uint16)
    sa_h = sa.cpu().numpy()
    idx = api.SuffixIndex(ctx, Td, sa, n, 32)
    q = 700_001                                                  # two full chunks and a ragged third
    oa, sa_ = api.gen_queries("substring", Th, n, q // 2, seed=5)
    ob, sb = api.gen_queries("random", None, 0, q - q // 2, seed=6)
    off = np.concatenate([oa, ob[1:] + oa[-1]])
    sym = np.concatenate([sa_, sb, np.zeros(8, np.uint16)])
    o, s = _dev(off, sym)
    itv_d = idx.find(o, s, q)
    pos_d, cnt_d = idx.locate(itv_d, q, 20)
    want_itv = itv_d.cpu().numpy().view(np.uint64)
    want_cnt = cnt_d.cpu().numpy().view(np.uint32)
    want_pos = pos_d.cpu().numpy().view(np.uint64)
    sample = np.arange(0, q, 1013)
    sub_off = np.zeros(len(sample) + 1, np.uint64)
    sub_off[1:] = np.cumsum(off[sample + 1] - off[sample])
    sub_sym = np.concatenate([sym[int(off[i]):int(off[i + 1])] for i in sample])
    assert np.array_equal(want_itv.reshape(q, 2)[sample].ravel(), oracle.find_batch(Th[:n], sa_h, sub_off, sub_sym))
    for index in (idx, api.SuffixIndex(ctx, Td, sa.cpu().pin_memory(), n, 32, table=idx.table)):
        itv_h, cnt_h, poff_h, pos_h, total = index.query_host(off, sym, 20)
        assert np.array_equal(itv_h, want_itv)
        assert np.array_equal(cnt_h, want_cnt) and total == int(want_cnt.sum()) and int(poff_h[-1]) == total
        assert np.array_equal(poff_h[:-1], np.concatenate([[0], np.cumsum(want_cnt.astype(np.uint64))[:-1]]))
        for i in list(range(0, q, 4999)) + [262143, 262144, 524287, 524288, q - 1]:
            assert np.array_equal(pos_h[int(poff_h[i]):int(poff_h[i + 1])], want_pos[i, :want_cnt[i]]), i
    # counts only
    itv_h, _, _, _, total = idx.query_host(off, sym, 0)
    assert np.array_equal(itv_h, want_itv) and total == 0
    # a positions buffer that is too small: refused, and the caller learns how many words are needed
    small = {"pos": np.zeros(1000, np.uint64)}
    with pytest.raises(api.CascadeError) as e:
        idx.query_host(off, sym, 20, small)
    assert e.value.code == 3
