"""The build driven part by part (5-byte lanes, ranks local to a part, suffix lists in host memory) against the golden
fixtures and the oracle: byte-for-byte equal sa40 arrays, also with every position pushed above 2^32, and the part jobs
called one by one through the C ABI as a host pipeline would call them."""
import ctypes
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


def _padded(T):
    from cascade_b200 import api
    return np.concatenate([np.ascontiguousarray(T, np.uint16), np.zeros(api.TEXT_PAD, np.uint16)])


@pytest.mark.parametrize("p,part_suffixes", [(1, 0), (3, 50), (64, 7), (64, 5000)])
def test_golden_sa_fixtures(ctx, p, part_suffixes):
    from cascade_b200 import api
    g = np.load(os.path.join(GOLDEN, "sa_fixtures.npz"))
    for name in [k[2:] for k in g.files if k.startswith("T_")]:
        T, want = g["T_" + name], g["SA_" + name]
        sa, st = api.build_sa_streamed(ctx, _padded(T), len(T), p, part_suffixes=part_suffixes)
        got = sa40_to_u64(sa, len(T)).astype(np.uint32)
        assert np.array_equal(got, want), (name, p, part_suffixes)
        assert np.all(sa[5 * len(T):] == 0), "bytes past the array must stay untouched"


@pytest.mark.parametrize("n,sigma,p,part_suffixes", [(100000, 2, 16, 20000), (300000, 4, 8, 0), (1 << 20, 50000, 64, 100000), (777777, 3, 5, 1000)])
def test_random_texts_against_oracle(ctx, oracle, n, sigma, p, part_suffixes):
    from cascade_b200 import api
    rng = np.random.default_rng(n + sigma)
    T = rng.integers(0, sigma, n).astype(np.uint16)
    T[rng.integers(0, 300, n) == 0] = 0xFFFF
    sa, st = api.build_sa_streamed(ctx, _padded(T), n, p, part_suffixes=part_suffixes)
    want = oracle.build_sa40(T)
    assert np.array_equal(sa[:5 * n], want[:5 * n])


def test_zipf_and_repetitive_corpora_equal_the_resident_build(ctx, oracle):
    from cascade_b200 import api
    n = 1 << 21
    Th = api.gen_corpus_host(n, 0, 512)
    pinned_text = torch.from_numpy(Th.view(np.int16)).pin_memory()
    pinned_out = torch.zeros(5 * n + api.SA_PAD_BYTES, dtype=torch.uint8).pin_memory()
    sa, st = api.build_sa_streamed(ctx, pinned_text, n, 64, out=pinned_out, part_suffixes=300000)
    want = oracle.build_sa40(Th[:n])
    assert np.array_equal(pinned_out.numpy()[:5 * n], want[:5 * n])
    assert st.partitions > 8 and st.generations >= 1
    n = 600000
    T = api.gen_repeat_corpus_host(n, seed=0, base_docs=16, mean_doc=2048, mutate=0.001)
    sa, st = api.build_sa_streamed(ctx, T, n, 8, part_suffixes=150000)
    assert st.generations >= 6, "long shared suffixes need many doubling generations"
    assert oracle.is_correct(T[:n], sa)
    assert np.array_equal(sa[:5 * n], oracle.build_sa40(T[:n])[:5 * n])


def test_positions_above_32_bits(ctx, oracle):
    """With the test offset every lane, message and output entry carries position + 2^33 + 5: the 5-byte paths are
    exercised end to end on a text that the oracle can sort."""
    from cascade_b200 import api
    from cascade_b200._lib import lib
    n = 400000
    off = (1 << 33) + 5
    Th = api.gen_corpus_host(n, 3, 256)
    assert lib().csa_debug_set(4, off) == 0
    try:
        sa, st = api.build_sa_streamed(ctx, Th, n, 16, part_suffixes=90000)
    finally:
        assert lib().csa_debug_set(4, 0) == 0
    got = sa40_to_u64(sa, n)
    assert int(got.min()) >= off
    want = sa40_to_u64(oracle.build_sa40(Th[:n]), n)
    assert np.array_equal(got - np.uint64(off), want)


def test_part_jobs_called_one_by_one(ctx, oracle):
    """A host pipeline in a few lines: partition ids, parts of whole partitions, generation 0 and the later generations
    part by part with the exchange in between, then the final order; lists in device memory for one part, in host memory for
    the others. The result must be the oracle's array."""
    from cascade_b200 import api
    from cascade_b200._lib import Part, PartResult, c_u64, c_vp
    L = ctx.L
    n, p = 250_000, 8
    rng = np.random.default_rng(17)
    T = rng.integers(0, 6, n).astype(np.uint16)
    T[rng.integers(0, 200, n) == 0] = 0xFFFF
    Td = torch.from_numpy(_padded(T).view(np.int16)).cuda().view(torch.uint16)
    # splitters and partition ids
    ns = 8192
    samples = torch.zeros(2 * ns, dtype=torch.int64, device="cuda")
    ctx.check(L.csa_sample_kgrams(ctx.h, Td.data_ptr(), n, ns, 1, samples.data_ptr()))
    ctx.sync()
    sh = samples.cpu().numpy().view(np.uint64)
    piv = np.zeros(2 * (p - 1), np.uint64)
    p_eff = ctypes.c_uint32(0)
    assert L.csa_select_pivots(sh.ctypes.data, ns, p, piv.ctypes.data, ctypes.byref(p_eff)) == 0
    pe = p_eff.value
    pivd = torch.from_numpy(piv.view(np.int64)).cuda()
    pid = torch.zeros(n + 64, dtype=torch.int16, device="cuda")
    hist = torch.zeros(pe, dtype=torch.int64, device="cuda")
    ctx.check(L.csa_partition_ids(ctx.h, Td.data_ptr(), n, 0, n, pivd.data_ptr(), pe, pid.data_ptr(), hist.data_ptr()))
    ctx.sync()
    sizes = hist.cpu().numpy()
    assert sizes.sum() == n
    # two partitions to a part
    part_of_pid = (np.arange(pe) // 2).astype(np.uint16)
    parts = int(part_of_pid.max()) + 1
    pid_h = pid[:n].cpu().numpy().view(np.uint16)
    part_of_pos = part_of_pid[pid_h]
    store = c_vp()
    ctx.check(L.csa_store_create(ctx.h, Td.data_ptr(), n, pid.data_ptr(), part_of_pid.ctypes.data, pe, None, ctypes.byref(store)))
    try:
        lanes, ranks, active = [], [], []
        for u in range(parts):
            pos = np.flatnonzero(part_of_pos == u).astype(np.uint64)
            b = np.zeros(5 * len(pos) + 64, np.uint8)
            for k in range(5):
                b[:5 * len(pos)].reshape(-1, 5)[:, k] = ((pos >> np.uint64(8 * k)) & np.uint64(0xFF)).astype(np.uint8)
            if u == 1:      # this part's lists live in device memory
                lanes.append(torch.from_numpy(b).cuda()); ranks.append(torch.zeros(len(pos) + 16, dtype=torch.int32, device="cuda"))
            else:
                lanes.append(torch.from_numpy(b).pin_memory()); ranks.append(torch.zeros(len(pos) + 16, dtype=torch.int32).pin_memory())
            active.append(len(pos))
        count = list(active)
        for u in range(parts):
            pin, pout = Part(lanes[u].data_ptr(), None, count[u], u), PartResult(lanes[u].data_ptr(), ranks[u].data_ptr(), 0, 0)
            ctx.check(L.csa_rank_gen0(ctx.h, store, ctypes.byref(pin), ctypes.byref(pout)))
            ctx.sync()
            active[u] = int(pout.active)
            assert pout.messages == 0
        L.csa_store_drop_partition_ids(store)
        h, gens = 3, 0
        while sum(active) > 0:
            ctx.check(L.csa_store_reserve_messages(ctx.h, store, sum(active)))
            sent = 0
            for u in range(parts):
                if active[u] == 0:
                    continue
                pin = Part(lanes[u].data_ptr(), ranks[u].data_ptr(), active[u], u)
                pout = PartResult(lanes[u].data_ptr(), ranks[u].data_ptr(), 0, 0)
                ctx.check(L.csa_rank_gen(ctx.h, store, ctypes.byref(pin), h, ctypes.byref(pout)))
                ctx.sync()
                assert pout.active <= active[u] and pout.messages == active[u]
                sent += active[u]
                active[u] = int(pout.active)
            applied = c_u64(0)
            ctx.check(L.csa_exchange_messages(ctx.h, store, ctypes.byref(applied)))
            assert applied.value == sent
            h *= 2
            gens += 1
            assert gens < 40
        out = np.zeros(5 * n + 128, np.uint8)
        at = 0
        for u in range(parts):
            # ranks of a finished part are a permutation of its slots
            r = ranks[u][:count[u]].cpu().numpy()
            assert np.array_equal(np.sort(r), np.arange(count[u]))
            seg = torch.zeros(5 * count[u] + 64, dtype=torch.uint8).pin_memory()
            ctx.check(L.csa_rank_order(ctx.h, lanes[u].data_ptr(), ranks[u].data_ptr(), count[u], seg.data_ptr()))
            ctx.sync()
            out[5 * at:5 * (at + count[u])] = seg.numpy()[:5 * count[u]]
            at += count[u]
    finally:
        L.csa_store_destroy(store)
    assert gens >= 1
    assert np.array_equal(out[:5 * n], oracle.build_sa40(T)[:5 * n])


@pytest.mark.parametrize("bound_fraction,keep_array", [(0.0, True), (0.4, True), (0.4, False), (None, False)])
def test_lists_in_files_give_the_same_array(ctx, oracle, tmp_path, bound_fraction, keep_array):
    """Tiers of the part-by-part build: with a host bound of nothing every part's lists go through files, with 40 % of the
    lists' size the first parts stay in host memory; the array must be the oracle's, in memory and in the output file, and
    the scratch directory must be empty again afterwards."""
    from cascade_b200 import api
    n = 700_000
    Th = api.gen_corpus_host(n, 5, 384)
    scratch = tmp_path / "scratch"
    scratch.mkdir()
    out_path = tmp_path / "sa.bin"
    bound = None if bound_fraction is None else int(9 * n * bound_fraction)
    sa, st = api.build_sa_tiered(ctx, Th, n, 32, part_suffixes=60_000, host_list_bytes=bound, scratch_dir=scratch, output_path=out_path,
                                 out=None if keep_array else False)
    want = oracle.build_sa40(Th[:n])[:5 * n]
    assert np.array_equal(np.fromfile(out_path, dtype=np.uint8), want)
    if keep_array:
        assert np.array_equal(sa[:5 * n], want)
    assert list(scratch.iterdir()) == []
    assert st.host_parts + st.file_parts >= 10
    if bound_fraction == 0.0:
        assert st.host_parts == 0 and st.file_bytes_written >= 9 * n and st.file_bytes_read >= 9 * n
    elif bound_fraction is None:
        assert st.file_parts == 0 and st.file_bytes_written == 0
    else:
        assert st.host_parts > 0 and st.file_parts > 0


def test_tiered_build_refusals(ctx, tmp_path):
    from cascade_b200 import api
    n = 100_000
    Th = api.gen_corpus_host(n, 1, 256)
    with pytest.raises(api.CascadeError) as e:      # the bound is passed and there is nowhere to put the lists
        api.build_sa_tiered(ctx, Th, n, 8, part_suffixes=20_000, host_list_bytes=1000)
    assert e.value.code == 3 and "scratch" in str(e.value)
    with pytest.raises(api.CascadeError) as e:      # a scratch directory that does not exist
        api.build_sa_tiered(ctx, Th, n, 8, part_suffixes=20_000, host_list_bytes=1000, scratch_dir=tmp_path / "nowhere")
    assert e.value.code == 1
    with pytest.raises(api.CascadeError):           # no array and no file
        api.build_sa_tiered(ctx, Th, n, 8, out=False)
    sa, st = api.build_sa_streamed(ctx, Th, n, 8)    # the context still works
    assert st.n == n


def test_rank_shard_primitives(ctx):
    """The pieces a sharded rank store is driven with, one by one against numpy: positions ordered into runs per owner (by
    address or just by owner), a stretch answering requests and taking messages, answers put back into request order, and the
    outbox's split positions joined; a request outside the stretch is reported, not served."""
    L = ctx.L
    rng = np.random.default_rng(3)
    n, owners = 1_000_000, 3
    end = int(n - 1).bit_length()
    begin = end - 8
    unit = max(64, 1 << begin)
    stretch = (-(-n // owners) + unit - 1) // unit * unit
    m = 300_001
    pos = rng.integers(0, n, m).astype(np.uint64)
    pay = rng.integers(0, 1 << 31, m).astype(np.uint32)
    for by_address in (False, True):
        pd = torch.from_numpy(pos.view(np.int64)).cuda()
        yd = torch.from_numpy(pay.view(np.int32)).cuda()
        counts = np.zeros(owners, np.uint64)
        if by_address:
            pa, ya = torch.empty_like(pd), torch.empty_like(yd)
            wsb = L.csa_sort_workspace_bytes(m)
            ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
            in_alt = ctypes.c_int(0)
            torch.cuda.synchronize()
            ctx.check(L.csa_order_by_address(ctx.h, pd.data_ptr(), pa.data_ptr(), yd.data_ptr(), ya.data_ptr(), m, begin, end, stretch, owners, 1,
                                             counts.ctypes.data, ws.data_ptr(), wsb, ctypes.byref(in_alt)))
            ctx.sync()
            got_pos = (pa if in_alt.value else pd).cpu().numpy().view(np.uint64)
            order = (ya if in_alt.value else yd).cpu().numpy().view(np.uint32)
            assert np.all(np.diff((got_pos >> np.uint64(begin)).astype(np.int64)) >= 0), "buckets must ascend"
        else:
            po, yo, od = torch.empty_like(pd), torch.empty_like(yd), torch.empty(m, dtype=torch.int32, device="cuda")
            torch.cuda.synchronize()
            ctx.check(L.csa_bucket_by_owner(ctx.h, pd.data_ptr(), yd.data_ptr(), m, stretch, owners, counts.ctypes.data, po.data_ptr(), yo.data_ptr(), od.data_ptr()))
            ctx.sync()
            got_pos, order = po.cpu().numpy().view(np.uint64), od.cpu().numpy().view(np.uint32)
            assert np.array_equal(yo.cpu().numpy().view(np.uint32), pay[order])
        assert np.array_equal(counts, np.bincount((pos // np.uint64(stretch)).astype(np.int64), minlength=owners).astype(np.uint64))
        assert np.array_equal(got_pos, pos[order]) and np.array_equal(np.sort(order), np.arange(m, dtype=np.uint32))
        assert np.all(np.diff((got_pos // np.uint64(stretch)).astype(np.int64)) >= 0), "one run per owner, in owner order"
    # owner 1's stretch: apply messages, read them back, put the answers into the order of the requests
    lo, cnt = stretch, min(n, 2 * stretch) - stretch
    shard = torch.zeros(cnt + 16, dtype=torch.int32, device="cuda")
    mine = np.unique(pos[(pos >= lo) & (pos < lo + cnt)])
    ranks = rng.integers(1, 1 << 31, len(mine)).astype(np.uint32)
    md, rd = torch.from_numpy(mine.view(np.int64)).cuda(), torch.from_numpy(ranks.view(np.int32)).cuda()
    torch.cuda.synchronize()
    ctx.check(L.csa_rank_shard_apply(ctx.h, shard.data_ptr(), lo, cnt, md.data_ptr(), rd.data_ptr(), len(mine)))
    perm = rng.permutation(len(mine)).astype(np.uint32)
    asked = torch.from_numpy(mine[perm].view(np.int64)).cuda()
    ans = torch.zeros(len(mine), dtype=torch.int32, device="cuda")
    back = torch.zeros(len(mine), dtype=torch.int32, device="cuda")
    order_d = torch.from_numpy(perm.view(np.int32)).cuda()
    torch.cuda.synchronize()
    ctx.check(L.csa_rank_shard_read(ctx.h, shard.data_ptr(), lo, cnt, asked.data_ptr(), len(mine), ans.data_ptr()))
    ctx.check(L.csa_unbucket(ctx.h, order_d.data_ptr(), ans.data_ptr(), len(mine), back.data_ptr()))
    ctx.sync()
    assert np.array_equal(back.cpu().numpy().view(np.uint32), ranks)
    # the outbox keeps positions as low 32 and high 8 bits
    big = rng.integers(0, 1 << 40, 1000).astype(np.uint64)
    lo32 = torch.from_numpy((big & np.uint64(0xFFFFFFFF)).astype(np.uint32).view(np.int32)).cuda()
    hi8 = torch.from_numpy((big >> np.uint64(32)).astype(np.uint8)).cuda()
    joined = torch.zeros(1000, dtype=torch.int64, device="cuda")
    torch.cuda.synchronize()
    ctx.check(L.csa_outbox_positions(ctx.h, lo32.data_ptr(), hi8.data_ptr(), 1000, joined.data_ptr()))
    ctx.sync()
    assert np.array_equal(joined.cpu().numpy().view(np.uint64), big)
    # a request for a position of another stretch: answered with 0 and reported by the status word, no fault
    from cascade_b200 import api
    outside = torch.tensor([0], dtype=torch.int64, device="cuda")
    one = torch.full((1,), 7, dtype=torch.int32, device="cuda")
    torch.cuda.synchronize()
    ctx.check(L.csa_rank_shard_read(ctx.h, shard.data_ptr(), lo, cnt, outside.data_ptr(), 1, one.data_ptr()))
    with pytest.raises(api.CascadeError):
        ctx.sync()
    assert int(one.item()) == 0
    ctx.check(L.csa_rank_shard_read(ctx.h, shard.data_ptr(), lo, cnt, asked.data_ptr(), 1, one.data_ptr()))
    ctx.sync()                                        # the context works on
