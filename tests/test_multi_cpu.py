"""Host side of the multi-GPU build, on CPU: the shard plan, and the caller-supplied all-gather between two gloo ranks."""
import ctypes
import os
import socket
import sys

import numpy as np
import torch.multiprocessing as mp

from conftest import ROOT


def _check_plan(hist_all, world, policy):
    from cascade_b200 import multi
    part_off, owner, local_first, local_count, cursor = multi.plan_shards(hist_all, world, policy)
    p = hist_all.shape[1]
    sizes = hist_all.sum(axis=0)
    n = int(sizes.sum())
    assert part_off[0] == 0 and np.array_equal(np.diff(part_off.astype(np.int64)), sizes.astype(np.int64))
    assert owner.max() < world and int(local_count.sum()) == n
    if policy == 0:
        assert np.all(np.diff(owner.astype(np.int64)) >= 0)          # contiguous blocks of partitions
    elif p >= world:
        assert np.array_equal(owner, np.arange(p) % world)           # dealt round
    # every GPU keeps its partitions one after another, in increasing order, without gaps
    for g in range(world):
        at = 0
        for q in range(p):
            if owner[q] == g:
                assert local_first[q] == at
                at += int(sizes[q])
        assert at == local_count[g]
    for q in range(p):      # the ranks' runs inside a partition tile it exactly
        assert cursor[0, q] == 0
        for r in range(1, world):
            assert cursor[r, q] == cursor[r - 1, q] + hist_all[r - 1, q]
    return local_count


def test_plan_is_balanced_and_consistent():
    rng = np.random.default_rng(0)
    for policy in (0, 1):
        for world in (1, 2, 4, 8):
            for p in (1, 3, 64, 500):
                h = rng.integers(0, 1000, size=(world, p)).astype(np.uint64)
                local_count = _check_plan(h, world, policy)
                if p >= 64:
                    n = int(h.sum())
                    slack = 2 * int(h.sum(axis=0).max()) if policy == 0 else 0.35 * n / world      # dealing round balances on average only (the sizes here are random)
                    assert int(local_count.max()) <= n / world + slack
        # degenerate: everything in one partition, more GPUs than partitions
        h = np.zeros((4, 2), np.uint64)
        h[:, 1] = 10
        _check_plan(h, 4, policy)


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _gloo_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from cascade_b200 import multi
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    comm, keep = multi.make_comm(rank, world, None)
    p = 16
    mine = (np.arange(p, dtype=np.uint64) + 1) * np.uint64(rank + 1)           # this rank's partition sizes
    allh = np.zeros(world * p, np.uint64)
    rc = comm.allgather(None, mine.ctypes.data, allh.ctypes.data, mine.nbytes)   # the call the library makes
    assert rc == 0
    part_off, owner, local_first, local_count, cursor = multi.plan_shards(allh.reshape(world, p), world)
    q.put((rank, allh.tolist(), part_off.tolist(), owner.tolist(), local_first.tolist(), local_count.tolist()))
    dist.barrier()
    dist.destroy_process_group()


def test_allgather_callback_between_two_gloo_ranks():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gloo_worker, args=(r, world, port, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for pr in procs:
        pr.join(timeout=60)
        assert pr.exitcode == 0
    assert res[0][1:] == res[1][1:], "the ranks must see the same sizes and make the same plan"
    want = [(i + 1) * (r + 1) for r in range(world) for i in range(16)]
    assert res[0][1] == want


def _upload_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from cascade_b200 import multi
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    ok = True
    scratch = None
    for n in (1, 17, 100003):                       # shares are whole 16-byte pieces; the last rank's may be short or empty
        host = ((torch.arange(n, dtype=torch.int64) * 2654435761) % 65521).to(torch.int32).to(torch.uint16)
        dev = torch.zeros(n, dtype=torch.uint16)
        scratch = multi.upload_text_sharded(host, dev, scratch)
        ok = ok and torch.equal(dev.view(torch.int16), host.view(torch.int16))
    q.put((rank, ok))
    dist.barrier()
    dist.destroy_process_group()


def test_text_upload_in_shares_with_all_gather_between_three_gloo_ranks():
    world, port = 3, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_upload_worker, args=(r, world, port, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for pr in procs:
        pr.join(timeout=60)
        assert pr.exitcode == 0
    assert res == [(r, True) for r in range(world)]


def _shm_worker(rank, world, name, q):
    sys.path.insert(0, ROOT)
    from cascade_b200 import multi
    comm, close = multi.make_shm_comm(rank, world, name)
    out = []
    for rnd in range(200):                       # many rounds: the two payload buffers of a rank alternate
        mine = np.full(5, rank * 1000 + rnd, np.uint64)
        allv = np.zeros(5 * world, np.uint64)
        assert comm.allgather(comm.user, mine.ctypes.data, allv.ctypes.data, mine.nbytes) == 0
        out.append(allv.reshape(world, 5)[:, 0].tolist())
    big = np.zeros(49 * 1024, np.uint8)          # beyond the per-rank payload limit: refused, not truncated
    assert comm.allgather(comm.user, big.ctypes.data, big.ctypes.data, big.nbytes) != 0
    q.put((rank, out))
    close()


def test_shared_memory_allgather_between_processes():
    world, name = 3, f"/cascade_b200_test_{os.getpid()}"
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_shm_worker, args=(r, world, name, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for pr in procs:
        pr.join(timeout=60)
        assert pr.exitcode == 0
    for rank, out in res:
        for rnd, row in enumerate(out):
            assert row == [r * 1000 + rnd for r in range(world)]


def _open(lib, name, rank, world):
    from cascade_b200._lib import Comm
    comm = Comm()
    rc = lib.csa_comm_open_shm(name.encode(), rank, world, 1, ctypes.byref(comm))
    return rc, comm


def test_a_leftover_object_of_the_same_name_is_replaced_not_reused():
    """A finished or crashed job may leave its object behind (its round counters are far ahead, its payloads are old). The
    next job with that name must start from a fresh object: rank 0 replaces it, the other ranks refuse the old one."""
    import threading
    from multiprocessing import shared_memory
    from cascade_b200._lib import lib
    L = lib()
    name, world = f"/cascade_b200_stale_{os.getpid()}", 2
    # the old job's object: same size, marked live, every rank 57 rounds in, payloads full of junk
    slot = 64 + 2 * 48 * 1024
    size = 64 + world * slot
    old = shared_memory.SharedMemory(name=name.lstrip("/"), create=True, size=size)
    buf = np.frombuffer(old.buf, dtype=np.uint8)
    buf[:] = 0xAB
    np.frombuffer(old.buf, dtype=np.uint64, count=2)[:] = (0x4353415F4C495645, world)
    for g in range(world):
        np.frombuffer(old.buf, dtype=np.uint64, count=1, offset=64 + g * slot)[:] = 57
    res = {}

    def rank_body(rank, delay):
        import time
        time.sleep(delay)
        rc, comm = _open(L, name, rank, world)
        assert rc == 0
        got = []
        for rnd in range(3):
            mine = np.full(4, 100 * rank + rnd, np.uint64)
            allv = np.zeros(4 * world, np.uint64)
            got.append((comm.allgather(comm.user, mine.ctypes.data, allv.ctypes.data, mine.nbytes), allv.reshape(world, 4)[:, 0].tolist()))
        res[rank] = got
        L.csa_comm_close_shm(ctypes.byref(comm), 1 if rank == 0 else 0)

    # rank 1 arrives first and finds only the leftover; it must wait for rank 0's fresh object
    ts = [threading.Thread(target=rank_body, args=(1, 0.0)), threading.Thread(target=rank_body, args=(0, 0.3))]
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=60)
    del buf
    old.close()
    try:
        old.unlink()
    except FileNotFoundError:
        pass
    for rank in range(world):
        assert res[rank] == [(0, [rnd, 100 + rnd]) for rnd in range(3)], res


def test_a_missing_rank_makes_the_others_fail_within_the_limit():
    import threading
    import time
    from cascade_b200._lib import lib
    L = lib()
    name, world = f"/cascade_b200_missing_{os.getpid()}", 3
    out = {}

    def rank_body(rank):
        rc, comm = _open(L, name, rank, world)
        assert rc == 0
        assert L.csa_comm_shm_set_timeout(ctypes.byref(comm), 1.0) == 0
        mine = np.full(2, rank, np.uint64)
        allv = np.zeros(2 * world, np.uint64)
        t0 = time.perf_counter()
        rc = comm.allgather(comm.user, mine.ctypes.data, allv.ctypes.data, mine.nbytes)
        out[rank] = (rc, time.perf_counter() - t0)
        L.csa_comm_close_shm(ctypes.byref(comm), 1 if rank == 0 else 0)

    ts = [threading.Thread(target=rank_body, args=(r,)) for r in (0, 1)]        # rank 2 never comes
    for t in ts:
        t.start()
    for t in ts:
        t.join(timeout=60)
    for r in (0, 1):
        rc, dt = out[r]
        assert rc != 0 and 0.9 < dt < 10.0, out
    # a rank other than 0 that finds no object at all gives up too
    os.environ["CASCADE_COMM_TIMEOUT_S"] = "0.5"
    try:
        t0 = time.perf_counter()
        rc, _ = _open(L, name + "_nobody", 1, 2)
        assert rc == 6 and time.perf_counter() - t0 < 10.0
    finally:
        del os.environ["CASCADE_COMM_TIMEOUT_S"]


def test_stretches_are_whole_address_buckets_and_cover_the_text():
    from cascade_b200 import multi
    for n in (1, 63, 64, 65, 1000, 700_001, 2_000_000_000, 4_500_000_000, 16_000_000_000, (1 << 40) - 1):
        begin, end = multi.address_bits(n)
        assert 0 <= begin < end and (n - 1) >> end == 0 and end - begin <= 16
        assert end - begin <= 8 or begin > 9, "two digit passes only for texts whose one-pass buckets would pass the L2"
        for world in (1, 2, 3, 4, 8):
            bounds = [multi.shard_bounds(n, world, r) for r in range(world)]
            stretch = bounds[0][0]
            assert stretch % 64 == 0 and stretch % (1 << begin) == 0 and stretch * world >= n
            at = 0
            for s, lo, hi in bounds:
                assert s == stretch and lo == min(n, at) and lo <= hi <= n and hi - lo <= stretch
                at += stretch
            assert bounds[-1][2] == n and sum(hi - lo for _, lo, hi in bounds) == n


def _sharded_host_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist
    from cascade_b200 import multi
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # every rank's view of small per-rank arrays
    seen = multi._gather_small(np.array([rank, 10 * rank + 1], np.int64))
    # the entries that follow a rank's stretch: rank 0 holds 5 entries, rank 1 two, rank 2 none, rank 3 four
    valid = [5, 2, 0, 4][rank]
    local = torch.arange(100 * rank, 100 * rank + 8, dtype=torch.int16)
    halo = multi._halo_from_next(local, valid, 4)
    # runs per destination: rank r sends (d + 1) entries worth r * 1000 + d to rank d, twice as many bytes when width is 2
    counts = [d + 1 for d in range(world)]
    incoming = [rank + 1] * world
    send = torch.cat([torch.full((d + 1,), rank * 1000 + d, dtype=torch.int64) for d in range(world)])
    got = multi._exchange(send, counts, incoming)
    send2 = torch.cat([torch.full((2 * (d + 1),), rank * 1000 + d, dtype=torch.int32) for d in range(world)])
    got2 = multi._exchange(send2, counts, incoming, width=2)
    q.put((rank, seen.tolist(), halo.tolist(), got.tolist(), got2.tolist()))
    dist.barrier()
    dist.destroy_process_group()


def test_halo_exchange_and_runs_between_four_gloo_ranks():
    """The host-side pieces of the build with text and rank store sharded by position: what every rank learns of the others'
    counts, the entries that follow a stretch (taken from as many following ranks as it needs, zeros past the end), and the
    all-to-all of per-destination runs."""
    world, port = 4, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_sharded_host_worker, args=(r, world, port, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for pr in procs:
        pr.join(timeout=60)
        assert pr.exitcode == 0
    for rank, seen, halo, got, got2 in res:
        assert seen == [[r, 10 * r + 1] for r in range(world)]
        want = [s * 1000 + rank for s in range(world) for _ in range(rank + 1)]
        assert got == want and got2 == [x for x in want for _ in range(2)]
    assert res[0][2] == [100, 101, 300, 301]           # two entries of rank 1, none of rank 2, then rank 3's
    assert res[1][2] == [300, 301, 302, 303]
    assert res[2][2] == [300, 301, 302, 303]
    assert res[3][2] == [0, 0, 0, 0]                   # nothing follows the last stretch


def test_partitions_are_grouped_into_parts_in_order():
    """Parts are runs of whole partitions in partition order, each within the bound unless one partition alone passes it; the
    ranks of a sharded build own runs of consecutive parts whose sizes differ by at most one part."""
    import pytest
    from cascade_b200 import api, multi
    rng = np.random.default_rng(5)
    for p, bound in ((1, 100), (64, 1000), (300, 50), (4096, 1 << 20)):
        sizes = rng.integers(0, 400, p).astype(np.uint64)
        part_of_pid, part_off = multi.group_partitions_into_parts(sizes, bound)
        parts = len(part_off) - 1
        assert part_off[0] == 0 and part_off[-1] == int(sizes.sum()) and np.all(np.diff(part_of_pid.astype(np.int64)) >= 0)
        assert int(part_of_pid[-1]) == parts - 1 and np.all(np.diff(part_of_pid.astype(np.int64)) <= 1)
        for u in range(parts):
            inside = sizes[part_of_pid == u]
            assert int(inside.sum()) == part_off[u + 1] - part_off[u]
            assert int(inside.sum()) <= bound or int(np.count_nonzero(inside)) == 1
        for world in (1, 2, 3, 8):
            owner = [u * world // parts for u in range(parts)]
            held = np.bincount(owner, minlength=world)
            assert owner == sorted(owner) and held.max() - held.min() <= 1
    with pytest.raises(api.CascadeError):
        multi.group_partitions_into_parts(np.array([1 << 31], np.uint64), 1 << 27)
