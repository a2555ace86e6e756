"""The sharded build (csa_build_sa_multi) against the single-GPU build: the ranks' slices, concatenated, are the same
bytes. Two ranks run as two processes that meet through gloo; they use two GPUs where the box has them and share one
otherwise (the kernels never wait on a peer on the device, so ranks on one GPU cannot block one another)."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

from conftest import ROOT

pytestmark = pytest.mark.gpu


def test_world_of_one_equals_the_single_gpu_build():
    from cascade_b200 import api, multi
    ctx = api.Context(0)
    try:
        n = 2_000_000
        T = api.gen_corpus_device(ctx, n, 3, 512)
        ref, _ = api.build_sa(ctx, T, n, 16)
        comm, keep = multi.make_comm(0, 1, None)
        out, segs, st = multi.build_sa_multi(ctx, comm, T, n, 16)
        assert segs[0][0] == 0 and sum(c for _, c in segs) == n and all(segs[k][0] + segs[k][1] == segs[k + 1][0] for k in range(len(segs) - 1))
        assert torch.equal(out[:5 * n], ref[:5 * n])
    finally:
        ctx.close()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, n, p, kind, policy, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from cascade_b200 import api, multi
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dev = rank % torch.cuda.device_count()
    torch.cuda.set_device(dev)
    ctx = api.Context(dev)
    if kind == "zipf":
        T = api.gen_corpus_device(ctx, n, 7, 512)
    else:
        Th = api.gen_repeat_corpus_host(n, seed=1, base_docs=8, mean_doc=1024, mutate=0.002)
        T = torch.from_numpy(Th.view(np.int16)).cuda().view(torch.uint16)
    if kind == "zipf" and policy == 1:
        comm, keep = multi.make_shm_comm(rank, world, f"/cascade_b200_t{port}", policy)      # the in-library shared-memory all-gather
    else:
        comm, keep = multi.make_comm(rank, world, None, policy)                              # the caller's torch.distributed all-gather
    for _ in range(2):      # twice: the second build reuses the peers' mappings
        out, segs, st = multi.build_sa_multi(ctx, comm, T, n, p)
    sl = out[:5 * sum(c for _, c in segs)].cpu().numpy()
    ref = None
    if rank == 0:
        r, _ = api.build_sa(ctx, T, n, p)
        ref = r[:5 * n].cpu().numpy()
    q.put((rank, segs, sl, ref, st.generations, st.peer_bytes))
    dist.barrier()
    if callable(keep) and not hasattr(keep, "restype"):
        keep()
    ctx.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,n,p,kind,policy", [(2, 3_000_000, 16, "zipf", 1), (2, 400_000, 8, "repeat", 1), (3, 1_000_003, 5, "zipf", 1),
                                                    (2, 1_500_000, 16, "zipf", 0), (2, 1_200_000, 300, "zipf", 1)])
def test_sharded_build_equals_the_single_gpu_build(world, n, p, kind, policy):
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, p, kind, policy, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    res = sorted(_collect(procs, q, world), key=lambda x: x[0])
    for pr in procs:
        pr.join(timeout=120)
        assert pr.exitcode == 0
    ref = res[0][3]
    covered = np.zeros(n, np.uint8)
    for rank, segs, sl, _, gens, peer in res:
        at = 0
        for first, count in segs:       # a rank's output holds its partitions one after another
            assert np.array_equal(sl[5 * at:5 * (at + count)], ref[5 * first:5 * (first + count)]), f"rank {rank}'s segment at {first} differs"
            covered[first:first + count] += 1
            at += count
        assert 5 * at == sl.size
        if policy == 0 and segs:
            assert all(segs[k][0] + segs[k][1] == segs[k + 1][0] for k in range(len(segs) - 1)), "contiguous blocks give one contiguous slice"
    assert np.all(covered == 1), "the ranks' segments tile the suffix array exactly"
    if kind == "repeat":
        assert res[0][4] >= 5
    assert sum(r[5] for r in res) > 0      # ranks and positions did cross between the GPUs' memories


def test_a_failing_all_gather_ends_the_build_with_a_comm_error_and_the_context_stays_usable():
    from cascade_b200 import api, multi
    from cascade_b200._lib import ALLGATHER_FN, Comm
    ctx = api.Context(0)
    try:
        n = 500_000
        T = api.gen_corpus_device(ctx, n, 3, 512)
        calls = []

        def broken(user, send, recv, nbytes):
            calls.append(int(nbytes))
            return 1 if len(calls) >= 2 else multi.make_comm(0, 1, None)[0].allgather(user, send, recv, nbytes)
        fn = ALLGATHER_FN(broken)
        with pytest.raises(api.CascadeError) as e:
            multi.build_sa_multi(ctx, Comm(0, 1, 1, fn, None), T, n, 8)
        assert e.value.code == 6 and len(calls) == 2          # CSA_E_COMM at the second all-gather; no further calls on a dead communicator
        assert len(set(calls)) == 1, "every all-gather of a build has one size"
        comm, keep = multi.make_comm(0, 1, None)
        out, segs, st = multi.build_sa_multi(ctx, comm, T, n, 8)
        ref, _ = api.build_sa(ctx, T, n, 8)
        assert torch.equal(out[:5 * n], ref[:5 * n])
    finally:
        ctx.close()


def _failing_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import time
    import torch.distributed as dist
    from cascade_b200 import api, multi
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dev = rank % torch.cuda.device_count()
    torch.cuda.set_device(dev)
    ctx = api.Context(dev)
    n, p = 1_000_000, 8
    T = api.gen_corpus_device(ctx, n, 7, 512)
    comm, close = multi.make_shm_comm(rank, world, f"/cascade_b200_f{port}")
    # rank 1's output buffer is too small for its slice: it alone can tell, yet both ranks must leave the build, and soon
    code = 0
    t0 = time.perf_counter()
    try:
        multi.build_sa_multi(ctx, comm, T, n, p, capacity=(1000 if rank == 1 else n))
    except api.CascadeError as e:
        code = e.code
    dt = time.perf_counter() - t0
    out, segs, st = multi.build_sa_multi(ctx, comm, T, n, p)           # the same contexts and communicator build normally afterwards
    ref, _ = api.build_sa(ctx, T, n, p)
    at, same = 0, True
    for first, count in segs:
        same = same and bool(torch.equal(out[5 * at:5 * (at + count)], ref[5 * first:5 * (first + count)]))
        at += count
    q.put((rank, code, dt, same))
    dist.barrier()
    close()
    ctx.close()
    dist.destroy_process_group()


def test_a_rank_that_fails_alone_takes_every_rank_out_of_the_build():
    world, port = 2, _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    res = sorted(q.get(timeout=240) for _ in range(world))
    for pr in procs:
        pr.join(timeout=120)
        assert pr.exitcode == 0
    assert res[1][1] == 3 and res[0][1] == 6, res          # CSA_E_NOMEM where it happened, CSA_E_COMM on the peer
    assert all(r[2] < 30 and r[3] for r in res), res


def _collect(procs, q, world, limit=240):
    """One result per rank from the queue. A rank that fails leaves the others waiting in a collective: they are ended at once
    instead of after their timeouts."""
    import queue as queue_module
    import time as time_module
    res, deadline = [], time_module.time() + limit
    while len(res) < world:
        try:
            res.append(q.get(timeout=1))
        except queue_module.Empty:
            failed = [pr for pr in procs if pr.exitcode not in (None, 0)]
            if failed or time_module.time() > deadline:
                for pr in procs:
                    if pr.is_alive():
                        pr.terminate()
                pytest.fail("a rank failed" if failed else "the ranks did not finish in time")
    return res


def _streamed_worker(rank, world, port, n, p, part_suffixes, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from cascade_b200 import api, multi
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dev = rank % torch.cuda.device_count()
    torch.cuda.set_device(dev)
    ctx = api.Context(dev)
    T = api.gen_corpus_device(ctx, n, 11, 256)
    # where the parts' lists live: wherever the device has room (one rank), all in host memory (two), some of each (three)
    budget = {1: None, 2: 0, 3: 9 * 130_000}[world]
    segs, info = multi.build_sa_streamed_multi(ctx, T, n, p, part_suffixes=part_suffixes, workers=2, list_budget_bytes=budget)
    assert (info["lists_on_host"] == 0) if world == 1 else (info["lists_on_device"] == 0) if world == 2 else (info["lists_on_device"] > 0 and info["lists_on_host"] > 0)
    ref = None
    if rank == 0:
        r, _ = api.build_sa(ctx, T, n, 16)
        ref = r[:5 * n].cpu().numpy()
    q.put((rank, [(f, c, t.numpy().copy()) for f, c, t in segs], ref, info["generations"], info["parts"]))
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world", [1, 2, 3])
def test_part_at_a_time_build_over_several_ranks(world):
    """Every rank ranks the parts it owns with its lists in its own host memory; the rank stores are replicas kept equal by
    an all-reduce after generation 0 and an all-gather of the outboxes after every later generation. The ranks' parts,
    put together, are the resident build's array."""
    n, p, part_suffixes = 700_001, 64, 50_000
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_streamed_worker, args=(r, world, port, n, p, part_suffixes, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    res = sorted(_collect(procs, q, world), key=lambda x: x[0])
    for pr in procs:
        pr.join(timeout=120)
        assert pr.exitcode == 0
    ref = res[0][2]
    covered = np.zeros(n, np.uint8)
    for rank, segs, _, gens, parts in res:
        assert parts >= 10 and gens >= 1
        for first, count, lanes in segs:
            assert np.array_equal(lanes, ref[5 * first:5 * (first + count)]), f"rank {rank}'s part at {first} differs"
            covered[first:first + count] += 1
    assert np.all(covered == 1)


def _sharded_worker(rank, world, port, n, p, part_suffixes, window, on_device, offset, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist
    from cascade_b200 import api, multi
    from cascade_b200._lib import lib
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    dev = rank % torch.cuda.device_count()
    torch.cuda.set_device(dev)
    ctx = api.Context(dev)
    T = api.gen_corpus_device(ctx, n, 11, 256)
    _, lo, hi = multi.shard_bounds(n, world, rank)
    mine = T[lo:hi].clone()                      # all that this rank gives the build
    if offset:
        assert lib().csa_debug_set(4, offset) == 0
    try:
        segs, info = multi.build_sa_sharded(ctx, mine, n, p, part_suffixes=part_suffixes, window_suffixes=window, lists_on_device=on_device)
        if on_device:
            # the same build with the parts left in device memory: the same bytes, and one range of the array per rank
            dsegs, _ = multi.build_sa_sharded(ctx, mine, n, p, part_suffixes=part_suffixes, window_suffixes=window, lists_on_device=True, output="device")
            assert len(dsegs) == len(segs)
            for (f, c, t), (df, dc, dt) in zip(segs, dsegs):
                assert (f, c) == (df, dc) and dt.is_cuda and torch.equal(dt.cpu(), t)
            assert all(a[0] + a[1] == b[0] for a, b in zip(dsegs[:-1], dsegs[1:])), "a rank's parts are consecutive ranges"
    finally:
        lib().csa_debug_set(4, 0)
    ref = None
    if rank == 0:
        r, _ = api.build_sa(ctx, T, n, 16)
        ref = r[:5 * n].cpu().numpy()
    q.put((rank, [(f, c, t.numpy().copy()) for f, c, t in segs], ref, info["generations"], info["parts"]))
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,n,p,part_suffixes,window,on_device,offset", [
    (1, 300_001, 64, 40_000, 100_000, True, 0),
    (2, 700_001, 64, 50_000, 120_000, False, 0),
    (3, 700_001, 300, 50_000, 1 << 28, True, 0),
    (3, 1_000, 8, 100, 300, None, 0),                        # stretches of a few hundred positions
    (3, 100, 4, 30, 50, None, 0),                            # the last rank holds no position at all
    (2, 5_000, 1, 1 << 27, 1 << 28, True, 0),                # one partition, one part
    (2, 400_000, 32, 60_000, 1 << 28, True, (1 << 33) + 5),   # every lane above 2^32
])
def test_build_with_text_and_rank_store_sharded_by_position(world, n, p, part_suffixes, window, on_device, offset):
    """Nothing is replicated: a rank holds its stretch of the text, of the partition ids and of the rank store only; keys and
    ranks travel between the ranks. The parts, put together, are the resident build's array (shifted by the test offset)."""
    from conftest import sa40_to_u64
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_sharded_worker, args=(r, world, port, n, p, part_suffixes, window, on_device, offset, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    res = sorted(_collect(procs, q, world), key=lambda x: x[0])
    for pr in procs:
        pr.join(timeout=120)
        assert pr.exitcode == 0
    ref = res[0][2]
    want = sa40_to_u64(ref, n) + np.uint64(offset)
    covered = np.zeros(n, np.uint8)
    for rank, segs, _, gens, parts in res:
        assert gens >= (1 if n >= 100_000 else 0)
        for first, count, lanes in segs:
            assert np.array_equal(sa40_to_u64(lanes, count), want[first:first + count]), f"rank {rank}'s part at {first} differs"
            covered[first:first + count] += 1
    assert np.all(covered == 1)
