"""Multi-GPU build, one process per GPU: the host plumbing (torch.distributed) around csa_build_sa_multi.

The library asks its caller for ONE collective, an all-gather of small host buffers (partition sizes, IPC handles,
active counts; it also serves as the barrier between the steps). Here it is torch.distributed.all_gather, on CPU
tensors under gloo and on device tensors under NCCL. All bulk data moves inside the library's kernels as peer loads
and stores.
"""
import ctypes
import json
import os
import time

import numpy as np
import torch
import torch.distributed as dist

from . import api
from ._lib import ALLGATHER_FN, BuildStats, Comm, c_u64


def make_comm(rank, world, device=None, policy=1):
    """Returns (Comm, keepalive). `device` is the torch device for NCCL groups, None for gloo. policy: 0 deals the partitions
    to the GPUs in contiguous blocks, 1 (default) interleaves them."""
    def _allgather(user, send, recv, nbytes):
        try:
            n = int(nbytes)
            src = np.ctypeslib.as_array(ctypes.cast(send, ctypes.POINTER(ctypes.c_uint8)), shape=(n,))
            dst = np.ctypeslib.as_array(ctypes.cast(recv, ctypes.POINTER(ctypes.c_uint8)), shape=(n * world,))
            if world == 1:
                dst[:] = src
                return 0
            t = torch.from_numpy(src.copy())
            if device is not None:
                t = t.to(device)
            out = [torch.empty_like(t) for _ in range(world)]
            dist.all_gather(out, t)
            for r in range(world):
                dst[r * n:(r + 1) * n] = out[r].cpu().numpy()
            return 0
        except Exception as e:  # the C side turns a non-zero return into CSA_E_COMM
            print(f"[cascade_b200.multi] all-gather failed on rank {rank}: {e}", flush=True)
            return 1

    fn = ALLGATHER_FN(_allgather)
    return Comm(rank, world, policy, fn, None), fn


def make_shm_comm(rank, world, name, policy=1):
    """A communicator whose all-gather runs in the library over POSIX shared memory (ranks of one box). `name` must be the
    same on all ranks and unique to the job. Returns (Comm, close): call close() after the last build."""
    from ._lib import lib
    comm = Comm()
    rc = lib().csa_comm_open_shm(name.encode(), rank, world, policy, ctypes.byref(comm))
    if rc != 0:
        raise api.CascadeError(rc, "csa_comm_open_shm")

    def close():
        lib().csa_comm_close_shm(ctypes.byref(comm), 1 if rank == 0 else 0)
    return comm, close


def plan_shards(hist_all, world, policy=1):
    """Host-side shard plan (csa_plan_shards) from hist_all[world][p]. Returns (part_off, owner, local_first, local_count, cursor_all)."""
    from ._lib import lib
    hist_all = np.ascontiguousarray(hist_all, dtype=np.uint64)
    p = hist_all.shape[1]
    part_off = np.zeros(p + 1, np.uint64)
    owner = np.zeros(p, np.uint32)
    local_first = np.zeros(p, np.uint64)
    local_count = np.zeros(world, np.uint64)
    cursor = np.zeros((world, p), np.uint64)
    rc = lib().csa_plan_shards(hist_all.ctypes.data, p, world, policy, part_off.ctypes.data, owner.ctypes.data, local_first.ctypes.data,
                               local_count.ctypes.data, cursor.ctypes.data)
    if rc != 0:
        raise api.CascadeError(rc, "csa_plan_shards")
    return part_off, owner, local_first, local_count, cursor


def build_sa_multi(ctx, comm, text_dev, n, p, seed=0, out=None, capacity=None):
    """This rank's part of the suffix array of text_dev[0, n). Returns (sa40 tensor, segments, stats): the tensor holds the
    rank's partitions one after another; segments = [(first global rank, count), ...] in that order."""
    world = comm.world
    if capacity is None:
        capacity = n if world == 1 else min(n, n // world + n // max(1, min(p, 8)) + 1024)
    if out is None:
        out = torch.zeros(5 * capacity + api.SA_PAD_BYTES, dtype=torch.uint8, device=text_dev.device)
    st = BuildStats()
    seg_first = np.zeros(max(1, p), np.uint64)
    seg_count = np.zeros(max(1, p), np.uint64)
    seg_c = ctypes.c_uint32(0)
    torch.cuda.synchronize(text_dev.device)
    ctx.check(ctx.L.csa_build_sa_multi(ctx.h, ctypes.byref(comm), text_dev.data_ptr(), n, p, seed, out.data_ptr(), capacity,
                                       seg_first.ctypes.data, seg_count.ctypes.data, ctypes.byref(seg_c), ctypes.byref(st)))
    segs = [(int(seg_first[k]), int(seg_count[k])) for k in range(seg_c.value)]
    return out, segs, st


class ShardedIndex:
    """A query index sharded by suffix-array range over the ranks of a process group: every rank holds the whole text, the
    slice [first, first + count) of the 5-byte suffix array and a sample table over its slice. A batch is searched by every
    rank in its slice; the per-slice counts add up to the global interval (one all-reduce of 16 bytes per query), and every
    rank contributes the positions whose ranks it holds (one all-reduce of the position rows)."""

    def __init__(self, ctx, text_dev, sa40_slice_dev, n, first, count, stride=32):
        self.local = api.SuffixIndex(ctx, text_dev, sa40_slice_dev, n, stride, sa_first=first, sa_entries=count)
        self.n, self.first, self.count = n, first, count

    def find(self, off_dev, sym_dev, q, reduce=True):
        itv = self.local.find(off_dev, sym_dev, q)
        if reduce and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(itv, op=dist.ReduceOp.SUM)
        return itv

    def locate(self, itv_global_dev, q, max_pos=100, reduce=True):
        rows = torch.zeros(q * max_pos, dtype=torch.int64, device=itv_global_dev.device)
        self.local.locate_window(itv_global_dev, q, max_pos, rows)
        if reduce and dist.is_initialized() and dist.get_world_size() > 1:
            dist.all_reduce(rows, op=dist.ReduceOp.SUM)
        cnt = torch.clamp(itv_global_dev[1::2] - itv_global_dev[0::2], max=max_pos).to(torch.int32)
        return rows.view(q, max_pos), cnt


def upload_text_sharded(text_host, text_dev, scratch=None):
    """Fills this rank's device copy of the text from host memory with every rank copying only its own 1/world share over
    PCIe; the shares then meet by one all-gather over NVLink (NCCL). text_host: pinned uint16 tensor, text_dev: device uint16
    tensor of the same length, the same on every rank. Returns the scratch tensor for reuse."""
    world, rank = dist.get_world_size(), dist.get_rank()
    host_bytes, dev_bytes = text_host.view(torch.uint8), text_dev.view(torch.uint8)
    total = dev_bytes.numel()
    share = (-(-total // world) + 15) // 16 * 16                  # equal shares, whole 16-byte pieces
    if scratch is None or scratch.numel() != share * world:
        scratch = torch.empty(share * world, dtype=torch.uint8, device=text_dev.device)
    lo, hi = min(total, rank * share), min(total, (rank + 1) * share)
    mine = scratch[rank * share:(rank + 1) * share]
    if hi > lo:
        mine[:hi - lo].copy_(host_bytes[lo:hi], non_blocking=True)
    dist.all_gather_into_tensor(scratch, mine)
    dev_bytes.copy_(scratch[:total])
    return scratch


def _max_over_ranks(x, device):
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _sum_over_ranks(x, device):
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def bench(args, rank, world, local):
    """The N > 1 arm of bench.py: the same corpus (strong scaling), partitions sharded over the ranks."""
    import bench as B
    dev = torch.device("cuda", local)
    ctx = api.Context(local)
    name = [f"/cascade_b200_{os.getpid()}_{int(time.time())}"]
    dist.broadcast_object_list(name, src=0)            # one name for the job's shared-memory object
    comm, close_comm = make_shm_comm(rank, world, name[0])
    n, p = args.tokens, B.C2_PARTITIONS
    peak, peak_kind = B.measured_peak_gbs()
    T = api.gen_corpus_device(ctx, n, 0, B.C2_MEAN_DOC)          # every rank makes the same text in its own HBM
    cap = min(n, n // world + n // 8 + 1024)
    out = torch.zeros(5 * cap + api.SA_PAD_BYTES, dtype=torch.uint8, device=dev)
    for _ in range(args.warmup):
        build_sa_multi(ctx, comm, T, n, p, out=out, capacity=cap)
    ctx.L.csa_set_pass_timing(ctx.h, 1)
    ctx.reset_counters()
    dist.barrier()
    torch.cuda.synchronize()
    step_ms, launches, peer = [], 0, 0
    with B.ClockSampler(local) as clocks:
        for _ in range(args.steps):
            _, segs, st = build_sa_multi(ctx, comm, T, n, p, out=out, capacity=cap)
            count = sum(c for _, c in segs)
            step_ms.append(_max_over_ranks(st.ms_total, dev))
            launches += st.kernel_launches
            peer += st.peer_bytes
        dist.barrier()
        torch.cuda.synchronize()
    ms = sum(step_ms) / len(step_ms)
    pm, pc, pr, pb = ctypes.c_double(0), c_u64(0), c_u64(0), c_u64(0)
    ctx.L.csa_get_pass_timing(ctx.h, ctypes.byref(pm), ctypes.byref(pc), ctypes.byref(pr), ctypes.byref(pb))
    ctx.L.csa_set_pass_timing(ctx.h, 0)
    achieved = pb.value / (pm.value * 1e-3) / 1e9 if pm.value > 0 else 0.0

    # cheap check of this rank's slice: sizes add up, and sampled neighbours are in order on their first 4 symbols
    total = _sum_over_ranks(count, dev)
    ok = 1.0
    if count > 1:
        g = torch.Generator(device=dev).manual_seed(rank)
        r = torch.randint(0, count - 1, (min(count - 1, 1 << 20),), device=dev, generator=g)
        e = out[:5 * count].view(count, 5)
        def entry(ix):
            v = e[ix].to(torch.int64)
            return v[:, 0] | (v[:, 1] << 8) | (v[:, 2] << 16) | (v[:, 3] << 24) | (v[:, 4] << 32)
        Ts = T.view(torch.int16)
        def key4(ps):
            return sum((Ts[ps + k].to(torch.int64) & 0xFFFF) << (48 - 16 * k) for k in range(4))
        a, c = key4(entry(r)), key4(entry(r + 1))
        ok = float(bool(((a >> 1) <= (c >> 1)).all()))      # compare as unsigned through a 63-bit view
        del a, c, e, Ts
    torch.cuda.empty_cache()
    ok_all = _sum_over_ranks(ok, dev) == world and total == n

    # end to end: pinned host text in, this rank's slice of the 5-byte array out
    e2e = None
    if not args.no_e2e:
        th = torch.empty(n + api.TEXT_PAD, dtype=torch.uint16).pin_memory()
        th.copy_(T.cpu())
        oh = torch.empty(5 * cap + api.SA_PAD_BYTES, dtype=torch.uint8).pin_memory()
        ts = []
        scratch = None
        for it in range(1 + max(1, min(args.steps, 2))):
            dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            scratch = upload_text_sharded(th, T, scratch)         # 1/world of the text per rank over PCIe, the rest over NVLink
            _, segs, st = build_sa_multi(ctx, comm, T, n, p, out=out, capacity=cap)
            count = sum(c for _, c in segs)
            oh[:5 * count].copy_(out[:5 * count], non_blocking=True)
            torch.cuda.synchronize()
            dt = _max_over_ranks(time.perf_counter() - t0, dev)
            if it > 0:
                ts.append(dt)
        e_ms = 1e3 * sum(ts) / len(ts)
        e2e = {"value": n / (e_ms * 1e-3), "unit": B.UNIT, "h2d_bytes_per_step": 2 * n, "d2h_bytes_per_step": 5 * n, "ms_per_step": e_ms,
               "api": "upload_text_sharded (1/N of the pinned host text per rank, all-gather over NVLink) + csa_build_sa_multi + a pinned copy "
                      "of the rank's sa40 slice out"}
        del scratch
        torch.cuda.empty_cache()
    # ---- batched queries on the index sharded by suffix-array range (BASELINE config 5 over N GPUs) ---------------------
    query = None
    if args.queries > 0:
        comm0, close0 = make_shm_comm(rank, world, name[0] + "_q", policy=0)     # contiguous blocks: one slice of the array per rank
        sl, segs0, _ = build_sa_multi(ctx, comm0, T, n, p, out=out, capacity=cap)
        close0()
        first0, count0 = (segs0[0][0], sum(c for _, c in segs0)) if segs0 else (0, 0)
        sh = ShardedIndex(ctx, T, sl, n, first0, count0, stride=32)
        q = args.queries
        qa = [None, None, None, None]
        if rank == 0:
            tn = T.cpu().view(torch.int16).numpy().view(np.uint16)
            oa, sa_ = api.gen_queries("substring", tn, n, q // 2, seed=1)
            ob, sb = api.gen_queries("random", None, 0, q - q // 2, seed=2)
            qa = [np.concatenate([oa, ob[1:] + oa[-1]]), np.concatenate([sa_, sb, np.zeros(8, np.uint16)])]
        objs = [qa[0], qa[1]]
        dist.broadcast_object_list(objs, src=0)
        od = torch.from_numpy(objs[0].view(np.int64)).to(dev)
        sd = torch.from_numpy(objs[1].view(np.int16)).to(dev)
        for _ in range(2):
            itv = sh.find(od, sd, q)
        dist.barrier(); torch.cuda.synchronize()
        t0 = time.perf_counter()
        itv = sh.find(od, sd, q)
        rows, cnt = sh.locate(itv, q, 100)
        torch.cuda.synchronize()
        dq = _max_over_ranks(time.perf_counter() - t0, dev)
        query = {"value": q / dq, "unit": f"queries/s (count + locate <= 100, suffix array sharded by range over {world} GPUs, text replicated)",
                 "queries": q, "counts_hash": f"{api.counts_hash(itv.cpu().numpy().view(np.uint64)):016x}", "positions": int(cnt.sum().item())}
    launches_all = _sum_over_ranks(launches, dev)
    peer_all = _sum_over_ranks(peer, dev)
    if rank == 0:
        line = {"metric": B.METRIC, "value": n / (ms * 1e-3), "unit": B.UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
                "config": B.workload_config(args, world), "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": int(launches_all),
                "roofline": {"bound": "hbm", "kernel": "onesweep_pass_kernel (one 8-bit digit pass of the LSD radix sort), rank 0", "achieved": achieved,
                             "peak": peak, "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}", "traffic": None,
                             "passes": pc.value, "records": pr.value, "pass_ms_total": pm.value},
                "nvlink": {"peer_bytes_per_step_all_ranks": peer_all / args.steps, "generations": st.generations,
                           "note": "positions to partition owners + ranks to and from position owners, 4 bytes each, (G-1)/G of them remote"},
                "phases_ms_rank0": {"partition": st.ms_partition, "gen0": st.ms_gen0, "doubling": st.ms_doubling, "output": st.ms_output},
                "query": query,
                "verified": {"slices_add_up_to_n": total == n, "sampled_neighbours_in_order": ok_all}}
        print(json.dumps(line))
    dist.barrier()
    close_comm()
    ctx.close()
    dist.destroy_process_group()
