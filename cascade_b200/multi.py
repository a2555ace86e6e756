"""Multi-GPU build, one process per GPU: the host plumbing (torch.distributed) around csa_build_sa_multi.

The library asks its caller for ONE collective, an all-gather of small host buffers (partition sizes, IPC handles,
active counts; it also serves as the barrier between the steps). Here it is torch.distributed.all_gather, on CPU
tensors under gloo and on device tensors under NCCL. All bulk data moves inside the library's kernels as peer loads
and stores.
"""
import ctypes
import os

import numpy as np
import torch
import torch.distributed as dist

from . import api
from ._lib import ALLGATHER_FN, BuildStats, Comm


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


def _locate_packed(self, itv_global_dev, q, max_pos=100, reduce=True):
    """Packed positions of global intervals: (pos, pos_off, cnt) with query i's positions at pos[pos_off[i]:pos_off[i + 1]], in
    rank order. Every shard fills in the entries whose ranks it holds; one all-reduce of the packed array (a ninth of the
    q x max_pos rows on the benchmark's queries) puts them together."""
    dev = itv_global_dev.device
    cnt_t = torch.clamp(itv_global_dev[1::2] - itv_global_dev[0::2], max=max_pos)
    total = int(cnt_t.sum().item())
    pos = torch.zeros(max(1, total), dtype=torch.int64, device=dev)
    cnt = torch.empty(q, dtype=torch.int32, device=dev)
    poff = torch.empty(q + 1, dtype=torch.int64, device=dev)
    tot = torch.zeros(1, dtype=torch.int64, device=dev)
    loc = self.local
    torch.cuda.synchronize(dev)
    loc.ctx.check(loc.ctx.L.csa_locate_window_packed(loc.ctx.h, ctypes.byref(loc.c), itv_global_dev.data_ptr(), q, max_pos, cnt.data_ptr(), poff.data_ptr(),
                                                     pos.data_ptr(), tot.data_ptr()))
    loc.ctx.sync()
    if reduce and dist.is_initialized() and dist.get_world_size() > 1:
        dist.all_reduce(pos, op=dist.ReduceOp.SUM)
    return pos[:total], poff, cnt


ShardedIndex.locate_packed = _locate_packed


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


def group_partitions_into_parts(sizes, part_suffixes):
    """Runs of whole partitions, each run below part_suffixes suffixes (a partition larger than that is a part of its own).
    Returns (part_of_pid uint16[p], part_off int list of parts + 1 entries), as csa_build_sa_streamed groups them."""
    part_of_pid = np.zeros(len(sizes), np.uint16)
    part_off, cur, total = [0], 0, 0
    for q, s in enumerate(int(x) for x in sizes):
        if s >= 1 << 31:
            raise api.CascadeError(4, "a partition holds 2^31 suffixes or more; ask for more partitions")
        if cur > 0 and cur + s > part_suffixes:
            part_off.append(total)
            cur = 0
        part_of_pid[q] = len(part_off) - 1
        cur += s
        total += s
    part_off.append(total)
    return part_of_pid, part_off


def build_sa_streamed_multi(ctx, text_dev, n, p=4096, seed=0, part_suffixes=1 << 27, workers=3, host=None, window_bytes=8 << 30,
                            list_budget_bytes=None):
    """The part-at-a-time build over the GPUs of a process group (one process per GPU; also works alone), written on the
    library's part jobs: every rank holds the whole text and a replica of the rank store on its device, owns the parts u with
    u mod world == rank, keeps their suffix lists (5-byte lanes + 4-byte ranks) in its own pinned host memory and streams them
    through its GPU over its own PCIe link on `workers` contexts. Between generations the ranks exchange their (position, rank)
    messages: after generation 0 the replicas (zero where a rank wrote nothing) are added up by one all-reduce; after a later
    generation every rank's outbox is all-gathered (NCCL over NVLink) and applied to every replica.
    Returns (segments, info): segments = [(first global rank, count, pinned uint8 tensor of 5 * count bytes)] for the
    rank's parts in the order of their ranks, info = timings and counts. `host` may be a dict that keeps the pinned list
    buffers between calls (pinning gigabytes takes seconds).
    Residency of the lists (the reference plans its tiers likewise, src/Residency_Plan.cpp): a part's list stays in device
    memory while the device has room for it (list_budget_bytes, or what is free after the text, the rank store, the job
    workspaces and the largest outboxes), and lives in pinned host memory otherwise; list_budget_bytes = 0 keeps every list on
    the host. The final order always lands in the pinned host segments."""
    import threading
    import time
    from ._lib import Part, PartResult, c_u64, c_vp
    L = ctx.L
    dev = text_dev.device
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    info = {"ms": {}}

    def sync_all():
        ctx.sync()
        torch.cuda.synchronize(dev)

    def mark(name, t0):
        sync_all()
        info["ms"][name] = info["ms"].get(name, 0.0) + 1e3 * (time.perf_counter() - t0)

    def total_over_ranks(x):
        if world == 1:
            return int(x)
        t = torch.tensor([int(x)], dtype=torch.int64, device=dev)
        dist.all_reduce(t)
        return int(t.item())

    t_all = time.perf_counter()
    # ---- splitters and partition ids: the same on every rank (the same samples of the same text) ------------------------------
    t0 = time.perf_counter()
    pe, piv = 1, None
    if p > 1:
        ns = min(1 << 19, max(1024, 32 * p * max(1, int(n).bit_length())))
        samples = torch.empty(2 * ns, dtype=torch.int64, device=dev)
        torch.cuda.synchronize(dev)
        ctx.check(L.csa_sample_kgrams(ctx.h, text_dev.data_ptr(), n, ns, seed, samples.data_ptr()))
        piv = np.zeros(2 * (p - 1), np.uint64)
        p_out = ctypes.c_uint32(0)
        ctx.check(L.csa_select_pivots_dev(ctx.h, samples.data_ptr(), ns, p, piv.ctypes.data, ctypes.byref(p_out)))
        pe = p_out.value
        del samples
    pivd = torch.from_numpy(piv.view(np.int64)).to(dev) if pe > 1 else None
    # every rank computes the ids of its own stretch of positions; the stretches meet by one all-gather (NVLink)
    stretch = (-(-n // world) + 4095) // 4096 * 4096               # equal stretches, whole 4096 positions
    pid = torch.empty(world * stretch + 64, dtype=torch.int16, device=dev)
    hist = torch.zeros(max(pe, 1), dtype=torch.int64, device=dev)
    torch.cuda.synchronize(dev)
    my_first, my_end = min(n, rank * stretch), min(n, (rank + 1) * stretch)
    step = 1 << 28
    if pe > 1:
        ctx.check(L.csa_install_pivots(ctx.h, piv.ctypes.data, pe))
    try:
        for first in range(my_first, my_end, step):
            c = min(step, my_end - first)
            ctx.check(L.csa_partition_ids(ctx.h, text_dev.data_ptr(), n, first, c, pivd.data_ptr() if pivd is not None else None, pe,
                                          pid.data_ptr() + 2 * first, hist.data_ptr()))
        ctx.sync()
    finally:
        L.csa_install_pivots(ctx.h, None, 0)
    if world > 1:
        pb = pid.view(torch.uint8)             # the collective libraries take bytes, not 16-bit integers
        dist.all_gather([pb[2 * g * stretch:2 * (g + 1) * stretch] for g in range(world)], pb[2 * rank * stretch:2 * (rank + 1) * stretch].clone())
        dist.all_reduce(hist)
    sizes = hist.cpu().numpy()
    part_of_pid, part_off = group_partitions_into_parts(sizes, part_suffixes)
    parts = len(part_off) - 1
    if part_off[-1] != n:
        raise api.CascadeError(5, "partition sizes do not add up to n")
    own = [u for u in range(parts) if u % world == rank]
    size = [part_off[u + 1] - part_off[u] for u in range(parts)]
    mark("partition_ids", t0)

    # ---- the store (a replica of the rank store on every GPU) and this rank's lists in pinned host memory --------------------
    t0 = time.perf_counter()
    R = torch.zeros(n + 16, dtype=torch.int32, device=dev)
    store = c_vp()
    torch.cuda.synchronize(dev)
    ctx.check(L.csa_store_create(ctx.h, text_dev.data_ptr(), n, pid.data_ptr(), part_of_pid.ctypes.data, pe, R.data_ptr(), ctypes.byref(store)))
    ctxs = [ctx]
    try:
        own_first, at = {}, 0
        for u in own:
            own_first[u] = at
            at += size[u]
        own_total = at
        host = host if host is not None else {}
        if host.get("lanes") is None or host["lanes"].numel() < 5 * own_total + 64:
            host["lanes"] = torch.empty(5 * own_total + 64, dtype=torch.uint8).pin_memory()
            host["ranks"] = torch.empty(own_total + 16, dtype=torch.int32).pin_memory()
        lanes_h, ranks_h = host["lanes"], host["ranks"]
        mark("pinned_lists", t0)
        # ---- the part jobs, on `workers` contexts (streams and scratch), one host thread each ---------------------------------
        ctxs += [api.Context(dev.index) for _ in range(max(0, min(workers, len(own)) - 1))]
        active = {u: size[u] for u in own}

        def over_parts(todo, job):
            it, lock, errors, job_s = iter(todo), threading.Lock(), [], []

            def body(c):
                torch.cuda.set_device(dev)
                while not errors:
                    with lock:
                        u = next(it, None)
                    if u is None:
                        return
                    try:
                        t1 = time.perf_counter()
                        job(c, u)
                        t2 = time.perf_counter()
                        c.sync()
                        job_s.append((t2 - t1, time.perf_counter() - t2))
                    except Exception as e:        # noqa: BLE001 - reported after the workers have joined
                        errors.append(e)
            ts = [threading.Thread(target=body, args=(c,)) for c in ctxs[1:]]
            for t in ts:
                t.start()
            body(ctxs[0])
            for t in ts:
                t.join()
            if errors:
                raise errors[0]
            if os.environ.get("CSA_DEBUG") and job_s:
                print(f"[csa multi {rank}/{world}] {job.__name__}: {len(job_s)} jobs, in the call {1e3 * sum(a for a, _ in job_s) / len(job_s):.1f} ms, "
                      f"waiting for the lists to be out {1e3 * sum(b for _, b in job_s) / len(job_s):.1f} ms on average", flush=True)

        # which lists stay on the device
        largest = max([size[u] for u in own], default=1)
        if list_budget_bytes is None:
            torch.cuda.empty_cache()                # what an earlier build left in the allocator's cache counts as free
            free_b, _ = torch.cuda.mem_get_info(dev)
            reserve = 3 * int(L.csa_part_workspace_bytes(largest)) + window_bytes + 2 * 9 * int(0.7 * n) + (6 << 30)
            budget = max(0, free_b - reserve)
        else:
            budget = int(list_budget_bytes)
        res_first, used = {}, 0
        for u in own:
            if 9 * (used + size[u]) + 256 <= budget:
                res_first[u] = used
                used += size[u]
        dev_lanes = torch.empty(5 * used + 64, dtype=torch.uint8, device=dev)
        dev_ranks = torch.empty(used + 16, dtype=torch.int32, device=dev)
        info["list_budget_bytes"] = int(budget)
        info["lists_on_device"] = len(res_first)
        info["lists_on_host"] = len(own) - len(res_first)

        def host_segment(u):
            return lanes_h.data_ptr() + 5 * own_first[u]

        def lists(u):
            if u in res_first:
                return dev_lanes.data_ptr() + 5 * res_first[u], dev_ranks.data_ptr() + 4 * res_first[u]
            return host_segment(u), ranks_h.data_ptr() + 4 * own_first[u]

        # ---- generation 0, a window of parts at a time: the window's lanes are picked out of the partition ids into a device
        # buffer (one sweep over the ids per window; the parts' sizes are known, so every lane has its place), and the parts are
        # ranked from there; only their ranked lists travel to the host.
        t0 = time.perf_counter()
        window = max(1, min(len(own), int(window_bytes // (5 * largest + 64)))) if own else 1
        win_buf = torch.empty(5 * sum(sorted((size[u] for u in own), reverse=True)[:window]) + 256, dtype=torch.uint8, device=dev)
        first_d = torch.empty(parts, dtype=torch.int64, device=dev)
        cursor_d = torch.zeros(parts, dtype=torch.int64, device=dev)
        win_first = {}

        def gen0(c, u):
            lp, rp = lists(u)
            pin, pout = Part(win_buf.data_ptr() + 5 * win_first[u], None, size[u], u), PartResult(lp, rp, 0, 0)
            c.check(L.csa_rank_gen0(c.h, store, ctypes.byref(pin), ctypes.byref(pout)))
            active[u] = int(pout.active)

        for w0 in range(0, len(own), window):
            wparts = own[w0:w0 + window]
            pf = np.full(parts, -1, np.int64)
            at = 0
            for u in wparts:
                win_first[u] = at
                pf[u] = at
                at += size[u]
            first_d.copy_(torch.from_numpy(pf))
            cursor_d.zero_()
            torch.cuda.synchronize(dev)
            sweep = 1 << 30
            for first in range(0, n, sweep):
                ctx.check(L.csa_scatter_lanes(ctx.h, store, first, min(sweep, n - first), first_d.data_ptr(), cursor_d.data_ptr(), win_buf.data_ptr()))
            ctx.sync()
            over_parts(wparts, gen0)
        del win_buf
        L.csa_store_drop_partition_ids(store)
        del pid
        if world > 1:
            dist.all_reduce(R)          # every position was ranked by exactly one GPU; the others hold zero there
        total_active = total_over_ranks(sum(active.values()))
        info["active_after_gen0"] = total_active
        mark("gen0", t0)

        # ---- doubling generations --------------------------------------------------------------------------------------------------
        t0 = time.perf_counter()
        h, gens, exchanged = 3, 0, 0
        info["active_per_generation"] = []
        while total_active > 0:
            info["active_per_generation"].append(total_active)
            a_own = sum(active.values())
            box_l = torch.empty(a_own + 16, dtype=torch.int32, device=dev)     # positions: low 32 bits
            box_h = torch.empty(a_own + 16, dtype=torch.uint8, device=dev)     #            high 8 bits
            box_r = torch.empty(a_own + 16, dtype=torch.int32, device=dev)     # ranks
            torch.cuda.synchronize(dev)
            ctx.check(L.csa_store_use_outbox(store, box_l.data_ptr(), box_h.data_ptr(), box_r.data_ptr(), a_own))

            def gen(c, u, h=h):
                lp, rp = lists(u)
                pin, pout = Part(lp, rp, active[u], u), PartResult(lp, rp, 0, 0)
                c.check(L.csa_rank_gen(c.h, store, ctypes.byref(pin), h, ctypes.byref(pout)))
                active[u] = int(pout.active)
            over_parts([u for u in own if active[u] > 0], gen)
            sent = int(L.csa_store_outbox_count(store))
            assert sent == a_own
            if world == 1:
                ctx.check(L.csa_store_apply_messages(ctx.h, store, box_l.data_ptr(), box_h.data_ptr(), box_r.data_ptr(), sent))
                ctx.sync()
            else:
                counts = torch.zeros(world, dtype=torch.int64, device=dev)
                counts[rank] = sent
                dist.all_reduce(counts)
                cs = [int(x) for x in counts.cpu()]
                row = (max(cs) + 16 + 15) // 16 * 16          # messages per rank in the gathered arrays, padded
                gathered = []
                for box, dt in ((box_l, torch.int32), (box_h, torch.uint8), (box_r, torch.int32)):
                    snd = torch.zeros(row, dtype=dt, device=dev)
                    snd[:sent] = box[:sent]
                    allb = torch.empty(world * row, dtype=dt, device=dev)
                    dist.all_gather([allb[g * row:(g + 1) * row] for g in range(world)], snd)
                    gathered.append(allb)
                torch.cuda.synchronize(dev)
                al, ah, ar = gathered
                for g in range(world):
                    ctx.check(L.csa_store_apply_messages(ctx.h, store, al.data_ptr() + 4 * g * row, ah.data_ptr() + g * row, ar.data_ptr() + 4 * g * row, cs[g]))
                ctx.sync()
                exchanged += 9 * sum(cs[g] for g in range(world) if g != rank)
                del gathered, al, ah, ar
            ctx.check(L.csa_store_use_outbox(store, None, None, None, 0))
            del box_l, box_h, box_r
            total_active = total_over_ranks(sum(active.values()))
            h *= 2
            gens += 1
            if gens > 45:
                raise api.CascadeError(5, "doubling did not terminate")
        info["generations"] = gens
        info["nvlink_bytes_received"] = exchanged + (4 * n * (world - 1) // world if world > 1 else 0)
        mark("doubling", t0)

        # ---- every part into its final order, in place -------------------------------------------------------------------------------
        t0 = time.perf_counter()

        def order(c, u):
            lp, rp = lists(u)
            c.check(L.csa_rank_order(c.h, lp, rp, size[u], host_segment(u)))
        over_parts(own, order)
        mark("output", t0)
        del dev_lanes, dev_ranks
    finally:
        for c in ctxs[1:]:
            c.close()
        L.csa_store_destroy(store)
    info["ms"]["total"] = 1e3 * (time.perf_counter() - t_all)
    info.update({"partitions": pe, "parts": parts, "own_parts": len(own), "own_suffixes": own_total,
                 "launches": sum(c.launches for c in ctxs[:1])})
    segments = [(part_off[u], size[u], lanes_h[5 * own_first[u]:5 * (own_first[u] + size[u])]) for u in own]
    return segments, info


# ---- the part-at-a-time build with nothing replicated: text, partition ids and rank store sharded by position ------------------

def address_bits(n):
    """(begin_bit, end_bit) of the address bits by which requests and messages are ordered on their way to the owners: the top
    8 bits of a position while a bucket of the rank store then stays within 128 MB, about the L2 (one digit pass), else the top
    16 (two passes; at 4.5e9 positions the second pass cost what the better locality of the writes saved)."""
    end = max(1, int(n - 1).bit_length())
    begin = max(0, end - 8)
    if begin > 25:
        begin = end - 16
    return begin, end


def shard_bounds(n, world, rank):
    """Equal stretches of whole address buckets (and whole 64 positions): (stretch, first position, end) of `rank`'s share of a
    text of n symbols."""
    unit = max(64, 1 << address_bits(n)[0])
    stretch = (-(-n // world) + unit - 1) // unit * unit
    lo = min(n, rank * stretch)
    return stretch, lo, min(n, lo + stretch)


def _exchange(send, send_counts, recv_counts, width=1):
    """All-to-all of one tensor cut into per-rank runs (counts in units of `width` elements). The collective library does it
    between GPUs; a process group without device all-to-all (several test ranks on one GPU) goes through host memory."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    if world == 1:
        return send[:send_counts[0] * width].clone()
    recv = torch.empty(sum(recv_counts) * width, dtype=send.dtype, device=send.device)
    ss, rs = [c * width for c in send_counts], [c * width for c in recv_counts]
    if dist.get_backend() == "nccl":
        dist.all_to_all_single(recv, send[:sum(ss)].contiguous(), rs, ss)
    else:
        r_host = torch.empty(sum(rs), dtype=send.dtype)
        dist.all_to_all_single(r_host, send[:sum(ss)].cpu().contiguous(), rs, ss)
        recv.copy_(r_host)
    return recv


def _gather_small(t):
    """All ranks' copies of a small host-side integer array (numpy int64), as one array [world, len]."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    if world == 1:
        return t[None, :].copy()
    dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend() == "nccl" else torch.device("cpu")
    mine = torch.from_numpy(np.ascontiguousarray(t, dtype=np.int64)).to(dev)
    out = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(out, mine)
    return torch.stack(out).cpu().numpy()


def _halo_from_next(local, valid, k):
    """The k entries that follow this rank's stretch of a position-sharded array: the first entries of the next ranks' stretches
    (zero past the end of the array). local: device tensor whose first `valid` entries are this rank's."""
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    out = torch.zeros(k, dtype=local.dtype, device=local.device)
    if world == 1:
        return out
    head = torch.zeros(k, dtype=torch.int32, device=local.device)
    m = min(k, valid)
    head[:m] = local[:m].to(torch.int32)
    heads = [torch.empty_like(head) for _ in range(world)]
    dist.all_gather(heads, head)
    valids = _gather_small(np.array([m], np.int64))[:, 0]
    at = 0
    for g in range(rank + 1, world):
        take = min(int(valids[g]), k - at)
        if take > 0:
            out[at:at + take] = heads[g][:take].to(local.dtype)
            at += take
        if at == k:
            break
    return out


def build_sa_sharded(ctx, text_shard, n, p=4096, seed=0, part_suffixes=1 << 27, window_suffixes=None, lists_on_device=None, host=None, output="host"):
    """The part-at-a-time build with NOTHING replicated: rank r of the process group holds the symbols of its stretch of
    positions only (shard_bounds), and the same stretch of the partition ids and of the rank store; a rank owns a run of
    consecutive parts (part u belongs to rank u * world // parts), so its parts in final order are ONE range of the suffix array. The GPU that holds a stretch of the text makes the generation-0 keys of its positions
    and sends (lane, key) to the parts' owners; in a later generation the owner of a part asks the owners of the positions
    h further on for their ranks, and new ranks travel back to the positions' owners as messages. Device memory per GPU:
    8 n / world bytes (2 text + 2 partition ids until generation 0 is over + 4 ranks) plus the lists of its parts (9 bytes per
    suffix, on the device while they fit, else in pinned host memory) plus one part's workspace and the windows in flight
    (window_suffixes per rank and window of generation 0, 52 bytes each; None: what the free memory allows).
    text_shard: device uint16 tensor with this rank's symbols first. `host` may be a dict that keeps the pinned buffers between
    calls. output = "host": the parts end in pinned host memory; "device": they stay in this GPU's memory (the lists must be
    resident), which is where a ShardedIndex over the same ranks wants its slice of the array.
    Returns (segments, info) as build_sa_streamed_multi."""
    import time
    from ._lib import Part, PartResult, c_vp
    L = ctx.L
    dev = text_shard.device
    world = dist.get_world_size() if dist.is_initialized() else 1
    rank = dist.get_rank() if dist.is_initialized() else 0
    stretch, lo, hi = shard_bounds(n, world, rank)
    cnt = hi - lo
    HALO = 64
    info = {"ms": {}, "nvlink_bytes_sent": 0}

    def mark(name, t0):
        ctx.sync()
        torch.cuda.synchronize(dev)
        info["ms"][name] = info["ms"].get(name, 0.0) + 1e3 * (time.perf_counter() - t0)

    def total_over_ranks(x):
        if world == 1:
            return int(x)
        t = torch.tensor([int(x)], dtype=torch.int64, device=dev)
        dist.all_reduce(t)
        return int(t.item())

    def sent(counts, bytes_each):
        info["nvlink_bytes_sent"] += bytes_each * sum(int(c) for g, c in enumerate(counts) if g != rank)

    t_all = time.perf_counter()
    t0 = time.perf_counter()
    # ---- this rank's stretch of the text with the symbols that follow it -------------------------------------------------------
    T = torch.zeros(cnt + HALO + api.TEXT_PAD, dtype=torch.uint16, device=dev)
    T[:cnt] = text_shard[:cnt]
    T[cnt:cnt + HALO] = _halo_from_next(T.view(torch.int16), cnt, HALO).view(torch.uint16)
    known = min(cnt + HALO, n - lo)                      # symbols of the text in T; zeros follow

    # ---- splitters from samples of every stretch ----------------------------------------------------------------------------------
    pe, piv = 1, None
    if p > 1:
        ns_all = min(1 << 19, max(1024, 32 * p * max(1, int(n).bit_length())))
        ns = max(64, ns_all // world)
        samples = torch.zeros(2 * ns, dtype=torch.int64, device=dev)
        torch.cuda.synchronize(dev)
        if cnt > 0:
            ctx.check(L.csa_sample_kgrams(ctx.h, T.data_ptr(), cnt, ns, seed + rank, samples.data_ptr()))
            ctx.sync()
        if world > 1:
            every = [torch.empty_like(samples) for _ in range(world)]
            dist.all_gather(every, samples)
            have = _gather_small(np.array([cnt > 0], np.int64))[:, 0]
            samples = torch.cat([e for e, ok in zip(every, have) if ok])
        samples = samples.contiguous()
        piv = np.zeros(2 * (p - 1), np.uint64)
        p_out = ctypes.c_uint32(0)
        torch.cuda.synchronize(dev)
        ctx.check(L.csa_select_pivots_dev(ctx.h, samples.data_ptr(), samples.numel() // 2, p, piv.ctypes.data, ctypes.byref(p_out)))
        pe = p_out.value
        del samples
    pivd = torch.from_numpy(piv.view(np.int64)).to(dev) if pe > 1 else None

    # ---- partition ids of this stretch, with the 3 ids that follow it -------------------------------------------------------------
    pid = torch.zeros(cnt + 64, dtype=torch.int16, device=dev)
    hist = torch.zeros(max(pe, 1), dtype=torch.int64, device=dev)
    torch.cuda.synchronize(dev)
    if pe > 1:
        ctx.check(L.csa_install_pivots(ctx.h, piv.ctypes.data, pe))
    try:
        step = 1 << 28
        for first in range(0, cnt, step):
            ctx.check(L.csa_partition_ids(ctx.h, T.data_ptr(), known, first, min(step, cnt - first), pivd.data_ptr() if pivd is not None else None, pe,
                                          pid.data_ptr() + 2 * first, hist.data_ptr()))
        ctx.sync()
    finally:
        L.csa_install_pivots(ctx.h, None, 0)
    pid[cnt:cnt + 3] = _halo_from_next(pid, cnt, 3)
    if world > 1:
        dist.all_reduce(hist)
    sizes = hist.cpu().numpy()
    part_of_pid, part_off = group_partitions_into_parts(sizes, part_suffixes)
    parts = len(part_off) - 1
    if part_off[-1] != n:
        raise api.CascadeError(5, "partition sizes do not add up to n")
    size = [int(part_off[u + 1] - part_off[u]) for u in range(parts)]
    owner = [u * world // parts for u in range(parts)]
    own = [u for u in range(parts) if owner[u] == rank]
    mark("partition_ids", t0)

    t0 = time.perf_counter()
    R = torch.zeros(cnt + 16, dtype=torch.int32, device=dev)              # this stretch of the rank store
    unused = torch.zeros(16, dtype=torch.int32, device=dev)               # the store object keeps no rank array of its own here
    store = c_vp()
    torch.cuda.synchronize(dev)
    ctx.check(L.csa_store_create(ctx.h, T.data_ptr(), n, pid.data_ptr(), part_of_pid.ctypes.data, pe, unused.data_ptr(), ctypes.byref(store)))
    try:
        # how many positions of every part each rank holds
        local_d = torch.zeros(parts, dtype=torch.int64, device=dev)
        torch.cuda.synchronize(dev)             # the zeros are written on torch's stream, the counts on the context's
        if cnt > 0:
            ctx.check(L.csa_part_sizes(ctx.h, store, 0, cnt, parts, local_d.data_ptr()))
            ctx.sync()
        held = _gather_small(local_d.cpu().numpy())                       # [world, parts]
        if not np.array_equal(held.sum(axis=0), np.array(size)):
            raise api.CascadeError(5, "the ranks' counts of a part do not add up to its size")

        # where this rank's lists live
        own_first, at = {}, 0
        for u in own:
            own_first[u] = at
            at += size[u]
        own_total = at
        largest = max(size) if size else 1
        host = host if host is not None else {}
        if window_suffixes is None:
            window_suffixes = host.get("window_suffixes")
        if lists_on_device is None:
            lists_on_device = host.get("lists_on_device")
        free_b = None
        if lists_on_device is None or window_suffixes is None:
            torch.cuda.empty_cache()                # what an earlier build left in the allocator's cache counts as free
            free_b, _ = torch.cuda.mem_get_info(dev)
            free_b -= int(L.csa_part_workspace_bytes(largest)) + 40 * largest + (6 << 30)      # a job's workspace, a part's pieces put together
        if lists_on_device is None:
            lists_on_device = 9 * own_total + 52 * (1 << 26) < free_b
            host["lists_on_device"] = lists_on_device
        if window_suffixes is None:
            # a window's lanes and keys lie twice on a GPU: as picked out of its stretch, and as received for its parts
            room = free_b - (9 * own_total if lists_on_device else 0)
            window_suffixes = max(1 << 24, min(1 << 31, room // 2 // 52))
            if world > 1:
                window_suffixes = int(_gather_small(np.array([window_suffixes], np.int64)).min())
            host["window_suffixes"] = window_suffixes
        if lists_on_device:
            lanes_all = torch.empty(5 * own_total + 64, dtype=torch.uint8, device=dev)
            ranks_all = torch.empty(own_total + 16, dtype=torch.int32, device=dev)
        else:
            if host.get("lanes") is None or host["lanes"].numel() < 5 * own_total + 64:
                host["lanes"] = torch.empty(5 * own_total + 64, dtype=torch.uint8).pin_memory()
                host["ranks"] = torch.empty(own_total + 16, dtype=torch.int32).pin_memory()
            lanes_all, ranks_all = host["lanes"], host["ranks"]
        if output == "device":
            if not lists_on_device:
                raise api.CascadeError(3, "the array can stay on the device only where the parts' lists are resident there")
            out_lanes = lanes_all                   # every part is put into its final order in place
        else:
            if host.get("out") is None or host["out"].numel() < 5 * own_total + 64:
                host["out"] = torch.empty(5 * own_total + 64, dtype=torch.uint8).pin_memory()
            out_lanes = host["out"]
        info["lists_on_device"] = bool(lists_on_device)

        def lists(u):
            return lanes_all.data_ptr() + 5 * own_first[u], ranks_all.data_ptr() + 4 * own_first[u]

        addr_begin, addr_end = address_bits(n)

        def bucket(pos, payload, want_order, c=ctx):
            """pos (and payload, or the entries' indexes) ordered by address: one run per owner, ascending buckets inside.
            Returns (counts, positions, payload or order). c: the context (stream and scratch) that does the work."""
            m = int(pos.numel())
            counts = np.zeros(world, np.uint64)
            if m == 0:
                return [0] * world, pos, torch.empty(0, dtype=torch.int32, device=dev)
            pos_alt = torch.empty(m + 8, dtype=torch.int64, device=dev)
            pay = payload if payload is not None else torch.empty(m + 8, dtype=torch.int32, device=dev)
            pay_alt = torch.empty(m + 8, dtype=torch.int32, device=dev)
            wsb = int(L.csa_sort_workspace_bytes(m))
            ws = torch.empty(wsb, dtype=torch.uint8, device=dev)
            in_alt = ctypes.c_int(0)
            torch.cuda.current_stream(dev).synchronize()
            c.check(L.csa_order_by_address(c.h, pos.data_ptr(), pos_alt.data_ptr(), pay.data_ptr(), pay_alt.data_ptr(), m, addr_begin, addr_end, stretch, world,
                                           1 if want_order else 0, counts.ctypes.data, ws.data_ptr(), wsb, ctypes.byref(in_alt)))
            c.sync()
            del ws
            return [int(c) for c in counts], (pos_alt if in_alt.value else pos), (pay_alt if in_alt.value else pay)

        def route_messages(pos, ranks):
            """(position, rank) messages to the owners of the positions, applied to their stretch of the rank store."""
            t1 = time.perf_counter()
            counts, pos_b, rank_b = bucket(pos, ranks, False)
            incoming = [int(c) for c in _gather_small(np.array(counts, np.int64))[:, rank]] if world > 1 else counts
            mark("route_bucket", t1)
            t1 = time.perf_counter()
            sent(counts, 12)
            got_pos = _exchange(pos_b, counts, incoming)
            got_rank = _exchange(rank_b, counts, incoming)
            del pos_b, rank_b
            mark("route_exchange", t1)
            t1 = time.perf_counter()
            m = int(got_pos.numel())
            if m:
                torch.cuda.synchronize(dev)
                ctx.check(L.csa_rank_shard_apply(ctx.h, R.data_ptr(), lo, cnt, got_pos.data_ptr(), got_rank.data_ptr(), m))
                ctx.sync()
            del got_pos, got_rank
            mark("route_apply", t1)
            return m

        def outbox_tensors(capacity):
            box_l = torch.empty(capacity + 16, dtype=torch.int32, device=dev)
            box_h = torch.empty(capacity + 16, dtype=torch.uint8, device=dev)
            box_r = torch.empty(capacity + 16, dtype=torch.int32, device=dev)
            torch.cuda.synchronize(dev)
            ctx.check(L.csa_store_use_outbox(store, box_l.data_ptr(), box_h.data_ptr(), box_r.data_ptr(), capacity))
            return box_l, box_h, box_r

        def flush_outbox(box):
            """The outbox, in runs of 2^29 messages (as many runs on every rank as the rank with the most messages needs)."""
            box_l, box_h, box_r = box
            m = int(L.csa_store_outbox_count(store))
            ctx.sync()
            applied, run = 0, 1 << 29
            runs = -(-m // run)
            if world > 1:
                runs = int(_gather_small(np.array([runs], np.int64)).max())
            for k in range(runs):
                a, b = min(m, k * run), min(m, (k + 1) * run)
                pos = torch.empty(b - a + 8, dtype=torch.int64, device=dev)
                torch.cuda.synchronize(dev)
                ctx.check(L.csa_outbox_positions(ctx.h, box_l.data_ptr() + 4 * a, box_h.data_ptr() + a, b - a, pos.data_ptr()))
                ctx.sync()
                applied += route_messages(pos[:b - a], box_r[a:b])
                del pos
            ctx.check(L.csa_store_use_outbox(store, None, None, None, 0))
            return m, applied
        mark("setup", t0)

        # ---- generation 0, a window of parts at a time ---------------------------------------------------------------------------------
        # Every rank picks the window's positions out of its stretch with their keys, the runs travel to the parts' owners, and
        # an owner ranks a part once its pieces from all ranks lie one after another.
        t0 = time.perf_counter()
        active = {u: 0 for u in own}
        windows, cur, cur_n = [], [], 0
        for u in range(parts):
            if cur and cur_n + size[u] > window_suffixes * world:
                windows.append(cur)
                cur, cur_n = [], 0
            cur.append(u)
            cur_n += size[u]
        if cur:
            windows.append(cur)
        first_d = torch.empty(parts, dtype=torch.int64, device=dev)
        cursor_d = torch.zeros(parts, dtype=torch.int64, device=dev)
        for wparts in windows:
            by_owner = sorted(wparts, key=lambda u: (owner[u], u))
            pf = np.full(parts, -1, np.int64)
            at = 0
            for u in by_owner:
                pf[u] = at
                at += int(held[rank, u])
            mine_n = at
            send_counts = [sum(int(held[rank, u]) for u in wparts if owner[u] == g) for g in range(world)]
            my_parts = [u for u in wparts if owner[u] == rank]
            recv_counts = [sum(int(held[g, u]) for u in my_parts) for g in range(world)]
            st_lanes = torch.empty(5 * mine_n + 64, dtype=torch.uint8, device=dev)
            st_keys = torch.empty(mine_n + 8, dtype=torch.int64, device=dev)
            first_d.copy_(torch.from_numpy(pf))
            cursor_d.zero_()
            torch.cuda.synchronize(dev)
            sweep = 1 << 30
            t1 = time.perf_counter()
            for first in range(0, cnt, sweep):
                ctx.check(L.csa_scatter_lanes_keys(ctx.h, store, T.data_ptr() + 2 * first, pid.data_ptr() + 2 * first, lo + first, min(sweep, cnt - first),
                                                   first_d.data_ptr(), cursor_d.data_ptr(), st_lanes.data_ptr(), st_keys.data_ptr()))
            mark("gen0_scan", t1)
            t1 = time.perf_counter()
            sent(send_counts, 13)
            got_lanes = _exchange(st_lanes, send_counts, recv_counts, width=5)
            got_keys = _exchange(st_keys, send_counts, recv_counts)
            del st_lanes, st_keys
            mark("gen0_keys_to_owners", t1)
            t1 = time.perf_counter()
            box = outbox_tensors(sum(size[u] for u in my_parts))
            src_at = np.concatenate([[0], np.cumsum(recv_counts)])[:world].astype(np.int64)      # where each rank's block starts
            for u in my_parts:
                pieces_l, pieces_k = [], []
                for g in range(world):
                    a = int(src_at[g]) + sum(int(held[g, v]) for v in my_parts if v < u)
                    c = int(held[g, u])
                    pieces_l.append(got_lanes[5 * a:5 * (a + c)])
                    pieces_k.append(got_keys[a:a + c])
                filled = [g for g in range(world) if int(held[g, u]) > 0]
                if len(filled) == 1:                   # the part's records came from one rank: they lie in one piece already
                    pl, pk = pieces_l[filled[0]], pieces_k[filled[0]]
                else:
                    pl = torch.cat(pieces_l + [torch.zeros(64, dtype=torch.uint8, device=dev)])
                    pk = torch.cat(pieces_k + [torch.zeros(8, dtype=torch.int64, device=dev)])
                torch.cuda.synchronize(dev)
                lp, rp = lists(u)
                pin, pout = Part(pl.data_ptr(), None, size[u], u), PartResult(lp, rp, 0, 0)
                ctx.check(L.csa_rank_gen0_keys(ctx.h, store, ctypes.byref(pin), pk.data_ptr(), ctypes.byref(pout)))
                ctx.sync()
                active[u] = int(pout.active)
                del pl, pk
            del got_lanes, got_keys
            mark("gen0_rank", t1)
            t1 = time.perf_counter()
            flush_outbox(box)
            del box
            mark("gen0_ranks_to_owners", t1)
        L.csa_store_drop_partition_ids(store)
        del pid
        total_active = total_over_ranks(sum(active.values()))
        info["active_after_gen0"] = total_active
        mark("gen0", t0)

        # ---- doubling generations: the ranks go through their parts in step, one part each per round -----------------------------
        # Fetching the second ranks of a round's part (requests out, answers back: this thread, a context of its own, the
        # collective) runs while the part of the round before is ranked (a second thread, the main context). Nothing that the
        # two touch is shared: a job reads and writes its own part's lists and appends to the outbox; the rank store changes only
        # after the generation's last part.
        import threading
        t0 = time.perf_counter()
        h, gens = 3, 0
        info["active_per_generation"] = []
        rounds = -(-parts // world)
        fetch_ctx = api.Context(dev.index)
        mine = torch.cuda.current_stream(dev)

        def lap(name, t1):
            info["ms"][name] = info["ms"].get(name, 0.0) + 1e3 * (time.perf_counter() - t1)

        def rank_job(u, a, second, failures):
            try:
                torch.cuda.set_device(dev)
                lp, rp = lists(u)
                pin, pout = Part(lp, rp, a, u), PartResult(lp, rp, 0, 0)
                ctx.check(L.csa_rank_gen_ranks(ctx.h, store, ctypes.byref(pin), second.data_ptr(), ctypes.byref(pout)))
                ctx.sync()
                active[u] = int(pout.active)
            except Exception as e:        # noqa: BLE001 - raised on the main thread after the join
                failures.append(e)

        try:
            while total_active > 0:
                info["active_per_generation"].append(total_active)
                box = outbox_tensors(sum(active.values()))
                running, failures = None, []
                for k in range(rounds):
                    u = own[k] if k < len(own) else None
                    a = active[u] if u is not None else 0
                    t1 = time.perf_counter()
                    ask = torch.empty(a + 8, dtype=torch.int64, device=dev)
                    if a:
                        mine.synchronize()
                        fetch_ctx.check(L.csa_part_positions(fetch_ctx.h, store, lists(u)[0], a, h, ask.data_ptr()))
                        fetch_ctx.sync()
                    sc, ask_b, order = bucket(ask[:a], None, True, fetch_ctx)
                    rc_ = [int(c) for c in _gather_small(np.array(sc, np.int64))[:, rank]] if world > 1 else sc
                    sent(sc, 8)
                    asked = _exchange(ask_b, sc, rc_)
                    m = int(asked.numel())
                    answers = torch.empty(m + 8, dtype=torch.int32, device=dev)
                    if m:
                        mine.synchronize()
                        fetch_ctx.check(L.csa_rank_shard_read(fetch_ctx.h, R.data_ptr(), lo, cnt, asked.data_ptr(), m, answers.data_ptr()))
                        fetch_ctx.sync()
                    sent(rc_, 4)
                    back = _exchange(answers, rc_, sc)
                    second = None
                    if a:
                        second = torch.empty(a + 8, dtype=torch.int32, device=dev)
                        mine.synchronize()
                        fetch_ctx.check(L.csa_unbucket(fetch_ctx.h, order.data_ptr(), back.data_ptr(), a, second.data_ptr()))
                        fetch_ctx.sync()
                    del ask, ask_b, asked, answers, back, order
                    lap("doubling_fetch", t1)
                    t1 = time.perf_counter()
                    if running is not None:
                        running.join()
                        if failures:
                            raise failures[0]
                    lap("doubling_wait_for_rank", t1)
                    running = None
                    if a:
                        running = threading.Thread(target=rank_job, args=(u, a, second, failures))
                        running.start()
                t1 = time.perf_counter()
                if running is not None:
                    running.join()
                    if failures:
                        raise failures[0]
                lap("doubling_wait_for_rank", t1)
                t1 = time.perf_counter()
                flush_outbox(box)
                del box
                lap("doubling_ranks_to_owners", t1)
                total_active = total_over_ranks(sum(active.values()))
                h *= 2
                gens += 1
                if gens > 45:
                    raise api.CascadeError(5, "doubling did not terminate")
        finally:
            fetch_ctx.close()
        info["generations"] = gens
        mark("doubling", t0)

        # ---- every part into its final order -------------------------------------------------------------------------------------------
        t0 = time.perf_counter()
        for u in own:
            lp, rp = lists(u)
            ctx.check(L.csa_rank_order(ctx.h, lp, rp, size[u], out_lanes.data_ptr() + 5 * own_first[u]))
        ctx.sync()
        mark("output", t0)
        del ranks_all
        if output != "device":
            del lanes_all
    finally:
        L.csa_store_destroy(store)
    info["ms"]["total"] = 1e3 * (time.perf_counter() - t_all)
    info.update({"partitions": pe, "parts": parts, "own_parts": len(own), "own_suffixes": own_total, "launches": ctx.launches,
                 "device_bytes_per_position": 8.0 / world})
    segments = [(int(part_off[u]), size[u], out_lanes[5 * own_first[u]:5 * (own_first[u] + size[u])]) for u in own]
    return segments, info
