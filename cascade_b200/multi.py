"""Multi-GPU build, one process per GPU: the host plumbing (torch.distributed) around csa_build_sa_multi.

The library asks its caller for ONE collective, an all-gather of small host buffers (partition sizes, IPC handles,
active counts; it also serves as the barrier between the steps). Here it is torch.distributed.all_gather, on CPU
tensors under gloo and on device tensors under NCCL. All bulk data moves inside the library's kernels as peer loads
and stores.
"""
import ctypes

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
