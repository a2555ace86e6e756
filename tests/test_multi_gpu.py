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
        out, first, count, st = multi.build_sa_multi(ctx, comm, T, n, 16)
        assert (first, count) == (0, n)
        assert torch.equal(out[:5 * n], ref[:5 * n])
    finally:
        ctx.close()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, n, p, kind, q):
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
    comm, keep = multi.make_comm(rank, world, None)
    for _ in range(2):      # twice: the second build reuses the peers' mappings
        out, first, count, st = multi.build_sa_multi(ctx, comm, T, n, p)
    sl = out[:5 * count].cpu().numpy()
    ref = None
    if rank == 0:
        r, _ = api.build_sa(ctx, T, n, p)
        ref = r[:5 * n].cpu().numpy()
    q.put((rank, first, count, sl, ref, st.generations, st.peer_bytes))
    dist.barrier()
    ctx.close()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,n,p,kind", [(2, 3_000_000, 16, "zipf"), (2, 400_000, 8, "repeat"), (3, 1_000_003, 5, "zipf")])
def test_sharded_build_equals_the_single_gpu_build(world, n, p, kind):
    port = _free_port()
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, p, kind, q)) for r in range(world)]
    for pr in procs:
        pr.start()
    res = sorted((q.get(timeout=600) for _ in range(world)), key=lambda x: x[0])
    for pr in procs:
        pr.join(timeout=120)
        assert pr.exitcode == 0
    ref = res[0][4]
    at = 0
    for rank, first, count, sl, _, gens, peer in res:
        assert first == at, "slices must be contiguous in rank order"
        assert np.array_equal(sl, ref[5 * first:5 * (first + count)]), f"rank {rank}'s slice differs"
        at += count
    assert at == n
    if kind == "repeat":
        assert res[0][5] >= 5
    assert sum(r[6] for r in res) > 0      # ranks and positions did cross between the GPUs' memories
