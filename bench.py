#!/usr/bin/env python
"""Benchmark of the suffix-array build (and the batched query engine) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--tokens T] [--queries Q]

One step = one whole build of the suffix array of the seeded Zipf corpus (BASELINE config 2 at N = 1: 2e9 u16 tokens,
K = 8 splitters, 64 partitions, everything resident in one GPU's HBM). `value` times the build with the text already
in HBM (CUDA events on the library's stream); `e2e` times the host-buffer entry point (pinned host text in, 5-byte
suffix array out, copies inside the timed region). Prints ONE JSON line on rank 0.
"""
import argparse
import ctypes
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "sa_build_suffixes_per_s"
UNIT = "suffixes/s"
C2_TOKENS = 2_000_000_000
C2_PARTITIONS = 64
C2_MEAN_DOC = 1024
C5_QUERIES = 4_000_000
# DRAM read + write of one launch of the digit-pass kernel over 31.25 M records (the partition size of config 2), from the ncu
# capture summarised in profiles/onesweep_pass_kernel__sort_31m_records.md; the algorithmic bytes of that launch are 750e6.
ONESWEEP_TRAFFIC = 707.9e6


def measured_peak_gbs():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.stop, self.t = index, [], False, None

    def _run(self):
        while not self.stop:
            try:
                out = subprocess.run(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits"],
                                     capture_output=True, text=True, timeout=5).stdout.strip()
                if out:
                    self.rows.append([x.strip() for x in out.split(",")])
            except Exception:
                pass
            time.sleep(0.1)

    def __enter__(self):
        self.t = threading.Thread(target=self._run, daemon=True)
        self.t.start()
        return self

    def __exit__(self, *a):
        self.stop = True
        self.t.join(timeout=6)

    def summary(self):
        sm = [float(r[0]) for r in self.rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in self.rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [nm for k, nm in enumerate(names) if any(len(r) > 3 + k and r[3 + k].lower().startswith("active") for r in self.rows)]
        busy = [x for x in sm if x > 0.5 * (max(mx) if mx else 1)] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(self.rows)}


def ref_lib():
    p = os.path.join(ROOT, "oracle", "_ref", "libcascade_ref.so")
    if os.path.exists(p):
        return ctypes.CDLL(p), "reference"
    subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "liboracle.so"], stdout=subprocess.DEVNULL)
    return ctypes.CDLL(os.path.join(ROOT, "oracle", "liboracle.so")), "port"


def cpu_build_once(L, kind, T, n, out):
    """One CPU build of the sample with all host threads: the reference's comparator under a parallel sort
    (oracle/_ref), or the C port's parallel merge sort."""
    t0 = time.perf_counter()
    if kind == "reference":
        L.ref_build_sa40_parallel(T.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(n), out.ctypes.data_as(ctypes.c_void_p))
    else:
        L.orc_build_sa40(T.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(n), out.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(0))
    return time.perf_counter() - t0


def cpu_threads(L, kind):
    if kind == "reference":
        L.ref_thread_count.restype = ctypes.c_uint
        return int(L.ref_thread_count())
    L.orc_max_threads.restype = ctypes.c_int
    return int(L.orc_max_threads())


def cpu_baseline(sample_tokens, mean_doc, queries):
    """Times the reference's CPU paths on a bounded sample of the same corpus: the comparison-sort builder on all host
    threads, then the reference's batched host search over the sample's index."""
    from cascade_b200 import api
    L, kind = ref_lib()
    T = api.gen_corpus_host(sample_tokens, 0, mean_doc)
    out = np.zeros(5 * sample_tokens + 128, np.uint8)
    dt = cpu_build_once(L, kind, T, sample_tokens, out)
    res = {"value": sample_tokens / dt, "unit": UNIT, "cores": cpu_threads(L, kind), "kind": kind,
           "sample": f"first {sample_tokens} tokens of the same seeded Zipf corpus, one comparison-sort build ({dt:.2f} s)"}
    if queries:
        off, sym = api.gen_queries("substring", T, sample_tokens, queries // 2, seed=1)
        off2, sym2 = api.gen_queries("random", None, 0, queries - queries // 2, seed=2)
        off = np.concatenate([off, off2[1:] + off[-1]])
        sym = np.concatenate([sym, sym2, np.zeros(8, np.uint16)])
        itv = np.zeros(2 * queries, np.uint64)
        t0 = time.perf_counter()
        if kind == "reference":
            L.ref_host_search_find(T.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(sample_tokens), out.ctypes.data_as(ctypes.c_void_p),
                                   off.ctypes.data_as(ctypes.c_void_p), sym.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(queries),
                                   itv.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint(0), ctypes.c_uint(32))
        else:
            L.orc_find_batch(T.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(sample_tokens), out.ctypes.data_as(ctypes.c_void_p),
                             off.ctypes.data_as(ctypes.c_void_p), sym.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(queries),
                             itv.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(0))
        dq = time.perf_counter() - t0
        res["query"] = {"value": queries / dq, "unit": "queries/s (count only, host search)", "queries": queries,
                        "sample": f"index of the {sample_tokens}-token sample"}
    return res


def run_reference(args):
    """The reference arm: the reference's own CPU builder on the box's host cores, on bounded samples of the workload."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from cascade_b200 import api
    L, kind = ref_lib()
    sample = min(args.tokens, args.ref_sample)
    T = api.gen_corpus_host(sample, 0, C2_MEAN_DOC)
    out = np.zeros(5 * sample + 128, np.uint8)
    for _ in range(args.warmup):
        cpu_build_once(L, kind, T, sample, out)
    times = [cpu_build_once(L, kind, T, sample, out) for _ in range(args.steps)]
    ms = 1e3 * sum(times) / len(times)
    v = sample / (ms * 1e-3)
    cores = cpu_threads(L, kind)
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
            "config": workload_config(args, args.gpus),
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": cores, "kind": kind,
                             "sample": f"each step builds the first {sample} tokens of the workload's corpus with the reference's CPU comparison-sort builder"},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line))


def workload_config(args, n_gpus):
    return {"workload": "in-HBM suffix-array build, BASELINE config 2" if args.tokens == C2_TOKENS else "in-HBM suffix-array build (reduced size)",
            "tokens": args.tokens, "symbol_bytes": 2, "vocab": 50257, "zipf_s": 1.1, "mean_doc": C2_MEAN_DOC, "separator": 65535,
            "partitions": C2_PARTITIONS, "kgram": 8, "output": "sa40", "seed": 0, "gpus": n_gpus,
            "l2": "inputs (4 GB text, 24 GB of sort records per pass at full size) exceed the 126 MB L2; no flush needed"}


def run_ours(args):
    import torch
    from cascade_b200 import api
    from cascade_b200._lib import c_u64

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        torch.cuda.set_device(local)
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    if world > 1:
        from cascade_b200 import multi
        return multi.bench(args, rank, world, local)

    torch.cuda.set_device(local)
    ctx = api.Context(local)
    n, p = args.tokens, C2_PARTITIONS
    peak, peak_kind = measured_peak_gbs()
    T = api.gen_corpus_device(ctx, n, 0, C2_MEAN_DOC)
    out = torch.zeros(5 * n + api.SA_PAD_BYTES, dtype=torch.uint8, device=T.device)

    for _ in range(args.warmup):
        api.build_sa(ctx, T, n, p, out=out)
    ctx.L.csa_set_pass_timing(ctx.h, 1)
    ctx.reset_counters()
    torch.cuda.synchronize()
    step_ms, launches, stats = [], 0, None
    with ClockSampler(local) as clocks:
        t0 = time.perf_counter()
        for _ in range(args.steps):
            _, st = api.build_sa(ctx, T, n, p, out=out)
            step_ms.append(st.ms_total)
            launches += st.kernel_launches
            stats = st
        torch.cuda.synchronize()
        wall_ms = 1e3 * (time.perf_counter() - t0) / args.steps
    ms = sum(step_ms) / len(step_ms)
    pm, pc, pr, pb = ctypes.c_double(0), c_u64(0), c_u64(0), c_u64(0)
    ctx.L.csa_get_pass_timing(ctx.h, ctypes.byref(pm), ctypes.byref(pc), ctypes.byref(pr), ctypes.byref(pb))
    ctx.L.csa_set_pass_timing(ctx.h, 0)
    # algorithmic bytes: one read and one write of every record of every pass (12-byte key + position records; 8-byte
    # records in the keys-only passes that order rank updates by address)
    achieved = pb.value / (pm.value * 1e-3) / 1e9 if pm.value > 0 else 0.0
    roofline = {"bound": "hbm", "kernel": "onesweep_pass_kernel (one 8-bit digit pass of the LSD radix sort)", "achieved": achieved, "peak": peak,
                "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}",
                "traffic": ONESWEEP_TRAFFIC, "traffic_note": "bytes per launch over 31.25 M records (algorithmic: 750e6), ncu capture in profiles/",
                "passes": pc.value, "records": pr.value, "pass_ms_total": pm.value, "share_of_step": pm.value / (ms * args.steps)}

    # ---- end to end through the host-buffer entry point --------------------------------------------------------------
    e2e = None
    if not args.no_e2e:
        th = torch.empty(n + api.TEXT_PAD, dtype=torch.uint16).pin_memory()
        th.copy_(T.cpu())
        oh = torch.empty(5 * n + api.SA_PAD_BYTES, dtype=torch.uint8).pin_memory()
        api.build_sa_host(ctx, th, n, p, out=oh)      # warm-up (grows the arena)
        ts = []
        for _ in range(max(1, min(args.steps, 2))):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            api.build_sa_host(ctx, th, n, p, out=oh)
            ts.append(time.perf_counter() - t0)
        e_ms = 1e3 * sum(ts) / len(ts)
        e2e = {"value": n / (e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": 2 * n, "d2h_bytes_per_step": 5 * n, "ms_per_step": e_ms,
               "api": "csa_build_sa_host (pinned host text in, sa40 out)"}
        # the two entry points must give the same bytes
        same = bool(torch.equal(oh[:5 * n].cuda(), out[:5 * n]))
        e2e["matches_device_path"] = same
    else:
        th = None

    # ---- batched queries on the index just built (BASELINE config 5) ------------------------------------------------
    query = None
    if args.queries > 0:
        if th is None:
            th = T.cpu()
        tn = th.view(torch.int16).numpy().view(np.uint16)
        q = args.queries
        oa, sa_ = api.gen_queries("substring", tn, n, q // 2, seed=1)
        ob, sb = api.gen_queries("random", None, 0, q - q // 2, seed=2)
        off = np.concatenate([oa, ob[1:] + oa[-1]])
        sym = np.concatenate([sa_, sb, np.zeros(8, np.uint16)])
        idx = api.SuffixIndex(ctx, T, out, n, 32)
        od = torch.from_numpy(off.view(np.int64)).cuda()
        sd = torch.from_numpy(sym.view(np.int16)).cuda()
        for _ in range(2):                       # warm: the timed call then finds its result buffers in torch's pool
            itv = idx.find(od, sd, q)
            pos, cnt = idx.locate(itv, q, 100)
        del pos, cnt
        t0 = time.perf_counter()
        itv = idx.find(od, sd, q)
        pos, cnt = idx.locate(itv, q, 100)
        dq = time.perf_counter() - t0
        fails, first = idx.certify(od, sd, q, itv)
        offp = torch.from_numpy(off.view(np.int64)).pin_memory()
        symp = torch.from_numpy(sym.view(np.int16)).pin_memory()
        bufs = {"itv": torch.empty(2 * q, dtype=torch.int64).pin_memory(), "cnt": torch.empty(q, dtype=torch.int32).pin_memory(),
                "pos_off": torch.empty(q + 1, dtype=torch.int64).pin_memory(), "pos": torch.empty(q * 100, dtype=torch.int64).pin_memory()}
        idx.query_host(offp, symp, 100, bufs)
        t0 = time.perf_counter()
        r = idx.query_host(offp, symp, 100, bufs)
        dqe = time.perf_counter() - t0
        itv_np = bufs["itv"].numpy().view(np.uint64)
        # the same index with the suffix array left in pinned host memory (the device reads it over PCIe)
        pinned = None
        if not args.no_e2e:
            sa_pinned = torch.empty(5 * n + api.SA_PAD_BYTES, dtype=torch.uint8).pin_memory()
            sa_pinned.copy_(out.cpu())
            idx_h = api.SuffixIndex(ctx, T, sa_pinned, n, 32, table=idx.table)
            pos_h, cnt_h = idx_h.locate(idx_h.find(od, sd, q), q, 100)
            del pos_h, cnt_h
            t0 = time.perf_counter()
            itv_h = idx_h.find(od, sd, q)
            pos_h, cnt_h = idx_h.locate(itv_h, q, 100)
            dqh = time.perf_counter() - t0
            pinned = {"value": q / dqh, "unit": "queries/s (count + locate <= 100, suffix array in pinned host memory, text and table in HBM)",
                      "same_intervals": bool(torch.equal(itv_h, itv))}
        query = {"value": q / dq, "unit": "queries/s (count + locate <= 100, index in HBM, batch in HBM)", "queries": q,
                 "e2e": {"value": q / dqe, "unit": "queries/s (host batch in, intervals + positions out)",
                         "h2d_bytes": int(off.nbytes + sym.nbytes), "d2h_bytes": int(q * 16 + q * 4 + (q + 1) * 8 + r[4] * 8)},
                 "sa_in_pinned_host_memory": pinned, "certificate_failures": fails, "positions": r[4], "counts_hash": f"{api.counts_hash(itv_np):016x}", "table_stride": 32}

    line = {"metric": METRIC, "value": n / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "wall_ms_per_step": wall_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
            "config": workload_config(args, 1), "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": int(launches),
            "roofline": roofline,
            "phases_ms": {"partition": stats.ms_partition, "gen0": stats.ms_gen0, "doubling": stats.ms_doubling, "output": stats.ms_output},
            "build": {"partitions": stats.partitions, "generations": stats.generations, "max_partition": stats.max_partition,
                      "active_after_gen0": stats.active_after_gen0, "sort_passes_per_step": stats.sort_passes},
            "query": query}
    if not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(min(n, args.cpu_sample), C2_MEAN_DOC, min(args.queries, 1_000_000))
    print(json.dumps(line))
    ctx.close()


def run_micro_sort(args):
    """The radix sort alone on uniformly random 64-bit keys with 32-bit values: per-pass device time and GB/s."""
    import torch
    from cascade_b200 import api
    from cascade_b200._lib import c_u64, c_int
    ctx = api.Context(0)
    if args.variant >= 0:
        assert ctx.L.csa_debug_set(1, args.variant) == 0
    n = args.records
    g = torch.Generator(device="cuda").manual_seed(1)
    keys0 = torch.randint(-(1 << 62), 1 << 62, (n,), device="cuda", dtype=torch.int64, generator=g)
    keys, ka = keys0.clone(), torch.empty_like(keys0)
    vals, va = torch.arange(n, device="cuda", dtype=torch.int32), torch.empty(n, device="cuda", dtype=torch.int32)
    wsb = ctx.L.csa_sort_workspace_bytes(n)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    peak, kind = measured_peak_gbs()
    whole_ms = []
    for it in range(args.warmup + args.steps):
        keys.copy_(keys0)
        torch.cuda.synchronize()
        if it == args.warmup:
            ctx.L.csa_set_pass_timing(ctx.h, 1)
            ctx.reset_counters()
        in_alt = c_int(0)
        t0 = time.perf_counter()
        ctx.check(ctx.L.csa_sort_pairs(ctx.h, keys.data_ptr(), ka.data_ptr(), vals.data_ptr(), va.data_ptr(), 4, n, 0, args.bits, ws.data_ptr(), wsb,
                                       ctypes.byref(in_alt)))
        ctx.sync()
        if it >= args.warmup:
            whole_ms.append((time.perf_counter() - t0) * 1e3)
    pm, pc, pr, pb = ctypes.c_double(0), c_u64(0), c_u64(0), c_u64(0)
    ctx.L.csa_get_pass_timing(ctx.h, ctypes.byref(pm), ctypes.byref(pc), ctypes.byref(pr), ctypes.byref(pb))
    gbs = pb.value / (pm.value * 1e-3) / 1e9
    print(json.dumps({"micro": "sort", "records": n, "bits": args.bits, "passes": pc.value, "ms_per_pass": pm.value / max(1, pc.value),
                      "achieved_gbs": gbs, "peak_gbs": peak, "frac": gbs / peak, "peak_kind": kind, "variant": args.variant,
                      "whole_sort_ms": sum(whole_ms) / len(whole_ms), "outside_passes_ms": sum(whole_ms) / len(whole_ms) - pm.value / args.steps}))
    ctx.close()


def run_repeat(args):
    """BASELINE config 3, the worst case for prefix doubling: 4096 base documents (geometric, mean 2048, Zipf tokens), then
    copies of random base documents with 0.1 % of their tokens replaced, 1e9 tokens in all. Reports the build alone."""
    import torch
    from cascade_b200 import api
    n = args.tokens if args.tokens != C2_TOKENS else 1_000_000_000
    ctx = api.Context(0)
    t0 = time.perf_counter()
    Th = api.gen_repeat_corpus_host(n, seed=0, base_docs=4096, mean_doc=2048, mutate=0.001)
    T = torch.from_numpy(Th.view(np.int16)).cuda().view(torch.uint16)
    gen_s = time.perf_counter() - t0
    out = torch.zeros(5 * n + api.SA_PAD_BYTES, dtype=torch.uint8, device="cuda")
    for _ in range(max(1, args.warmup - 2)):
        api.build_sa(ctx, T, n, C2_PARTITIONS, out=out)
    ms, st = [], None
    for _ in range(args.steps):
        _, st = api.build_sa(ctx, T, n, C2_PARTITIONS, out=out)
        ms.append(st.ms_total)
    # sampled order check on the device: neighbours compared on their first 64 symbols (undecided pairs count as consistent)
    g = torch.Generator(device="cuda").manual_seed(0)
    r = torch.randint(0, n - 1, (1 << 20,), device="cuda", generator=g)
    b = out[:5 * n].view(n, 5)
    def entry(idx):
        e = b[idx].to(torch.int64)
        return e[:, 0] | (e[:, 1] << 8) | (e[:, 2] << 16) | (e[:, 3] << 24) | (e[:, 4] << 32)
    pa, pb = entry(r), entry(r + 1)
    Tl = T.view(torch.int16)
    undecided = torch.ones_like(pa, dtype=torch.bool)
    bad = torch.zeros_like(undecided)
    for k in range(64):
        xa = torch.where(pa + k < n, Tl[torch.clamp(pa + k, max=n)].to(torch.int64) & 0xFFFF, torch.full_like(pa, -1))
        xb = torch.where(pb + k < n, Tl[torch.clamp(pb + k, max=n)].to(torch.int64) & 0xFFFF, torch.full_like(pb, -1))
        bad |= undecided & (xa > xb)
        undecided &= (xa == xb) & (xa >= 0)
    m = sum(ms) / len(ms)
    print(json.dumps({"metric": METRIC, "value": n / (m * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps, "ms_per_step": m,
                      "config": {"workload": "repetitive corpus, BASELINE config 3", "tokens": n, "base_docs": 4096, "mean_doc": 2048, "mutate": 0.001,
                                 "partitions": C2_PARTITIONS}, "generations": st.generations,
                      "active_per_generation": [int(x) for x in st.active_per_gen[:st.generations]],
                      "phases_ms": {"partition": st.ms_partition, "gen0": st.ms_gen0, "doubling": st.ms_doubling, "output": st.ms_output},
                      "sort_passes": st.sort_passes, "order_violations_in_1M_sampled_neighbours": int(bad.sum().item()),
                      "host_generation_s": gen_s}))
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--tokens", type=int, default=C2_TOKENS)
    ap.add_argument("--queries", type=int, default=C5_QUERIES)
    ap.add_argument("--cpu-sample", type=int, default=1 << 25)
    ap.add_argument("--ref-sample", type=int, default=1 << 24)
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--workload", default="zipf", choices=["zipf", "repeat"],
                    help="zipf: BASELINE config 2; repeat: config 3 (1e9 tokens of near-duplicate documents, build only)")
    ap.add_argument("--micro", default=None, choices=["sort"], help="time one kernel family alone instead of the build")
    ap.add_argument("--records", type=int, default=31_250_000)
    ap.add_argument("--bits", type=int, default=64)
    ap.add_argument("--variant", type=int, default=-1, help="shape of the digit-pass kernel (test hook), -1 = default")
    args = ap.parse_args()
    if args.micro == "sort":
        return run_micro_sort(args)
    if args.workload == "repeat":
        return run_repeat(args)
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
