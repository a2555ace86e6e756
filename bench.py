#!/usr/bin/env python
"""Benchmark of the suffix-array build (and the batched query engine) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--tokens T] [--queries Q]

One step = one whole build of the suffix array of the seeded Zipf corpus (BASELINE config 2 at N = 1: 2e9 u16 tokens,
K = 8 splitters, 64 partitions, everything resident in one GPU's HBM). `value` times the build with the text already
in HBM (CUDA events on the library's stream); `e2e` times the host-buffer entry point (pinned host text in, 5-byte
suffix array out, copies inside the timed region). Every array that a number is quoted on is checked in full on the
device (permutation + order of every neighbouring pair) outside the timed region. Prints ONE JSON line on rank 0.

`--impl reference` times the reference's own CPU builder on the box's host cores, on a bounded sample of the same corpus;
it loads nothing but the CPU checkers under oracle/.
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
C3_TOKENS = 1_000_000_000
C5_QUERIES = 4_000_000
# DRAM read + write per record of one launch of the digit-pass kernel (24 B algorithmic), from an ncu capture of a launch over
# 1e8 records (a 1e8-token build); traffic grows with the records of a launch, so the benchmark scales it to its own launch
# (generation 0 moves all n records per launch). It is a figure from that capture, not measured by the run that prints it.
ONESWEEP_TRAFFIC_PER_RECORD_FROM_PROFILE = 23.71


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


# ---- the CPU side: the reference's own code (oracle/_ref) or the C restatement (oracle/liboracle.so) -------------------------

def zipf_cdf(vocab=50257, s=1.1):
    """64-bit inverse-CDF thresholds of Zipf(s) over ranks 1..vocab (the same table as cascade_b200.api.zipf_cdf, kept here
    so that the CPU arm needs nothing of the product)."""
    w = np.arange(1, vocab + 1, dtype=np.float64) ** (-s)
    c = np.cumsum(w)
    c /= c[-1]
    t = np.minimum(np.floor(c * 18446744073709551616.0), 18446744073709551615.0)
    out = np.array([int(x) if x < 18446744073709551615.0 else 0xFFFFFFFFFFFFFFFF for x in t], dtype=np.uint64)
    out[-1] = np.uint64(0xFFFFFFFFFFFFFFFF)
    return out


def host_threads():
    try:
        return len(os.sched_getaffinity(0))
    except Exception:
        return os.cpu_count() or 1


class CpuSide:
    """The CPU checkers, with their thread count set by hand: a launcher such as torch.distributed.run exports
    OMP_NUM_THREADS=1 to its children, which would leave all but one core idle."""

    def __init__(self):
        self.threads = host_threads()
        os.environ["OMP_NUM_THREADS"] = str(self.threads)          # read by the OpenMP runtime when it is first loaded
        orc = os.path.join(ROOT, "oracle", "liboracle.so")
        if not os.path.exists(orc):
            subprocess.check_call(["make", "-C", os.path.join(ROOT, "oracle"), "liboracle.so"], stdout=subprocess.DEVNULL)
        self.orc = ctypes.CDLL(orc)
        self.orc.orc_set_threads(ctypes.c_int(self.threads))
        ref = os.path.join(ROOT, "oracle", "_ref", "libcascade_ref.so")
        self.ref = ctypes.CDLL(ref) if os.path.exists(ref) else None
        if self.ref is not None:
            self.ref.ref_set_threads(ctypes.c_int(self.threads))
        self.kind = "reference" if self.ref is not None else "port"

    def corpus(self, n, mean_doc, seed=0):
        cdf = zipf_cdf()
        T = np.zeros(n + 64, dtype=np.uint16)
        self.orc.orc_gen_corpus(T.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(0), ctypes.c_uint64(n), ctypes.c_uint64(seed),
                                ctypes.c_uint32(mean_doc), cdf.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint32(len(cdf)))
        return T

    def build_once(self, T, n, out):
        """One CPU build with all host threads: the reference's comparator under a parallel sort (oracle/_ref), or the C
        port's parallel merge sort."""
        t0 = time.perf_counter()
        if self.ref is not None:
            self.ref.ref_build_sa40_parallel(T.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(n), out.ctypes.data_as(ctypes.c_void_p))
        else:
            self.orc.orc_build_sa40(T.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(n), out.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(0))
        return time.perf_counter() - t0

    def cores(self):
        if self.ref is not None:
            self.ref.ref_thread_count.restype = ctypes.c_uint
            return max(int(self.ref.ref_thread_count()), self.threads)
        self.orc.orc_max_threads.restype = ctypes.c_int
        return int(self.orc.orc_max_threads())

    def find(self, T, n, sa40, off, sym, q, itv):
        vp = ctypes.c_void_p
        if self.ref is not None:
            self.ref.ref_host_search_find(T.ctypes.data_as(vp), ctypes.c_uint64(n), sa40.ctypes.data_as(vp), off.ctypes.data_as(vp),
                                          sym.ctypes.data_as(vp), ctypes.c_uint64(q), itv.ctypes.data_as(vp), ctypes.c_uint(0), ctypes.c_uint(32))
        else:
            self.orc.orc_find_batch(T.ctypes.data_as(vp), ctypes.c_uint64(n), sa40.ctypes.data_as(vp), off.ctypes.data_as(vp),
                                    sym.ctypes.data_as(vp), ctypes.c_uint64(q), itv.ctypes.data_as(vp), ctypes.c_int(0))


def cpu_baseline(sample_tokens, mean_doc, queries):
    """Times the reference's CPU paths on a bounded sample of the same corpus: the comparison-sort builder on all host
    threads, then the reference's batched host search over the sample's index."""
    from cascade_b200 import api
    cpu = CpuSide()
    T = cpu.corpus(sample_tokens, mean_doc)
    out = np.zeros(5 * sample_tokens + 128, np.uint8)
    dt = cpu.build_once(T, sample_tokens, out)
    res = {"value": sample_tokens / dt, "unit": UNIT, "cores": cpu.cores(), "kind": cpu.kind,
           "sample": f"first {sample_tokens} tokens of the same seeded Zipf corpus, one comparison-sort build ({dt:.2f} s)"}
    if queries:
        off, sym = api.gen_queries("substring", T, sample_tokens, queries // 2, seed=1)
        off2, sym2 = api.gen_queries("random", None, 0, queries - queries // 2, seed=2)
        off = np.concatenate([off, off2[1:] + off[-1]])
        sym = np.concatenate([sym, sym2, np.zeros(8, np.uint16)])
        itv = np.zeros(2 * queries, np.uint64)
        t0 = time.perf_counter()
        cpu.find(T, sample_tokens, out, off, sym, queries, itv)
        dq = time.perf_counter() - t0
        res["query"] = {"value": queries / dq, "unit": "queries/s (count only, host search)", "queries": queries,
                        "sample": f"index of the {sample_tokens}-token sample"}
    return res


def workload_config(args, n_gpus):
    return {"workload": "in-HBM suffix-array build, BASELINE config 2" if args.tokens == C2_TOKENS else "in-HBM suffix-array build (reduced size)",
            "tokens": args.tokens, "symbol_bytes": 2, "vocab": 50257, "zipf_s": 1.1, "mean_doc": C2_MEAN_DOC, "separator": 65535,
            "partitions": C2_PARTITIONS, "kgram": 8, "output": "sa40", "seed": 0, "gpus": n_gpus,
            "l2": "inputs (4 GB text, 24 GB of sort records per pass at full size) exceed the 126 MB L2; no flush needed"}


def run_reference(args):
    """The reference arm: the reference's own CPU builder on all host cores, each step one build of a bounded sample of the
    workload's corpus. Under a multi-rank launch rank 0 alone works. Nothing of the product is loaded."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cpu = CpuSide()
    sample = min(args.tokens, args.ref_sample)
    T = cpu.corpus(sample, C2_MEAN_DOC)
    out = np.zeros(5 * sample + 128, np.uint8)
    for _ in range(args.warmup):
        cpu.build_once(T, sample, out)
    times = [cpu.build_once(T, sample, out) for _ in range(args.steps)]
    ms = 1e3 * sum(times) / len(times)
    v = sample / (ms * 1e-3)
    cfg = workload_config(args, args.gpus)
    cfg["workload"] += f" -- CPU arm: each step sorts a sample, the first {sample} tokens of that corpus"
    cfg["reference_sample_tokens"] = sample
    what = "the reference's CPU comparison-sort builder" if cpu.kind == "reference" else "the C port of the reference's CPU builder"
    line = {"impl": "reference", "metric": METRIC, "value": v, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
            "config": cfg,
            "cpu_baseline": {"value": v, "unit": UNIT, "cores": cpu.cores(), "kind": cpu.kind,
                             "sample": f"each step builds the first {sample} tokens of the workload's corpus with {what} on all host threads"},
            "e2e": {"value": v, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
    print(json.dumps(line))


# ---- the GPU side -----------------------------------------------------------------------------------------------------

def pass_roofline(ctx, peak, peak_kind, step_ms_total, traffic):
    from cascade_b200._lib import c_u64
    pm, pc, pr, pb = ctypes.c_double(0), c_u64(0), c_u64(0), c_u64(0)
    ctx.L.csa_get_pass_timing(ctx.h, ctypes.byref(pm), ctypes.byref(pc), ctypes.byref(pr), ctypes.byref(pb))
    ctx.L.csa_set_pass_timing(ctx.h, 0)
    # algorithmic bytes: one read and one write of every record of every pass (12-byte key + position records; 8-byte
    # records in the keys-only passes that order rank updates by address)
    achieved = pb.value / (pm.value * 1e-3) / 1e9 if pm.value > 0 else 0.0
    r = {"bound": "hbm", "kernel": "one 8-bit digit pass of the LSD radix sort (onesweep_seg_pass_kernel over all partitions in generation 0, onesweep_pass_kernel "
                                   "over the tied suffixes later: the same tile code)", "achieved": achieved, "peak": peak,
         "unit": "GB/s", "frac": achieved / peak, "peak_kind": f"of {peak_kind}", "traffic": traffic,
         "passes": pc.value, "records": pr.value, "pass_ms_total": pm.value}
    if traffic is not None:
        r["traffic_note"] = ("DRAM bytes of one generation-0 launch (all records of the build; algorithmic: 24 B per record), scaled by the records from an ncu "
                             "capture of the same kernel over 1e8 records (23.71 B per record); not measured by this run")
    if step_ms_total:
        r["share_of_step"] = pm.value / step_ms_total
    return r


def sort_baselines(ctx, records=31_250_000, reps=5):
    """The product's radix sort and the library sort the reference calls (cub::DeviceRadixSort::SortPairs), both on `records`
    random (u64 key, u32 value) records, all 64 key bits: whole-sort device milliseconds side by side."""
    import torch
    from cascade_b200._lib import c_int
    n = records
    g = torch.Generator(device="cuda").manual_seed(1)
    keys0 = torch.randint(-(1 << 62), 1 << 62, (n,), device="cuda", dtype=torch.int64, generator=g)
    keys, ka = keys0.clone(), torch.empty_like(keys0)
    vals, va = torch.arange(n, device="cuda", dtype=torch.int32), torch.empty(n, device="cuda", dtype=torch.int32)
    wsb = ctx.L.csa_sort_workspace_bytes(n)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    ours = []
    for it in range(reps + 1):
        keys.copy_(keys0)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        s = torch.cuda.ExternalStream(ctx.stream())
        e0.record(s)
        in_alt = c_int(0)
        ctx.check(ctx.L.csa_sort_pairs(ctx.h, keys.data_ptr(), ka.data_ptr(), vals.data_ptr(), va.data_ptr(), 4, n, 0, 64, ws.data_ptr(), wsb,
                                       ctypes.byref(in_alt)))
        e1.record(s)
        ctx.sync()
        if it > 0:
            ours.append(e0.elapsed_time(e1))
    del keys, ka, vals, va, ws, keys0
    torch.cuda.empty_cache()
    res = {"records": n, "key_bits": 64, "value_bytes": 4, "ours_ms": sum(ours) / len(ours),
           "ours_gbs_per_pass": 8 * 2 * 12 * n / (sum(ours) / len(ours) * 1e-3) / 1e9}
    so = os.path.join(ROOT, "bench_cub_sort.so")
    if os.path.exists(so):
        L = ctypes.CDLL(so)
        ms = ctypes.c_double(0)
        rc = L.cub_sort_pairs_ms(ctypes.c_ulonglong(n), ctypes.c_int(64), ctypes.c_int(reps), ctypes.byref(ms))
        if rc == 0:
            res["cub_ms"] = ms.value
            res["cub_gbs_per_pass"] = 8 * 2 * 12 * n / (ms.value * 1e-3) / 1e9
            res["ours_over_cub"] = ms.value / res["ours_ms"]
        else:
            res["cub_error"] = rc
    else:
        res["cub_error"] = "bench_cub_sort.so is not built"
    res["note"] = ("whole sort, device time; cub::DeviceRadixSort::SortPairs is the call the reference makes, built here for sm_100a as a "
                   "benchmark-only baseline; the per-pass figure divides 8 passes x 24 B per record by the time")
    return res


def run_config3(ctx, args):
    """BASELINE config 3, the worst case for prefix doubling: 4096 base documents (geometric, mean 2048, Zipf tokens), then
    copies of random base documents with 0.1 % of their tokens replaced. Build alone, then the full check of the array."""
    import torch
    from cascade_b200 import api
    n = args.config3_tokens
    t0 = time.perf_counter()
    Th = api.gen_repeat_corpus_host(n, seed=0, base_docs=4096, mean_doc=2048, mutate=0.001)
    T = torch.from_numpy(Th.view(np.int16)).cuda().view(torch.uint16)
    del Th
    gen_s = time.perf_counter() - t0
    out = torch.zeros(5 * n + api.SA_PAD_BYTES, dtype=torch.uint8, device="cuda")
    api.build_sa(ctx, T, n, C2_PARTITIONS, out=out)
    ms, st = [], None
    for _ in range(max(1, min(args.steps, 3))):
        _, st = api.build_sa(ctx, T, n, C2_PARTITIONS, out=out)
        ms.append(st.ms_total)
    v = api.validate_sa(ctx, T, n, out)
    m = sum(ms) / len(ms)
    res = {"value": n / (m * 1e-3), "unit": UNIT, "ms_per_step": m, "steps": len(ms),
           "config": {"workload": "repetitive corpus, BASELINE config 3", "tokens": n, "base_docs": 4096, "mean_doc": 2048, "mutate": 0.001,
                      "partitions": C2_PARTITIONS},
           "generations": st.generations, "active_per_generation": [int(x) for x in st.active_per_gen[:st.generations]],
           "phases_ms": {"partition": st.ms_partition, "gen0": st.ms_gen0, "doubling": st.ms_doubling, "output": st.ms_output},
           "sort_passes": st.sort_passes, "validated": v["ok"], "validation": v, "host_generation_s": gen_s}
    del T, out
    torch.cuda.empty_cache()
    return res


def make_queries(api, tn, n, q):
    oa, sa_ = api.gen_queries("substring", tn, n, q // 2, seed=1)
    ob, sb = api.gen_queries("random", None, 0, q - q // 2, seed=2)
    return np.concatenate([oa, ob[1:] + oa[-1]]), np.concatenate([sa_, sb, np.zeros(8, np.uint16)])


def run_ours(args):
    import torch
    from cascade_b200 import api

    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        return run_ours_multi(args)

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
    roofline = pass_roofline(ctx, peak, peak_kind, ms * args.steps, ONESWEEP_TRAFFIC_PER_RECORD_FROM_PROFILE * n)
    validation = api.validate_sa(ctx, T, n, out)         # the whole array, outside the timed region

    # ---- end to end through the host-buffer entry point --------------------------------------------------------------
    e2e = None
    th = None
    if not args.no_e2e:
        th = torch.empty(n + api.TEXT_PAD, dtype=torch.uint16).pin_memory()
        th.copy_(T.cpu())
        oh = torch.empty(5 * n + api.SA_PAD_BYTES, dtype=torch.uint8).pin_memory()
        api.build_sa_host(ctx, th, n, p, out=oh)      # warm-up (grows the arena)
        ts = []
        for _ in range(args.steps):
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            api.build_sa_host(ctx, th, n, p, out=oh)
            ts.append(time.perf_counter() - t0)
        e_ms = 1e3 * sum(ts) / len(ts)
        e2e = {"value": n / (e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": 2 * n, "d2h_bytes_per_step": 5 * n, "ms_per_step": e_ms,
               "steps": len(ts), "api": "csa_build_sa_host (pinned host text in, sa40 out)"}
        # the two entry points must give the same bytes
        e2e["matches_device_path"] = bool(torch.equal(oh[:5 * n].cuda(), out[:5 * n]))
        del oh

    # ---- batched queries on the index just built (BASELINE config 5) ------------------------------------------------
    query = None
    if args.queries > 0:
        if th is None:
            th = T.cpu()
        tn = th.view(torch.int16).numpy().view(np.uint16)
        q = args.queries
        off, sym = make_queries(api, tn, n, q)
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
        tq = []
        for _ in range(3):
            t0 = time.perf_counter()
            r = idx.query_host(offp, symp, 100, bufs)
            tq.append(time.perf_counter() - t0)
        dqe = min(tq)
        itv_np = bufs["itv"].numpy().view(np.uint64)
        same_host = bool(np.array_equal(itv_np, itv.cpu().numpy().view(np.uint64)))
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
            del sa_pinned, idx_h, pos_h, cnt_h, itv_h
        query = {"value": q / dq, "unit": "queries/s (count + locate <= 100, index in HBM, batch in HBM)", "queries": q,
                 "e2e": {"value": q / dqe, "unit": "queries/s (host batch in, intervals + positions out; best of 3)",
                         "h2d_bytes": int(off.nbytes + sym.nbytes), "d2h_bytes": int(q * 16 + q * 4 + (q + 1) * 8 + r[4] * 8),
                         "same_intervals_as_device_path": same_host},
                 "sa_in_pinned_host_memory": pinned, "certificate_failures": fails, "positions": r[4], "counts_hash": f"{api.counts_hash(itv_np):016x}", "table_stride": 32}
        del idx, od, sd, pos, cnt, itv, bufs
    del th
    torch.cuda.empty_cache()

    line = {"metric": METRIC, "value": n / (ms * 1e-3), "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms,
            "wall_ms_per_step": wall_ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
            "config": workload_config(args, 1), "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": int(launches),
            "roofline": roofline, "validated": validation["ok"], "validation": validation,
            "phases_ms": {"partition": stats.ms_partition, "gen0": stats.ms_gen0, "doubling": stats.ms_doubling, "output": stats.ms_output},
            "build": {"partitions": stats.partitions, "generations": stats.generations, "max_partition": stats.max_partition,
                      "active_after_gen0": stats.active_after_gen0, "sort_passes_per_step": stats.sort_passes,
                      "active_per_generation": [int(x) for x in stats.active_per_gen[:stats.generations]]},
            "query": query}
    del T, out
    torch.cuda.empty_cache()
    if not args.no_sort_baseline:
        line["sort_baseline"] = sort_baselines(ctx)
    if args.config3_tokens > 0:
        line["config3"] = run_config3(ctx, args)
    if not args.no_cpu:
        line["cpu_baseline"] = cpu_baseline(min(n, args.cpu_sample), C2_MEAN_DOC, min(args.queries, 1_000_000))
    print(json.dumps(line))
    ctx.close()


def _max_over_ranks(x, device):
    import torch
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def _sum_over_ranks(x, device):
    import torch
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def run_ours_multi(args):
    """N > 1: the same corpus (strong scaling), partitions sharded over the ranks, one process per GPU."""
    import torch
    import torch.distributed as dist
    from cascade_b200 import api, multi

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    ctx = api.Context(local)
    name = [f"/cascade_b200_{os.getpid()}_{int(time.time())}"]
    dist.broadcast_object_list(name, src=0)            # one name for the job's shared-memory object
    comm, close_comm = multi.make_shm_comm(rank, world, name[0])
    n, p = args.tokens, C2_PARTITIONS
    peak, peak_kind = measured_peak_gbs()
    T = api.gen_corpus_device(ctx, n, 0, C2_MEAN_DOC)          # every rank makes the same text in its own HBM
    cap = min(n, n // world + n // 8 + 1024)
    out = torch.zeros(5 * cap + api.SA_PAD_BYTES, dtype=torch.uint8, device=dev)
    for _ in range(args.warmup):
        multi.build_sa_multi(ctx, comm, T, n, p, out=out, capacity=cap)
    ctx.L.csa_set_pass_timing(ctx.h, 1)
    ctx.reset_counters()
    dist.barrier()
    torch.cuda.synchronize()
    step_ms, launches, peer = [], 0, 0
    with ClockSampler(local) as clocks:
        for _ in range(args.steps):
            _, segs, st = multi.build_sa_multi(ctx, comm, T, n, p, out=out, capacity=cap)
            step_ms.append(_max_over_ranks(st.ms_total, dev))
            launches += st.kernel_launches
            peer += st.peer_bytes
            per_gen = [int(x) for x in st.peer_bytes_per_gen[:st.generations + 1]]
        dist.barrier()
        torch.cuda.synchronize()
    ms = sum(step_ms) / len(step_ms)
    roofline = pass_roofline(ctx, peak, peak_kind, None, None)
    roofline["kernel"] += ", rank 0"
    count = sum(c for _, c in segs)
    total = _sum_over_ranks(count, dev)

    # The whole array, checked in full on rank 0: every rank lays its segments into a zeroed buffer of the full size, the
    # buffers are summed over the ranks, and rank 0 runs the device validator on the sum.
    full = torch.zeros(5 * n + api.SA_PAD_BYTES, dtype=torch.uint8, device=dev)
    at = 0
    for first, c in segs:
        full[5 * first:5 * (first + c)] = out[5 * at:5 * (at + c)]
        at += c
    dist.all_reduce(full, op=dist.ReduceOp.SUM)
    validation = api.validate_sa(ctx, T, n, full) if rank == 0 else None
    del full
    torch.cuda.empty_cache()

    # end to end: pinned host text in, this rank's slice of the 5-byte array out
    e2e = None
    if not args.no_e2e:
        th = torch.empty(n + api.TEXT_PAD, dtype=torch.uint16).pin_memory()
        th.copy_(T.cpu())
        oh = torch.empty(5 * cap + api.SA_PAD_BYTES, dtype=torch.uint8).pin_memory()
        ts = []
        scratch = None
        for it in range(1 + args.steps):
            dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            scratch = multi.upload_text_sharded(th, T, scratch)         # 1/world of the text per rank over PCIe, the rest over NVLink
            _, segs, st = multi.build_sa_multi(ctx, comm, T, n, p, out=out, capacity=cap)
            count = sum(c for _, c in segs)
            oh[:5 * count].copy_(out[:5 * count], non_blocking=True)
            torch.cuda.synchronize()
            dt = _max_over_ranks(time.perf_counter() - t0, dev)
            if it > 0:
                ts.append(dt)
        e_ms = 1e3 * sum(ts) / len(ts)
        e2e = {"value": n / (e_ms * 1e-3), "unit": UNIT, "h2d_bytes_per_step": 2 * n, "d2h_bytes_per_step": 5 * n, "ms_per_step": e_ms, "steps": len(ts),
               "api": "upload_text_sharded (1/N of the pinned host text per rank, all-gather over NVLink) + csa_build_sa_multi + a pinned copy "
                      "of the rank's sa40 slice out"}
        del scratch, th, oh
        torch.cuda.empty_cache()
    # ---- batched queries on the index sharded by suffix-array range (BASELINE config 5 over N GPUs) ---------------------
    query = None
    if args.queries > 0:
        comm0, close0 = multi.make_shm_comm(rank, world, name[0] + "_q", policy=0)     # contiguous blocks: one slice of the array per rank
        sl, segs0, _ = multi.build_sa_multi(ctx, comm0, T, n, p, out=out, capacity=cap)
        close0()
        first0, count0 = (segs0[0][0], sum(c for _, c in segs0)) if segs0 else (0, 0)
        sh = multi.ShardedIndex(ctx, T, sl, n, first0, count0, stride=32)
        q = args.queries
        objs = [None, None]
        if rank == 0:
            tn = T.cpu().view(torch.int16).numpy().view(np.uint16)
            objs = list(make_queries(api, tn, n, q))
        dist.broadcast_object_list(objs, src=0)
        od = torch.from_numpy(objs[0].view(np.int64)).to(dev)
        sd = torch.from_numpy(objs[1].view(np.int16)).to(dev)
        for _ in range(2):
            itv = sh.find(od, sd, q)
            pos, poff, cnt = sh.locate_packed(itv, q, 100)
        del pos, poff, cnt
        dist.barrier(); torch.cuda.synchronize()
        t0 = time.perf_counter()
        itv = sh.find(od, sd, q)
        pos, poff, cnt = sh.locate_packed(itv, q, 100)
        torch.cuda.synchronize()
        dq = _max_over_ranks(time.perf_counter() - t0, dev)
        query = {"value": q / dq, "unit": f"queries/s (count + locate <= 100 into packed positions, suffix array sharded by range over {world} GPUs, text replicated; each shard answers at once the "
                                           f"patterns outside its range, one all-reduce of the intervals and one of the packed positions)",
                 "queries": q, "counts_hash": f"{api.counts_hash(itv.cpu().numpy().view(np.uint64)):016x}", "positions": int(cnt.sum().item())}
    launches_all = _sum_over_ranks(launches, dev)
    peer_all = _sum_over_ranks(peer, dev)
    pg = torch.zeros(49, dtype=torch.float64, device=dev)
    pg[:len(per_gen)] = torch.tensor(per_gen, dtype=torch.float64, device=dev)
    dist.all_reduce(pg)
    per_gen_all = [int(x) for x in pg[:st.generations + 1].cpu()]
    if rank == 0:
        line = {"metric": METRIC, "value": n / (ms * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
                "ms_per_step": ms, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
                "config": workload_config(args, world), "clocks": clocks.summary(), "e2e": e2e, "gpu_launches": int(launches_all),
                "roofline": roofline,
                "nvlink": {"peer_bytes_per_step_all_ranks": peer_all / args.steps, "generations": st.generations,
                           "peer_bytes_per_generation_all_ranks": per_gen_all,
                           "note": "bytes written into other GPUs' memory; [0] = positions and generation-0 keys to the partitions' owners (12 B) and the first "
                                   "ranks to the positions' owners (8 B), [t] = doubling generation t: rank requests and responses (4 B each) and rank updates "
                                   "(8 B); (G-1)/G of the records are remote"},
                "phases_ms_rank0": {"partition": st.ms_partition, "gen0": st.ms_gen0, "doubling": st.ms_doubling, "output": st.ms_output},
                "query": query, "validated": bool(validation["ok"] and total == n), "validation": validation}
        print(json.dumps(line))
    dist.barrier()
    close_comm()
    ctx.close()
    dist.destroy_process_group()


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


def run_c4(args):
    """A scaled-down stand-in for BASELINE config 4: the part-at-a-time build (suffix lists in pinned host memory, 5-byte
    lanes, 4096 partitions) on a corpus of more than 2^32 tokens, so that every position-carrying path runs beyond 32 bits for
    real, on N GPUs of one box (strong scaling: the same corpus at every N). Each rank owns the parts u with u mod N == rank and
    streams their lists over its own PCIe link; ranks cross NVLink between generations. Wall time of the whole build with
    the text resident on the devices, max over ranks; the array is then put together and checked in full on rank 0's device."""
    import torch
    import torch.distributed as dist
    from cascade_b200 import api, multi
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n = args.tokens if args.tokens != C2_TOKENS else 4_500_000_000
    p = 4096
    ps = args.part_suffixes or (1 << 27)
    ctx = api.Context(local)
    T = api.gen_corpus_device(ctx, n, 0, C2_MEAN_DOC)            # every rank makes the same text in its own HBM
    host, times, infos = {}, [], []
    with ClockSampler(local) as clocks:
        for it in range(1 + max(1, min(args.steps, 3))):            # the first build pins the host lists and is not counted
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            segs, info = multi.build_sa_streamed_multi(ctx, T, n, p, part_suffixes=ps, host=host,
                                                       list_budget_bytes=None if args.list_budget_gb < 0 else int(args.list_budget_gb * 1e9))
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            if world > 1:
                dt = _max_over_ranks(dt, dev)
            if it > 0:
                times.append(dt)
                infos.append(info)
    info = infos[-1]
    sec = sum(times) / len(times)
    # the whole array on rank 0's device, checked in full
    full = torch.zeros(5 * n + api.SA_PAD_BYTES, dtype=torch.uint8, device=dev)
    for first, count, lanes in segs:
        full[5 * first:5 * (first + count)].copy_(lanes, non_blocking=True)
    torch.cuda.synchronize()
    if world > 1:
        dist.all_reduce(full)
    v = api.validate_sa(ctx, T, n, full) if rank == 0 else None
    del full
    torch.cuda.empty_cache()
    c_driver = None
    if world == 1 and not args.no_e2e:
        # the same build through the one-call C entry point, host text in (its own pinned rank list is kept by the context)
        th = torch.empty(n + api.TEXT_PAD, dtype=torch.uint16).pin_memory()
        th.copy_(T)
        oh = host["lanes"]                                          # 5 n + 64 bytes, pinned: the output array
        ts = []
        for it in range(2):
            t0 = time.perf_counter()
            _, st = api.build_sa_streamed(ctx, th, n, p, out=oh, part_suffixes=ps)
            ts.append(time.perf_counter() - t0)
        c_driver = {"value": n / ts[-1], "unit": UNIT, "ms_per_step": 1e3 * ts[-1], "api": "csa_build_sa_streamed (pinned host text in, sa40 out in pinned host memory)",
                    "phases_ms": {"partition": st.ms_partition, "gen0": st.ms_gen0, "doubling": st.ms_doubling, "output": st.ms_output}}
    file_tier = None
    if world == 1 and args.scratch:
        # the same again with the lists of the parts beyond --host-list-gb in files below --scratch (page cache included: the
        # files are written and read back within seconds, so this times the file path, not a drive)
        if c_driver is None:
            th = torch.empty(n + api.TEXT_PAD, dtype=torch.uint16).pin_memory()
            th.copy_(T)
            oh = host["lanes"]
        oh.zero_()
        t0 = time.perf_counter()
        _, st = api.build_sa_tiered(ctx, th, n, p, out=oh, part_suffixes=ps, host_list_bytes=int(args.host_list_gb * 1e9), scratch_dir=args.scratch)
        dt = time.perf_counter() - t0
        full = oh[:5 * n + api.SA_PAD_BYTES].to(dev)
        vf = api.validate_sa(ctx, T, n, full)
        del full
        file_tier = {"value": n / dt, "unit": UNIT, "ms_per_step": 1e3 * dt, "api": "csa_build_sa_tiered", "host_list_gb": args.host_list_gb,
                     "host_parts": st.host_parts, "file_parts": st.file_parts, "file_gb_read": st.file_bytes_read / 1e9,
                     "file_gb_written": st.file_bytes_written / 1e9, "validated": bool(vf["ok"]),
                     "phases_ms": {"partition": st.ms_partition, "gen0": st.ms_gen0, "doubling": st.ms_doubling, "output": st.ms_output}}
    own_active = info["active_per_generation"]
    if rank == 0:
        print(json.dumps({"metric": METRIC, "value": n / sec, "unit": UNIT, "n_gpus": world, "steps": len(times), "warmup": 1, "ms_per_step": 1e3 * sec,
                          "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
                          "config": {"workload": "part-at-a-time build with the suffix lists in pinned host memory: a scaled-down stand-in for BASELINE config 4 "
                                                 "(64e9 tokens on 1-8 GPUs under a 512 GB host cap); text and rank store on every GPU (--workload c4-sharded shards them)", "tokens": n, "beyond_2_32_positions": n > (1 << 32),
                                     "partitions_asked": p, "part_suffixes": ps, "mean_doc": C2_MEAN_DOC, "vocab": 50257, "seed": 0, "gpus": world,
                                     "lists_on_device_rank0": info["lists_on_device"], "lists_on_host_rank0": info["lists_on_host"],
                                     "list_budget_gb": "what is free" if args.list_budget_gb < 0 else args.list_budget_gb},
                          "timed": "wall clock of the whole build, text resident on every device: partition ids, lanes to the host, every generation's lists over "
                                   "PCIe both ways, rank exchange over NVLink, final order; max over ranks",
                          "clocks": clocks.summary(), "partitions": info["partitions"], "parts": info["parts"], "generations": info["generations"],
                          "active_per_generation": own_active, "phases_ms_rank0": info["ms"], "gpu_launches": info["launches"],
                          "nvlink_bytes_received_rank0": info["nvlink_bytes_received"],
                          "pcie_bytes_rank0": {"h2d": 5 * info["own_suffixes"] + 9 * info["own_suffixes"] + 9 * sum(own_active) // world,
                                               "d2h": 5 * info["own_suffixes"] + 9 * info["own_suffixes"] + 9 * sum(own_active) // world + 5 * info["own_suffixes"]},
                          "validated": bool(v["ok"]), "validation": v, "one_call_entry_point": c_driver, "lists_in_files": file_tier}))
    if world > 1:
        dist.barrier()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


def run_c4_sharded(args):
    """The part-at-a-time build with nothing replicated (cascade_b200/multi.py: build_sa_sharded): every rank makes and holds its
    own stretch of the corpus only, and the same stretch of the partition ids and the rank store; keys and ranks travel between
    the GPUs. Strong scaling on a corpus beyond 2^32 tokens; wall time of the whole build, max over ranks. Where the whole
    text, the whole array and the checker's workspace fit one device, the array is put together and checked in full on rank 0."""
    import torch
    import torch.distributed as dist
    from cascade_b200 import api, multi
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    n = args.tokens if args.tokens != C2_TOKENS else 4_500_000_000
    p = 4096
    ps = args.part_suffixes or (1 << 27)
    ctx = api.Context(local)
    _, lo, hi = multi.shard_bounds(n, world, rank)
    mine = api.gen_corpus_device_window(ctx, lo, hi - lo, 0, C2_MEAN_DOC)
    host, times, infos = {}, [], []
    with ClockSampler(local) as clocks:
        for it in range(1 + max(1, min(args.steps, 2))):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            segs, info = multi.build_sa_sharded(ctx, mine, n, p, part_suffixes=ps, host=host)
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            if world > 1:
                dt = _max_over_ranks(dt, dev)
            if it > 0:
                times.append(dt)
                infos.append(info)
    info = infos[-1]
    sec = sum(times) / len(times)
    # once more with the parts left in the GPUs' memory (each rank one range of the array), as a sharded index wants them
    resident = None
    if info["lists_on_device"] or world > 1:
        ok = torch.tensor([int(bool(info["lists_on_device"]))], dtype=torch.int64, device=dev)
        if world > 1:
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()):
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            dsegs, dinfo = multi.build_sa_sharded(ctx, mine, n, p, part_suffixes=ps, host=host, output="device")
            torch.cuda.synchronize()
            dt = time.perf_counter() - t0
            if world > 1:
                dt = _max_over_ranks(dt, dev)
            same = all(torch.equal(d[2].cpu(), h_[2]) for d, h_ in zip(dsegs, segs))
            resident = {"ms_per_step": 1e3 * dt, "value": n / dt, "unit": UNIT, "equal_to_the_host_copy_rank0": bool(same), "output_ms_rank0": dinfo["ms"]["output"]}
            del dsegs
    del mine
    torch.cuda.empty_cache()
    v = None
    need = 2 * n + 5 * n + int(ctx.L.csa_validate_workspace_bytes(n)) + (2 << 30)
    free_b, _ = torch.cuda.mem_get_info(dev)
    fits = torch.tensor([int(need < free_b and not args.partial_check)], dtype=torch.int64, device=dev)
    if world > 1:
        dist.all_reduce(fits, op=dist.ReduceOp.MIN)
    if int(fits.item()):
        full = torch.zeros(5 * n + api.SA_PAD_BYTES, dtype=torch.uint8, device=dev)
        for first, count, lanes in segs:
            full[5 * first:5 * (first + count)].copy_(lanes, non_blocking=True)
        torch.cuda.synchronize()
        if world > 1:
            dist.all_reduce(full)
        if rank == 0:
            T = api.gen_corpus_device(ctx, n, 0, C2_MEAN_DOC)
            v = api.validate_sa(ctx, T, n, full)
            del T
        del full
    else:
        # Too large for one device to check in full. Two checks that do not depend on the size: (1) the sums of all entries and of
        # their squares modulo 2^64, added up over the ranks, must be those of 0 .. n-1 (a permutation has them; a lost or doubled
        # position almost surely has not); (2) sampled neighbours SA[i], SA[i+1] from every rank's parts are compared symbol by
        # symbol on rank 0, which makes the whole text again for that.
        mask = (1 << 64) - 1
        s1 = s2 = 0
        pairs = []
        g = torch.Generator(device="cpu").manual_seed(1234 + rank)
        per_seg = max(1, 250_000 // max(1, len(segs)))
        for first, count, lanes in segs:
            step = 1 << 26
            for a in range(0, count, step):
                b = min(count, a + step)
                x = lanes[5 * a:5 * b].to(dev).view(-1, 5).to(torch.int64)
                v = x[:, 0] | (x[:, 1] << 8) | (x[:, 2] << 16) | (x[:, 3] << 24) | (x[:, 4] << 32)
                s1 = (s1 + int(v.sum().item())) & mask
                s2 = (s2 + int((v * v).sum().item())) & mask
                if b - a > 1:
                    at = torch.randint(0, b - a - 1, (max(1, per_seg * (b - a) // count),), generator=g).to(dev)
                    pairs.append(torch.stack([v[at], v[at + 1]], dim=1))
                del x, v
        sums = torch.tensor([s1 - (1 << 64) if s1 >= (1 << 63) else s1, s2 - (1 << 64) if s2 >= (1 << 63) else s2], dtype=torch.int64, device=dev)
        pairs = torch.cat(pairs) if pairs else torch.zeros((0, 2), dtype=torch.int64, device=dev)
        if world > 1:
            dist.all_reduce(sums)                     # 64-bit sums wrap, which is the arithmetic modulo 2^64 that is wanted
            cnts = [torch.zeros(1, dtype=torch.int64, device=dev) for _ in range(world)]
            dist.all_gather(cnts, torch.tensor([pairs.shape[0]], dtype=torch.int64, device=dev))
            most = max(int(c.item()) for c in cnts)
            padded = torch.zeros((most, 2), dtype=torch.int64, device=dev)
            padded[:pairs.shape[0]] = pairs
            every = [torch.empty_like(padded) for _ in range(world)]
            dist.all_gather(every, padded)
            pairs = torch.cat([e[:int(c.item())] for e, c in zip(every, cnts)])
        if rank == 0:
            want1 = (n * (n - 1) // 2) & mask
            want2 = ((n - 1) * n * (2 * n - 1) // 6) & mask
            got1, got2 = int(sums[0].item()) & mask, int(sums[1].item()) & mask
            T = api.gen_corpus_device(ctx, n, 0, C2_MEAN_DOC).view(torch.int16)
            x, y = pairs[:, 0], pairs[:, 1]
            undecided = torch.ones(x.shape[0], dtype=torch.bool, device=dev)
            wrong = torch.zeros_like(undecided)
            for k in range(64):
                # symbols as unsigned 16-bit values; past the end of the text a suffix has ended, which sorts first
                sx = torch.where(x + k < n, T[torch.clamp(x + k, max=n)].to(torch.int32) & 0xFFFF, torch.full_like(x, -1, dtype=torch.int32))
                sy = torch.where(y + k < n, T[torch.clamp(y + k, max=n)].to(torch.int32) & 0xFFFF, torch.full_like(y, -1, dtype=torch.int32))
                wrong |= undecided & (sx > sy)
                undecided &= sx == sy
            v = {"kind": "sums of entries and of squares mod 2^64 over all ranks + sampled neighbours compared to a depth of 64 symbols",
                 "sum_ok": got1 == want1, "sum_of_squares_ok": got2 == want2, "neighbours_sampled": int(x.shape[0]),
                 "neighbours_out_of_order": int(wrong.sum().item()), "neighbours_equal_to_depth_64": int(undecided.sum().item()),
                 "ok": got1 == want1 and got2 == want2 and int(wrong.sum().item()) == 0}
            del T
    sent_all = info["nvlink_bytes_sent"]
    if world > 1:
        t = torch.tensor([sent_all], dtype=torch.int64, device=dev)
        dist.all_reduce(t)
        sent_all = int(t.item())
    if rank == 0:
        print(json.dumps({"metric": METRIC, "value": n / sec, "unit": UNIT, "n_gpus": world, "steps": len(times), "warmup": 1, "ms_per_step": 1e3 * sec,
                          "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "u64", "data": "synthetic",
                          "config": {"workload": "part-at-a-time build with text, partition ids and rank store sharded by position (nothing replicated): "
                                                 "a scaled-down stand-in for BASELINE config 4", "tokens": n, "beyond_2_32_positions": n > (1 << 32),
                                     "partitions_asked": p, "part_suffixes": ps, "mean_doc": C2_MEAN_DOC, "vocab": 50257, "seed": 0, "gpus": world,
                                     "device_bytes_per_position_per_gpu": 8.0 / world, "lists_on_device": info["lists_on_device"]},
                          "timed": "wall clock of the whole build from each rank's stretch of the text in its HBM to the parts in final order in pinned host "
                                   "memory; max over ranks",
                          "clocks": clocks.summary(), "partitions": info["partitions"], "parts": info["parts"], "generations": info["generations"],
                          "active_per_generation": info["active_per_generation"], "phases_ms_rank0": info["ms"], "gpu_launches": info["launches"],
                          "nvlink_bytes_sent_all_ranks": sent_all, "array_left_on_the_devices": resident,
                          "validated": bool(v["ok"]) if "out_of_order" in v else "in part: too large for one device to check in full", "validation": v}))
    if world > 1:
        dist.barrier()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


def run_repeat(args):
    """BASELINE config 3 alone (it is also a key of the default line)."""
    from cascade_b200 import api
    if args.tokens != C2_TOKENS:
        args.config3_tokens = args.tokens
    ctx = api.Context(0)
    r = run_config3(ctx, args)
    r.update({"metric": METRIC, "n_gpus": 1})
    print(json.dumps(r))
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
    ap.add_argument("--ref-sample", type=int, default=1 << 26, help="tokens that one step of the CPU reference arm sorts")
    ap.add_argument("--config3-tokens", type=int, default=C3_TOKENS, help="size of the repetitive corpus reported under `config3` (0 = skip)")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    ap.add_argument("--no-sort-baseline", action="store_true")
    ap.add_argument("--workload", default="zipf", choices=["zipf", "repeat", "c4", "c4-sharded"],
                    help="zipf: BASELINE config 2; repeat: config 3 alone (1e9 tokens of near-duplicate documents, build only); "
                         "c4: the part-at-a-time build on more than 2^32 tokens (one-GPU stand-in for config 4)")
    ap.add_argument("--part-suffixes", type=int, default=0, help="c4: most suffixes of a part (0 = the library's default, 2^27)")
    ap.add_argument("--list-budget-gb", type=float, default=-1.0,
                    help="c4: device memory (GB) that may hold parts' suffix lists; 0 keeps every list in pinned host memory, -1 (default) takes what is free")
    ap.add_argument("--scratch", default=None, help="c4: a directory; the build is then also run with lists in files there (csa_build_sa_tiered)")
    ap.add_argument("--host-list-gb", type=float, default=0.0, help="c4 with --scratch: host memory for lists, 9 bytes a suffix; parts beyond it use files")
    ap.add_argument("--partial-check", action="store_true", help="c4-sharded: use the checks for arrays too large for one device even where the full check fits")
    ap.add_argument("--micro", default=None, choices=["sort"], help="time one kernel family alone instead of the build")
    ap.add_argument("--records", type=int, default=31_250_000)
    ap.add_argument("--bits", type=int, default=64)
    ap.add_argument("--variant", type=int, default=-1, help="shape of the digit-pass kernel (test hook), -1 = default")
    args = ap.parse_args()
    if args.impl == "reference":
        return run_reference(args)
    if args.micro == "sort":
        return run_micro_sort(args)
    if args.workload == "c4":
        return run_c4(args)
    if args.workload == "c4-sharded":
        return run_c4_sharded(args)
    if args.workload == "repeat":
        return run_repeat(args)
    run_ours(args)


if __name__ == "__main__":
    main()
