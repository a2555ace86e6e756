"""Python face of the C ABI (include/cascade_b200.h): thin wrappers that pass torch / numpy buffers as plain
pointers. torch is used for device memory only; every computation happens in the library's own kernels.
"""
import ctypes
import os

import numpy as np
import torch

from ._lib import BuildStats, Index, c_int, c_u64, c_vp, lib

TEXT_PAD = 64
SA_PAD_BYTES = 128
K = 8

_ERR = {1: "invalid argument", 2: "CUDA error", 3: "out of memory", 4: "size limit", 5: "device status", 6: "exchange failed"}


class CascadeError(RuntimeError):
    def __init__(self, code, text):
        super().__init__(f"cascade_b200: {_ERR.get(code, code)} ({code}): {text}")
        self.code = code


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, torch.Tensor):
        return x.data_ptr()
    if isinstance(x, np.ndarray):
        return x.ctypes.data
    return x


class Context:
    """One library context (stream, status word, scratch) on a device."""

    def __init__(self, device=0):
        self.L = lib()
        self.device = device
        h = c_vp()
        rc = self.L.csa_ctx_create(device, ctypes.byref(h))
        if rc != 0:
            raise CascadeError(rc, "csa_ctx_create")
        self.h = h

    def close(self):
        if self.h:
            self.L.csa_ctx_destroy(self.h)
            self.h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def check(self, rc):
        if rc != 0:
            raise CascadeError(rc, self.L.csa_last_error(self.h).decode())

    def sync(self):
        st = c_u64(0)
        rc = self.L.csa_sync(self.h, ctypes.byref(st))
        if rc != 0:
            raise CascadeError(rc, f"status bits {st.value}: " + self.L.csa_last_error(self.h).decode())

    def stream(self):
        """The context's cudaStream_t as an integer (for torch.cuda.ExternalStream)."""
        return int(self.L.csa_ctx_stream(self.h))

    @property
    def launches(self):
        return int(self.L.csa_kernel_launches(self.h))

    def reset_counters(self):
        self.L.csa_reset_counters(self.h)


# ---- synthetic workloads -----------------------------------------------------------------------------------------

def zipf_cdf(vocab=50257, s=1.1):
    """64-bit inverse-CDF thresholds of Zipf(s) over ranks 1..vocab: token r is drawn when u <= cdf[r]."""
    w = np.arange(1, vocab + 1, dtype=np.float64) ** (-s)
    c = np.cumsum(w)
    c /= c[-1]
    t = np.minimum(np.floor(c * 18446744073709551616.0), 18446744073709551615.0)
    out = np.array([int(x) if x < 18446744073709551615.0 else 0xFFFFFFFFFFFFFFFF for x in t], dtype=np.uint64)
    out[-1] = np.uint64(0xFFFFFFFFFFFFFFFF)
    return out


def gen_corpus_host(n, seed=0, mean_doc=512, cdf=None):
    """The seeded Zipf corpus on the host: n symbols followed by TEXT_PAD zeros (numpy uint16)."""
    cdf = zipf_cdf() if cdf is None else cdf
    T = np.zeros(n + TEXT_PAD, dtype=np.uint16)
    rc = lib().csa_gen_corpus_host(T.ctypes.data, 0, n, seed, mean_doc, cdf.ctypes.data, len(cdf))
    if rc != 0:
        raise CascadeError(rc, "csa_gen_corpus_host")
    return T


def gen_corpus_device(ctx, n, seed=0, mean_doc=512, cdf=None):
    """The same corpus made on the device: a torch uint16 tensor of n + TEXT_PAD symbols."""
    cdf = zipf_cdf() if cdf is None else cdf
    dev = torch.device("cuda", ctx.device)
    cdf_t = torch.from_numpy(cdf.view(np.int64)).to(dev)
    T = torch.zeros(n + TEXT_PAD, dtype=torch.uint16, device=dev)
    torch.cuda.synchronize(dev)
    ctx.check(ctx.L.csa_gen_corpus_dev(ctx.h, T.data_ptr(), n, seed, mean_doc, cdf_t.data_ptr(), len(cdf)))
    ctx.sync()
    return T


def gen_corpus_device_window(ctx, first, count, seed=0, mean_doc=512, cdf=None):
    """The symbols first .. first + count - 1 of the same corpus, followed by TEXT_PAD zeros: one GPU's stretch of a sharded text."""
    cdf = zipf_cdf() if cdf is None else cdf
    dev = torch.device("cuda", ctx.device)
    cdf_t = torch.from_numpy(cdf.view(np.int64)).to(dev)
    T = torch.zeros(count + TEXT_PAD, dtype=torch.uint16, device=dev)
    torch.cuda.synchronize(dev)
    ctx.check(ctx.L.csa_gen_corpus_dev_window(ctx.h, T.data_ptr(), first, count, seed, mean_doc, cdf_t.data_ptr(), len(cdf)))
    ctx.sync()
    return T


def gen_repeat_corpus_host(n, seed=0, base_docs=4096, mean_doc=2048, mutate=0.001, vocab=50257, cdf=None):
    """The repetitive corpus: `base_docs` Zipf documents, then copies of random base documents with a fraction
    `mutate` of their tokens replaced by uniform ids, each preceded by 0xFFFF, cut at n symbols (numpy, host)."""
    cdf = zipf_cdf(vocab) if cdf is None else cdf
    rng = np.random.Generator(np.random.PCG64(seed))
    lens = 1 + np.floor(np.log1p(-rng.random(base_docs)) / np.log1p(-1.0 / mean_doc)).astype(np.int64)
    starts = np.concatenate([[0], np.cumsum(lens)])
    u = rng.integers(0, 2**63, size=int(starts[-1]), dtype=np.int64).astype(np.uint64) * np.uint64(2)
    base = np.searchsorted(cdf, u, side="left").astype(np.uint16)
    out = np.zeros(n + TEXT_PAD, dtype=np.uint16)
    at = 0
    d = 0
    while at < n:
        b = d if d < base_docs else int(rng.integers(0, base_docs))
        doc = base[starts[b]:starts[b + 1]].copy()
        if d >= base_docs and mutate > 0:
            m = rng.random(len(doc)) < mutate
            doc[m] = rng.integers(0, vocab, size=int(m.sum()), dtype=np.int64).astype(np.uint16)
        out[at] = 0xFFFF
        at += 1
        take = min(len(doc), n - at)
        if take > 0:
            out[at:at + take] = doc[:take]
            at += take
        d += 1
    out[n:] = 0
    return out


def gen_queries(kind, text_host, n, q, lens=tuple(range(1, 17)), vocab=50257, seed=1):
    """A query batch as the reference's `query gen` makes it: kind 'substring' or 'random'. Returns (off, sym)."""
    lens_a = np.asarray(lens, dtype=np.uint32)
    cap = int(q) * int(lens_a.max()) + 1
    off = np.zeros(q + 1, dtype=np.uint64)
    sym = np.zeros(cap, dtype=np.uint16)
    k = {"substring": 0, "random": 1}[kind]
    rc = lib().csa_gen_queries_host(k, _ptr(text_host) if k == 0 else None, n, q, lens_a.ctypes.data, len(lens_a), vocab, seed,
                                    off.ctypes.data, sym.ctypes.data, cap)
    if rc != 0:
        raise CascadeError(rc, "csa_gen_queries_host")
    return off, sym[:int(off[-1])].copy()


def counts_hash(itv):
    itv = np.ascontiguousarray(itv, dtype=np.uint64)
    return int(lib().csa_counts_hash(itv.ctypes.data, itv.size // 2))


# ---- sort ----------------------------------------------------------------------------------------------------------

def sort_pairs(ctx, keys, vals, begin_bit=0, end_bit=64):
    """Sorts (int64-as-u64 keys, int32/int64 vals) device tensors; returns the sorted (keys, vals) tensors."""
    n = keys.numel()
    ka, va = torch.empty_like(keys), torch.empty_like(vals)
    wsb = ctx.L.csa_sort_workspace_bytes(n)
    ws = torch.empty(wsb, dtype=torch.uint8, device=keys.device)
    torch.cuda.synchronize(keys.device)
    in_alt = c_int(0)
    ctx.check(ctx.L.csa_sort_pairs(ctx.h, keys.data_ptr(), ka.data_ptr(), vals.data_ptr(), va.data_ptr(), vals.element_size(), n,
                                   begin_bit, end_bit, ws.data_ptr(), wsb, ctypes.byref(in_alt)))
    ctx.sync()
    return (ka, va) if in_alt.value else (keys, vals)


# ---- build ---------------------------------------------------------------------------------------------------------

def stats_dict(st):
    d = {k: getattr(st, k) for k, _ in st._fields_ if k != "active_per_gen"}
    d["active_per_gen"] = [int(x) for x in st.active_per_gen[:max(1, st.generations)]]
    return d


def build_sa(ctx, text_dev, n, p=1, seed=0, out=None):
    """Suffix array of text_dev[0, n) (a device uint16 tensor with TEXT_PAD zeros after n). Returns (sa40, stats):
    sa40 is a device uint8 tensor of 5 n + SA_PAD_BYTES bytes."""
    dev = text_dev.device
    if out is None:
        out = torch.zeros(5 * n + SA_PAD_BYTES, dtype=torch.uint8, device=dev)
    st = BuildStats()
    torch.cuda.synchronize(dev)
    ctx.check(ctx.L.csa_build_sa(ctx.h, text_dev.data_ptr(), n, p, seed, out.data_ptr(), ctypes.byref(st)))
    return out, st


def build_sa_host(ctx, text_host, n, p=1, seed=0, out=None):
    """The same from host memory (numpy array or pinned torch tensor): copies in, builds, copies the 5 n bytes out."""
    if out is None:
        out = np.zeros(5 * n + SA_PAD_BYTES, dtype=np.uint8)
    st = BuildStats()
    ctx.check(ctx.L.csa_build_sa_host(ctx.h, _ptr(text_host), n, p, seed, _ptr(out), ctypes.byref(st)))
    return out, st


def build_sa_streamed(ctx, text_host, n, p=64, seed=0, out=None, part_suffixes=0):
    """The build driven part by part (csa_build_sa_streamed): text and output in host memory (numpy arrays or pinned torch
    tensors), suffix lists streamed through the device, positions up to 2^40. Returns (sa40, stats)."""
    if out is None:
        out = np.zeros(5 * n + SA_PAD_BYTES, dtype=np.uint8)
    st = BuildStats()
    ctx.check(ctx.L.csa_build_sa_streamed(ctx.h, _ptr(text_host), n, p, seed, _ptr(out), part_suffixes, ctypes.byref(st)))
    return out, st


def build_sa_tiered(ctx, text_host, n, p=64, seed=0, out=None, part_suffixes=0, host_list_bytes=None, scratch_dir=None, output_path=None):
    """The part-by-part build with the lists in tiers (csa_build_sa_tiered): lists of the first parts in host memory up to
    host_list_bytes (None: no bound), the others in files below scratch_dir; output_path names a file that receives the
    array, and with out=False no array is kept in memory at all. Returns (sa40 or None, stats)."""
    from ._lib import TierOptions
    if out is None:
        out = np.zeros(5 * n + SA_PAD_BYTES, dtype=np.uint8)
    opts = TierOptions(part_suffixes, 2**64 - 1 if host_list_bytes is None else host_list_bytes,
                       None if scratch_dir is None else os.fsencode(scratch_dir), None if output_path is None else os.fsencode(output_path))
    st = BuildStats()
    ctx.check(ctx.L.csa_build_sa_tiered(ctx.h, _ptr(text_host), n, p, seed, None if out is False else _ptr(out), ctypes.byref(opts), ctypes.byref(st)))
    return (None if out is False else out), st


def validate_sa(ctx, text_dev, n, sa40_dev):
    """Exact check of a whole suffix array on the device (csa_validate_sa). Returns a dict with the counts of entries out of
    range, duplicate entries and neighbouring pairs out of order, the first bad rank, and `ok`."""
    wsb = ctx.L.csa_validate_workspace_bytes(n)
    ws = torch.empty(wsb, dtype=torch.uint8, device=text_dev.device)
    res = torch.zeros(4, dtype=torch.int64, device=text_dev.device)
    torch.cuda.synchronize(text_dev.device)
    ctx.check(ctx.L.csa_validate_sa(ctx.h, text_dev.data_ptr(), n, sa40_dev.data_ptr(), ws.data_ptr(), wsb, res.data_ptr()))
    ctx.sync()
    r = res.cpu().numpy().view(np.uint64)
    del ws
    return {"out_of_range": int(r[0]), "duplicates": int(r[1]), "out_of_order": int(r[2]),
            "first_bad_rank": None if int(r[3]) == 2**64 - 1 else int(r[3]), "ok": int(r[0]) == 0 and int(r[1]) == 0 and int(r[2]) == 0}


# ---- queries -------------------------------------------------------------------------------------------------------

class SuffixIndex:
    """Text, suffix array and sample table of one index on a device (the reference's Suffix_Index + Sample_Table)."""

    def __init__(self, ctx, text_dev, sa40_dev, n, stride=32, table=None, sa_first=0, sa_entries=None):
        """sa40_dev may also be a pinned host tensor: the device then reads the suffix array over PCIe. With sa_entries
        given, sa40_dev holds only the slice [sa_first, sa_first + sa_entries) of the suffix array (one shard of a sharded
        index): find() then returns per-slice counts that add up over the shards, see ShardedIndex in multi.py."""
        self.ctx, self.text, self.sa40, self.n, self.stride = ctx, text_dev, sa40_dev, n, stride
        self.sa_first, self.sa_entries = sa_first, (n if sa_entries is None else sa_entries)
        entries = max(1, (self.sa_entries + stride - 1) // stride)
        if table is not None:
            self.table = table
        else:
            self.table = torch.zeros(2 * entries, dtype=torch.int64, device=text_dev.device)
            torch.cuda.synchronize(text_dev.device)
            ctx.check(ctx.L.csa_table_build_slice(ctx.h, text_dev.data_ptr(), n, sa40_dev.data_ptr(), self.sa_entries, stride, self.table.data_ptr()))
            ctx.sync()
        self.c = Index(text_dev.data_ptr(), sa40_dev.data_ptr(), self.table.data_ptr(), n, stride, self.sa_entries, sa_first)

    def locate_window(self, itv_global_dev, q, max_pos, rows):
        """Adds this slice's share of the positions of global intervals to rows (a zero-initialised q x max_pos int64 tensor)."""
        torch.cuda.synchronize(self.text.device)
        self.ctx.check(self.ctx.L.csa_locate_window(self.ctx.h, ctypes.byref(self.c), itv_global_dev.data_ptr(), q, max_pos, rows.data_ptr()))
        self.ctx.sync()
        return rows

    def find(self, off_dev, sym_dev, q):
        itv = torch.empty(2 * q, dtype=torch.int64, device=self.text.device)     # every interval is written
        torch.cuda.synchronize(self.text.device)
        self.ctx.check(self.ctx.L.csa_find(self.ctx.h, ctypes.byref(self.c), off_dev.data_ptr(), sym_dev.data_ptr(), q, itv.data_ptr()))
        self.ctx.sync()
        return itv

    def locate(self, itv_dev, q, max_pos=100):
        """Rows of up to max_pos positions per query, in rank order, and how many each row holds; a row's entries beyond its
        count are unspecified (the buffer is not cleared: clearing 800 B per query would cost as much as the lookup)."""
        pos = torch.empty(q * max_pos, dtype=torch.int64, device=self.text.device)
        cnt = torch.empty(q, dtype=torch.int32, device=self.text.device)
        torch.cuda.synchronize(self.text.device)
        self.ctx.check(self.ctx.L.csa_locate(self.ctx.h, ctypes.byref(self.c), itv_dev.data_ptr(), q, max_pos, pos.data_ptr(), cnt.data_ptr()))
        self.ctx.sync()
        return pos.view(q, max_pos), cnt

    def certify(self, off_dev, sym_dev, q, itv_dev):
        res = torch.zeros(2, dtype=torch.int64, device=self.text.device)
        torch.cuda.synchronize(self.text.device)
        self.ctx.check(self.ctx.L.csa_certify(self.ctx.h, ctypes.byref(self.c), off_dev.data_ptr(), sym_dev.data_ptr(), q, itv_dev.data_ptr(),
                                              res.data_ptr()))
        self.ctx.sync()
        r = res.cpu().numpy().view(np.uint64)
        return int(r[0]), int(r[1])

    def query_host(self, off, sym, max_pos=100, bufs=None):
        """Count + locate from host arrays. Returns (itv, cnt, pos_off, pos) numpy arrays; `bufs` may carry
        preallocated (pinned) host buffers {itv, cnt, pos_off, pos}."""
        q = len(off) - 1
        b = bufs or {}
        itv = b.get("itv") if b.get("itv") is not None else np.zeros(2 * q, dtype=np.uint64)
        cnt = b.get("cnt") if b.get("cnt") is not None else np.zeros(q, dtype=np.uint32)
        poff = b.get("pos_off") if b.get("pos_off") is not None else np.zeros(q + 1, dtype=np.uint64)
        pos = b.get("pos") if b.get("pos") is not None else np.zeros(max(1, q * max_pos), dtype=np.uint64)
        cap = pos.numel() if isinstance(pos, torch.Tensor) else pos.size
        total = c_u64(0)
        self.ctx.check(self.ctx.L.csa_query_host(self.ctx.h, ctypes.byref(self.c), _ptr(off), _ptr(sym), q, max_pos, _ptr(itv), _ptr(cnt),
                                                 _ptr(poff), _ptr(pos), cap, ctypes.byref(total)))
        return itv, cnt, poff, pos, int(total.value)
