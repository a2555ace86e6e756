import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

ORACLE_DIR = os.path.join(ROOT, "oracle")
ORACLE_LIB = os.path.join(ORACLE_DIR, "liboracle.so")
REF_LIB = os.path.join(ORACLE_DIR, "_ref", "libcascade_ref.so")
GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


def pytest_collection_modifyitems(config, items):
    # Files run in name order; the file whose name starts with test_zz is collected last by that order.
    items.sort(key=lambda it: (os.path.basename(str(it.fspath)).startswith("test_zz"),))


def _build_oracle():
    src = os.path.join(ORACLE_DIR, "cascade_oracle.c")
    if not os.path.exists(ORACLE_LIB) or os.path.getmtime(ORACLE_LIB) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", ORACLE_DIR, "liboracle.so"], stdout=subprocess.DEVNULL)


class Oracle:
    """ctypes face of the C restatement (test infrastructure only)."""

    def __init__(self, path, prefix):
        self.L = ctypes.CDLL(path)
        self.p = prefix
        self.is_ref = prefix == "ref_"

    @staticmethod
    def _pad_text(T):
        T = np.ascontiguousarray(T, dtype=np.uint16)
        return np.concatenate([T, np.zeros(64, np.uint16)])

    def build_sa40(self, T, threads=0):
        n = len(T)
        Tp = self._pad_text(T)
        out = np.zeros(5 * n + 128, np.uint8)
        if self.is_ref:
            self.L.ref_build_sa40(Tp.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(n), out.ctypes.data_as(ctypes.c_void_p))
        else:
            rc = self.L.orc_build_sa40(Tp.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(n), out.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(threads))
            assert rc == 0
        return out

    def is_correct(self, T, sa40):
        n = len(T)
        Tp = self._pad_text(T)
        f = self.L.ref_is_correct_sa40 if self.is_ref else self.L.orc_is_correct_sa40
        f.restype = ctypes.c_int
        return f(Tp.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(n), np.ascontiguousarray(sa40).ctypes.data_as(ctypes.c_void_p)) == 1

    def find_one(self, T, sa40, P):
        n = len(T)
        Tp = self._pad_text(T)
        P = np.ascontiguousarray(P, dtype=np.uint16)
        lo, hi = ctypes.c_uint64(0), ctypes.c_uint64(0)
        f = self.L.ref_find_one if self.is_ref else self.L.orc_find_one
        f(Tp.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(n), np.ascontiguousarray(sa40).ctypes.data_as(ctypes.c_void_p),
          P.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(len(P)), ctypes.byref(lo), ctypes.byref(hi))
        return lo.value, hi.value

    def brute_find(self, T, P):
        n = len(T)
        Tp = self._pad_text(T)
        P = np.ascontiguousarray(P, dtype=np.uint16)
        lo, hi = ctypes.c_uint64(0), ctypes.c_uint64(0)
        f = self.L.ref_brute_find if self.is_ref else self.L.orc_brute_find
        f(Tp.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(n), P.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(len(P)),
          ctypes.byref(lo), ctypes.byref(hi))
        return lo.value, hi.value

    def certify(self, T, sa40, P, lo, hi):
        n = len(T)
        Tp = self._pad_text(T)
        P = np.ascontiguousarray(P, dtype=np.uint16)
        f = self.L.ref_certify if self.is_ref else self.L.orc_certify
        f.restype = ctypes.c_int
        return f(Tp.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(n), np.ascontiguousarray(sa40).ctypes.data_as(ctypes.c_void_p),
                 P.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(len(P)), ctypes.c_uint64(lo), ctypes.c_uint64(hi)) == 1

    def find_batch(self, T, sa40, off, sym, threads=0):
        """Intervals of a batch: the oracle's loop over find_one, or the reference's host_search::find."""
        n = len(T)
        Tp = self._pad_text(T)
        q = len(off) - 1
        off = np.ascontiguousarray(off, dtype=np.uint64)
        sym = np.ascontiguousarray(np.concatenate([sym, np.zeros(1, np.uint16)]), dtype=np.uint16)
        out = np.zeros(2 * q, np.uint64)
        sa = np.ascontiguousarray(sa40)
        if self.is_ref:
            self.L.ref_host_search_find(Tp.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(n), sa.ctypes.data_as(ctypes.c_void_p),
                                        off.ctypes.data_as(ctypes.c_void_p), sym.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(q),
                                        out.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint(threads), ctypes.c_uint(32))
        else:
            self.L.orc_find_batch(Tp.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(n), sa.ctypes.data_as(ctypes.c_void_p),
                                  off.ctypes.data_as(ctypes.c_void_p), sym.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(q),
                                  out.ctypes.data_as(ctypes.c_void_p), ctypes.c_int(threads))
        return out

    def locate_batch(self, sa40, itv, max_pos):
        assert not self.is_ref
        q = len(itv) // 2
        itv = np.ascontiguousarray(itv, dtype=np.uint64)
        pos = np.zeros(q * max_pos, np.uint64)
        cnt = np.zeros(q, np.uint32)
        self.L.orc_locate_batch(np.ascontiguousarray(sa40).ctypes.data_as(ctypes.c_void_p), itv.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(q),
                                ctypes.c_uint32(max_pos), pos.ctypes.data_as(ctypes.c_void_p), cnt.ctypes.data_as(ctypes.c_void_p))
        return pos.reshape(q, max_pos), cnt

    def counts_hash(self, itv):
        itv = np.ascontiguousarray(itv, dtype=np.uint64)
        f = self.L.ref_counts_hash if self.is_ref else self.L.orc_counts_hash
        f.restype = ctypes.c_uint64
        return f(itv.ctypes.data_as(ctypes.c_void_p), ctypes.c_uint64(len(itv) // 2))


@pytest.fixture(scope="session")
def oracle():
    _build_oracle()
    return Oracle(ORACLE_LIB, "orc_")


@pytest.fixture(scope="session")
def reference():
    """The reference's own CPU code, where its compiled library is present; else the test is skipped."""
    if not os.path.exists(REF_LIB):
        pytest.skip("oracle/_ref/libcascade_ref.so is not built here")
    return Oracle(REF_LIB, "ref_")


def sa40_to_u64(sa40, n):
    b = np.ascontiguousarray(sa40[:5 * n]).reshape(n, 5).astype(np.uint64)
    return b[:, 0] | (b[:, 1] << np.uint64(8)) | (b[:, 2] << np.uint64(16)) | (b[:, 3] << np.uint64(24)) | (b[:, 4] << np.uint64(32))


def fixture_texts():
    """Small texts with the shapes the reference's own tests use (src/test_query.cu:317-367, dataset/make-corner-case.py):
    alphabets of 2..65536 symbols with separators, periodic, Fibonacci, all-zero, zero-tailed."""
    rng = np.random.default_rng(3)
    out = {}
    for n in (1, 2, 3, 15, 16, 17, 1000, 20000):
        for sigma in (2, 3, 4, 16, 256, 65536):
            alpha = np.arange(sigma, dtype=np.int64) if sigma == 65536 else (np.arange(sigma, dtype=np.int64) * 65535) // max(1, sigma - 1)
            T = alpha[rng.integers(0, sigma, n)]
            T[rng.integers(0, 50, n) == 0] = 0xFFFF
            out[f"rand_n{n}_s{sigma}"] = T.astype(np.uint16)
    out["periodic_ab"] = np.array([7 if i % 2 else 3 for i in range(3000)], np.uint16)
    fib, prev = [1], [0]
    while len(fib) < 2500:
        fib, prev = fib + prev, fib
    out["fibonacci"] = np.array(fib, np.uint16)
    out["all_zero_4"] = np.zeros(4, np.uint16)
    out["all_zero_1000"] = np.zeros(1000, np.uint16)
    out["all_max_100"] = np.full(100, 0xFFFF, np.uint16)
    c = rng.integers(1, 4, 5000).astype(np.uint16)      # the corner-case corpus: tiny alphabet 1..3 plus 16 trailing zeros
    out["corner_case"] = np.concatenate([c, np.zeros(16, np.uint16)])
    z = rng.integers(0, 2, 4000).astype(np.uint16)      # many zero runs, zero tail
    z[-9:] = 0
    out["binary_zero_tail"] = z
    return out


def fixture_queries(T, rng, count):
    """Query shapes of the reference's fixture (src/test_query.cu:221-270): substrings (maybe past the end), random,
    mutated substrings, zero-tails; lengths from its list."""
    lens = [0, 1, 2, 3, 4, 5, 7, 8, 9, 15, 16, 17, 31, 32, 33, 64, 100]
    n = len(T)
    alpha = np.unique(T)
    qs = []
    for k in range(count):
        m = lens[int(rng.integers(0, len(lens)))]
        pos = int(rng.integers(0, n))
        sub = [int(T[pos + i]) if pos + i < n else int(alpha[rng.integers(0, len(alpha))]) for i in range(m)]
        kind = k % 5
        if kind in (0, 1):
            P = sub
        elif kind == 2:
            P = [int(alpha[rng.integers(0, len(alpha))]) for _ in range(m)]
        elif kind == 3:
            P = sub
            if m:
                P[int(rng.integers(0, m))] = int(alpha[rng.integers(0, len(alpha))])
        else:
            tail = min(n, 1 + int(rng.integers(0, 9)))
            P = [int(x) for x in T[n - tail:]] + [0] * (1 + int(rng.integers(0, 9)))
        qs.append(np.array(P, np.uint16))
    off = np.zeros(len(qs) + 1, np.uint64)
    off[1:] = np.cumsum([len(x) for x in qs])
    sym = np.concatenate(qs) if qs and off[-1] > 0 else np.zeros(0, np.uint16)
    return off, sym.astype(np.uint16), qs
