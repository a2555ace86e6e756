"""The C-ABI library loads and exports every entry point that include/cascade_b200.h declares. CPU only: no
compute call is made."""
import ctypes
import os
import re

import numpy as np

from conftest import ROOT


def _declared():
    src = open(os.path.join(ROOT, "include", "cascade_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(csa_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_are_exported():
    from cascade_b200 import _lib
    L = ctypes.CDLL(_lib.LIB_PATH)
    names = _declared()
    assert len(names) >= 25
    for n in names:
        assert hasattr(L, n), f"{n} is declared in the header but not exported"
    assert set(_lib.exported_names()) == set(names)


def test_loader_sets_signatures_and_version():
    from cascade_b200._lib import lib
    assert b"sm_100a" in lib().csa_version()


def test_host_generators_are_deterministic(oracle):
    from cascade_b200 import api
    cdf = api.zipf_cdf()
    assert cdf.dtype == np.uint64 and np.all(np.diff(cdf.astype(np.float64)) >= 0) and cdf[-1] == np.uint64(2**64 - 1)
    a = api.gen_corpus_host(200000, seed=0, mean_doc=512, cdf=cdf)
    b = api.gen_corpus_host(200000, seed=0, mean_doc=512, cdf=cdf)
    assert np.array_equal(a, b) and a[0] == 0xFFFF and np.all(a[200000:] == 0)
    seps = np.flatnonzero(a[:200000] == 0xFFFF)
    assert np.all(np.diff(seps) >= 2)                       # documents hold at least one token
    assert 300 < 200000 / len(seps) < 800                   # mean document length near 512
    tok = a[:200000][a[:200000] != 0xFFFF]
    assert tok.max() < 50257 and 0.10 < np.mean(tok == 0) < 0.18   # Zipf(1.1): the top token has about 14 % of the mass
    c = api.gen_corpus_host(1000, seed=1, mean_doc=512, cdf=cdf)
    assert not np.array_equal(a[:1000], c[:1000])

    off, sym = api.gen_queries("substring", a, 200000, 500, seed=1)
    off2, sym2 = api.gen_queries("substring", a, 200000, 500, seed=1)
    assert np.array_equal(off, off2) and np.array_equal(sym, sym2)
    lens = np.diff(off.astype(np.int64))
    assert lens.min() >= 1 and lens.max() <= 16
    offr, symr = api.gen_queries("random", None, 0, 500, seed=2)
    assert symr.max() < 50257
    itv = np.arange(40, dtype=np.uint64) * np.uint64(3)
    assert api.counts_hash(itv) == oracle.counts_hash(itv)


def test_select_pivots_host():
    from cascade_b200._lib import lib
    rng = np.random.default_rng(0)
    s = rng.integers(0, 50, size=(1000, 2)).astype(np.uint64)
    piv = np.zeros(2 * 15, np.uint64)
    p_out = ctypes.c_uint32(0)
    assert lib().csa_select_pivots(s.ctypes.data, 1000, 16, piv.ctypes.data, ctypes.byref(p_out)) == 0
    k = p_out.value - 1
    pairs = [tuple(piv[2 * i:2 * i + 2]) for i in range(k)]
    assert 1 <= p_out.value <= 16 and pairs == sorted(set(pairs))
    # all-equal samples cannot be split
    s[:] = 7
    assert lib().csa_select_pivots(s.ctypes.data, 1000, 16, piv.ctypes.data, ctypes.byref(p_out)) == 0 and p_out.value == 2
