"""The C restatement (oracle/) against the golden vectors made by the reference's own CPU code, and against that code
itself where its compiled library is present. CPU only."""
import json
import os

import numpy as np
import pytest

import conftest
from conftest import GOLDEN, sa40_to_u64


def _known():
    with open(os.path.join(GOLDEN, "known_answers.json")) as f:
        return json.load(f)


def test_known_answer_table(oracle):
    for c in _known():
        T, P = np.array(c["text"], np.uint16), np.array(c["pattern"], np.uint16)
        sa = oracle.build_sa40(T)
        assert [int(x) for x in sa40_to_u64(sa, len(T))] == c["sa"]
        lo, hi = oracle.find_one(T, sa, P)
        assert (lo, hi) == (c["lo"], c["hi"]) and hi - lo == c["count"]
        assert oracle.brute_find(T, P) == (lo, hi)
        assert oracle.certify(T, sa, P, lo, hi)
        if len(T) > 1:
            assert not oracle.certify(T, sa, P, lo, hi + 1) or hi == len(T)


def test_sa_fixtures(oracle):
    g = np.load(os.path.join(GOLDEN, "sa_fixtures.npz"))
    names = [k[2:] for k in g.files if k.startswith("T_")]
    assert len(names) > 50
    for name in names:
        T, want = g["T_" + name], g["SA_" + name]
        sa = oracle.build_sa40(T, threads=3)
        assert np.array_equal(sa40_to_u64(sa, len(T)).astype(np.uint32), want), name
        assert oracle.is_correct(T, sa), name
        if len(T) > 1:
            bad = sa.copy()
            bad[0:5], bad[5:10] = sa[5:10].copy(), sa[0:5].copy()
            assert not oracle.is_correct(T, bad), name


def test_query_fixtures(oracle):
    g = np.load(os.path.join(GOLDEN, "query_fixtures.npz"))
    s = np.load(os.path.join(GOLDEN, "sa_fixtures.npz"))
    for name in [k[4:] for k in g.files if k.startswith("off_")]:
        T = s["T_" + name]
        sa = oracle.build_sa40(T)
        off, sym, want = g["off_" + name], g["sym_" + name], g["itv_" + name]
        got = oracle.find_batch(T, sa, off, sym, threads=2)
        assert np.array_equal(got, want), name
        pos, cnt = oracle.locate_batch(sa, got, 100)
        full = sa40_to_u64(sa, len(T))
        for i in range(len(off) - 1):
            lo, hi = int(got[2 * i]), int(got[2 * i + 1])
            c = min(100, hi - lo)
            assert cnt[i] == c and np.array_equal(pos[i, :c], full[lo:lo + c])


def test_against_reference_library(oracle, reference):
    rng = np.random.default_rng(5)
    for n, sigma in ((500, 2), (3000, 5), (4000, 60000)):
        T = rng.integers(0, sigma, n).astype(np.uint16)
        a, b = oracle.build_sa40(T), reference.build_sa40(T)
        assert np.array_equal(a[:5 * n], b[:5 * n])
        assert reference.is_correct(T, a) and oracle.is_correct(T, b)
        off, sym, qs = conftest.fixture_queries(T, rng, 100)
        ia, ib = oracle.find_batch(T, a, off, sym), reference.find_batch(T, a, off, sym, threads=2)
        assert np.array_equal(ia, ib)
        assert oracle.counts_hash(ia) == reference.counts_hash(ib)
        for i, P in enumerate(qs[:20]):
            assert reference.brute_find(T, P) == (int(ia[2 * i]), int(ia[2 * i + 1]))
