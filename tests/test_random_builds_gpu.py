"""Seeded random texts through every single-GPU build entry point, each result byte for byte against the oracle's array.
The texts mix what the fixed cases keep apart: one symbol only, tiny and huge alphabets, long runs, periodic stretches, copied
documents and document separators, lengths from one symbol up. CASCADE_RANDOM_BUILDS sets the number of cases (default 24)."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _text(rng):
    n = int(rng.choice([1, 2, 3, 5, 17, 255, 256, 257, 4095, 4097, 30_000, 120_000, int(rng.integers(1, 250_000))]))
    sigma = int(rng.choice([1, 2, 3, 5, 50, 5000, 65536]))
    T = rng.integers(0, sigma, n).astype(np.uint16)
    kind = int(rng.integers(0, 5))
    if kind == 1 and n > 8:                         # long runs of one symbol
        for _ in range(int(rng.integers(1, 6))):
            a = int(rng.integers(0, n)); T[a:a + int(rng.integers(1, n // 2 + 1))] = T[a]
    elif kind == 2 and n > 8:                       # periodic stretches
        period = int(rng.integers(1, 9))
        a = int(rng.integers(0, n // 2)); b = int(rng.integers(a, n)) + 1
        T[a:b] = np.resize(T[a:a + period], b - a)
    elif kind == 3 and n > 64:                      # copies of one stretch, some with a symbol changed
        L = int(rng.integers(8, n // 4 + 8))
        src = T[:L].copy()
        for _ in range(int(rng.integers(1, 8))):
            a = int(rng.integers(0, n - L + 1)); T[a:a + L] = src
            if rng.integers(0, 2):
                T[a + int(rng.integers(0, L))] ^= 1
    if rng.integers(0, 2) and n > 4:                # document separators, top of the symbol order
        T[rng.integers(0, n, max(1, n // 300))] = 0xFFFF
    if rng.integers(0, 4) == 0:
        T[-1] = 0                                   # a text that ends in the smallest symbol
    return T


def test_random_texts_through_every_build(oracle, tmp_path):
    from cascade_b200 import api
    cases = int(os.environ.get("CASCADE_RANDOM_BUILDS", "24"))
    first = int(os.environ.get("CASCADE_RANDOM_BUILDS_SEED", "0"))
    scratch = tmp_path / "scratch"
    scratch.mkdir()
    ctx = api.Context(0)
    try:
        for case in range(first, first + cases):
            rng = np.random.default_rng(1000 + case)
            T = _text(rng)
            n = len(T)
            p = int(rng.choice([1, 2, 7, 64, 300]))
            part = int(rng.choice([0, 1, 1000, 50_000]))
            want = oracle.build_sa40(T)[:5 * n]
            Tp = np.concatenate([T, np.zeros(api.TEXT_PAD, np.uint16)])
            Td = torch.from_numpy(Tp.view(np.int16)).cuda().view(torch.uint16)
            tag = (case, n, p, part)
            sa, _ = api.build_sa(ctx, Td, n, p)
            assert np.array_equal(sa[:5 * n].cpu().numpy(), want), ("resident", tag)
            sa, _ = api.build_sa_host(ctx, Tp, n, p)
            assert np.array_equal(sa[:5 * n], want), ("host", tag)
            sa, _ = api.build_sa_streamed(ctx, Tp, n, p, part_suffixes=part)
            assert np.array_equal(sa[:5 * n], want), ("streamed", tag)
            sa, st = api.build_sa_tiered(ctx, Tp, n, p, part_suffixes=part, host_list_bytes=int(rng.choice([0, 9 * n // 2])), scratch_dir=scratch)
            assert np.array_equal(sa[:5 * n], want), ("tiered", tag)
            v = api.validate_sa(ctx, Td, n, torch.from_numpy(sa).cuda())
            assert v["ok"], ("validate", tag, v)
        assert list(scratch.iterdir()) == []
    finally:
        ctx.close()
