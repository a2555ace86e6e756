"""Seeded random texts and query batches through the query engine's placements (suffix array on the device, in pinned host
memory, sharded by range) and strides, every interval, count and position against the oracle's host search.
CASCADE_RANDOM_QUERIES sets the number of cases (default 16)."""
import os

import numpy as np
import pytest
import torch

import conftest
from test_random_builds_gpu import _text

pytestmark = pytest.mark.gpu


def test_random_indexes_and_batches(oracle):
    from cascade_b200 import api, multi
    cases = int(os.environ.get("CASCADE_RANDOM_QUERIES", "16"))
    first = int(os.environ.get("CASCADE_RANDOM_QUERIES_SEED", "0"))
    ctx = api.Context(0)
    try:
        for case in range(first, first + cases):
            rng = np.random.default_rng(5000 + case)
            T = _text(rng)
            n = len(T)
            if n > 60_000:
                T = T[:60_000]; n = len(T)
            stride = int(rng.choice([1, 2, 3, 32, 64, 4096]))
            max_pos = int(rng.choice([1, 7, 100]))
            q = int(rng.choice([1, 33, 400]))
            tag = (case, n, stride, max_pos, q)
            sa = oracle.build_sa40(T)
            Tp = np.concatenate([T, np.zeros(api.TEXT_PAD, np.uint16)])
            td = torch.from_numpy(Tp.view(np.int16)).cuda().view(torch.uint16)
            off, sym, _ = conftest.fixture_queries(T, rng, q)
            o = torch.from_numpy(off.view(np.int64)).cuda()
            s = torch.from_numpy(np.concatenate([sym, np.zeros(8, np.uint16)]).view(np.int16)).cuda()
            want = oracle.find_batch(T, sa, off, sym)
            wp, wc = oracle.locate_batch(sa, want, max_pos)
            sa_dev = torch.from_numpy(np.ascontiguousarray(sa)).cuda()
            for where, sa_t in (("device", sa_dev), ("pinned", torch.from_numpy(np.ascontiguousarray(sa)).pin_memory())):
                idx = api.SuffixIndex(ctx, td, sa_t, n, stride)
                itv = idx.find(o, s, q)
                assert np.array_equal(itv.cpu().numpy().view(np.uint64), want), (where, tag)
                assert idx.certify(o, s, q, itv)[0] == 0, (where, tag)
                pos, cnt = idx.locate(itv, q, max_pos)
                assert np.array_equal(cnt.cpu().numpy().view(np.uint32), wc), (where, tag)
                pn = pos.cpu().numpy().view(np.uint64).reshape(q, max_pos)
                for i in range(q):
                    assert np.array_equal(pn[i, :wc[i]], wp[i, :wc[i]]), (where, tag, i)
                itv_h, cnt_h, poff_h, pos_h, total = idx.query_host(off, np.concatenate([sym, np.zeros(8, np.uint16)]), max_pos)
                assert np.array_equal(itv_h, want) and np.array_equal(cnt_h, wc) and total == int(wc.sum()), (where, "host", tag)
                for i in range(q):
                    assert np.array_equal(pos_h[int(poff_h[i]):int(poff_h[i + 1])], wp[i, :wc[i]]), (where, "host", tag, i)
            # slices of the suffix array, each with its own table; starts are multiples of 4 entries
            if n >= 16:
                cuts = sorted(set([0, n] + [int(c) // 4 * 4 for c in rng.integers(1, n, 3)]))
                total_itv = torch.zeros(2 * q, dtype=torch.int64, device="cuda")
                shards = []
                for a, b in zip(cuts[:-1], cuts[1:]):
                    sl = np.concatenate([sa[5 * a:5 * b], np.zeros(128, np.uint8)])
                    shards.append(multi.ShardedIndex(ctx, td, torch.from_numpy(sl).cuda(), n, a, b - a, stride=stride))
                    total_itv += shards[-1].find(o, s, q, reduce=False)
                assert np.array_equal(total_itv.cpu().numpy().view(np.uint64), want), ("sharded", tag, cuts)
                packed = None
                for sh in shards:
                    pos, poff, cnt = sh.locate_packed(total_itv, q, max_pos, reduce=False)
                    packed = pos.clone() if packed is None else packed + pos
                pk, po = packed.cpu().numpy().view(np.uint64), poff.cpu().numpy()
                assert np.array_equal(cnt.cpu().numpy().view(np.uint32), wc), ("sharded", tag)
                for i in range(q):
                    assert np.array_equal(pk[int(po[i]):int(po[i + 1])], wp[i, :wc[i]]), ("sharded", tag, cuts, i)
    finally:
        ctx.close()
