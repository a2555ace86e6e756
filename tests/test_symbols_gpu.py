"""Texts of 1-byte and 4-byte symbols: mapped onto 16-bit symbols in numeric order, their suffix array is the one of the
original text (checked against the oracle on the equally mapped text, whose suffixes compare the same way)."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    from cascade_b200 import api
    c = api.Context(0)
    yield c
    c.close()


def test_one_byte_symbols(ctx, oracle):
    from cascade_b200 import api
    rng = np.random.default_rng(5)
    n = 300_000
    t8 = rng.integers(0, 256, n).astype(np.uint8)
    t8[rng.integers(0, 50, n) == 0] = 255
    d8 = torch.from_numpy(t8).cuda()
    out = torch.full((n + api.TEXT_PAD,), 7, dtype=torch.int16, device="cuda")
    ctx.check(ctx.L.csa_text_from_u8(ctx.h, d8.data_ptr(), n, out.data_ptr()))
    ctx.sync()
    got = out.cpu().numpy().view(np.uint16)
    assert np.array_equal(got[:n], t8.astype(np.uint16)) and np.all(got[n:] == 0)
    sa, _ = api.build_sa(ctx, out.view(torch.uint16), n, 8)
    assert np.array_equal(sa.cpu().numpy()[:5 * n], oracle.build_sa40(t8.astype(np.uint16))[:5 * n])


def test_four_byte_symbols_by_rank(ctx, oracle):
    from cascade_b200 import api
    rng = np.random.default_rng(6)
    n = 400_000
    alphabet = np.unique(np.concatenate([rng.integers(0, 2**32, 40_000, dtype=np.uint64), [0, 1, 2**32 - 1, 2**31, 65535, 65536]]).astype(np.uint32))
    t32 = alphabet[np.minimum((rng.pareto(1.2, n) * 20).astype(np.int64), len(alphabet) - 1)]
    d32 = torch.from_numpy(t32.view(np.int32)).cuda()
    out = torch.zeros(n + api.TEXT_PAD, dtype=torch.int16, device="cuda")
    alpha_d = torch.zeros(65536, dtype=torch.int32, device="cuda")
    distinct = ctypes.c_uint32(0)
    ctx.check(ctx.L.csa_text_from_u32(ctx.h, d32.data_ptr(), n, out.data_ptr(), alpha_d.data_ptr(), ctypes.byref(distinct)))
    ctx.sync()
    want_alpha, want_ranks = np.unique(t32, return_inverse=True)
    assert distinct.value == len(want_alpha)
    assert np.array_equal(alpha_d.cpu().numpy().view(np.uint32)[:distinct.value], want_alpha)
    got = out.cpu().numpy().view(np.uint16)
    assert np.array_equal(got[:n], want_ranks.astype(np.uint16)) and np.all(got[n:] == 0)
    sa, _ = api.build_sa(ctx, out.view(torch.uint16), n, 16)
    # ranks keep the order of the symbols, so the oracle on the ranks sorts the suffixes of the 32-bit text
    assert np.array_equal(sa.cpu().numpy()[:5 * n], oracle.build_sa40(want_ranks.astype(np.uint16))[:5 * n])
    # more distinct symbols than 16 bits hold: refused
    many = torch.arange(70_000, dtype=torch.int32, device="cuda") * 3
    rc = ctx.L.csa_text_from_u32(ctx.h, many.data_ptr(), 70_000, out.data_ptr(), alpha_d.data_ptr(), ctypes.byref(distinct))
    assert rc == 4 and b"70000 distinct" in ctx.L.csa_last_error(ctx.h)
