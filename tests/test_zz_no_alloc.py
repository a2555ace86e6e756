"""csa_sort_pairs_static: the sort for hosts that may not allocate device memory (a plugin inside another runtime whose
pool owns the device, a service pinned to a fixed memory budget). It is called through the C ABI twice in a row, with
different inputs, and each result must equal csa_sort_pairs's on the same input, bit for bit; the second call checks that
what the first left in the shared fixed scratch does no harm. The file sorts last so that a failure here cannot hide
another test's."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _reference_sort(ctx, keys, vals, b0, b1):
    from cascade_b200 import api
    return api.sort_pairs(ctx, keys.clone(), vals.clone(), b0, b1)


def _static_sort(L, keys, vals, b0, b1):
    k, v = keys.clone(), vals.clone()
    ka, va = torch.empty_like(k), torch.empty_like(v)
    torch.cuda.synchronize()
    in_alt = ctypes.c_int(-1)
    rc = L.csa_sort_pairs_static(None, k.data_ptr(), ka.data_ptr(), v.data_ptr(), va.data_ptr(), k.numel(), b0, b1, ctypes.byref(in_alt))
    assert rc == 0, rc
    return (ka, va) if in_alt.value else (k, v)


def test_static_sort_matches_the_workspace_sort_twice_in_a_row():
    from cascade_b200 import api
    from cascade_b200._lib import lib
    L = lib()
    ctx = api.Context(0)
    try:
        g = torch.Generator(device="cuda").manual_seed(11)
        cases = [(1_000_003, 0, 64), (3_141_593, 5, 43)]
        for n, b0, b1 in cases:      # two calls in a row on the one shared scratch array
            keys = torch.randint(-(1 << 62), 1 << 62, (n,), device="cuda", dtype=torch.int64, generator=g)
            vals = torch.randint(0, 1 << 31, (n,), device="cuda", dtype=torch.int32, generator=g)
            want_k, want_v = _reference_sort(ctx, keys, vals, b0, b1)
            got_k, got_v = _static_sort(L, keys, vals, b0, b1)
            assert torch.equal(got_k, want_k) and torch.equal(got_v, want_v), (n, b0, b1)
        # a small sort after the large ones, constant digits included (the static variant never skips a pass)
        keys = (torch.arange(5000, device="cuda", dtype=torch.int64) * 7919) % 1000
        vals = torch.arange(5000, device="cuda", dtype=torch.int32)
        want_k, want_v = _reference_sort(ctx, keys, vals, 0, 64)
        got_k, got_v = _static_sort(L, keys, vals, 0, 64)
        assert torch.equal(got_k, want_k) and torch.equal(got_v, want_v)
    finally:
        ctx.close()


def test_static_sort_edges_against_a_comparison_sort():
    """The sizes around a tile and at the limit, a list that starts on an odd 8-byte boundary, a caller's own stream; checked
    against a stable comparison sort of the same records, not against the library's other sort."""
    from cascade_b200._lib import lib
    L = lib()
    g = torch.Generator(device="cuda").manual_seed(23)
    stream = torch.cuda.Stream()
    for n in (1, 2, 4095, 4096, 4097, 1 << 22):
        base_k = torch.randint(-(1 << 62), 1 << 62, (n + 1,), device="cuda", dtype=torch.int64, generator=g)
        base_v = torch.arange(n + 1, device="cuda", dtype=torch.int32)
        for odd in (0, 1):
            k, v = base_k[odd:odd + n].clone() if not odd else base_k[1:], base_v[odd:odd + n].clone() if not odd else base_v[1:]
            if odd:
                assert k.data_ptr() % 16 == 8
            k0, v0 = k.clone(), v.clone()
            ka, va = torch.empty(n + 1, dtype=torch.int64, device="cuda")[odd:odd + n], torch.empty(n + 1, dtype=torch.int32, device="cuda")[odd:odd + n]
            torch.cuda.synchronize()
            in_alt = ctypes.c_int(-1)
            rc = L.csa_sort_pairs_static(ctypes.c_void_p(stream.cuda_stream), k.data_ptr(), ka.data_ptr(), v.data_ptr(), va.data_ptr(), n, 0, 64, ctypes.byref(in_alt))
            assert rc == 0, (n, odd, rc)
            gk, gv = (ka, va) if in_alt.value else (k, v)
            order = torch.sort(k0 ^ (-(1 << 63)), stable=True).indices
            assert torch.equal(gk, k0[order]) and torch.equal(gv, v0[order]), (n, odd)


def test_static_sort_refuses_more_than_its_fixed_scratch_holds():
    from cascade_b200._lib import lib
    L = lib()
    n = (1 << 22) + 1
    k = torch.zeros(n, dtype=torch.int64, device="cuda")
    v = torch.zeros(n, dtype=torch.int32, device="cuda")
    in_alt = ctypes.c_int(0)
    rc = L.csa_sort_pairs_static(None, k.data_ptr(), k.data_ptr(), v.data_ptr(), v.data_ptr(), n, 0, 64, ctypes.byref(in_alt))
    assert rc == 4          # CSA_E_LIMIT
