"""The hand-written radix sort (through the C ABI) against a stable comparison sort of the same records."""
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


def _check(ctx, keys, vals, b0, b1):
    from cascade_b200 import api
    k0, v0 = keys.clone(), vals.clone()
    ko, vo = api.sort_pairs(ctx, keys, vals, b0, b1)
    width = b1 - b0
    if width >= 64:
        mk = k0 ^ (-(1 << 63))          # unsigned order on int64 storage
    else:
        mk = (k0 >> b0) & ((1 << width) - 1)
    order = torch.sort(mk, stable=True).indices
    assert torch.equal(k0[order], ko)
    assert torch.equal(v0[order], vo)


@pytest.mark.parametrize("n", [1, 2, 3, 31, 255, 4095, 4096, 4097, 100003, 1 << 20])
def test_sort_random_full_keys(ctx, n):
    g = torch.Generator(device="cuda").manual_seed(n)
    keys = torch.randint(-(1 << 62), 1 << 62, (n,), device="cuda", dtype=torch.int64, generator=g) * 2 + (torch.arange(n, device="cuda") & 1)
    _check(ctx, keys, torch.arange(n, device="cuda", dtype=torch.int32), 0, 64)


@pytest.mark.parametrize("bits", [(0, 8), (3, 40), (16, 17), (0, 56), (40, 64)])
def test_sort_bit_ranges_are_stable(ctx, bits):
    n = 300007
    g = torch.Generator(device="cuda").manual_seed(7)
    keys = torch.randint(-(1 << 62), 1 << 62, (n,), device="cuda", dtype=torch.int64, generator=g)
    _check(ctx, keys, torch.arange(n, device="cuda", dtype=torch.int32), *bits)


def test_sort_skewed_digits_and_skipped_passes(ctx):
    n = 1 << 21
    g = torch.Generator(device="cuda").manual_seed(1)
    keys = (torch.randint(0, 7, (n,), device="cuda", dtype=torch.int64, generator=g) << 20) | 5     # most digits are constant
    _check(ctx, keys, torch.arange(n, device="cuda", dtype=torch.int32), 0, 64)
    keys = torch.zeros(n, device="cuda", dtype=torch.int64)                                         # every pass is skipped
    _check(ctx, keys, torch.arange(n, device="cuda", dtype=torch.int32), 0, 64)


def test_sort_64_bit_values(ctx):
    n = 1 << 20
    g = torch.Generator(device="cuda").manual_seed(2)
    keys = torch.randint(0, 1 << 40, (n,), device="cuda", dtype=torch.int64, generator=g)
    _check(ctx, keys, torch.arange(n, device="cuda", dtype=torch.int64) * 3, 0, 40)


@pytest.mark.parametrize("n", [1, 2, 5, 4097, 300008])
def test_sort_of_a_list_on_an_odd_8_byte_boundary(ctx, n):
    """A partition's records start wherever the partition starts: keys 8-byte aligned only, values 4-byte aligned only."""
    g = torch.Generator(device="cuda").manual_seed(n)
    keys = torch.randint(-(1 << 62), 1 << 62, (n + 1,), device="cuda", dtype=torch.int64, generator=g)[1:]
    vals = torch.arange(n + 1, device="cuda", dtype=torch.int32)[1:]
    assert keys.data_ptr() % 16 == 8
    _check(ctx, keys, vals, 0, 64)


def test_sort_many_tiles(ctx):
    n = 20_000_003
    g = torch.Generator(device="cuda").manual_seed(3)
    keys = torch.randint(-(1 << 62), 1 << 62, (n,), device="cuda", dtype=torch.int64, generator=g)
    _check(ctx, keys, torch.arange(n, device="cuda", dtype=torch.int32), 0, 64)


def test_sort_in_several_launches_per_pass(ctx):
    """Sorts larger than one launch's share run as several launches per pass whose digit offsets chain up."""
    from cascade_b200._lib import lib
    assert lib().csa_debug_set(0, 16) == 0
    try:
        n = 1_000_003
        g = torch.Generator(device="cuda").manual_seed(9)
        keys = torch.randint(-(1 << 62), 1 << 62, (n,), device="cuda", dtype=torch.int64, generator=g)
        _check(ctx, keys, torch.arange(n, device="cuda", dtype=torch.int32), 0, 64)
        keys = torch.randint(0, 1 << 20, (n,), device="cuda", dtype=torch.int64, generator=g)
        _check(ctx, keys, torch.arange(n, device="cuda", dtype=torch.int32), 0, 20)
    finally:
        assert lib().csa_debug_set(0, 29) == 0


def test_a_wait_that_cannot_succeed_runs_out_and_is_reported_without_a_fault(ctx):
    """With the test hooks on, the tiles of a pass are numbered from 1: tile 0, on which tile 1 waits, never comes. Every
    bounded wait of the pass must run out, the kernels must return, nothing of the failed passes may be written, the host
    must get CSA_E_DEVICE with the look-back bit from csa_sync, and the context must sort correctly afterwards."""
    from cascade_b200 import api
    from cascade_b200._lib import lib
    L = lib()
    n = 200_000
    g = torch.Generator(device="cuda").manual_seed(5)
    keys = torch.randint(-(1 << 62), 1 << 62, (n,), device="cuda", dtype=torch.int64, generator=g)
    vals = torch.arange(n, device="cuda", dtype=torch.int32)
    assert L.csa_debug_set(2, 64) == 0 and L.csa_debug_set(3, 1) == 0
    try:
        with pytest.raises(api.CascadeError) as e:
            api.sort_pairs(ctx, keys.clone(), vals.clone(), 0, 16)
        assert e.value.code == 5 and "status bits 1" in str(e.value)
    finally:
        assert L.csa_debug_set(3, 0) == 0 and L.csa_debug_set(2, 1 << 22) == 0
    _check(ctx, keys, vals, 0, 64)


def _sort_segments(ctx, keys, vals, seg_off, b0, b1):
    from cascade_b200._lib import c_int
    import ctypes
    n, segs = keys.numel(), len(seg_off) - 1
    ka = torch.empty_like(keys)
    va = torch.empty_like(vals) if vals is not None else None
    wsb = ctx.L.csa_sort_segments_workspace_bytes(n, segs)
    ws = torch.empty(wsb, dtype=torch.uint8, device="cuda")
    off = np.ascontiguousarray(seg_off, dtype=np.uint64)
    in_alt = c_int(0)
    torch.cuda.synchronize()
    ctx.check(ctx.L.csa_sort_segments(ctx.h, keys.data_ptr(), ka.data_ptr(), vals.data_ptr() if vals is not None else None, va.data_ptr() if va is not None else None,
                                      off.ctypes.data, segs, b0, b1, ws.data_ptr(), wsb, ctypes.byref(in_alt)))
    ctx.sync()
    assert in_alt.value == ((b1 - b0 + 7) // 8) % 2
    return (ka, va) if in_alt.value else (keys, vals)


@pytest.mark.parametrize("bits", [(0, 64), (0, 20), (8, 40)])
def test_segments_of_one_array_sorted_in_one_set_of_launches(ctx, bits):
    """Ragged segments (empty, one record, exactly one tile, many tiles, constant keys, keys that differ in one byte only),
    each sorted stably on its own; records never leave their segment."""
    g = torch.Generator(device="cuda").manual_seed(11)
    sizes = [0, 1, 6144, 6145, 5, 100_003, 0, 300_000, 12_288, 7, 250_000, 1]
    seg_off = np.concatenate([[0], np.cumsum(sizes)])
    n = int(seg_off[-1])
    keys = torch.randint(-(1 << 62), 1 << 62, (n,), device="cuda", dtype=torch.int64, generator=g)
    a, b = int(seg_off[7]), int(seg_off[8])
    keys[a:b] = 0x1234_5678_9ABC_DEF0                       # a constant segment: every pass copies it over
    a, b = int(seg_off[10]), int(seg_off[11])
    keys[a:b] = (keys[a:b] & 0xFF00) | 0x0101_0101_0101_0001  # one varying byte: the other passes copy it over
    vals = torch.arange(n, device="cuda", dtype=torch.int32)
    k0, v0 = keys.clone(), vals.clone()
    ko, vo = _sort_segments(ctx, keys, vals, seg_off, *bits)
    width = bits[1] - bits[0]
    for s in range(len(sizes)):
        a, b = int(seg_off[s]), int(seg_off[s + 1])
        if a == b:
            continue
        mk = (k0[a:b] ^ (-(1 << 63))) if width >= 64 else ((k0[a:b] >> bits[0]) & ((1 << width) - 1))
        order = torch.sort(mk, stable=True).indices
        assert torch.equal(k0[a:b][order], ko[a:b]), (s, bits)
        assert torch.equal(v0[a:b][order], vo[a:b]), (s, bits)
    # keys only
    ko2, _ = _sort_segments(ctx, k0.clone(), None, seg_off, *bits)
    assert torch.equal(ko2, ko)
