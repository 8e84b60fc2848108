"""The decode attention entry point that allocates nothing, reached through its
exported C symbol, against the regular entry point.

Programs that cannot call cudaMalloc (a server whose arena owns the whole GPU,
a loop that must not stall other streams, a plain C host) use
``agv_attention_decode_static``: its scratch is a fixed array inside the
library.  This file is collected last, so a run that stops at the first failure
has run every other test before it; it also passes alone in a fresh process.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"
SCRATCH_FLOATS = 4 * 1024 * 1024


def _rnd(*shape, dtype, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(dtype).to(DEV)


def _static(lib, q, out, k_pool, v_pool, table, slots, positions, page, cap, nh, nkv, hd, scale,
            window, max_keys):
    code = 0 if q.dtype == torch.float32 else 1
    vp = lambda t: ctypes.c_void_p(t.data_ptr())
    return lib.agv_attention_decode_static(
        vp(q), ctypes.c_longlong(q.stride(0)), vp(out), code, vp(k_pool), vp(v_pool), vp(table),
        vp(slots), vp(positions), table.shape[1], page, cap, q.shape[0], nh, nkv, hd,
        ctypes.c_float(scale), window, max_keys,
        ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_static_scratch_entry_point_matches_the_regular_one(dtype):
    from agave_b200 import kernels
    lib = kernels.library()
    lib.agv_attention_decode_static.restype = ctypes.c_int
    PAGE, nh, nkv, hd = 64, 4, 1, 128
    max_pages, n_pages = 10, 30
    k_pool = _rnd(n_pages, PAGE, nkv, hd, dtype=dtype, seed=1, scale=0.3)
    v_pool = _rnd(n_pages, PAGE, nkv, hd, dtype=dtype, seed=2)
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(3)).int()
    table = perm.reshape(3, max_pages).contiguous().to(DEV)
    cap = max_pages * PAGE
    tol = 2e-5 if dtype == torch.float32 else 8e-3
    # two calls in a row; the second has other lengths, slots and window, so what the
    # first call left in the shared array would show if it were read
    cases = [([600, 130, 1], [1, 2, 0], 0, 640), ([64, 333, 2], [2, -1, 1], 100, 100)]
    for lens, slot_list, window, max_keys in cases:
        slots = torch.tensor(slot_list, dtype=torch.int32, device=DEV)
        positions = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
        q = _rnd(3, nh * hd, dtype=dtype, seed=10 + lens[0], scale=0.3)
        ref = torch.full((3, nh * hd), float("nan"), dtype=dtype, device=DEV)
        kernels.attention_decode_split(q, ref, k_pool, v_pool, table, slots, positions, PAGE, cap,
                                       nh, nkv, hd, 0.5, window, max_keys)
        out = torch.full_like(ref, float("nan"))
        rc = _static(lib, q, out, k_pool, v_pool, table, slots, positions, PAGE, cap, nh, nkv, hd,
                     0.5, window, max_keys)
        assert rc == 0, lib.agv_last_error().decode()
        torch.cuda.synchronize()
        assert torch.isfinite(out.float()).all()
        err = (out.double() - ref.double()).abs().max().item()
        assert err <= tol * ref.double().abs().max().item(), err


def test_static_scratch_entry_point_recovers_from_a_call_with_too_small_max_keys():
    """max_keys sizes the grid.  A call that understates it leaves that entry's arrival
    count unfinished; the counters live inside the library, where no caller can clear
    them, so every call clears the ones it uses before its kernel runs and the next call
    is right again."""
    from agave_b200 import kernels
    lib = kernels.library()
    lib.agv_attention_decode_static.restype = ctypes.c_int
    dtype = torch.float32
    PAGE, nh, nkv, hd = 64, 4, 1, 64
    max_pages, n_pages = 10, 20
    k_pool = _rnd(n_pages, PAGE, nkv, hd, dtype=dtype, seed=1, scale=0.3)
    v_pool = _rnd(n_pages, PAGE, nkv, hd, dtype=dtype, seed=2)
    table = torch.arange(n_pages, dtype=torch.int32).reshape(2, max_pages).contiguous().to(DEV)
    cap = max_pages * PAGE
    slots = torch.tensor([0, 1], dtype=torch.int32, device=DEV)
    positions = torch.tensor([599, 299], dtype=torch.int32, device=DEV)
    q = _rnd(2, nh * hd, dtype=dtype, seed=5, scale=0.3)
    ref = torch.empty((2, nh * hd), dtype=dtype, device=DEV)
    kernels.attention_decode_split(q, ref, k_pool, v_pool, table, slots, positions, PAGE, cap, nh,
                                   nkv, hd, 0.5, 0, 640)
    out = torch.zeros_like(ref)
    # 600 keys announced as at most 128: two chunks run, their count never reaches ten
    rc = _static(lib, q, out, k_pool, v_pool, table, slots, positions, PAGE, cap, nh, nkv, hd,
                 0.5, 0, 128)
    assert rc == 0
    for _ in range(2):
        out = torch.full_like(ref, float("nan"))
        rc = _static(lib, q, out, k_pool, v_pool, table, slots, positions, PAGE, cap, nh, nkv,
                     hd, 0.5, 0, 640)
        assert rc == 0, lib.agv_last_error().decode()
        torch.cuda.synchronize()
        err = (out.double() - ref.double()).abs().max().item()
        assert err <= 2e-5 * ref.double().abs().max().item(), err


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    from agave_b200 import kernels
    lib = kernels.library()
    lib.agv_attention_decode_static.restype = ctypes.c_int
    nh, nkv, hd, PAGE = 4, 1, 256, 64
    B, max_keys = 64, 8192                  # 64 * 4 * 128 chunks * 258 values: far too many
    chunk, n_splits = kernels.attention_decode_plan(hd, torch.bfloat16, max_keys)
    assert B * nh * n_splits * (hd + 2) > SCRATCH_FLOATS
    k_pool = torch.zeros((2, PAGE, nkv, hd), dtype=torch.bfloat16, device=DEV)
    table = torch.zeros((B, 128), dtype=torch.int32, device=DEV)
    slots = torch.full((B,), -1, dtype=torch.int32, device=DEV)
    positions = torch.zeros(B, dtype=torch.int32, device=DEV)
    q = torch.zeros((B, nh * hd), dtype=torch.bfloat16, device=DEV)
    out = torch.zeros_like(q)
    rc = _static(lib, q, out, k_pool, k_pool, table, slots, positions, PAGE, 8192, nh, nkv, hd,
                 1.0, 0, max_keys)
    assert rc != 0
    msg = lib.agv_last_error().decode()
    assert "scratch" in msg and str(SCRATCH_FLOATS) in msg
