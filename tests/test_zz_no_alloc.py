"""The allocation-free GEMM entry point, called through its exported C symbol.

Some embedders cannot hand the library a workspace: they run under a frozen memory
pool or inside callbacks where cudaMalloc is forbidden.  For them
``pg_gemm_bf16_tn_noalloc`` keeps its split-K scratch in a fixed array inside the
library.  This test calls that symbol directly with ctypes (no wrapper, nothing
allocated on its behalf except the operands and output the caller owns anyway) and
checks it against the regular entry point on two back-to-back calls, so leftovers of
the first call in the shared scratch must not disturb the second.  It is collected
last so that a failure here cannot hide another test's result.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, x, w, y, status):
    t, k = x.shape
    m = w.shape[0]
    vp, ll, ci = ctypes.c_void_p, ctypes.c_longlong, ctypes.c_int
    fn = lib.pg_gemm_bf16_tn_noalloc
    fn.restype = ci
    rc = fn(vp(x.data_ptr()), vp(w.data_ptr()), vp(y.data_ptr()), ci(t), ci(m), ci(k), ll(x.stride(0)), ll(w.stride(0)), ll(y.stride(0)),
            vp(status.data_ptr()), vp(torch.cuda.current_stream().cuda_stream))
    return rc


def test_noalloc_gemm_matches_regular_entry_point_twice_in_a_row():
    from pegainfer_b200 import _native
    from pegainfer_b200.ops import cuda as K

    lib = _native.load()
    lib.pg_last_error.restype = ctypes.c_char_p
    dev = "cuda:0"
    torch.manual_seed(11)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    # (128, 4096, 4096) and (200, 1000, 4104) take the workspace split-K path: their f32 partial
    # sums and tile counters live in the library's built-in array, which is what this entry point
    # is for.  The same shape runs twice in a row and two shapes alternate, so whatever one call
    # leaves in the shared array must not disturb the next.  The narrow shapes reduce on chip.
    scratch_shapes = [(128, 4096, 4096), (200, 1000, 4104)]
    scratch_bytes = (8 << 20) - (64 << 10)
    for t, m, k in scratch_shapes:
        plan = K.gemm_plan(t, m, k)
        tiles = ((m + 127) // 128) * ((t + plan["bn"] - 1) // plan["bn"])
        assert plan["cluster"] == 1 and plan["splits"] > 1, f"{t}x{m}x{k} does not use the split-K workspace: {plan}"
        assert tiles * 2 * plan["bn"] * 128 * 4 <= scratch_bytes, "at least two splits must fit the built-in scratch"
    shapes = [scratch_shapes[0], scratch_shapes[0], scratch_shapes[1], scratch_shapes[0], (64, 4096, 4096), (48, 1000, 520), scratch_shapes[1]]
    for t, m, k in shapes:
        x = (torch.randn(t, k, device=dev) * 0.5).bfloat16()
        w = (torch.randn(m, k, device=dev) * 0.05).bfloat16()
        y = torch.full((t, m), float("nan"), dtype=torch.bfloat16, device=dev)
        rc = _call(lib, x, w, y, status)
        assert rc == 0, lib.pg_last_error().decode()
        torch.cuda.synchronize()
        ref = K.linear(x, w).float()
        exact = x.float() @ w.float().t()
        err = (y.float() - ref).abs()
        tol = 2 ** -7 * exact.abs() + 2e-2 * (k / 1024) ** 0.5
        assert torch.isfinite(y.float()).all()
        assert (err <= tol).all(), f"{t}x{m}x{k}: max diff to the regular entry point {err.max().item()}"
        assert (y.float() - exact).abs().le(tol).all()
    assert int(status.item()) == 0


def test_noalloc_gemm_rejects_problems_beyond_its_scratch():
    from pegainfer_b200 import _native

    lib = _native.load()
    lib.pg_last_error.restype = ctypes.c_char_p
    dev = "cuda:0"
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    # 16385 row tiles of 128 -> one more than the counters can hold; K tiny so it stays small
    m = 128 * 16384 + 1
    x = torch.zeros(1, 8, dtype=torch.bfloat16, device=dev)
    w = torch.zeros(m, 8, dtype=torch.bfloat16, device=dev)
    y = torch.zeros(1, m, dtype=torch.bfloat16, device=dev)
    rc = _call(lib, x, w, y, status)
    assert rc != 0
    assert b"exceed the built-in scratch limit" in lib.pg_last_error()
