"""The allocation-free GEMM entry point (``mx_gemm_bf16_static``, csrc/no_alloc.h).

Some users of the kernel library are handed their input and output buffers and nothing else:
they run behind a fixed memory plan, or inside a section of another runtime where asking for
device memory is not allowed, so they cannot provide the workspace that ``mx_gemm_bf16`` needs.
For them the library carries its own fixed scratch array. This test calls that entry point the
way such a user would — straight through the exported C symbol, passing raw pointers — and checks
that two calls in a row give the same numbers as the regular entry point, and that a problem
beyond the documented limits is refused instead of launched.

Collected last on purpose (file name sorts after the other tests), so a run that stops at the
first failure has already exercised everything else.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _close(got, want, rtol=2e-2, atol=2e-2):
    err = (got.float() - want.float()).abs()
    bad = (err > atol + rtol * want.float().abs()).sum().item()
    assert bad == 0, f"{bad} mismatches, max err {err.max().item():.4g}"


def _symbol():
    from mlxcel_b200.ops import _lib

    lib = ctypes.CDLL(str(_lib.lib_path()))
    fn = lib.mx_gemm_bf16_static
    vp, i, f = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [vp, vp, vp, vp, vp, i, i, i, i, i, i, i, i, i, i, f, f, vp]
    fn.restype = i
    err = lib.mx_gemm_bf16_static_error
    err.argtypes, err.restype = [i], ctypes.c_char_p
    return fn, err


def _status(clear: int = 1) -> int:
    """The bounded-wait status word of the library's own scratch array (0 = every launch completed)."""
    from mlxcel_b200.ops import _lib

    lib = ctypes.CDLL(str(_lib.lib_path()))
    lib.mx_gemm_bf16_static_status.argtypes, lib.mx_gemm_bf16_static_status.restype = [ctypes.c_int], ctypes.c_int
    return lib.mx_gemm_bf16_static_status(clear)


def test_static_scratch_gemm_matches_regular_entry_point_twice():
    from mlxcel_b200 import ops

    fn, err = _symbol()
    dev = torch.device("cuda")
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device=dev).manual_seed(0)
    # (M, N, K): the second shape splits K over several CTAs, so the scratch partials and
    # counters left by the first call are reused by the second.
    for (M, N, K) in [(48, 512, 4096), (64, 1024, 2048)]:
        x = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
        w = (torch.randn(N, K, generator=g, device=dev) * 0.05).to(torch.bfloat16)
        res = torch.randn(M, N, generator=g, device=dev).to(torch.bfloat16)
        want = ops.linear(x, w, residual=res, force_mode=2)      # existing entry point
        for call in range(2):                                      # two calls in a row
            out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
            rc = fn(x.data_ptr(), w.data_ptr(), out.data_ptr(), None, res.data_ptr(), M, N, K, K, K, N, N,
                    2, 0, 0, 0.0, 0.0, stream)
            assert rc == 0, err(rc)
            torch.cuda.synchronize()
            _close(out, want)
            assert torch.equal(out, want), f"call {call}: split-K sum order must match"
            # and against plain PyTorch in fp32 (the regular entry point runs the same kernel)
            _close(out, x.float() @ w.float().t() + res.float())
            assert _status() == 0


def test_static_scratch_gemm_other_shapes_against_fp32():
    """Two column tiles (M = 192), a gated epilogue, and a shape whose preferred split count does not
    fit the 8 MiB array (the dispatcher trims it), each against the fp32 product, twice."""
    from mlxcel_b200 import ops

    fn, err = _symbol()
    dev = torch.device("cuda")
    stream = torch.cuda.current_stream().cuda_stream
    g = torch.Generator(device=dev).manual_seed(1)
    for (M, N, K, gated) in [(192, 512, 2048, False), (40, 256, 1024, True), (256, 3072, 4096, False)]:
        x = torch.randn(M, K, generator=g, device=dev).to(torch.bfloat16)
        rows = 2 * N if gated else N
        w = (torch.randn(rows, K, generator=g, device=dev) * 0.03).to(torch.bfloat16)
        acc = x.float() @ w.float().t()
        if gated:
            want32 = torch.nn.functional.silu(acc[:, :N]) * acc[:, N:]
            want = ops.glu_linear(x, w, N, "silu", force_mode=2)
        else:
            want32 = acc
            want = ops.linear(x, w, force_mode=2)
        for call in range(2):
            out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device=dev)
            rc = fn(x.data_ptr(), w.data_ptr(), out.data_ptr(), None, None, M, N, K, K, K, N, 0,
                    3 if gated else 0, 0, N if gated else 0, 0.0, 0.0, stream)
            assert rc == 0, err(rc)
            torch.cuda.synchronize()
            _close(out, want32, rtol=3e-2, atol=3e-2)
            _close(out, want)
            assert _status() == 0


def test_static_scratch_gemm_refuses_oversize():
    fn, err = _symbol()
    x = torch.zeros(8, 64, dtype=torch.bfloat16, device="cuda")
    rc = fn(x.data_ptr(), x.data_ptr(), x.data_ptr(), None, None, 257, 64, 64, 64, 64, 64, 0, 0, 0, 0, 0.0, 0.0,
            torch.cuda.current_stream().cuda_stream)
    assert rc == -70 and b"exceeds" in err(rc)
    rc = fn(None, x.data_ptr(), x.data_ptr(), None, None, 8, 64, 64, 64, 64, 64, 0, 0, 0, 0, 0.0, 0.0, None)
    assert rc == -72
