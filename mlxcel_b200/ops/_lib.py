"""ctypes binding of ``lib/libmlxcel_b200.so`` (the sm_100a kernel library).

The library is the only GPU code path: when a CUDA device is present and the library cannot
be loaded, every op raises instead of falling back to PyTorch, so a missing build can not
pass silently.
"""
from __future__ import annotations

import ctypes
import os
from pathlib import Path

import torch

_LIB = None
_LIB_ERR: str | None = None
_PKG = Path(__file__).resolve().parent.parent


def lib_path() -> Path:
    return _PKG / "lib" / "libmlxcel_b200.so"


def load(required: bool = True):
    """Return the loaded kernel library (building it when sources are newer and nvcc exists)."""
    global _LIB, _LIB_ERR
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not path.exists() or os.environ.get("MLXCEL_B200_REBUILD") == "1":
        try:
            from .. import _build

            _build.build_cuda()
        except Exception as e:  # pragma: no cover - build environment specific
            _LIB_ERR = f"build failed: {e}"
    if path.exists():
        if os.environ.get("MLXCEL_B200_AUTOTUNE", "") in ("1", "cache"):
            from .. import autotune      # cached launch knobs go into the environment before the library reads them

            autotune.apply_cached()
        try:
            _LIB = ctypes.CDLL(str(path))
            _declare(_LIB)
            if os.environ.get("MLXCEL_B200_ROPE_VEC", "1") == "0" and hasattr(_LIB, "mx_set_rope_vec"):
                _LIB.mx_set_rope_vec(0)
            if os.environ.get("MLXCEL_B200_MOE_ALIGN_FAST", "1") == "0" and hasattr(_LIB, "mx_set_moe_align_fast"):
                _LIB.mx_set_moe_align_fast(0)
            return _LIB
        except OSError as e:
            _LIB_ERR = str(e)
    if required:
        raise RuntimeError(
            f"mlxcel_b200 CUDA kernel library is not available ({_LIB_ERR or 'not built'}); "
            "run `python -c 'import __graft_entry__ as g; g.build()'`")
    return None


_vp = ctypes.c_void_p
_i = ctypes.c_int
_ll = ctypes.c_longlong
_f = ctypes.c_float


def _declare(lib) -> None:
    sig = {
        "mx_gemm_bf16": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _f, _f,
                         _vp, _ll, _i, _i, _vp, _vp],
        "mx_gemm_comm": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _vp, _vp,
                         _vp, _vp, _vp, _ll, _ll, _vp, _ll, _vp, _vp],
        "mx_allreduce_comm": [_vp, _vp, _vp, _ll, _i, _i, _i, _vp, _vp, _vp, _vp, _vp, _ll, _ll, _vp, _vp,
                              _vp, _vp, _vp],
        "mx_qmv_allreduce": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i, _i,
                             _vp, _vp, _vp, _vp, _ll, _ll, _vp, _vp, _vp, _vp],
        "mx_moe_qgemv": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _ll, _ll, _vp],
        "mx_row_ssq": [_vp, _i, _i, _ll, _vp, _vp],
        "mx_add_rmsnorm": [_vp, _vp, _vp, _vp, _vp, _i, _i, _f, _f, _vp],
        "mx_head_rmsnorm": [_vp, _vp, _i, _i, _i, _ll, _f, _vp],
        "mx_rope_append": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _f, _i, _i, _i, _i,
                           _i, _i, _i, _f, _i, _vp],
        "mx_paged_decode": [_vp, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i,
                            _i, _i, _i, _f, _f, _i, _i, _vp],
        "mx_paged_prefill": [_vp, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i,
                             _i, _i, _i, _i, _i, _f, _f, _i, _vp],
        "mx_paged_prefill_tc": [_vp, _ll, _vp, _vp, _ll, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i,
                                _i, _i, _i, _f, _vp, _vp],
        "mx_embedding": [_vp, _vp, _vp, _i, _i, _i, _f, _vp],
        "mx_argmax": [_vp, _i, _ll, _vp, _i, _i, _vp],
        "mx_sample": [_vp, _i, _ll, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _vp],
        "mx_apply_penalties": [_vp, _i, _ll, _vp, _i, _vp, _vp, _vp, _i, _i, _vp],
        "mx_spec_verify": [_vp, _i, _ll, _vp, _vp, _vp, _vp, _i, _i, _i, _vp],
        "mx_swiglu": [_vp, _vp, _i, _i, _i, _f, _f, _vp],
        "mx_read_status": [_vp, _i],
        "mx_qmm_affine": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _vp, _ll, _vp],
        "mx_dequantize": [_vp, _vp, _vp, _vp, _ll, _i, _i, _i, _i, _vp],
        "mx_moe_route": [_vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
        "mx_moe_align": [_vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
        "mx_moe_gather_rows_n": [_vp, _vp, _vp, _vp, _i, _i, _vp],
        "mx_moe_align_n": [_vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _vp],
        "mx_moe_scatter_rows_n": [_vp, _vp, _vp, _vp, _i, _i, _vp],
        "mx_moe_combine_n": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
        "mx_qmv": [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _i, _i, _vp],
        "mx_grouped_gemm_bf16": [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, _f, _f, _vp, _ll,
                                 _vp, _vp],
    }
    for name, args in sig.items():
        fn = getattr(lib, name, None)
        if fn is None:
            continue
        fn.argtypes = args
        fn.restype = _i
    for name in ("mx_gemm_workspace_bytes",):
        fn = getattr(lib, name, None)
        if fn is not None:
            fn.restype = _ll
            fn.argtypes = []
    fn = getattr(lib, "mx_paged_decode_scratch_floats", None)
    if fn is not None:
        fn.restype = _ll
        fn.argtypes = [_i, _i, _i, _i]
    fn = getattr(lib, "mx_build_info", None)
    if fn is not None:
        fn.restype = ctypes.c_char_p
        fn.argtypes = []


class GemmExtras(ctypes.Structure):
    """Mirror of ``MxGemmExtras`` (csrc/api.h): the optional per-call arguments of the GEMM entry
    points — packed-weight format, deferred-RMSNorm buffers, NVLS multicast addresses."""

    _fields_ = [("wq", _i), ("q_group", _i), ("ssq_in", _vp), ("ssq_out", _vp), ("ssq_eps", _f),
                ("ssq_inv_dim", _f), ("flags_mc", _vp), ("recv_mc", _vp), ("out_mc", _vp)]


def gemm_extras(wq: int = 0, q_group: int = 0, row_norm=None, ssq_out=None, flags_mc: int = 0,
                recv_mc: int = 0, out_mc: int = 0):
    """Builds the extras argument of one GEMM call (``None`` when the call needs none). The returned
    object must stay referenced until the call returns (pass ``ctypes.byref`` of it)."""
    if not (wq or row_norm is not None or ssq_out is not None or flags_mc):
        return None
    ex = GemmExtras()
    ex.wq, ex.q_group = int(wq), int(q_group)
    if row_norm is not None:
        ex.ssq_in = row_norm.ssq.buf.data_ptr()
        ex.ssq_eps = float(row_norm.eps)
        ex.ssq_inv_dim = 1.0 / row_norm.dim
    if ssq_out is not None:
        ex.ssq_out = ssq_out.buf.data_ptr()
    if flags_mc:
        ex.flags_mc, ex.recv_mc, ex.out_mc = flags_mc or None, recv_mc or None, out_mc or None
    return ex


def ref_or_null(ex):
    return ctypes.byref(ex) if ex is not None else None


class KernelError(RuntimeError):
    pass


def check(rc: int, name: str) -> None:
    if rc != 0:
        raise KernelError(f"{name} failed with code {rc}")


def ptr(t: torch.Tensor | None) -> int | None:
    """Address of an optional kernel operand. A pageable host tensor here would hand a kernel a pointer
    it cannot read (an illegal-address fault that takes the context down), so it is refused."""
    if t is None:
        return None
    if not t.is_cuda and not t.is_pinned():
        raise ValueError(f"a host tensor (shape {tuple(t.shape)}, {t.dtype}) was passed to a CUDA kernel")
    return t.data_ptr()


def stream() -> int:
    return torch.cuda.current_stream().cuda_stream


# ----------------------------------------------------------------------------- workspaces
_WS: dict[int, torch.Tensor] = {}
_LAUNCHES = 0


def workspace(device: torch.device) -> torch.Tensor:
    """Per-device scratch buffer (status word, tile counters, split-K partials), zeroed once."""
    idx = device.index if device.index is not None else torch.cuda.current_device()
    ws = _WS.get(idx)
    if ws is None:
        nbytes = int(load().mx_gemm_workspace_bytes())
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=torch.device("cuda", idx))
        _WS[idx] = ws
    return ws


def count_launch(n: int = 1) -> None:
    global _LAUNCHES
    _LAUNCHES += n


def launches() -> int:
    """Number of kernel launches issued through this library since import."""
    return _LAUNCHES


def read_status(device: torch.device, clear: bool = True) -> int:
    """Device status word of the workspace (0 = no kernel reported a bounded-wait failure)."""
    ws = workspace(device)
    return int(load().mx_read_status(ws.data_ptr(), 1 if clear else 0))
