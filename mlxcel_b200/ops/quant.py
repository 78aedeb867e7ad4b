"""MLX quantization formats: quantizers (for random-init checkpoints and tests), the PyTorch
reference dequantizer, and the quantized linear dispatch.

Layout facts (reference: src/lib/mlxcel-core/src/layers.rs:2322-2522 and
src/lib/mlxcel-core/cpp/mlx_cxx_kernels.cpp:3073-3152):

* affine: ``w ≈ q * scale + bias`` per group of ``group_size`` inputs; ``q`` packed LSB-first
  along the input dimension into uint32 (a contiguous little-endian bit stream for 3/5/6 bits);
  scales/biases ``[out, in/group]`` in the activation dtype;
  invariant ``packed_in * 32 == bits * in``.
* mxfp4 / mxfp8: e2m1 / e4m3 values with one e8m0 scale (uint8) per 32 inputs, no biases.
"""
from __future__ import annotations

import os

import torch

from . import _lib
from ..models.weights import QuantizedTensor

_E2M1 = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0])
_MODE_ID = {"affine": 0, "mxfp4": 1, "mxfp8": 2}


# ----------------------------------------------------------------------------- bit packing
def pack_bits(q: torch.Tensor, bits: int) -> torch.Tensor:
    """q: integer tensor [..., in] with values < 2**bits → uint32 words [..., in*bits/32]."""
    *lead, n = q.shape
    assert (n * bits) % 32 == 0
    qv = q.to(torch.int64).reshape(-1, n)
    bitpos = torch.arange(n, device=q.device, dtype=torch.int64) * bits
    words = torch.zeros(qv.shape[0], n * bits // 32 + 1, dtype=torch.int64, device=q.device)
    wi, sh = bitpos // 32, bitpos % 32
    lo = (qv << sh) & 0xFFFFFFFF
    hi = (qv << sh) >> 32
    words.scatter_add_(1, wi.expand_as(qv), lo)
    words.scatter_add_(1, (wi + 1).expand_as(qv), hi)
    words = words[:, :-1] & 0xFFFFFFFF
    # keep the bit pattern in an int32 tensor (torch has limited uint32 support)
    words = torch.where(words >= 2 ** 31, words - 2 ** 32, words).to(torch.int32)
    return words.reshape(*lead, n * bits // 32)


def unpack_bits(words: torch.Tensor, bits: int, n: int) -> torch.Tensor:
    *lead, nw = words.shape
    w = words.to(torch.int64).reshape(-1, nw) & 0xFFFFFFFF
    w = torch.cat([w, torch.zeros(w.shape[0], 1, dtype=torch.int64, device=w.device)], dim=1)
    bitpos = torch.arange(n, device=words.device, dtype=torch.int64) * bits
    wi, sh = bitpos // 32, bitpos % 32
    lo = w.gather(1, wi.expand(w.shape[0], n)) >> sh
    hi = w.gather(1, (wi + 1).expand(w.shape[0], n)) << (32 - sh)
    return ((lo | hi) & ((1 << bits) - 1)).reshape(*lead, n)


# ----------------------------------------------------------------------------- quantizers
def quantize_affine(w: torch.Tensor, bits: int = 4, group_size: int = 64,
                    dtype=torch.bfloat16) -> QuantizedTensor:
    """MLX affine quantization: per group, scale = (max - min) / (2^bits - 1), bias = min
    (with MLX's sign convention that keeps the larger-magnitude edge exact)."""
    *lead, out, inn = w.shape
    g = w.float().reshape(*lead, out, inn // group_size, group_size)
    wmax, wmin = g.amax(-1, keepdim=True), g.amin(-1, keepdim=True)
    nlev = float((1 << bits) - 1)
    # MLX keeps the group edge of larger magnitude exactly representable: the scale is negative
    # when that edge is the maximum (codes then count down from it).
    mask = wmin.abs() > wmax.abs()
    scale = ((wmax - wmin) / nlev).clamp_min(1e-7)
    scale = torch.where(mask, scale, -scale)
    edge = torch.where(mask, wmin, wmax)
    q0 = torch.round(edge / scale)
    scale = torch.where(q0 != 0, edge / q0, scale)
    bias = torch.where(q0 == 0, torch.zeros_like(edge), edge)
    scale = scale.to(dtype).float()
    bias = bias.to(dtype).float()
    q = torch.round((g - bias) / scale).clamp(0, nlev).to(torch.int64)
    packed = pack_bits(q.reshape(*lead, out, inn), bits)
    return QuantizedTensor(packed, scale.squeeze(-1).to(dtype), bias.squeeze(-1).to(dtype), bits,
                           group_size, "affine")


def quantize_mxfp4(w: torch.Tensor) -> QuantizedTensor:
    """e2m1 values with e8m0 = ceil-pow2(amax / 6) per 32 inputs."""
    *lead, out, inn = w.shape
    g = w.float().reshape(*lead, out, inn // 32, 32)
    amax = g.abs().amax(-1, keepdim=True).clamp_min(2.0 ** -126)
    e = torch.ceil(torch.log2(amax / 6.0)).clamp(-127, 127)
    scale = torch.pow(2.0, e)
    x = (g / scale).clamp(-6.0, 6.0)
    tab = _E2M1.to(w.device)
    idx = (x.abs().unsqueeze(-1) - tab).abs().argmin(-1)
    code = idx | ((x < 0).to(torch.int64) << 3)
    packed = pack_bits(code.reshape(*lead, out, inn), 4)
    s8 = (e + 127).to(torch.uint8).squeeze(-1)
    return QuantizedTensor(packed, s8, None, 4, 32, "mxfp4")


def quantize_nvfp4(w: torch.Tensor) -> QuantizedTensor:
    """e2m1 values with one e4m3 scale (amax / 6, rounded to fp8) per 16 inputs (MLX mode ``nvfp4``)."""
    *lead, out, inn = w.shape
    g = w.float().reshape(*lead, out, inn // 16, 16)
    s8 = (g.abs().amax(-1, keepdim=True) / 6.0).clamp(2.0 ** -9, 448.0).to(torch.float8_e4m3fn)
    x = (g / s8.float()).clamp(-6.0, 6.0)
    tab = _E2M1.to(w.device)
    idx = (x.abs().unsqueeze(-1) - tab).abs().argmin(-1)
    code = idx | ((x < 0).to(torch.int64) << 3)
    packed = pack_bits(code.reshape(*lead, out, inn), 4)
    return QuantizedTensor(packed, s8.view(torch.uint8).squeeze(-1), None, 4, 16, "nvfp4")


def quantize_mxfp8(w: torch.Tensor) -> QuantizedTensor:
    *lead, out, inn = w.shape
    g = w.float().reshape(*lead, out, inn // 32, 32)
    amax = g.abs().amax(-1, keepdim=True).clamp_min(2.0 ** -126)
    e = torch.ceil(torch.log2(amax / 448.0)).clamp(-127, 127)
    scale = torch.pow(2.0, e)
    x8 = (g / scale).clamp(-448.0, 448.0).to(torch.float8_e4m3fn)
    code = x8.view(torch.uint8).to(torch.int64)
    packed = pack_bits(code.reshape(*lead, out, inn), 8)
    s8 = (e + 127).to(torch.uint8).squeeze(-1)
    return QuantizedTensor(packed, s8, None, 8, 32, "mxfp8")


def quantize(w: torch.Tensor, mode: str = "affine", bits: int = 4, group_size: int = 64,
             dtype=torch.bfloat16) -> QuantizedTensor:
    if mode == "affine":
        return quantize_affine(w, bits, group_size, dtype)
    if mode == "mxfp4":
        return quantize_mxfp4(w)
    if mode == "mxfp8":
        return quantize_mxfp8(w)
    if mode == "nvfp4":
        return quantize_nvfp4(w)
    raise ValueError(mode)


def quantize_chunked(w: torch.Tensor, mode: str = "affine", bits: int = 4, group_size: int = 64,
                     max_elems: int = 1 << 24) -> QuantizedTensor:
    """:func:`quantize` over slices of the leading dimension, so that the integer temporaries of the
    packing stay small next to large (stacked-expert, vocabulary-sized) tensors."""
    lead = w.shape[0]
    per = max(1, w.numel() // max(lead, 1))
    step = max(1, max_elems // per)
    if step >= lead:
        return quantize(w, mode, bits, group_size, dtype=w.dtype if w.dtype != torch.float32 else torch.bfloat16)
    parts = [quantize(w[i:i + step], mode, bits, group_size,
                      dtype=w.dtype if w.dtype != torch.float32 else torch.bfloat16) for i in range(0, lead, step)]
    cat = lambda xs: torch.cat(xs, dim=0) if xs[0] is not None else None  # noqa: E731
    p0 = parts[0]
    return QuantizedTensor(cat([p.packed for p in parts]), cat([p.scales for p in parts]),
                           cat([p.biases for p in parts]), p0.bits, p0.group_size, p0.mode)


def quantize_model_weights(w, dense: tuple | None = None, experts: tuple | None = None, lm_head: bool = False):
    """Quantize a model's projections in place: ``dense`` = (mode, bits, group) for qkv / o / gate-up /
    down (and the LM head when ``lm_head``), ``experts`` = the same for the stacked expert matrices.
    Tensors whose input dimension is not a multiple of the group stay as they are. This is how the
    synthetic benchmark configurations get MLX-format packed weights out of random bf16 ones."""
    def q(v, spec):
        if v is None or spec is None or isinstance(v, QuantizedTensor) or v.shape[-1] % spec[2]:
            return v
        return quantize_chunked(v, *spec)

    for lw in w.layers:
        for name in ("wqkv", "wo", "w_gate_up", "w_down"):
            setattr(lw, name, q(getattr(lw, name), dense))
        for name in ("experts_gate_up", "experts_down"):
            setattr(lw, name, q(getattr(lw, name), experts))
        if torch.cuda.is_available():
            torch.cuda.empty_cache()
    if lm_head and dense is not None and w.lm_head is not w.embed:
        w.lm_head = q(w.lm_head, dense)
    return w


# ----------------------------------------------------------------------------- dequantize
def dequantize_ref(qt: QuantizedTensor, dtype=torch.float32) -> torch.Tensor:
    *lead, out, inn = qt.shape
    q = unpack_bits(qt.packed, qt.bits, inn)
    g = qt.group_size
    if qt.mode == "affine":
        v = q.float().reshape(*lead, out, inn // g, g) * qt.scales.float().unsqueeze(-1) + \
            qt.biases.float().unsqueeze(-1)
    else:
        if qt.mode == "nvfp4":                  # the scale byte is an e4m3 number, not an exponent
            sc = qt.scales.view(torch.float8_e4m3fn).float().unsqueeze(-1)
        else:
            sc = torch.pow(2.0, qt.scales.float() - 127.0).unsqueeze(-1)
        if qt.mode in ("mxfp4", "nvfp4"):
            tab = _E2M1.to(q.device)
            val = tab[(q & 7)] * torch.where((q & 8) != 0, -1.0, 1.0)
        else:
            val = q.to(torch.uint8).view(torch.float8_e4m3fn).float()
        v = val.reshape(*lead, out, inn // g, g) * sc
    return v.reshape(*lead, out, inn).to(dtype)


def dequantize(qt: QuantizedTensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """bf16 dequantization (CUDA kernel on device tensors)."""
    if not qt.packed.is_cuda:
        return dequantize_ref(qt, torch.bfloat16)
    *lead, n, inn = qt.shape
    rows = n
    for d in lead:
        rows *= d
    if out is None:
        out = torch.empty(*lead, n, inn, dtype=torch.bfloat16, device=qt.packed.device)
    lib = _lib.load()
    rc = lib.mx_dequantize(qt.packed.data_ptr(), qt.scales.data_ptr(), _lib.ptr(qt.biases),
                           out.data_ptr(), rows, inn, qt.bits, qt.group_size, _MODE_ID[qt.mode],
                           _lib.stream())
    _lib.count_launch()
    _lib.check(rc, "mx_dequantize")
    return out


# ----------------------------------------------------------------------------- linear
_TMP: dict = {}


_FUSED_WQ = {("affine", 4): 1, ("affine", 8): 2, ("mxfp4", 4): 3}
_FUSED_QGEMM = os.environ.get("MLXCEL_B200_FUSED_QGEMM", "1") != "0"
_QMV_MAX_M = int(os.environ.get("MLXCEL_B200_QMV_MAX_M", "1"))   # rows served by the GEMV kernel


def fused_wq(qt: QuantizedTensor, M: int, K: int) -> int:
    """Format code of the fused dequant GEMM for this tensor and batch, 0 when not covered."""
    if not _FUSED_QGEMM or M > 256 or K % 64 or qt.packed.dim() != 2:
        return 0
    if qt.group_size not in (32, 64, 128) or qt.group_size > K:
        return 0
    return _FUSED_WQ.get((qt.mode, qt.bits), 0)


def tile_for_gemm(qt: QuantizedTensor) -> torch.Tensor:
    """Re-tile a 2-D quantized matrix for the fused dequant GEMM (built once, cached on the tensor).

    The checkpoint keeps every output row's packed values contiguous ([N, K*bits/32] words); a
    128-row x 64-value MMA operand tile then consists of 128 pieces of 32 (4-bit) or 64 (8-bit)
    bytes, 2 KB or more apart, and its scales sit in yet another tensor. The kernel wants each
    (row tile, k-block) as ONE contiguous block that a single TMA box brings in:

        uint8 [T, K/64, 128 + E, W]    W = 64*bits/8 bytes per row, T = ceil(N / 128) (zero-padded)
        rows 0..127   packed values of the 128 weight rows
        rows 128..    scales [2 halves of the k-block][128 rows], then biases likewise (affine),
                      bf16 (affine) or e8m0 bytes (mxfp4)
    """
    cached = getattr(qt, "_gemm_tiles", None)
    if cached is not None:
        return cached
    N, K = qt.shape[-2], qt.shape[-1]
    bits, group = qt.bits, qt.group_size
    T, nkb, W = (N + 127) // 128, K // 64, 64 * bits // 8
    pad = T * 128 - N
    by = qt.packed.contiguous().view(torch.uint8).view(N, nkb, W)
    if pad:
        by = torch.cat([by, torch.zeros(pad, nkb, W, dtype=torch.uint8, device=by.device)], 0)
    vals = by.view(T, 128, nkb, W).permute(0, 2, 1, 3)                     # [T, nkb, 128, W]

    def per_half(v):   # [N, K/group] -> bytes [T, nkb, 2 * 128 * itemsize]
        halves = torch.arange(2 * nkb, device=v.device) * 32 // group      # group of every 32-value half
        e = v.index_select(1, halves)                                      # [N, 2*nkb]
        if pad:
            e = torch.cat([e, torch.zeros(pad, 2 * nkb, dtype=e.dtype, device=e.device)], 0)
        e = e.view(T, 128, nkb, 2).permute(0, 2, 3, 1).contiguous()        # [T, nkb, 2, 128]
        return e.view(torch.uint8).view(T, nkb, -1)

    extra = per_half(qt.scales)
    if qt.biases is not None:
        extra = torch.cat([extra, per_half(qt.biases)], dim=-1)
    assert extra.shape[-1] % W == 0
    tiles = torch.cat([vals, extra.view(T, nkb, -1, W)], dim=2).contiguous()
    qt._gemm_tiles = tiles
    return tiles


def tile_experts_for_gemm(qt: QuantizedTensor, glu_inter: int | None = None) -> torch.Tensor:
    """Stacked expert weights ``[E, N, K]`` (``N = 2 * glu_inter`` rows = gate then up when gated) in
    the block layout of ``tile_for_gemm``, per expert: the row tiles of the gate part followed by
    those of the up part (each part zero-padded to a multiple of 128 rows on its own, so that a gate
    tile and its up tile are a fixed number of tiles apart). Returns uint8
    ``[E, tiles_per_expert, K/64, rows, W]``; cached on the tensor."""
    cached = getattr(qt, "_gemm_tiles", None)
    if cached is not None:
        return cached
    E, N, K = qt.shape
    bits, group = qt.bits, qt.group_size
    nkb, W = K // 64, 64 * bits // 8
    parts = [(0, N)] if glu_inter is None else [(0, glu_inter), (glu_inter, 2 * glu_inter)]
    by = qt.packed.contiguous().view(torch.uint8).view(E, N, nkb, W)
    halves = torch.arange(2 * nkb, device=by.device) * 32 // group

    def half_bytes(v, r0, r1, pad):   # [E, N, K/group] -> [E, T, nkb, bytes]
        e = v[:, r0:r1].index_select(2, halves)
        if pad:
            e = torch.cat([e, torch.zeros(E, pad, 2 * nkb, dtype=e.dtype, device=e.device)], 1)
        T = e.shape[1] // 128
        e = e.view(E, T, 128, nkb, 2).permute(0, 1, 3, 4, 2).contiguous()      # [E, T, nkb, 2, 128]
        return e.view(torch.uint8).view(E, T, nkb, -1)

    out = []
    for r0, r1 in parts:
        n = r1 - r0
        T = (n + 127) // 128
        pad = T * 128 - n
        v = by[:, r0:r1]
        if pad:
            v = torch.cat([v, torch.zeros(E, pad, nkb, W, dtype=torch.uint8, device=by.device)], 1)
        vals = v.view(E, T, 128, nkb, W).permute(0, 1, 3, 2, 4)              # [E, T, nkb, 128, W]
        extra = half_bytes(qt.scales, r0, r1, pad)
        if qt.biases is not None:
            extra = torch.cat([extra, half_bytes(qt.biases, r0, r1, pad)], dim=-1)
        out.append(torch.cat([vals, extra.view(E, T, nkb, -1, W)], dim=3))
    tiles = torch.cat(out, dim=1).contiguous()
    qt._gemm_tiles = tiles
    return tiles


def quant_extras(qt: QuantizedTensor, wq: int, **kw):
    """(pointer to the re-tiled packed weights, extras describing them) for one GEMM call."""
    tiles = tile_for_gemm(qt)
    return tiles.data_ptr(), _lib.gemm_extras(wq=wq, q_group=qt.group_size, **kw)


def _fused_qgemm(x, qt, wq, out, bias, residual, inter=None, act=None, alpha=1.702, limit=7.0):
    """Packed weights straight into the tcgen05 GEMM (dequantised by its transform warps)."""
    from . import _ACT_TO_EPI, EPI_BIAS, EPI_NONE, EPI_RESIDUAL

    M, K = x.shape
    N = qt.shape[-2] if inter is None else inter
    if out is None:
        out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
    if inter is None:
        epi = EPI_RESIDUAL if residual is not None else (EPI_BIAS if bias is not None else EPI_NONE)
    else:
        epi = _ACT_TO_EPI[act]
    ws = _lib.workspace(x.device)
    lib = _lib.load()
    w_ptr, ex = quant_extras(qt, wq)
    rc = lib.mx_gemm_bf16(x.data_ptr(), w_ptr, out.data_ptr(), _lib.ptr(bias), _lib.ptr(residual), M, N, K,
                          x.stride(0), 0, out.stride(0),
                          residual.stride(0) if residual is not None else 0, epi, 0, inter or 0, float(alpha),
                          float(limit), ws.data_ptr(), ws.numel(), 0, 0, _lib.stream(), _lib.ref_or_null(ex))
    _lib.count_launch()
    _lib.check(rc, "mx_gemm_bf16 (packed weights)")
    return out


def qglu_linear(x: torch.Tensor, qt: QuantizedTensor, inter: int, act: str, bias=None, alpha=1.702,
                limit=7.0) -> torch.Tensor:
    """Gated projection over packed weights: one kernel (dequantise + two accumulators + activation)
    when the fused path covers the format, else quantized linear followed by the activation."""
    from . import swiglu

    M, K = x.shape
    if (x.is_cuda and _QGEMV4 and 0 < M <= 8 and qt.bits == 4 and qt.mode in ("affine", "mxfp4") and qt.packed.dim() == 2
            and K % 32 == 0 and x.is_contiguous() and (bias is None or bias.dtype == torch.bfloat16)):
        # decode-sized: gate and up rows streamed once, activation in the epilogue (one launch)
        from . import _ACT_TO_EPI
        out = torch.empty(M, inter, dtype=torch.bfloat16, device=x.device)
        rc = _lib.load().mx_moe_qgemv(x.data_ptr(), qt.packed.data_ptr(), qt.scales.data_ptr(), _lib.ptr(qt.biases),
                                      _lib.ptr(bias), _row_offsets(x.device, M).data_ptr(), out.data_ptr(), 1, inter, K,
                                      qt.group_size, 0 if qt.mode == "affine" else 1, _ACT_TO_EPI[act], float(alpha),
                                      float(limit), None, 0, 0, _lib.stream())
        if rc == 0:
            _lib.count_launch()
            return out
        if rc != -9:
            _lib.check(rc, "mx_moe_qgemv (dense, gated)")
    wq = fused_wq(qt, M, K) if x.is_cuda else 0
    if wq and x.stride(1) == 1 and M > 0 and inter % 128 == 0:   # gate / up start on tile boundaries
        return _fused_qgemm(x, qt, wq, None, bias, None, inter=inter, act=act, alpha=alpha, limit=limit)
    return swiglu(qlinear(x, qt, bias=bias), inter, act, alpha, limit)


# Dense use of the grouped half2 GEMV (one group of M rows). Off by default: measured at M = 1 on
# 6144 x 4096 it takes 29 us against 10.6 us for the one-warp-per-row GEMV (it pays for four token
# slots and for its staging pass); the grouped form is what wins for experts.
_QGEMV4 = os.environ.get("MLXCEL_B200_QGEMV4", "0") == "1"
_OFFSETS: dict = {}


def _row_offsets(device, M: int) -> torch.Tensor:
    """Device tensor [0, M]: the one-group offsets the grouped GEMV takes for a dense projection."""
    key = (device.index, M)
    t = _OFFSETS.get(key)
    if t is None:
        t = torch.tensor([0, M], dtype=torch.int32, device=device)
        _OFFSETS[key] = t
    return t


def qlinear(x: torch.Tensor, qt: QuantizedTensor, bias=None, residual=None, out=None) -> torch.Tensor:
    """``x @ dequant(w)^T (+ bias) (+ residual)``. M <= 8 rows stream the packed weights once
    through the GEMV kernel; up to 256 rows go to the tcgen05 GEMM whose transform warps dequantise
    the packed tiles in shared memory (weights are read once, at 4 or 8 bits); larger M dequantizes
    into a reused bf16 buffer and runs the dense GEMM (prefill is compute bound, so the extra pass
    is small there)."""
    from . import linear, reference as ref

    if not x.is_cuda:
        return ref.linear(x, dequantize_ref(qt), bias, residual)
    M, K = x.shape
    N = qt.shape[-2]
    lib = _lib.load()
    if (_QGEMV4 and 0 < M <= 8 and qt.bits == 4 and qt.mode in ("affine", "mxfp4") and qt.packed.dim() == 2 and K % 32 == 0
            and x.is_contiguous() and (bias is None or bias.dtype == torch.bfloat16)):
        # weight-streaming 4-bit GEMV (half2 arithmetic, activations in registers): the grouped
        # expert kernel with one group of M rows
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        rc = lib.mx_moe_qgemv(x.data_ptr(), qt.packed.data_ptr(), qt.scales.data_ptr(), _lib.ptr(qt.biases),
                              _lib.ptr(bias), _row_offsets(x.device, M).data_ptr(), out.data_ptr(), 1, N, K,
                              qt.group_size, 0 if qt.mode == "affine" else 1, 1 if bias is not None else 0, 0.0, 0.0,
                              _lib.ptr(residual), out.stride(0), residual.stride(0) if residual is not None else 0,
                              _lib.stream())
        if rc == 0:
            _lib.count_launch()
            return out
        if rc != -9:
            _lib.check(rc, "mx_moe_qgemv (dense)")
    if M > _QMV_MAX_M or qt.bits not in (4, 8):
        wq = fused_wq(qt, M, K)
        if wq and x.stride(1) == 1 and M > 0:
            return _fused_qgemm(x, qt, wq, out, bias, residual)
    if M <= 8 and qt.bits in (4, 8):
        if out is None:
            out = torch.empty(M, N, dtype=torch.bfloat16, device=x.device)
        rc = lib.mx_qmv(x.data_ptr(), qt.packed.data_ptr(), qt.scales.data_ptr(), _lib.ptr(qt.biases),
                        out.data_ptr(), _lib.ptr(residual), _lib.ptr(bias), M, N, K, qt.bits,
                        qt.group_size, _MODE_ID[qt.mode], x.stride(0), out.stride(0), _lib.stream())
        if rc == 0:
            _lib.count_launch()
            return out
        if rc != -9:
            _lib.check(rc, "mx_qmv")
    key = (x.device.index, N, K)
    tmp = _TMP.get(key)
    if tmp is None:
        tmp = torch.empty(N, K, dtype=torch.bfloat16, device=x.device)
        _TMP[key] = tmp
    dequantize(qt, tmp)
    return linear(x, tmp, bias=bias, residual=residual, out=out)
