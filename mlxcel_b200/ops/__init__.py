"""Operator layer.

Every function takes torch tensors. CUDA tensors run the hand-written sm_100a kernels of
``lib/libmlxcel_b200.so`` (and raise when that library is missing); CPU tensors run the plain
PyTorch statements in :mod:`mlxcel_b200.ops.reference`, which are also the test oracles.
"""
from __future__ import annotations

import os

from dataclasses import dataclass

import torch

from . import _lib, reference as ref
from .reference import (EPI_BIAS, EPI_CLIPPED_SWIGLU, EPI_GEGLU, EPI_NONE, EPI_RESIDUAL,  # noqa: F401
                        EPI_SWIGLU)

_ACT_TO_EPI = {"silu": EPI_SWIGLU, "gelu_tanh": EPI_GEGLU, "clipped_swiglu": EPI_CLIPPED_SWIGLU}


@dataclass
class KVLayer:
    """One layer's slice of the paged KV pool: ``[num_blocks, Hkv, block_size, D]``."""

    k: torch.Tensor
    v: torch.Tensor
    k_meta: torch.Tensor | None
    v_meta: torch.Tensor | None
    block_size: int
    kv_bits: int = 16


def _lib_call(name: str, *args) -> None:
    lib = _lib.load()
    rc = getattr(lib, name)(*args)
    _lib.count_launch()
    _lib.check(rc, name)


# ----------------------------------------------------------------------------- deferred RMSNorm
class SsqBuffer:
    """Per-token partial sums of squares of a residual stream, left by the kernel that produced it
    (a GEMM epilogue or ``row_ssq``) for the GEMM that consumes it un-normalised.
    fp32 words: [0] partial count (device-written), [1] row stride, data from word 8."""

    def __init__(self, max_tokens: int, max_parts: int, device):
        self.max_tokens, self.max_parts = max_tokens, max_parts
        self.buf = torch.zeros(8 + max_parts * max_tokens, dtype=torch.float32, device=device)
        self.buf[:2].view(torch.int32).copy_(torch.tensor([0, max_tokens], dtype=torch.int32))

    def fits(self, tokens: int, features: int) -> bool:
        return tokens <= self.max_tokens and (features + 127) // 128 <= self.max_parts


@dataclass
class RowNorm:
    ssq: SsqBuffer
    eps: float
    dim: int      # length of the normalised rows (the GEMM's K when nothing is sharded)


def row_ssq(x: torch.Tensor, ssq: SsqBuffer) -> None:
    """Starts a deferred-RMSNorm chain: sums of squares of the rows of ``x`` (one partial)."""
    rows, dim = x.shape
    assert x.is_cuda and x.stride(1) == 1 and rows <= ssq.max_tokens
    _lib_call("mx_row_ssq", x.data_ptr(), rows, dim, x.stride(0), ssq.buf.data_ptr(), _lib.stream())


# ----------------------------------------------------------------------------- GEMM
def linear(x: torch.Tensor, w: torch.Tensor, bias: torch.Tensor | None = None,
           residual: torch.Tensor | None = None, out: torch.Tensor | None = None,
           out_fp32: bool = False, force_mode: int = 0, force_splits: int = 0,
           row_norm: "RowNorm | None" = None, ssq_out: "SsqBuffer | None" = None) -> torch.Tensor:
    """``x[M,K] @ w[N,K]^T (+ bias) (+ residual)`` with bf16 operands, fp32 accumulation.

    ``row_norm``: deferred RMSNorm — ``x`` is un-normalised, the norm weight is folded into ``w`` and
    every output row is scaled by the 1/rms described by ``row_norm.ssq`` before the bias.
    ``ssq_out``: the kernel also leaves the per-tile sums of squares of its result rows there."""
    if not x.is_cuda:
        assert row_norm is None and ssq_out is None, "deferred RMSNorm is a CUDA-only path"
        return ref.linear(x, w, bias, residual, torch.float32 if out_fp32 else None)
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    M, K = x.shape
    N = w.shape[0]
    assert x.stride(1) == 1 and w.stride(1) == 1 and w.shape[1] == K
    if out is None:
        out = torch.empty(M, N, dtype=torch.float32 if out_fp32 else torch.bfloat16, device=x.device)
    if M == 0:
        return out
    epi = EPI_RESIDUAL if residual is not None else (EPI_BIAS if bias is not None else EPI_NONE)
    ws = _lib.workspace(x.device)
    ex = _lib.gemm_extras(row_norm=row_norm, ssq_out=ssq_out)
    _lib_call("mx_gemm_bf16", x.data_ptr(), w.data_ptr(), out.data_ptr(), _lib.ptr(bias),
              _lib.ptr(residual), M, N, K, x.stride(0), w.stride(0), out.stride(0),
              residual.stride(0) if residual is not None else 0, epi, 1 if out_fp32 else 0, 0,
              0.0, 0.0, ws.data_ptr(), ws.numel(), force_mode, force_splits, _lib.stream(),
              _lib.ref_or_null(ex))
    return out


def glu_linear(x: torch.Tensor, w: torch.Tensor, inter: int, act: str = "silu",
               bias: torch.Tensor | None = None, alpha: float = 1.702, limit: float = 7.0,
               out: torch.Tensor | None = None, force_mode: int = 0,
               force_splits: int = 0, row_norm: "RowNorm | None" = None) -> torch.Tensor:
    """``act(x @ w[:I]^T) * (x @ w[I:2I]^T)`` — gate/up projection with the activation fused
    into the GEMM epilogue (gate and up live in two TMEM accumulators)."""
    epi = _ACT_TO_EPI[act]
    if not x.is_cuda:
        return ref.glu_linear(x, w, inter, epi, bias, alpha, limit)
    M, K = x.shape
    assert w.shape[0] == 2 * inter and x.stride(1) == 1 and w.stride(1) == 1
    if out is None:
        out = torch.empty(M, inter, dtype=torch.bfloat16, device=x.device)
    if M == 0:
        return out
    ws = _lib.workspace(x.device)
    ex = _lib.gemm_extras(row_norm=row_norm)
    _lib_call("mx_gemm_bf16", x.data_ptr(), w.data_ptr(), out.data_ptr(), _lib.ptr(bias), None, M,
              inter, K, x.stride(0), w.stride(0), out.stride(0), 0, epi, 0, inter, float(alpha),
              float(limit), ws.data_ptr(), ws.numel(), force_mode, force_splits, _lib.stream(),
              _lib.ref_or_null(ex))
    return out


# ----------------------------------------------------------------------------- norms
def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor | None, weight: torch.Tensor, eps: float,
                w_bias: float = 0.0) -> tuple[torch.Tensor, torch.Tensor]:
    """``h = x + residual; y = rmsnorm(h) * (weight + w_bias)`` → ``(y, h)``.
    With ``residual=None`` the new residual is ``x`` itself."""
    if not x.is_cuda:
        return ref.add_rmsnorm(x, residual, weight, eps, w_bias)
    rows, dim = x.shape
    y = torch.empty_like(x)
    if residual is None:
        _lib_call("mx_add_rmsnorm", x.data_ptr(), None, weight.data_ptr(), y.data_ptr(), None, rows,
                  dim, float(eps), float(w_bias), _lib.stream())
        return y, x
    h = torch.empty_like(x)
    _lib_call("mx_add_rmsnorm", x.data_ptr(), residual.data_ptr(), weight.data_ptr(), y.data_ptr(),
              h.data_ptr(), rows, dim, float(eps), float(w_bias), _lib.stream())
    return y, h


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, w_bias: float = 0.0) -> torch.Tensor:
    return add_rmsnorm(x, None, weight, eps, w_bias)[0]


# ----------------------------------------------------------------------------- rope + append
def rope_append(qkv: torch.Tensor, positions: torch.Tensor, slot_mapping: torch.Tensor,
                inv_freq: torch.Tensor, kv: KVLayer, *, Hq: int, Hkv: int, D: int, rot_dim: int,
                traditional: bool = False, mscale: float = 1.0, q_norm_w=None, k_norm_w=None,
                norm_eps: float = 1e-6) -> None:
    """RoPE on q (in place in ``qkv``) and k, then append k/v rows into the paged pool."""
    if not qkv.is_cuda:
        return ref.rope_append(qkv, positions, slot_mapping, inv_freq, kv, Hq=Hq, Hkv=Hkv, D=D,
                               rot_dim=rot_dim, traditional=traditional, mscale=mscale,
                               q_norm_w=q_norm_w, k_norm_w=k_norm_w, norm_eps=norm_eps)
    T = qkv.shape[0]
    assert qkv.is_contiguous() and positions.dtype == torch.int32 and slot_mapping.dtype == torch.int32
    _lib_call("mx_rope_append", qkv.data_ptr(), positions.data_ptr(), slot_mapping.data_ptr(),
              inv_freq.data_ptr(), kv.k.data_ptr(), kv.v.data_ptr(), _lib.ptr(kv.k_meta),
              _lib.ptr(kv.v_meta), _lib.ptr(q_norm_w), _lib.ptr(k_norm_w), float(norm_eps), T, Hq,
              Hkv, D, rot_dim, kv.block_size, 1 if traditional else 0, float(mscale), kv.kv_bits,
              _lib.stream())


# ----------------------------------------------------------------------------- attention
_DEC_SCRATCH: dict[int, torch.Tensor] = {}


def _decode_scratch(device: torch.device, floats: int) -> torch.Tensor:
    idx = device.index if device.index is not None else torch.cuda.current_device()
    s = _DEC_SCRATCH.get(idx)
    if s is None or s.numel() < floats:
        s = torch.zeros(max(floats, 1 << 22), dtype=torch.float32, device=device)
        _DEC_SCRATCH[idx] = s
    return s


def decode_splits(B: int, Hkv: int, max_len: int, sms: int = 148) -> int:
    """KV splits per (sequence, kv head). Two 4-warp CTAs are resident per SM; when the
    (sequence, kv head) pairs alone fill the SMs a split only adds merge traffic."""
    pairs = max(1, B * Hkv)
    if pairs >= sms:
        return 1
    s = -(-2 * sms // pairs)
    return max(1, min(s, max(1, max_len // 256), 16))


def paged_decode(q: torch.Tensor, kv: KVLayer, block_tables: torch.Tensor,
                 context_lens: torch.Tensor, *, Hq: int, Hkv: int, D: int, scale: float,
                 window: int = 0, sinks: torch.Tensor | None = None, softcap: float = 0.0,
                 num_splits: int = 0, max_len: int = 0, out: torch.Tensor | None = None) -> torch.Tensor:
    """One query row per sequence. ``q`` may be a strided view (rows of the fused qkv buffer)."""
    B = q.shape[0]
    if not q.is_cuda:
        cu = torch.arange(B + 1, dtype=torch.int32)
        return ref.paged_attention(q, kv, block_tables, context_lens, cu, Hq=Hq, Hkv=Hkv, D=D,
                                   scale=scale, window=window, sinks=sinks, softcap=softcap)
    if out is None:
        out = torch.empty(B, Hq * D, dtype=torch.bfloat16, device=q.device)
    if B == 0:
        return out
    if num_splits <= 0:
        num_splits = decode_splits(B, Hkv, max_len or block_tables.shape[1] * kv.block_size)
    lib = _lib.load()
    floats = int(lib.mx_paged_decode_scratch_floats(B, Hq, D, num_splits))
    scratch = _decode_scratch(q.device, floats)
    _lib_call("mx_paged_decode", q.data_ptr(), q.stride(0), kv.k.data_ptr(), kv.v.data_ptr(),
              _lib.ptr(kv.k_meta), _lib.ptr(kv.v_meta), block_tables.data_ptr(),
              context_lens.data_ptr(), _lib.ptr(sinks), out.data_ptr(), scratch.data_ptr(), B, Hq,
              Hkv, D, kv.block_size, block_tables.shape[1], window, float(scale), float(softcap),
              kv.kv_bits, num_splits, _lib.stream())
    return out


_PREFILL_TC = os.environ.get("MLXCEL_B200_PREFILL_TC", "1") != "0"


def paged_prefill(q: torch.Tensor, kv: KVLayer, block_tables: torch.Tensor, cu_q: torch.Tensor,
                  context_lens: torch.Tensor, *, Hq: int, Hkv: int, D: int, scale: float,
                  max_q_len: int, window: int = 0, sinks: torch.Tensor | None = None,
                  softcap: float = 0.0, out: torch.Tensor | None = None) -> torch.Tensor:
    """Causal attention of query chunks against their sequences' paged KV (prefix + chunk)."""
    T = q.shape[0]
    if not q.is_cuda:
        return ref.paged_attention(q, kv, block_tables, context_lens, cu_q, Hq=Hq, Hkv=Hkv, D=D,
                                   scale=scale, window=window, sinks=sinks, softcap=softcap)
    if out is None:
        out = torch.empty(T, Hq * D, dtype=torch.bfloat16, device=q.device)
    if T == 0:
        return out
    S = context_lens.shape[0]
    if (_PREFILL_TC and kv.kv_bits == 16 and kv.block_size == 16 and D in (64, 128) and softcap == 0.0
            and kv.k.dtype == torch.bfloat16 and q.stride(0) % 8 == 0):
        # tensor-core (tcgen05) kernel; -10 = configuration not covered, fall through
        lib = _lib.load()
        ws = _lib.workspace(q.device)
        rc = lib.mx_paged_prefill_tc(q.data_ptr(), q.stride(0), kv.k.data_ptr(), kv.v.data_ptr(), kv.k.shape[0],
                                     block_tables.data_ptr(), cu_q.data_ptr(), context_lens.data_ptr(),
                                     _lib.ptr(sinks), out.data_ptr(), S, T, max_q_len, Hq, Hkv, D, kv.block_size,
                                     block_tables.shape[1], window, float(scale), ws.data_ptr(), _lib.stream())
        if rc != -10:
            _lib.count_launch()
            _lib.check(rc, "mx_paged_prefill_tc")
            return out
    _lib_call("mx_paged_prefill", q.data_ptr(), q.stride(0), kv.k.data_ptr(), kv.v.data_ptr(),
              _lib.ptr(kv.k_meta), _lib.ptr(kv.v_meta), block_tables.data_ptr(), cu_q.data_ptr(),
              context_lens.data_ptr(), _lib.ptr(sinks), out.data_ptr(), S, T, max_q_len, Hq, Hkv, D,
              kv.block_size, block_tables.shape[1], window, float(scale), float(softcap),
              kv.kv_bits, _lib.stream())
    return out


# ----------------------------------------------------------------------------- misc
def embedding(ids: torch.Tensor, table: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    if not table.is_cuda:
        return ref.embedding(ids, table, scale)
    T = ids.shape[0]
    out = torch.empty(T, table.shape[1], dtype=table.dtype, device=table.device)
    if T:
        _lib_call("mx_embedding", ids.data_ptr(), table.data_ptr(), out.data_ptr(), T,
                  table.shape[1], table.shape[0], float(scale), _lib.stream())
    return out


def swiglu(gate_up: torch.Tensor, inter: int, act: str = "silu", alpha: float = 1.702,
           limit: float = 7.0) -> torch.Tensor:
    """Gated activation on a fused ``[T, 2I]`` tensor (gate columns first) → ``[T, I]``."""
    if not gate_up.is_cuda:
        return ref.glu_act(_ACT_TO_EPI[act], gate_up[:, :inter].float(), gate_up[:, inter:].float(),
                           alpha, limit).to(gate_up.dtype)
    T = gate_up.shape[0]
    out = torch.empty(T, inter, dtype=gate_up.dtype, device=gate_up.device)
    if T:
        mode = {"silu": 0, "gelu_tanh": 1, "clipped_swiglu": 2}[act]
        _lib_call("mx_swiglu", gate_up.data_ptr(), out.data_ptr(), T, inter, mode, float(alpha),
                  float(limit), _lib.stream())
    return out


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    if not logits.is_cuda:
        return ref.argmax(logits)
    B, V = logits.shape
    if out is None:
        out = torch.empty(B, dtype=torch.int32, device=logits.device)
    if B:
        _lib_call("mx_argmax", logits.data_ptr(), 1 if logits.dtype == torch.float32 else 0,
                  logits.stride(0), out.data_ptr(), B, V, _lib.stream())
    return out


def sample(logits: torch.Tensor, temperature: torch.Tensor, top_k: torch.Tensor,
           top_p: torch.Tensor, min_p: torch.Tensor, seeds: torch.Tensor,
           steps: torch.Tensor, typical_p: torch.Tensor | None = None,
           top_n_sigma: torch.Tensor | None = None) -> tuple[torch.Tensor, torch.Tensor]:
    """Fused filter + Gumbel-max draw. Per-row parameter tensors live on the logits' device:
    temperature/top_p/min_p/typical_p/top_n_sigma fp32, top_k int32, seeds/steps int64 (read as uint64)."""
    if not logits.is_cuda:
        return ref.sample(logits, temperature, top_k, top_p, min_p, seeds, steps, typical_p, top_n_sigma)
    B, V = logits.shape
    toks = torch.empty(B, dtype=torch.int32, device=logits.device)
    lps = torch.empty(B, dtype=torch.float32, device=logits.device)
    if B:
        _lib_call("mx_sample", logits.data_ptr(), 1 if logits.dtype == torch.float32 else 0,
                  logits.stride(0), temperature.data_ptr(), top_k.data_ptr(), top_p.data_ptr(),
                  min_p.data_ptr(), _lib.ptr(typical_p), _lib.ptr(top_n_sigma), seeds.data_ptr(),
                  steps.data_ptr(), toks.data_ptr(), lps.data_ptr(), B, V, _lib.stream())
    return toks, lps


def apply_penalties(logits: torch.Tensor, history: torch.Tensor, rep: torch.Tensor,
                    freq: torch.Tensor, pres: torch.Tensor) -> torch.Tensor:
    """Repetition / frequency / presence penalties, in place on CUDA."""
    if not logits.is_cuda:
        return ref.apply_penalties(logits, history, rep, freq, pres)
    B, V = logits.shape
    _lib_call("mx_apply_penalties", logits.data_ptr(), 1 if logits.dtype == torch.float32 else 0,
              logits.stride(0), history.data_ptr(), history.shape[1], rep.data_ptr(),
              freq.data_ptr(), pres.data_ptr(), B, V, _lib.stream())
    return logits


def spec_verify(logits: torch.Tensor, draft: torch.Tensor):
    """logits [B, K, V], draft [B, K-1] int32 → (target [B,K], accept_len [B], next_token [B])."""
    if not logits.is_cuda:
        return ref.spec_verify(logits, draft)
    B, K, V = logits.shape
    flat = logits.reshape(B * K, V)
    target = torch.empty(B, K, dtype=torch.int32, device=logits.device)
    acc = torch.empty(B, dtype=torch.int32, device=logits.device)
    nxt = torch.empty(B, dtype=torch.int32, device=logits.device)
    _lib_call("mx_spec_verify", flat.data_ptr(), 1 if logits.dtype == torch.float32 else 0,
              flat.stride(0), draft.data_ptr(), target.data_ptr(), acc.data_ptr(), nxt.data_ptr(),
              B, K, V, _lib.stream())
    _lib.count_launch()
    return target, acc, nxt
