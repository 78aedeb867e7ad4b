"""Mixture-of-experts operators: routing, token permutation, grouped expert GEMMs, combine.

CUDA tensors run ``csrc/moe.cu`` + the grouped mode of the tcgen05 GEMM (``csrc/gemm.cu``);
CPU tensors run the plain PyTorch statements below (also the test oracles).
Reference behaviour: src/models/switch_layers.rs:98-220,2180-2250 and
src/models/gpt_oss.rs:402-446 of the reference.
"""
from __future__ import annotations

import os

import torch

from . import _lib, reference as ref
from . import _ACT_TO_EPI


# ----------------------------------------------------------------------------- reference
def route_ref(logits: torch.Tensor, k: int, mode: str, norm_topk: bool):
    lg = torch.nan_to_num(logits.float(), nan=float("-inf"))
    if mode == "softmax_topk":
        p = torch.softmax(lg, -1)
        w, ids = torch.topk(p, k, dim=-1)
        if norm_topk:
            w = w / w.sum(-1, keepdim=True)
    else:
        v, ids = torch.topk(lg, k, dim=-1)
        w = torch.softmax(v, -1)
    return ids.to(torch.int32), w.float()


def moe_ref(x, ids, wts, w_gate_up, w_down, inter, act, b_gate_up=None, b_down=None,
            e_begin=0, alpha=1.702, limit=7.0, dequant=None, gated=True):
    """Dense statement: for every (token, slot) routed to a local expert, run that expert's
    gated MLP (plain ``down(act(up x))`` when ``gated`` is false; ``w_gate_up`` then holds the up rows
    only) and accumulate the weighted result in fp32. Returns fp32 [T, H]."""
    T, H = x.shape
    El = w_gate_up.shape[0]
    out = torch.zeros(T, w_down.shape[1], dtype=torch.float32, device=x.device)
    epi = _ACT_TO_EPI[act] if gated else None
    for el in range(El):
        e = e_begin + el
        tok, slot = torch.nonzero(ids == e, as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x[tok].float()
        gu = xe @ w_gate_up[el].float().t()
        if b_gate_up is not None:
            gu = gu + b_gate_up[el].float()
        if gated:
            a = ref.glu_act(epi, gu[:, :inter], gu[:, inter:2 * inter], alpha, limit).to(x.dtype).float()
        else:
            from . import recurrent as rops
            a = rops.activation(gu.to(x.dtype), act).float()
        y = a @ w_down[el].float().t()
        if b_down is not None:
            y = y + b_down[el].float()
        y = y.to(x.dtype).float()
        out.index_add_(0, tok, y * wts[tok, slot].unsqueeze(-1))
    return out


def route_sigmoid_grouped(logits: torch.Tensor, k: int, bias: torch.Tensor | None, n_group: int, topk_group: int,
                          norm_topk: bool, scale: float, score: str = "sigmoid", norm_min: float = 1e-20,
                          group_score: str = "top2sum"):
    """DeepSeek-V3-style routing (GLM-4-MoE, dots1, ...): sigmoid scores; experts are CHOSEN by
    score + correction bias, restricted to the ``topk_group`` groups with the best sum of their two
    top biased scores, but WEIGHTED by the unbiased score (normalised over the k, times ``scale``).
    ``score="softmax"`` is the ERNIE-4.5-MoE variant (softmax probabilities, the same selection bias).
    Plain tensor ops on the small [T, E] matrix (reference src/models/switch_layers.rs group-limited
    routing masks). Returns (ids int32 [T, k], weights fp32 [T, k])."""
    T, E = logits.shape
    scores = torch.sigmoid(logits.float()) if score == "sigmoid" else torch.softmax(logits.float(), dim=-1)
    choice = scores if bias is None else scores + bias.float().reshape(1, E)
    if n_group > 1:
        grp = choice.view(T, n_group, E // n_group)
        # a group is ranked by the sum of its two best scores (V3) or by its best score (V2)
        gscore = grp.topk(min(2, E // n_group), dim=-1)[0].sum(-1) if group_score == "top2sum" else grp.amax(-1)
        keep = torch.zeros_like(gscore).scatter_(1, gscore.topk(topk_group, dim=-1)[1], 1.0)
        choice = choice.masked_fill(~keep.bool().unsqueeze(-1).expand(T, n_group, E // n_group).reshape(T, E), 0.0)
    ids = choice.topk(k, dim=-1)[1]
    w = scores.gather(1, ids)
    if norm_topk:
        w = w / (w.sum(-1, keepdim=True) + norm_min if score == "sigmoid" else w.sum(-1, keepdim=True).clamp(min=norm_min))
    return ids.to(torch.int32).contiguous(), (w * scale).contiguous()


def route_sparsemixer(logits: torch.Tensor, jitter_eps: float = 0.01):
    """Phi-MoE's inference-time SparseMixer (top-2): the first expert is the arg-max; its weight is its
    softmax probability among the experts whose logit lies within a relative margin ``2 * jitter_eps``
    of the maximum. The second expert and its weight come from the same rule with the first expert
    removed. Weights are not renormalised. Plain tensor ops on [T, E]
    (reference src/models/phimoe.rs). Returns (ids int32 [T, 2], weights fp32 [T, 2])."""
    s = logits.float()
    ids, ws = [], []
    for _ in range(2):
        top, idx = s.max(dim=-1, keepdim=True)
        factor = logits.float().abs().clamp(min=top)
        masked = s.masked_fill(((top - logits.float()) / factor) > 2 * jitter_eps, float("-inf"))
        ws.append(torch.softmax(masked, dim=-1).gather(-1, idx))
        ids.append(idx)
        s = s.scatter(-1, idx, float("-inf"))
    return torch.cat(ids, -1).to(torch.int32).contiguous(), torch.cat(ws, -1).contiguous()


# ----------------------------------------------------------------------------- CUDA
def route(logits: torch.Tensor, k: int, mode: str = "topk_softmax", norm_topk: bool = True):
    """Router logits [T, E] → (expert ids [T, k] int32, weights [T, k] fp32)."""
    if not logits.is_cuda:
        return route_ref(logits, k, mode, norm_topk)
    T, E = logits.shape
    ids = torch.empty(T, k, dtype=torch.int32, device=logits.device)
    wts = torch.empty(T, k, dtype=torch.float32, device=logits.device)
    lib = _lib.load()
    rc = lib.mx_moe_route(logits.contiguous().data_ptr(), ids.data_ptr(), wts.data_ptr(), T, E, k,
                          0 if mode == "softmax_topk" else 1, 1 if norm_topk else 0, _lib.stream())
    _lib.count_launch()
    _lib.check(rc, "mx_moe_route")
    return ids, wts


_QGEMV_MAX_ROWS = int(os.environ.get("MLXCEL_B200_MOE_QGEMV_MAX_ROWS", "16"))
# From this many rows per expert (on average) packed 4-bit experts are expanded to bf16 once and run
# through the dense grouped GEMM: the expansion is one pass over the layer's experts at memory speed,
# cheaper than unpacking every tile again inside the GEMM (measured on the gpt-oss-120b block:
# 3.5 ms against 7.6 ms at 2048 rows, 5.1 ms at 8192 rows). Below the streaming kernel's range
# nothing is left for the GEMM with unpack warps, so the default sends everything else here.
_DEQUANT_MIN_ROWS = int(os.environ.get("MLXCEL_B200_MOE_DEQUANT_MIN_ROWS", "1"))


def grouped_linear(xs: torch.Tensor, w: torch.Tensor, offsets: torch.Tensor, n_out: int,
                   bias: torch.Tensor | None = None, act: str | None = None, alpha: float = 1.702,
                   limit: float = 7.0, out: torch.Tensor | None = None, rows_hint: int | None = None) -> torch.Tensor:
    """Rows [offsets[e], offsets[e+1]) of ``xs`` times expert e's matrix ``w[e]``. With ``act``
    the expert matrices hold gate rows then up rows and the gated activation is fused.
    ``rows_hint``: how many of the rows are expected to be in use (defaults to all of them); packed
    4-bit experts with at most ``MLXCEL_B200_MOE_QGEMV_MAX_ROWS`` rows per expert on average take the
    weight-streaming grouped GEMV instead of the tensor-core GEMM."""
    from ..models.weights import QuantizedTensor
    from . import quant

    rows, K = xs.shape
    E = w.shape[0]
    if out is None:
        out = torch.empty(rows, n_out, dtype=torch.bfloat16, device=xs.device)
    epi = _ACT_TO_EPI[act] if act else (1 if bias is not None else 0)
    ws = _lib.workspace(xs.device)
    lib = _lib.load()
    if isinstance(w, QuantizedTensor):
        # Packed expert weights go straight into the grouped tcgen05 GEMM (unpacked by its transform
        # warps) when few rows are routed to each expert; only experts that received tokens are
        # read, at 4 bits per weight. Otherwise: dequantise all experts, dense grouped GEMM.
        wq = {("affine", 4): 1, ("mxfp4", 4): 3}.get((w.mode, w.bits), 0)
        used = rows if rows_hint is None else min(rows, rows_hint)
        if (wq and _QGEMV_MAX_ROWS > 0 and used <= _QGEMV_MAX_ROWS * E and w.packed.dim() == 3 and K % 32 == 0
                and (bias is None or bias.dtype == torch.bfloat16)):
            epi_gv = _ACT_TO_EPI[act] if act else (1 if bias is not None else 0)
            rc = lib.mx_moe_qgemv(xs.data_ptr(), w.packed.data_ptr(), w.scales.data_ptr(), _lib.ptr(w.biases),
                                  _lib.ptr(bias), offsets.data_ptr(), out.data_ptr(), E, n_out, K, w.group_size,
                                  0 if w.mode == "affine" else 1, epi_gv, float(alpha), float(limit), None, 0, 0,
                                  _lib.stream())
            if rc != -9:
                _lib.count_launch()
                _lib.check(rc, "mx_moe_qgemv")
                return out
        expand = _DEQUANT_MIN_ROWS > 0 and used >= _DEQUANT_MIN_ROWS * E
        if wq and quant._FUSED_QGEMM and not expand and K % 64 == 0 and w.group_size in (32, 64, 128):
            tiles = quant.tile_experts_for_gemm(w, n_out if act else None)
            ex = _lib.gemm_extras(wq=wq, q_group=w.group_size)
            rc = lib.mx_grouped_gemm_bf16(xs.data_ptr(), tiles.data_ptr(), out.data_ptr(), _lib.ptr(bias),
                                          offsets.data_ptr(), E, n_out, K, rows, epi, n_out if act else 0,
                                          float(alpha), float(limit), ws.data_ptr(), ws.numel(), _lib.stream(),
                                          _lib.ref_or_null(ex))
            if rc != -9:
                _lib.count_launch()
                _lib.check(rc, "mx_grouped_gemm_bf16 (packed experts)")
                return out
        w = quant.dequantize(w)
    rc = lib.mx_grouped_gemm_bf16(xs.data_ptr(), w.data_ptr(), out.data_ptr(), _lib.ptr(bias),
                                  offsets.data_ptr(), E, n_out, K, rows, epi, n_out if act else 0,
                                  float(alpha), float(limit), ws.data_ptr(), ws.numel(), _lib.stream(), None)
    _lib.count_launch()
    _lib.check(rc, "mx_grouped_gemm_bf16")
    return out


def moe_experts(x: torch.Tensor, ids: torch.Tensor, wts: torch.Tensor, w_gate_up, w_down, inter: int,
                act: str, b_gate_up=None, b_down=None, e_begin: int = 0, residual=None,
                alpha: float = 1.702, limit: float = 7.0, out: torch.Tensor | None = None,
                gated: bool = True, rows_hint: int | None = None) -> torch.Tensor:
    """Weighted sum over the LOCAL experts [e_begin, e_begin + E_local) of their gated MLPs (plain
    ``down(act(up x))`` experts when ``gated`` is false: grouped GEMM, activation kernel, grouped GEMM),
    plus ``residual`` when given. Returns bf16 [T, H] (written into ``out`` when given; rows whose
    experts are all elsewhere come out as the residual, or zero)."""
    T, H = x.shape
    k = ids.shape[1]
    El = w_gate_up.shape[0]
    if not x.is_cuda:
        from ..models.weights import QuantizedTensor
        from . import quant
        if isinstance(w_gate_up, QuantizedTensor):
            w_gate_up = quant.dequantize_ref(w_gate_up)
        if isinstance(w_down, QuantizedTensor):
            w_down = quant.dequantize_ref(w_down)
        o = moe_ref(x, ids, wts, w_gate_up, w_down, inter, act, b_gate_up, b_down, e_begin, alpha, limit, gated=gated)
        if residual is not None:
            o = o + residual.float()
        if out is not None:
            out.copy_(o.to(out.dtype))
            return out
        return o.to(x.dtype)
    dev = x.device
    lib = _lib.load()
    st = _lib.stream()
    pairs = T * k
    offsets = torch.empty(El + 1, dtype=torch.int32, device=dev)
    sorted_pair = torch.empty(pairs, dtype=torch.int32, device=dev)
    sorted_token = torch.empty(pairs, dtype=torch.int32, device=dev)
    rc = lib.mx_moe_align(ids.data_ptr(), offsets.data_ptr(), sorted_pair.data_ptr(),
                          sorted_token.data_ptr(), T, k, 0, e_begin, e_begin + El, st)
    _lib.check(rc, "mx_moe_align")
    total = offsets[El:]
    xs = torch.empty(pairs, H, dtype=x.dtype, device=dev)
    rc = lib.mx_moe_gather_rows_n(x.data_ptr(), sorted_token.data_ptr(), total.data_ptr(), xs.data_ptr(),
                                  pairs, H, st)
    _lib.check(rc, "mx_moe_gather_rows_n")
    _lib.count_launch(2)
    if gated:
        a = grouped_linear(xs, w_gate_up, offsets, inter, b_gate_up, act, alpha, limit, rows_hint=rows_hint)
    else:
        from . import recurrent as rops
        a = rops.activation(grouped_linear(xs, w_gate_up, offsets, inter, b_gate_up, None), act)
    y = grouped_linear(a, w_down, offsets, w_down.shape[1], b_down, None, rows_hint=rows_hint)
    if out is None:
        out = torch.empty(T, w_down.shape[1], dtype=x.dtype, device=dev)
    assert out.shape == (T, w_down.shape[1]) and out.is_contiguous() and out.dtype == x.dtype
    inv = torch.empty(pairs, dtype=torch.int32, device=dev)
    rc = lib.mx_moe_combine_n(y.data_ptr(), sorted_pair.data_ptr(), total.data_ptr(), inv.data_ptr(),
                              wts.data_ptr(), out.data_ptr(), _lib.ptr(residual), T, k,
                              w_down.shape[1], pairs, 0, st)
    _lib.count_launch(3)
    _lib.check(rc, "mx_moe_combine_n")
    return out


def moe_experts_rows(x: torch.Tensor, ids_c: torch.Tensor, row_map: torch.Tensor, n_rows: torch.Tensor, w_gate_up,
                     w_down, inter: int, act: str, b_gate_up=None, b_down=None, e_begin: int = 0,
                     alpha: float = 1.702, limit: float = 7.0, out: torch.Tensor | None = None,
                     rows_hint: int | None = None) -> torch.Tensor:
    """The local experts' gated MLPs over a COMPACT LIST of rows of a larger buffer: entry i (for
    i < ``n_rows[0]``, a count that lives on the device) is row ``row_map[i]`` of ``x`` and goes to expert
    ``ids_c[i]``; its output is written to the same row of ``out``. Rows that are not in the list are
    neither read nor written, and every kernel's work is bounded by the count, not by the size of
    ``x``: this is the expert stage of the all-to-all path, whose receive area is sized for the worst
    case (every rank sends all its pairs to one rank) while a step fills a small part of it."""
    R, H = x.shape
    El = w_gate_up.shape[0]
    if out is None:
        out = torch.zeros(R, w_down.shape[1], dtype=x.dtype, device=x.device)
    if not x.is_cuda:
        n = int(n_rows[0])
        rows = row_map[:n].long()
        o = moe_experts(x[rows], ids_c[:n].view(n, 1), torch.ones(n, 1), w_gate_up, w_down, inter, act, b_gate_up,
                        b_down, e_begin=e_begin, alpha=alpha, limit=limit)
        out[rows] = o.to(out.dtype)
        return out
    dev, lib, st = x.device, _lib.load(), _lib.stream()
    offsets = torch.empty(El + 1, dtype=torch.int32, device=dev)
    sorted_pair = torch.empty(R, dtype=torch.int32, device=dev)
    sorted_row = torch.empty(R, dtype=torch.int32, device=dev)
    rc = lib.mx_moe_align_n(ids_c.data_ptr(), n_rows.data_ptr(), row_map.data_ptr(), offsets.data_ptr(),
                            sorted_pair.data_ptr(), sorted_row.data_ptr(), R, 1, e_begin, e_begin + El, st)
    _lib.check(rc, "mx_moe_align_n")
    total = offsets[El:]
    xs = torch.empty(R, H, dtype=x.dtype, device=dev)
    rc = lib.mx_moe_gather_rows_n(x.data_ptr(), sorted_row.data_ptr(), total.data_ptr(), xs.data_ptr(), R, H, st)
    _lib.check(rc, "mx_moe_gather_rows_n")
    a = grouped_linear(xs, w_gate_up, offsets, inter, b_gate_up, act, alpha, limit, rows_hint=rows_hint)
    y = grouped_linear(a, w_down, offsets, w_down.shape[1], b_down, None, rows_hint=rows_hint)
    assert out.shape == (R, w_down.shape[1]) and out.is_contiguous() and out.dtype == x.dtype
    rc = lib.mx_moe_scatter_rows_n(y.data_ptr(), sorted_row.data_ptr(), total.data_ptr(), out.data_ptr(), R,
                                   w_down.shape[1], st)
    _lib.check(rc, "mx_moe_scatter_rows_n")
    _lib.count_launch(3)
    return out
