"""State-space / linear-attention step operators and small element-wise ops (hybrid families:
Mamba, Mamba2 / Jamba / Nemotron-H, Qwen3-Next GatedDeltaNet, BitNet). CUDA kernels in
``csrc/recurrent.cu``; the PyTorch statements below are the references and the CPU path."""
from __future__ import annotations

import ctypes

import torch
import torch.nn.functional as F

from . import _lib

_vp, _i, _f, _ll = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_longlong
_SIG = {
    "mx_ssm_update": [_vp] * 9 + [_i] * 6 + [_vp],
    "mx_selective_scan": [_vp] * 8 + [_i] * 5 + [_vp],
    "mx_causal_conv_varlen": [_vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _vp],
    "mx_ssm_scan_varlen": [_vp, _vp, _vp, _vp, _vp, _i, _vp, _i, _vp, _vp, _vp, _i, _vp, _vp, _vp] + [_i] * 7 + [_f, _f, _vp],
    "mx_gated_rmsnorm": [_vp, _vp, _i, _vp, _vp, _i, _i, _i, _f, _vp],
    "mx_gated_delta_update": [_vp] * 7 + [_i, _i, _i, _f, _vp],
    "mx_bitlinear": [_vp, _vp, _vp, _i, _i, _i, _f, _vp],
    "mx_activation": [_vp, _vp, _ll, _i, _f, _f, _f, _f, _vp],
    "mx_add3_layernorm": [_vp] * 7 + [_i, _i, _f, _vp],
    "mx_layernorm": [_vp, _vp, _vp, _vp, _i, _i, _f, _vp],
}


def _fn(name):
    lib = _lib.load()
    fn = getattr(lib, name)
    if fn.argtypes is None or len(fn.argtypes) == 0:
        fn.argtypes, fn.restype = _SIG[name], _i
    return fn


def _call(name, *args):
    rc = _fn(name)(*args)
    _lib.count_launch()
    _lib.check(rc, name)


# ----------------------------------------------------------------------------- Mamba2 step
def ssm_update_ref(state, x, dt, A, Bm, C, D=None, dt_bias=None, dt_softplus=True):
    B, H, Dh, N = state.shape
    G = Bm.shape[1]
    dtv = dt.float() + (dt_bias.float() if dt_bias is not None else 0.0)
    if dt_softplus:
        dtv = F.softplus(dtv)
    dA = torch.exp(dtv * A.float())                                    # [B, H]
    Bh = Bm.float().repeat_interleave(H // G, dim=1)                   # [B, H, N]
    Ch = C.float().repeat_interleave(H // G, dim=1)
    new = state * dA[..., None, None] + (dtv[..., None] * x.float())[..., None] * Bh[:, :, None, :]
    y = (new * Ch[:, :, None, :]).sum(-1)
    if D is not None:
        y = y + D.float()[None, :, None] * x.float()
    state.copy_(new)
    return y.to(x.dtype)


def ssm_update(state, x, dt, A, Bm, C, D=None, dt_bias=None, dt_softplus=True):
    """Mamba2 decode step. state [B,H,Dh,N] fp32 is updated in place; returns y [B,H,Dh]."""
    if not x.is_cuda:
        return ssm_update_ref(state, x, dt, A, Bm, C, D, dt_bias, dt_softplus)
    B, H, Dh, N = state.shape
    y = torch.empty_like(x)
    _call("mx_ssm_update", state.data_ptr(), x.data_ptr(), dt.data_ptr(), A.data_ptr(), Bm.data_ptr(), C.data_ptr(),
          _lib.ptr(D), _lib.ptr(dt_bias), y.data_ptr(), B, H, Dh, N, Bm.shape[1], 1 if dt_softplus else 0,
          _lib.stream())
    return y


# ----------------------------------------------------------------------------- Mamba1 scan
def selective_scan_ref(x, dt, A, Bm, C, D, state, dt_softplus=True):
    Bsz, L, Di = x.shape
    y = torch.empty(Bsz, L, Di, dtype=torch.float32, device=x.device)
    s = state.clone()
    for t in range(L):
        dtv = dt[:, t].float()
        if dt_softplus:
            dtv = F.softplus(dtv)
        xv = x[:, t].float()
        s = torch.exp(dtv[..., None] * A.float()[None]) * s + (dtv * xv)[..., None] * Bm[:, t].float()[:, None, :]
        y[:, t] = (s * C[:, t].float()[:, None, :]).sum(-1) + (D.float()[None] * xv if D is not None else 0.0)
    state.copy_(s)
    return y.to(x.dtype)


def selective_scan(x, dt, A, Bm, C, D, state, dt_softplus=True):
    """Mamba1 scan over L steps. state [B,Di,N] fp32 in place; returns y [B,L,Di]."""
    if not x.is_cuda:
        return selective_scan_ref(x, dt, A, Bm, C, D, state, dt_softplus)
    Bsz, L, Di = x.shape
    y = torch.empty_like(x)
    _call("mx_selective_scan", x.data_ptr(), dt.data_ptr(), A.data_ptr(), Bm.data_ptr(), C.data_ptr(), _lib.ptr(D),
          state.data_ptr(), y.data_ptr(), Bsz, L, Di, A.shape[1], 1 if dt_softplus else 0, _lib.stream())
    return y


# ----------------------------------------------------------------------------- Mamba2, ragged batch
def _pieces(cu):
    c = cu.tolist()
    return [(c[j], c[j + 1]) for j in range(len(c) - 1)]


def causal_conv_varlen_ref(xin, conv_state, slots, cu, reset, w, bias, silu=True):
    C, K = w.shape
    out = torch.empty(xin.shape[0], C, dtype=xin.dtype, device=xin.device)
    sl, rs = slots.tolist(), reset.tolist()
    for j, (t0, t1) in enumerate(_pieces(cu)):
        if t1 <= t0:
            continue
        hist = torch.zeros(K - 1, C, device=xin.device) if rs[j] else conv_state[sl[j]].clone()
        seq = torch.cat([hist, xin[t0:t1, :C].float()], dim=0)                       # [K-1+L, C]
        y = F.conv1d(seq.t().unsqueeze(0), w.float().unsqueeze(1), None if bias is None else bias.float(), groups=C)
        y = y[0].t()
        out[t0:t1] = (F.silu(y) if silu else y).to(xin.dtype)
        if K > 1:
            conv_state[sl[j]] = seq[-(K - 1):]
    return out


def causal_conv_varlen(xin, conv_state, slots, cu, reset, w, bias, silu=True, max_len: int | None = None):
    """Causal depth-wise conv + bias (+ SiLU) over a ragged batch of sequence pieces.

    xin [T, >=C] (the first C columns are convolved; may be a column slice with a row stride);
    conv_state [slots, K-1, C] fp32, advanced in place; slots / reset [S] int32; cu [S+1] int32;
    w [C, K] fp32; bias [C] fp32 or None; max_len: an upper bound of the longest piece (read back
    from ``cu`` when not given, which synchronises). Returns [T, C]."""
    if not xin.is_cuda:
        return causal_conv_varlen_ref(xin, conv_state, slots, cu, reset, w, bias, silu)
    C, K = w.shape
    assert xin.stride(1) == 1
    if max_len is None:
        max_len = int((cu[1:] - cu[:-1]).max().item()) if slots.numel() else 0
    out = torch.empty(xin.shape[0], C, dtype=xin.dtype, device=xin.device)
    _call("mx_causal_conv_varlen", xin.data_ptr(), xin.stride(0), conv_state.data_ptr(), slots.data_ptr(), cu.data_ptr(),
          reset.data_ptr(), w.data_ptr(), _lib.ptr(bias), out.data_ptr(), slots.numel(), int(max_len), C, K,
          1 if silu else 0, _lib.stream())
    return out


def ssm_scan_varlen_ref(state, slots, cu, reset, x, dt, A, Bm, Cm, D, dt_bias, dt_softplus=True, dt_limit=(0.0, float("inf"))):
    S, H, P, N = state.shape
    G = Bm.shape[1] // N
    y = torch.empty(x.shape[0], H * P, dtype=x.dtype, device=x.device)
    sl, rs = slots.tolist(), reset.tolist()
    for j, (t0, t1) in enumerate(_pieces(cu)):
        if t1 <= t0:
            continue
        s = torch.zeros(H, P, N, device=x.device) if rs[j] else state[sl[j]].clone()
        for t in range(t0, t1):
            dtv = dt[t].float() + (dt_bias.float() if dt_bias is not None else 0.0)
            if dt_softplus:
                dtv = F.softplus(dtv)
            dtv = dtv.clamp(dt_limit[0], dt_limit[1])
            xv = x[t].float().reshape(H, P)
            Bh = Bm[t].float().reshape(G, N).repeat_interleave(H // G, dim=0)
            Ch = Cm[t].float().reshape(G, N).repeat_interleave(H // G, dim=0)
            s = s * torch.exp(dtv * A.float())[:, None, None] + (dtv[:, None] * xv)[..., None] * Bh[:, None, :]
            yt = (s * Ch[:, None, :]).sum(-1)
            if D is not None:
                yt = yt + D.float()[:, None] * xv
            y[t] = yt.reshape(-1).to(x.dtype)
        state[sl[j]] = s
    return y


def ssm_scan_varlen(state, slots, cu, reset, x, dt, A, Bm, Cm, D=None, dt_bias=None, dt_softplus=True,
                    dt_limit=(0.0, float("inf")), n_short: int = 0):
    """Mamba2 recurrence over a ragged batch (decode rows are pieces of one token).

    state [slots, H, P, N] fp32 in place; x [T, H*P]; dt [T, H]; Bm, Cm [T, G*N] (column slices with a
    row stride are fine); A, D, dt_bias [H] fp32; n_short: the first n_short pieces hold exactly one
    token (they take the bandwidth-shaped kernel, the rest the row-per-thread one). Returns y [T, H*P]."""
    if not x.is_cuda:
        return ssm_scan_varlen_ref(state, slots, cu, reset, x, dt, A, Bm, Cm, D, dt_bias, dt_softplus, dt_limit)
    S, H, P, N = state.shape
    G = Bm.shape[1] // N
    assert x.stride(1) == 1 and dt.stride(1) == 1 and Bm.stride(1) == 1 and Cm.stride(0) == Bm.stride(0)
    y = torch.empty(x.shape[0], H * P, dtype=x.dtype, device=x.device)
    _call("mx_ssm_scan_varlen", state.data_ptr(), slots.data_ptr(), cu.data_ptr(), reset.data_ptr(), x.data_ptr(),
          x.stride(0), dt.data_ptr(), dt.stride(0), A.data_ptr(), Bm.data_ptr(), Cm.data_ptr(), Bm.stride(0),
          _lib.ptr(D), _lib.ptr(dt_bias), y.data_ptr(), slots.numel(), int(n_short), H, P, N, G, 1 if dt_softplus else 0,
          float(dt_limit[0]), float(min(dt_limit[1], 3.0e38)), _lib.stream())
    return y


def gated_rmsnorm(y, z, weight, eps: float, groups: int = 1):
    """RMSNorm(y * silu(z)) * weight, normalised over each of ``groups`` equal slices of a row
    (groups == 1: the whole row); z may be a column slice with a row stride."""
    if not y.is_cuda:
        v = (y.float() * F.silu(z.float())).reshape(y.shape[0], groups, -1)
        v = v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + eps)
        return (v.reshape(y.shape[0], -1) * weight.float()).to(y.dtype)
    rows, dim = y.shape
    assert z.stride(1) == 1 and y.is_contiguous() and dim % groups == 0
    out = torch.empty_like(y)
    _call("mx_gated_rmsnorm", y.data_ptr(), z.data_ptr(), z.stride(0), weight.data_ptr(), out.data_ptr(), rows,
          dim // groups, int(groups), float(eps), _lib.stream())
    return out


# ----------------------------------------------------------------------------- gated delta rule
def gated_delta_update_ref(S, q, k, v, g, beta, q_scale=1.0):
    Sn = S * torch.exp(g.float())[..., None, None]
    mem = (Sn * k.float()[..., :, None]).sum(-2)
    delta = (v.float() - mem) * beta.float()[..., None]
    Sn = Sn + k.float()[..., :, None] * delta[..., None, :]
    out = (Sn * (q.float() * q_scale)[..., :, None]).sum(-2)
    S.copy_(Sn)
    return out.to(q.dtype)


def gated_delta_update(S, q, k, v, g, beta, q_scale=1.0):
    """GatedDeltaNet decode step. S [B,Hv,Dk,Dv] fp32 in place; q,k [B,Hv,Dk]; v [B,Hv,Dv]; g, beta [B,Hv] fp32."""
    if not q.is_cuda:
        return gated_delta_update_ref(S, q, k, v, g, beta, q_scale)
    B, Hv, Dk, Dv = S.shape
    out = torch.empty_like(v)
    _call("mx_gated_delta_update", S.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), g.data_ptr(),
          beta.data_ptr(), out.data_ptr(), B * Hv, Dk, Dv, float(q_scale), _lib.stream())
    return out


# ----------------------------------------------------------------------------- BitLinear
def pack_ternary(w: torch.Tensor) -> torch.Tensor:
    """{-1,0,1} [N,K] → uint8 [N,K/4] (2 bits per value, code = value + 1, LSB first)."""
    c = (w.to(torch.int64) + 1).reshape(w.shape[0], -1, 4)
    return (c[..., 0] | (c[..., 1] << 2) | (c[..., 2] << 4) | (c[..., 3] << 6)).to(torch.uint8)


def bitlinear(x, w_packed, scale: float):
    M, K = x.shape
    N = w_packed.shape[0]
    if not x.is_cuda:
        c = w_packed.to(torch.int64)
        w = torch.stack([(c >> (2 * j)) & 3 for j in range(4)], dim=-1).reshape(N, K).float() - 1.0
        return ((x.float() @ w.t()) * scale).to(x.dtype)
    out = torch.empty(M, N, dtype=x.dtype, device=x.device)
    _call("mx_bitlinear", x.data_ptr(), w_packed.data_ptr(), out.data_ptr(), M, N, K, float(scale), _lib.stream())
    return out


# ----------------------------------------------------------------------------- element-wise
def gelu_tanh(x):
    if not x.is_cuda:
        return F.gelu(x.float(), approximate="tanh").to(x.dtype)
    y = torch.empty_like(x)
    _call("mx_activation", x.data_ptr(), y.data_ptr(), x.numel(), 0, 0.0, 0.0, 0.0, 0.0, _lib.stream())
    return y


_ACT_MODES = {"gelu_tanh": 0, "relu2": 2, "gelu": 3, "silu": 4}


def activation(x, kind: str):
    """Element-wise activation of a plain (non-gated) MLP: gelu_tanh | gelu (erf) | relu2 | silu."""
    if not x.is_cuda:
        v = x.float()
        r = {"gelu_tanh": lambda: F.gelu(v, approximate="tanh"), "gelu": lambda: F.gelu(v),
             "relu2": lambda: torch.relu(v).square(), "silu": lambda: F.silu(v)}[kind]()
        return r.to(x.dtype)
    x = x.contiguous()
    y = torch.empty_like(x)
    _call("mx_activation", x.data_ptr(), y.data_ptr(), x.numel(), _ACT_MODES[kind], 0.0, 0.0, 0.0, 0.0, _lib.stream())
    return y


def layernorm(x, weight, bias=None, eps: float = 1e-5):
    """LayerNorm over the last dimension of a 2-D tensor (bias optional)."""
    if not x.is_cuda:
        return F.layer_norm(x.float(), (x.shape[-1],), weight.float(), None if bias is None else bias.float(),
                            eps).to(x.dtype)
    x = x.contiguous()
    y = torch.empty_like(x)
    _call("mx_layernorm", x.data_ptr(), weight.data_ptr(), _lib.ptr(bias), y.data_ptr(), x.shape[0], x.shape[1],
          float(eps), _lib.stream())
    return y


def relu2(x):
    """relu(x)^2 (the MLP activation of Nemotron-H)."""
    if not x.is_cuda:
        return torch.relu(x.float()).square().to(x.dtype)
    x = x.contiguous()
    y = torch.empty_like(x)
    _call("mx_activation", x.data_ptr(), y.data_ptr(), x.numel(), 2, 0.0, 0.0, 0.0, 0.0, _lib.stream())
    return y


def xielu_ref(x, ap, an, beta, eps):
    v = x.float()
    return torch.where(v > 0, ap * v * v + beta * v, an * (torch.expm1(torch.clamp(v, max=eps)) - v) + beta * v).to(x.dtype)


def xielu(x, ap: float, an: float, beta: float = 0.5, eps: float = -1e-6):
    if not x.is_cuda:
        return xielu_ref(x, ap, an, beta, eps)
    y = torch.empty_like(x)
    _call("mx_activation", x.data_ptr(), y.data_ptr(), x.numel(), 1, float(ap), float(an), float(beta), float(eps),
          _lib.stream())
    return y


def add3_layernorm(a, b, c, weight, bias=None, eps: float = 1e-5):
    """(LayerNorm(a + b + c) * weight + bias, a + b + c)."""
    if not a.is_cuda:
        s = (a.float() + b.float() + c.float()).to(a.dtype)
        y = F.layer_norm(s.float(), (s.shape[-1],), weight.float(), None if bias is None else bias.float(), eps)
        return y.to(a.dtype), s
    rows, dim = a.shape
    y, s = torch.empty_like(a), torch.empty_like(a)
    _call("mx_add3_layernorm", a.data_ptr(), b.data_ptr(), c.data_ptr(), weight.data_ptr(), _lib.ptr(bias),
          s.data_ptr(), y.data_ptr(), rows, dim, float(eps), _lib.stream())
    return y, s
