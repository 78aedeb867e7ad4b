"""Gated DeltaNet mixer (Qwen3-Next linear-attention layers) with per-sequence state slots.

Per value head h with key / value sizes Dk, Dv and state S [Dk, Dv], for every token:
``S <- exp(g) S;  S <- S + k (x) (beta (v - S^T k));  y = S^T (q / sqrt(Dk))`` with q, k L2-normalised,
``beta = sigmoid(b)``, ``g = -exp(A_log) softplus(a + dt_bias)``; before that a causal depth-wise
conv + SiLU over [q | k | v]; after it RMSNorm per head times ``silu(z)`` and out_proj.
Reference: src/models/qwen3_next.rs and the ``gated_delta`` kernels
(src/lib/mlxcel-core/cpp/mlx_cxx_kernels.cpp:887-1500), here ``gated_delta_kernel`` in
``csrc/recurrent.cu``.

State slots, chunked prefill and the engine contract are those of :class:`Mamba2Model`; the conv tail is
``[slots, K-1, 2 Hk Dk + Hv Dv]`` (the same ragged conv kernel), the recurrent state
``[slots, Hv, Dk, Dv]`` fp32. The step kernel advances one token of every row it is given, so decode
rows go through it as one batch over gathered states and a prefill piece token by token (the chunked
form of the delta rule is not written).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .. import ops
from ..config import ModelConfig
from ..ops import recurrent as rops
from .decoder import LocalComm
from .mamba2 import Mamba2Model, Mamba2Weights


@dataclass
class GdnLayerWeights:
    norm: torch.Tensor        # [H] layer norm in front of the mixer (plain gain)
    in_proj: torch.Tensor     # [2 Hk Dk + 2 Hv Dv, H], rows ordered q | k | v | z
    in_proj_ba: torch.Tensor  # [2 Hv, H], rows ordered b | a
    conv_w: torch.Tensor      # [conv_dim, K] fp32
    dt_bias: torch.Tensor     # [Hv]
    A_log: torch.Tensor       # [Hv]
    gnorm: torch.Tensor       # [Dv]
    out_proj: torch.Tensor    # [H, Hv Dv]


def gdn_dims(cfg: ModelConfig) -> dict:
    m = cfg.extra["gdn"]
    Hk, Hv, Dk, Dv = m["k_heads"], m["v_heads"], m["k_dim"], m["v_dim"]
    return dict(Hk=Hk, Hv=Hv, Dk=Dk, Dv=Dv, K=m["d_conv"], key_dim=Hk * Dk, value_dim=Hv * Dv,
                conv_dim=2 * Hk * Dk + Hv * Dv)


def regroup_qkvz(w: torch.Tensor, d: dict) -> torch.Tensor:
    """Checkpoint layout of in_proj_qkvz: per key head [q | k | v (r heads) | z (r heads)] with
    r = Hv / Hk; returned: all q rows, all k rows, all v rows, all z rows."""
    Hk, Dk, Dv, r = d["Hk"], d["Dk"], d["Dv"], d["Hv"] // d["Hk"]
    g = w.view(Hk, 2 * Dk + 2 * r * Dv, -1)
    q, k, v, z = g[:, :Dk], g[:, Dk:2 * Dk], g[:, 2 * Dk:2 * Dk + r * Dv], g[:, 2 * Dk + r * Dv:]
    return torch.cat([t.reshape(-1, w.shape[-1]) for t in (q, k, v, z)], 0).contiguous()


def regroup_ba(w: torch.Tensor, d: dict) -> torch.Tensor:
    Hk, r = d["Hk"], d["Hv"] // d["Hk"]
    g = w.view(Hk, 2 * r, -1)
    return torch.cat([g[:, :r].reshape(-1, w.shape[-1]), g[:, r:].reshape(-1, w.shape[-1])], 0).contiguous()


class GdnModel(Mamba2Model):
    """State slots + mixer of the Gated DeltaNet layers (used as a component of the hybrid executor)."""

    def __init__(self, cfg: ModelConfig, weights: Mamba2Weights, max_seqs: int = 256, comm=None):
        self.cfg, self.w = cfg, weights
        self.comm = comm or LocalComm()
        assert self.comm.tp_size == 1, "the Gated DeltaNet executor is single-GPU"
        self.device = weights.final_norm.device
        self.dg = gdn_dims(cfg)
        self.Hq = self.Hkv = 1
        self.D = cfg.head_dim
        self.layer_range = range(cfg.num_hidden_layers)
        d, L = self.dg, len(weights.layers)
        self.conv_state = torch.zeros(L, max_seqs, d["K"] - 1, d["conv_dim"], dtype=torch.float32, device=self.device)
        self.ssm_state = torch.zeros(L, max_seqs, d["Hv"], d["Dk"], d["Dv"], dtype=torch.float32, device=self.device)
        self.slot_of: dict[int, int] = {}
        self.free = list(range(max_seqs - 1, -1, -1))
        self.A = [-torch.exp(lw.A_log.float()).contiguous() for lw in weights.layers]
        for lw in weights.layers:
            lw.conv_w = lw.conv_w.float().contiguous()
            lw.dt_bias = lw.dt_bias.float().contiguous()
        self._host_pieces = None

    def pieces(self, b):
        out = super().pieces(b)
        nd, ids = b.num_decode, b.seq_ids
        pcu = b.pf_cu_q_host or [0]
        self._host_pieces = [(self.slot_of[ids[nd + j]], nd + pcu[j], pcu[j + 1] - pcu[j], b.pf_starts[j] == 0)
                             for j in range(b.num_prefill_seqs)]
        return out

    def _mixer(self, li: int, lw: GdnLayerWeights, x: torch.Tensor, pieces) -> torch.Tensor:
        """x [T, H] normalised input. Returns the normed, gated output [T, Hv * Dv] (input of out_proj)."""
        d = self.dg
        Hk, Hv, Dk, Dv, kd, vd, cd = d["Hk"], d["Hv"], d["Dk"], d["Dv"], d["key_dim"], d["value_dim"], d["conv_dim"]
        slots, cu, reset, nd, max_len = pieces
        T = x.shape[0]
        proj = ops.linear(x, lw.in_proj)                                     # [T, q | k | v | z]
        ba = ops.linear(x, lw.in_proj_ba).float()                            # [T, b | a]
        qkv = rops.causal_conv_varlen(proj[:, :cd], self.conv_state[li], slots, cu, reset, lw.conv_w, None, True, max_len)
        z = proj[:, cd:].reshape(T, Hv, Dv)
        l2 = lambda t: t * torch.rsqrt(t.pow(2).sum(-1, keepdim=True) + 1e-6)  # noqa: E731  (eps inside the root)
        q = l2(qkv[:, :kd].float().view(T, Hk, Dk))
        k = l2(qkv[:, kd:2 * kd].float().view(T, Hk, Dk))
        v = qkv[:, 2 * kd:].reshape(T, Hv, Dv)
        if Hv != Hk:
            q, k = q.repeat_interleave(Hv // Hk, dim=1), k.repeat_interleave(Hv // Hk, dim=1)
        q, k = q.to(x.dtype).contiguous(), k.to(x.dtype).contiguous()
        beta = torch.sigmoid(ba[:, :Hv]).contiguous()
        g = (self.A[li] * F.softplus(ba[:, Hv:] + lw.dt_bias)).contiguous()   # log decay, <= 0
        y = torch.empty(T, Hv, Dv, dtype=x.dtype, device=x.device)
        st_all = self.ssm_state[li]
        scale = Dk ** -0.5
        if nd:
            sl = slots[:nd].long()
            st = st_all.index_select(0, sl)
            y[:nd] = rops.gated_delta_update(st, q[:nd], k[:nd], v[:nd].contiguous(), g[:nd], beta[:nd], scale)
            st_all.index_copy_(0, sl, st)
        for slot, r0, cnt, fresh in self._host_pieces:
            st = st_all[slot:slot + 1]
            if fresh:
                st.zero_()
            for t in range(r0, r0 + cnt):                                     # one step-kernel launch per token
                y[t:t + 1] = rops.gated_delta_update(st, q[t:t + 1], k[t:t + 1], v[t:t + 1].contiguous(), g[t:t + 1],
                                                     beta[t:t + 1], scale)
        yf = y.float()
        yn = yf * torch.rsqrt(yf.pow(2).mean(-1, keepdim=True) + self.cfg.rms_norm_eps) * lw.gnorm.float()
        return (yn.to(x.dtype).float() * F.silu(z.float())).to(x.dtype).reshape(T, vd)
