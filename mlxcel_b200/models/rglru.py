"""Real-gated linear recurrent unit mixer (RecurrentGemma / Griffin recurrent blocks) with per-sequence
state slots.

Per layer: ``y = gelu(W_y h)``, ``x = conv_K(W_x h)`` (causal, depth-wise), then the RG-LRU over x:
``i = sigmoid(blockdiag(W_i) x + b_i)``, ``r = sigmoid(blockdiag(W_r) x + b_r)``,
``a = exp(-8 r softplus(L))``, ``s_t = a_t s_{t-1} + sqrt(1 - a_t^2) (i_t x_t)`` (the first token of a
sequence enters with factor 1), output ``W_o (s * y)``. Reference: src/models/recurrent_gemma.rs.

The recurrence runs on the selective-scan kernel of the Mamba-1 mixers with one state column: with
``A = -8 softplus(L)`` and ``dt = r`` that kernel's decay ``exp(dt A)`` is ``a``, and feeding it
``x' = sqrt(1 - a^2) i x / r`` with ``B = C = 1`` makes its update ``dt x' B`` the RG-LRU input term and
its output ``C s`` the state. The block-diagonal gate products go through the grouped GEMM with the
heads as groups. State slots, chunked prefill and the engine contract are those of
:class:`Mamba1Model`; the state is the conv tail ``[slots, K-1, W]`` and ``s`` ``[slots, W, 1]`` fp32.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .. import ops
from ..config import ModelConfig
from ..ops import recurrent as rops
from .decoder import LocalComm
from .mamba1 import Mamba1Model
from .mamba2 import Mamba2Weights


@dataclass
class RglruLayerWeights:
    norm: torch.Tensor            # [H] (plain gain: the stored (weight - 1) has its one added at load)
    linear_y: torch.Tensor        # [W, H]
    linear_y_b: torch.Tensor
    linear_x: torch.Tensor        # [W, H]
    linear_x_b: torch.Tensor
    conv_w: torch.Tensor          # [W, K] fp32
    conv_b: torch.Tensor          # [W] fp32
    gate_in_w: torch.Tensor       # [heads, bw, bw] as Linear weights (out, in) of each head's block
    gate_in_b: torch.Tensor       # [W]
    gate_rec_w: torch.Tensor      # [heads, bw, bw]
    gate_rec_b: torch.Tensor      # [W]
    decay: torch.Tensor           # [W] the recurrent parameter L
    out_proj: torch.Tensor        # [H, W]
    out_proj_b: torch.Tensor | None = None


class RglruModel(Mamba1Model):
    """State slots + mixer of the RG-LRU layers (a component of the hybrid executor)."""

    def __init__(self, cfg: ModelConfig, weights: Mamba2Weights, max_seqs: int = 256, comm=None):
        self.cfg, self.w = cfg, weights
        self.comm = comm or LocalComm()
        assert self.comm.tp_size == 1, "the RG-LRU executor is single-GPU"
        self.device = weights.final_norm.device
        r = cfg.extra["rglru"]
        self.W, self.heads, self.K = int(r["width"]), int(r["heads"]), int(r["d_conv"])
        self.Hq = self.Hkv = 1
        self.D = cfg.head_dim
        self.layer_range = range(cfg.num_hidden_layers)
        L = len(weights.layers)
        self.conv_state = torch.zeros(L, max_seqs, self.K - 1, self.W, dtype=torch.float32, device=self.device)
        self.ssm_state = torch.zeros(L, max_seqs, self.W, 1, dtype=torch.float32, device=self.device)
        self.slot_of: dict[int, int] = {}
        self.free = list(range(max_seqs - 1, -1, -1))
        self.A = [(-8.0 * F.softplus(lw.decay.float())).reshape(self.W, 1).contiguous() for lw in weights.layers]
        for lw in weights.layers:
            lw.conv_w, lw.conv_b = lw.conv_w.float().contiguous(), lw.conv_b.float().contiguous()
        self._host_pieces = None

    def _block_diag(self, x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        """sigmoid(per-head x_h W_h^T + b) for x [T, W] and w [heads, bw, bw] (Linear orientation)."""
        T, nh = x.shape[0], self.heads
        bw = self.W // nh
        if x.is_cuda and T:
            from ..ops import moe as moe_ops
            xs = x.view(T, nh, bw).transpose(0, 1).reshape(nh * T, bw).contiguous()          # rows grouped by head
            offs = torch.arange(0, (nh + 1) * T, T, dtype=torch.int32, device=x.device)
            y = moe_ops.grouped_linear(xs, w, offs, bw).view(nh, T, bw).transpose(0, 1).reshape(T, self.W)
        else:
            y = torch.einsum("thi,hoi->tho", x.view(T, nh, bw).float(), w.float()).reshape(T, self.W)
        return torch.sigmoid(y.float() + b.float())

    def _mixer(self, li: int, lw: RglruLayerWeights, x: torch.Tensor, pieces) -> torch.Tensor:
        """x [T, H] normalised input. Returns ``s * gelu(W_y x)`` [T, W] (input of out_proj)."""
        slots, cu, reset, nd, max_len = pieces
        yb = rops.activation(ops.linear(x, lw.linear_y, bias=lw.linear_y_b), "gelu_tanh")
        xb = ops.linear(x, lw.linear_x, bias=lw.linear_x_b)
        xc = rops.causal_conv_varlen(xb, self.conv_state[li], slots, cu, reset, lw.conv_w, lw.conv_b, False, max_len)
        gi = self._block_diag(xc, lw.gate_in_w, lw.gate_in_b)
        gr = self._block_diag(xc, lw.gate_rec_w, lw.gate_rec_b)
        log_a = gr * self.A[li].view(1, -1)                                    # fp32 [T, W], <= 0
        mult = torch.sqrt((1.0 - torch.exp(2.0 * log_a)).clamp_min(0.0))
        dec_slots, pf = self._host_pieces
        for _slot, r0, cnt, fresh in pf:
            if fresh and cnt:
                mult[r0] = 1.0                                                   # a sequence's first token enters unscaled
        dt = gr.to(x.dtype)
        xin = (xc.float() * gi * mult / dt.float().clamp_min(1e-12)).to(x.dtype)
        ones = torch.ones(x.shape[0], 1, dtype=x.dtype, device=x.device)
        s = torch.empty_like(xin)
        st_all = self.ssm_state[li]
        if nd:
            sl = slots[:nd].long()
            st = st_all.index_select(0, sl)
            s[:nd] = rops.selective_scan(xin[:nd].unsqueeze(1).contiguous(), dt[:nd].unsqueeze(1).contiguous(), self.A[li],
                                         ones[:nd].unsqueeze(1).contiguous(), ones[:nd].unsqueeze(1).contiguous(), None, st,
                                         False)[:, 0]
            st_all.index_copy_(0, sl, st)
        for slot, r0, cnt, fresh in pf:
            st = st_all[slot:slot + 1]
            if fresh:
                st.zero_()
            s[r0:r0 + cnt] = rops.selective_scan(xin[r0:r0 + cnt].unsqueeze(0).contiguous(),
                                                 dt[r0:r0 + cnt].unsqueeze(0).contiguous(), self.A[li],
                                                 ones[r0:r0 + cnt].unsqueeze(0).contiguous(),
                                                 ones[r0:r0 + cnt].unsqueeze(0).contiguous(), None, st, False)[0]
        return (s.float() * yb.float()).to(x.dtype)
