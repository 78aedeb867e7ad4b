"""Gated short convolution mixer (LFM2 conv layers) with per-sequence state slots.

``[B | C | x] = in_proj(h)``; ``y = C * causal_conv_K(B * x)`` (depth-wise, no activation); ``out_proj(y)``.
The only state is the conv tail ``[slots, K-1, H]`` per layer, carried by the ragged conv kernel that
the Mamba mixers use (``causal_conv_varlen_kernel`` in ``csrc/recurrent.cu``). Reference:
src/models/lfm2.rs and its conv decode path (src/models/conv_decode.rs).

State slots, chunked prefill and the engine contract are those of :class:`Mamba2Model`.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..config import ModelConfig
from ..ops import recurrent as rops
from .decoder import LocalComm
from .mamba2 import Mamba2Model, Mamba2Weights


@dataclass
class ShortConvLayerWeights:
    norm: torch.Tensor            # [H]
    in_proj: torch.Tensor         # [3H, H], rows ordered B | C | x
    conv_w: torch.Tensor          # [H, K] fp32
    out_proj: torch.Tensor        # [H, H]
    in_proj_b: torch.Tensor | None = None
    conv_b: torch.Tensor | None = None
    out_proj_b: torch.Tensor | None = None


class ShortConvModel(Mamba2Model):
    """State slots + mixer of the short-conv layers (a component of the hybrid executor)."""

    def __init__(self, cfg: ModelConfig, weights: Mamba2Weights, max_seqs: int = 256, comm=None):
        self.cfg, self.w = cfg, weights
        self.comm = comm or LocalComm()
        assert self.comm.tp_size == 1, "the short-conv executor is single-GPU"
        self.device = weights.final_norm.device
        self.Hq = self.Hkv = 1
        self.D = cfg.head_dim
        self.layer_range = range(cfg.num_hidden_layers)
        K, H, L = int(cfg.extra["shortconv"]["d_conv"]), cfg.hidden_size, len(weights.layers)
        self.conv_state = torch.zeros(L, max_seqs, K - 1, H, dtype=torch.float32, device=self.device)
        self.ssm_state = torch.zeros(L, max_seqs, 1, dtype=torch.float32, device=self.device)   # no recurrent state
        self.slot_of: dict[int, int] = {}
        self.free = list(range(max_seqs - 1, -1, -1))
        for lw in weights.layers:
            lw.conv_w = lw.conv_w.float().contiguous()
            lw.conv_b = None if lw.conv_b is None else lw.conv_b.float().contiguous()

    def _mixer(self, li: int, lw: ShortConvLayerWeights, x: torch.Tensor, pieces) -> torch.Tensor:
        """x [T, H] normalised input. Returns ``C * conv(B * x)`` [T, H] (input of out_proj)."""
        H = x.shape[1]
        slots, cu, reset, nd, max_len = pieces
        bcx = ops.linear(x, lw.in_proj, bias=lw.in_proj_b)
        bx = (bcx[:, :H].float() * bcx[:, 2 * H:].float()).to(x.dtype)
        conv = rops.causal_conv_varlen(bx, self.conv_state[li], slots, cu, reset, lw.conv_w, lw.conv_b, False, max_len)
        return (bcx[:, H:2 * H].float() * conv.float()).to(x.dtype)
