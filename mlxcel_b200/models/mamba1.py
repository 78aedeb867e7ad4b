"""Mamba (first generation, selective scan per channel) language model on the serving engine.

Block: RMSNorm -> in_proj -> [x | z]; causal depth-wise conv + SiLU over x; x_proj -> [dt_low | B | C];
dt = softplus(dt_proj(dt_low)); per channel d and state column n:
``S[d, n] <- exp(dt[d] A[d, n]) S[d, n] + dt[d] B[n] x[d]``, ``y[d] = S[d, :] . C + D[d] x[d]``;
y * silu(z) -> out_proj -> residual. Reference: src/models/mamba.rs and the scan kernel
``mamba1_selective_scan`` (src/lib/mlxcel-core/cpp/mlx_cxx_kernels.cpp:2680), here
``selective_scan_kernel`` in ``csrc/recurrent.cu``.

State slots, chunked prefill and the engine contract are those of :class:`Mamba2Model`
(``models/mamba2.py``); only the mixer and the state shapes differ: conv tail ``[slots, K-1, d_inner]``
(the same ragged conv kernel) and SSM state ``[slots, d_inner, N]``. The scan kernel walks one
sequence per launch row, so decode rows go through it as a batch of length-1 sequences over gathered
states and every prefill piece as one sequence.
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
class Mamba1LayerWeights:
    norm: torch.Tensor        # [H]
    in_proj: torch.Tensor     # [2 * Di, H]
    conv_w: torch.Tensor      # [Di, K] fp32
    conv_b: torch.Tensor | None
    x_proj: torch.Tensor      # [R + 2N, Di]
    dt_proj: torch.Tensor     # [Di, R]
    dt_proj_b: torch.Tensor   # [Di]
    A_log: torch.Tensor       # [Di, N]
    D: torch.Tensor           # [Di]
    out_proj: torch.Tensor    # [H, Di]
    in_proj_b: torch.Tensor | None = None
    out_proj_b: torch.Tensor | None = None
    dt_norm: torch.Tensor | None = None      # Jamba: RMSNorm on the low-rank dt, on B and on C
    b_norm: torch.Tensor | None = None
    c_norm: torch.Tensor | None = None


def mamba1_dims(cfg: ModelConfig) -> dict:
    m = cfg.extra["mamba1"]
    return dict(Di=m["d_inner"], N=m["d_state"], K=m["d_conv"], R=m["dt_rank"])


def random_mamba1_weights(cfg: ModelConfig, seed: int = 0, dtype=torch.bfloat16, device="cpu", std: float = 0.02):
    d = mamba1_dims(cfg)
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, sc=std: (torch.randn(*s, generator=g) * sc).to(dtype).to(device)  # noqa: E731
    H, Di, N, K, R = cfg.hidden_size, d["Di"], d["N"], d["K"], d["R"]
    layers = []
    for _ in range(cfg.num_hidden_layers):
        layers.append(Mamba1LayerWeights(
            norm=torch.ones(H, dtype=dtype, device=device), in_proj=r(2 * Di, H),
            conv_w=(torch.randn(Di, K, generator=g) * 0.2).float().to(device),
            conv_b=(torch.randn(Di, generator=g) * 0.1).float().to(device),
            x_proj=r(R + 2 * N, Di), dt_proj=r(Di, R, sc=0.3),
            dt_proj_b=(torch.rand(Di, generator=g) * 2 - 4).to(dtype).to(device),
            A_log=torch.log(torch.arange(1, N + 1, dtype=torch.float32)).repeat(Di, 1).to(device),
            D=torch.ones(Di, dtype=torch.float32, device=device), out_proj=r(H, Di)))
    embed = r(cfg.vocab_size, H)
    return Mamba2Weights(embed=embed, layers=layers, final_norm=torch.ones(H, dtype=dtype, device=device),
                         lm_head=embed if cfg.tie_word_embeddings else r(cfg.vocab_size, H))


def load_mamba1_weights(path, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu") -> Mamba2Weights:
    """HF / MLX Mamba checkpoint (``backbone.layers.N.mixer.{in_proj, conv1d, x_proj, dt_proj, A_log, D,
    out_proj}``); quantized projections are dequantised at load."""
    from ..loading.checkpoint import TensorSource, _Getter

    src = TensorSource(path)
    g = _Getter(src, cfg, dtype, dequantize=True)
    d = mamba1_dims(cfg)
    pre = "backbone." if any(k.startswith("backbone.") for k in src.keys()) else "model."

    def need(t, name):
        if t is None:
            raise KeyError(f"{path}: missing tensor {name}")
        return t.to(device)

    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"{pre}layers.{i}."
        m = p + "mixer."
        cw = need(g.vec(m + "conv1d.weight"), m + "conv1d.weight")
        cw = cw.reshape(d["Di"], d["K"]) if cw.dim() == 2 or cw.shape[1] == 1 else cw.squeeze(-1)
        cb = g.vec(m + "conv1d.bias")
        layers.append(Mamba1LayerWeights(
            norm=need(g.vec(p + "norm.weight"), p + "norm.weight"),
            in_proj=need(g.mat(m + "in_proj"), m + "in_proj"), in_proj_b=g.vec(m + "in_proj.bias"),
            conv_w=cw.float(), conv_b=None if cb is None else cb.float().to(device),
            x_proj=need(g.mat(m + "x_proj"), m + "x_proj"), dt_proj=need(g.mat(m + "dt_proj"), m + "dt_proj"),
            dt_proj_b=need(g.vec(m + "dt_proj.bias"), m + "dt_proj.bias"),
            A_log=need(g.vec(m + "A_log"), m + "A_log").float(), D=need(g.vec(m + "D"), m + "D").float(),
            out_proj=need(g.mat(m + "out_proj"), m + "out_proj"), out_proj_b=g.vec(m + "out_proj.bias")))
    ename = next((pre + n for n in ("embeddings", "embedding", "embed_tokens") if src.has(pre + n + ".weight")),
                 pre + "embeddings")
    embed = need(g.mat(ename), ename)
    head = g.mat("lm_head") if src.has("lm_head.weight") and not cfg.tie_word_embeddings else None
    return Mamba2Weights(embed=embed, layers=layers,
                         final_norm=need(g.vec(pre + "norm_f.weight"), pre + "norm_f.weight"),
                         lm_head=embed if head is None else head.to(device))


class Mamba1Model(Mamba2Model):
    """Engine-facing executor of first-generation Mamba models."""

    def __init__(self, cfg: ModelConfig, weights: Mamba2Weights, max_seqs: int = 256, comm=None):
        self.cfg, self.w = cfg, weights
        self.comm = comm or LocalComm()
        assert self.comm.tp_size == 1, "the Mamba executor is single-GPU"
        self.device = weights.final_norm.device
        self.d1 = mamba1_dims(cfg)
        self.Hq = self.Hkv = 1
        self.D = cfg.head_dim
        self.layer_range = range(cfg.num_hidden_layers)
        d, L = self.d1, len(weights.layers)
        if d["N"] > 32:
            raise ValueError("the selective-scan kernel keeps one state column per lane: d_state <= 32")
        self.conv_state = torch.zeros(L, max_seqs, d["K"] - 1, d["Di"], dtype=torch.float32, device=self.device)
        self.ssm_state = torch.zeros(L, max_seqs, d["Di"], d["N"], dtype=torch.float32, device=self.device)
        self.slot_of: dict[int, int] = {}
        self.free = list(range(max_seqs - 1, -1, -1))
        self.A = [-torch.exp(lw.A_log.float()).contiguous() for lw in weights.layers]
        for lw in weights.layers:
            lw.conv_w = lw.conv_w.float().contiguous()
            lw.conv_b = None if lw.conv_b is None else lw.conv_b.float().contiguous()
            lw.D = lw.D.float().contiguous()
        self._host_pieces = None

    def pieces(self, b):
        out = super().pieces(b)
        # host copy of (slot, first row, row count) for the per-sequence scan launches
        nd = b.num_decode
        ids = b.seq_ids
        pcu = b.pf_cu_q_host or [0]
        self._host_pieces = ([self.slot_of[i] for i in ids[:nd]],
                             [(self.slot_of[ids[nd + j]], nd + pcu[j], pcu[j + 1] - pcu[j], b.pf_starts[j] == 0)
                              for j in range(b.num_prefill_seqs)])
        return out

    def _mixer(self, li: int, lw: Mamba1LayerWeights, x: torch.Tensor, pieces) -> torch.Tensor:
        """x [T, H] normalised input. Returns the gated scan output [T, d_inner] (input of out_proj)."""
        d = self.d1
        Di, N, R = d["Di"], d["N"], d["R"]
        slots, cu, reset, nd, max_len = pieces
        proj = ops.linear(x, lw.in_proj, bias=lw.in_proj_b)                 # [T, 2 Di]
        xs = rops.causal_conv_varlen(proj[:, :Di], self.conv_state[li], slots, cu, reset, lw.conv_w, lw.conv_b,
                                     True, max_len)                         # [T, Di]
        z = proj[:, Di:]
        ssm = ops.linear(xs, lw.x_proj)                                     # [T, R + 2N]
        dt_low, Bm, Cm = ssm[:, :R].contiguous(), ssm[:, R:R + N].contiguous(), ssm[:, R + N:].contiguous()
        if lw.dt_norm is not None:
            eps = self.cfg.rms_norm_eps
            dt_low, Bm, Cm = (ops.rmsnorm(dt_low, lw.dt_norm, eps, 0.0), ops.rmsnorm(Bm, lw.b_norm, eps, 0.0),
                              ops.rmsnorm(Cm, lw.c_norm, eps, 0.0))
        dt = ops.linear(dt_low, lw.dt_proj, bias=lw.dt_proj_b)              # [T, Di]; softplus in the scan
        y = torch.empty_like(xs)
        dec_slots, pf = self._host_pieces
        st_all = self.ssm_state[li]
        if nd:
            sl = slots[:nd].long()
            st = st_all.index_select(0, sl)                                 # decode rows: a batch of 1-token sequences
            y[:nd] = rops.selective_scan(xs[:nd].unsqueeze(1).contiguous(), dt[:nd].unsqueeze(1).contiguous(), self.A[li],
                                         Bm[:nd].unsqueeze(1).contiguous(), Cm[:nd].unsqueeze(1).contiguous(), lw.D, st,
                                         True)[:, 0]
            st_all.index_copy_(0, sl, st)
        for slot, r0, cnt, fresh in pf:
            st = st_all[slot:slot + 1]
            if fresh:
                st.zero_()
            y[r0:r0 + cnt] = rops.selective_scan(xs[r0:r0 + cnt].unsqueeze(0).contiguous(),
                                                 dt[r0:r0 + cnt].unsqueeze(0).contiguous(), self.A[li],
                                                 Bm[r0:r0 + cnt].unsqueeze(0).contiguous(),
                                                 Cm[r0:r0 + cnt].unsqueeze(0).contiguous(), lw.D, st, True)[0]
        return (y.float() * F.silu(z.float())).to(x.dtype)

    @torch.inference_mode()
    def forward_hidden(self, b, kv_layers=None, hidden_in: torch.Tensor | None = None) -> torch.Tensor:
        cfg = self.cfg
        pieces = self.pieces(b)
        h = hidden_in if hidden_in is not None else ops.embedding(b.token_ids, self.w.embed, cfg.embed_scale)
        for li, lw in enumerate(self.w.layers):
            x = ops.rmsnorm(h, lw.norm, cfg.rms_norm_eps, 0.0)
            h = ops.linear(self._mixer(li, lw, x, pieces), lw.out_proj, bias=lw.out_proj_b, residual=h)
        return h
