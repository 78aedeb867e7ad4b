"""Mamba2 (pure state-space) language model on the serving engine.

Block: RMSNorm -> in_proj -> [z | xBC | dt]; causal depth-wise conv (width d_conv) + SiLU over xBC;
x, B, C = split(xBC); per head h with scalar A_h:  S <- S * exp(dt A) + dt * x (x) B,  y = S C + D x;
gated RMSNorm (y * silu(z)) -> out_proj -> residual. Reference: src/models/mamba2.rs and the SSM
step kernel K10 of its kernel table (src/lib/mlxcel-core/cpp, ssm update), here `csrc/recurrent.cu`.

State instead of KV: every sequence owns one slot of two pools, the conv tail
``[slots, d_conv - 1, conv_dim]`` and the SSM state ``[slots, heads, head_dim, d_state]`` (fp32).
The engine's paged KV blocks are still counted (they pace admission) but hold nothing. A prefill
piece that starts at position 0 resets the slot, so chunked prefill carries the state from chunk to
chunk and preemption-by-recompute simply starts over. Prefix caching, CUDA graphs and the lookahead
pipeline are turned off for recurrent models (the state of a cached prefix is not in the pool).

Per layer the mixer is five launches whatever the batch holds: in_proj GEMM, ragged causal conv,
ragged state scan (decode rows are pieces of one token), gated RMSNorm, out_proj GEMM with the
residual added in its epilogue.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .. import ops
from ..config import ModelConfig
from ..ops import recurrent as rops
from .decoder import LocalComm, StepBatch


@dataclass
class Mamba2LayerWeights:
    norm: torch.Tensor        # [H]
    in_proj: torch.Tensor     # [2*d_inner + 2*G*N + heads, H]
    conv_w: torch.Tensor      # [conv_dim, d_conv]
    conv_b: torch.Tensor      # [conv_dim]
    dt_bias: torch.Tensor     # [heads]
    A_log: torch.Tensor       # [heads]
    D: torch.Tensor           # [heads]
    gnorm: torch.Tensor       # [d_inner]
    out_proj: torch.Tensor    # [H, d_inner]


@dataclass
class Mamba2Weights:
    embed: torch.Tensor
    layers: list
    final_norm: torch.Tensor
    lm_head: torch.Tensor


def mamba_dims(cfg: ModelConfig) -> dict:
    m = cfg.extra["mamba"]
    d_inner = m.get("d_inner", m.get("expand", 2) * cfg.hidden_size)
    P = m.get("head_dim", 64)
    G, N, K = m.get("n_groups", 1), m.get("d_state", 128), m.get("d_conv", 4)
    return dict(d_inner=d_inner, P=P, heads=d_inner // P, G=G, N=N, K=K, conv_dim=d_inner + 2 * G * N)


def random_mamba2_weights(cfg: ModelConfig, seed: int = 0, dtype=torch.bfloat16, device="cpu", std: float = 0.02):
    d = mamba_dims(cfg)
    g = torch.Generator().manual_seed(seed)
    r = lambda *s, sc=std: (torch.randn(*s, generator=g) * sc).to(dtype).to(device)  # noqa: E731
    H = cfg.hidden_size
    layers = []
    for _ in range(cfg.num_hidden_layers):
        layers.append(Mamba2LayerWeights(
            norm=torch.ones(H, dtype=dtype, device=device),
            in_proj=r(2 * d["d_inner"] + 2 * d["G"] * d["N"] + d["heads"], H),
            conv_w=r(d["conv_dim"], d["K"], sc=0.2), conv_b=r(d["conv_dim"], sc=0.1),
            dt_bias=(torch.rand(d["heads"], generator=g) * 2 - 3).float().to(device),
            A_log=torch.log(torch.rand(d["heads"], generator=g) * 15 + 1).float().to(device),
            D=torch.ones(d["heads"], dtype=torch.float32, device=device),
            gnorm=torch.ones(d["d_inner"], dtype=dtype, device=device),
            out_proj=r(H, d["d_inner"])))
    embed = r(cfg.vocab_size, H)
    return Mamba2Weights(embed=embed, layers=layers, final_norm=torch.ones(H, dtype=dtype, device=device),
                         lm_head=embed if cfg.tie_word_embeddings else r(cfg.vocab_size, H))


def load_mamba2_weights(path, cfg: ModelConfig, dtype=torch.bfloat16, device="cpu") -> Mamba2Weights:
    """HF / MLX Mamba2 checkpoint (``backbone.layers.N.mixer.*``; reference src/models/mamba2.rs:860-970).
    Quantized projections are dequantised at load: the mixer's GEMMs run on bf16 weights. The conv
    weight is accepted as ``[C, 1, K]`` (PyTorch) or ``[C, K, 1]`` (MLX)."""
    from ..loading.checkpoint import TensorSource, _Getter

    src = TensorSource(path)
    g = _Getter(src, cfg, dtype, dequantize=True)
    d = mamba_dims(cfg)
    pre = "backbone." if any(k.startswith("backbone.") for k in src.keys()) else "model."

    def need(t, name):
        if t is None:
            raise KeyError(f"{path}: missing tensor {name}")
        return t.to(device)

    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"{pre}layers.{i}."
        cw = need(g.vec(p + "mixer.conv1d.weight"), p + "mixer.conv1d.weight")
        cw = cw.reshape(d["conv_dim"], d["K"]) if cw.shape[1] == 1 or cw.dim() == 2 else cw.squeeze(-1)
        cb = g.vec(p + "mixer.conv1d.bias")
        layers.append(Mamba2LayerWeights(
            norm=need(g.vec(p + "norm.weight"), p + "norm.weight"),
            in_proj=need(g.mat(p + "mixer.in_proj"), p + "mixer.in_proj"),
            conv_w=cw.float(), conv_b=None if cb is None else cb.float().to(device),
            dt_bias=need(g.vec(p + "mixer.dt_bias"), p + "mixer.dt_bias").float(),
            A_log=need(g.vec(p + "mixer.A_log"), p + "mixer.A_log").float(),
            D=need(g.vec(p + "mixer.D"), p + "mixer.D").float(),
            gnorm=need(g.vec(p + "mixer.norm.weight"), p + "mixer.norm.weight"),
            out_proj=need(g.mat(p + "mixer.out_proj"), p + "mixer.out_proj")))
    ename = pre + ("embeddings" if src.has(pre + "embeddings.weight") else "embed_tokens")
    embed = need(g.mat(ename), ename)
    head = g.mat("lm_head") if src.has("lm_head.weight") else None
    return Mamba2Weights(embed=embed, layers=layers,
                         final_norm=need(g.vec(pre + "norm_f.weight"), pre + "norm_f.weight"),
                         lm_head=embed if head is None else head.to(device))


def mamba2_config_dict(cfg: ModelConfig) -> dict:
    """``config.json`` content (HF ``Mamba2Config`` keys) that :func:`ModelConfig.from_dict` reads back."""
    d = mamba_dims(cfg)
    lim = cfg.extra["mamba"].get("time_step_limit", (0.0, float("inf")))
    out = dict(model_type="mamba2", vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
               num_hidden_layers=cfg.num_hidden_layers, num_heads=d["heads"], head_dim=d["P"], state_size=d["N"],
               conv_kernel=d["K"], n_groups=d["G"], intermediate_size=d["d_inner"],
               layer_norm_epsilon=cfg.rms_norm_eps, tie_word_embeddings=cfg.tie_word_embeddings)
    if lim[1] != float("inf") or lim[0] != 0.0:
        out["time_step_limit"] = [lim[0], min(lim[1], 3.0e38)]
    return out


def save_mamba2_checkpoint(path, cfg_dict: dict, w: Mamba2Weights) -> None:
    """Write ``config.json`` + ``model.safetensors`` with the HF tensor names (tests, conversions)."""
    import json
    from pathlib import Path

    from safetensors.torch import save_file

    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    t = {"backbone.embeddings.weight": w.embed, "backbone.norm_f.weight": w.final_norm}
    if w.lm_head is not w.embed:
        t["lm_head.weight"] = w.lm_head
    for i, lw in enumerate(w.layers):
        p = f"backbone.layers.{i}."
        t.update({p + "norm.weight": lw.norm, p + "mixer.in_proj.weight": lw.in_proj,
                  p + "mixer.conv1d.weight": lw.conv_w.unsqueeze(1), p + "mixer.dt_bias": lw.dt_bias,
                  p + "mixer.A_log": lw.A_log, p + "mixer.D": lw.D, p + "mixer.norm.weight": lw.gnorm,
                  p + "mixer.out_proj.weight": lw.out_proj})
        if lw.conv_b is not None:
            t[p + "mixer.conv1d.bias"] = lw.conv_b
    save_file({k: v.detach().cpu().contiguous() for k, v in t.items()}, str(path / "model.safetensors"))
    (path / "config.json").write_text(json.dumps(cfg_dict))


class Mamba2Model:
    """Executor with the interface the engine expects from a model (``forward`` / ``forward_hidden``
    / ``logits``), plus ``release_seq`` so the engine can return a sequence's state slot."""

    recurrent = True

    def __init__(self, cfg: ModelConfig, weights: Mamba2Weights, max_seqs: int = 256, comm=None):
        self.cfg, self.w = cfg, weights
        self.comm = comm or LocalComm()
        assert self.comm.tp_size == 1, "the Mamba2 executor is single-GPU"
        self.device = weights.final_norm.device
        self.d = mamba_dims(cfg)
        self.Hq = self.Hkv = 1                 # (attention geometry the engine asks for; unused)
        self.D = cfg.head_dim
        self.layer_range = range(cfg.num_hidden_layers)
        d, L = self.d, len(weights.layers)
        self.conv_state = torch.zeros(L, max_seqs, d["K"] - 1, d["conv_dim"], dtype=torch.float32, device=self.device)
        self.ssm_state = torch.zeros(L, max_seqs, d["heads"], d["P"], d["N"], dtype=torch.float32, device=self.device)
        self.slot_of: dict[int, int] = {}
        self.free = list(range(max_seqs - 1, -1, -1))
        self.A = [-torch.exp(lw.A_log.float()) for lw in weights.layers]
        for lw in weights.layers:                          # the conv kernel reads fp32 taps and bias
            lw.conv_w = lw.conv_w.float().contiguous()
            lw.conv_b = None if lw.conv_b is None else lw.conv_b.float().contiguous()
            lw.D, lw.dt_bias = lw.D.float().contiguous(), lw.dt_bias.float().contiguous()
        lim = cfg.extra["mamba"].get("time_step_limit", (0.0, float("inf")))
        self.dt_limit = (float(lim[0]), float(lim[1]))
        self.norm_groups = int(cfg.extra["mamba"].get("norm_groups", 1))   # Nemotron-H: one norm per B/C group
        self.gate_mode = cfg.extra["mamba"].get("gate_mode", "gate_then_norm")

    # ------------------------------------------------------------------ state slots
    def _slot(self, seq_id: int, resets: bool) -> int:
        """State slot of a sequence; ``resets`` says that this step's kernels start it from zero."""
        s = self.slot_of.get(seq_id)
        if s is None:
            if not self.free:
                raise RuntimeError("no free recurrent-state slot (raise max_seqs)")
            s = self.free.pop()
            self.slot_of[seq_id] = s
            if not resets:
                self.conv_state[:, s].zero_()
                self.ssm_state[:, s].zero_()
        return s

    def release_seq(self, seq_id: int) -> None:
        s = self.slot_of.pop(seq_id, None)
        if s is not None:
            self.free.append(s)

    # ------------------------------------------------------------------ one mixer
    def _mixer(self, li: int, lw: Mamba2LayerWeights, x: torch.Tensor, pieces) -> torch.Tensor:
        """x [T, H] normalised input; pieces = (slots, cu, reset int32 device tensors, number of decode
        rows, longest piece). Returns the
        gated, normalised SSM output [T, d_inner] (the input of out_proj)."""
        d = self.d
        di, GN = d["d_inner"], d["G"] * d["N"]
        slots, cu, reset, nd, max_len = pieces
        proj = ops.linear(x, lw.in_proj)                       # [T, 2*di + 2GN + heads]
        z, xBC, dt = proj[:, :di], proj[:, di:di + d["conv_dim"]], proj[:, di + d["conv_dim"]:]
        conv = rops.causal_conv_varlen(xBC, self.conv_state[li], slots, cu, reset, lw.conv_w, lw.conv_b, True, max_len)
        y = rops.ssm_scan_varlen(self.ssm_state[li], slots, cu, reset, conv[:, :di], dt, self.A[li],
                                 conv[:, di:di + GN], conv[:, di + GN:], lw.D, lw.dt_bias, True, self.dt_limit, nd)
        mode = self.gate_mode
        if mode == "gate_then_norm":           # Mamba2, Nemotron-H, Granite: RMSNorm(y * silu(z))
            return rops.gated_rmsnorm(y, z, lw.gnorm, self.cfg.rms_norm_eps, self.norm_groups)
        if mode == "none":                      # Falcon-H1 without the mixer norm: y * silu(z)
            return (y.float() * torch.nn.functional.silu(z.float())).to(y.dtype)
        # norm_then_gate: grouped RMSNorm(y) * weight, then * silu(z)
        v = y.float().reshape(y.shape[0], self.norm_groups, -1)
        v = (v * torch.rsqrt(v.pow(2).mean(-1, keepdim=True) + self.cfg.rms_norm_eps)).reshape(y.shape[0], -1)
        return (v * lw.gnorm.float() * torch.nn.functional.silu(z.float())).to(y.dtype)

    def pieces(self, b: StepBatch):
        """Per-step description of the ragged batch for the mixer kernels: (slots, cu, reset) as int32
        device tensors (one host-to-device copy), the number of decode rows and the longest piece.
        Allocates a state slot for every new sequence."""
        ids = getattr(b, "seq_ids", None)
        if ids is None:
            raise RuntimeError("recurrent models need StepBatch.seq_ids (the engine fills them in)")
        nd = b.num_decode
        cu = list(range(nd + 1))
        reset = [0] * nd
        pcu = b.pf_cu_q_host or [0]
        for j in range(b.num_prefill_seqs):
            cu.append(nd + pcu[j + 1])
            reset.append(1 if b.pf_starts[j] == 0 else 0)
        slots = [self._slot(i, bool(r)) for i, r in zip(ids, reset)]
        S = len(slots)
        meta = torch.tensor(slots + reset + cu, dtype=torch.int32).to(self.device, non_blocking=True)
        return (meta[:S], meta[2 * S:], meta[S:2 * S], nd, max(1 if nd else 0, b.pf_max_q_len))

    # ------------------------------------------------------------------ forward
    @torch.inference_mode()
    def forward_hidden(self, b: StepBatch, kv_layers=None, hidden_in: torch.Tensor | None = None) -> torch.Tensor:
        cfg = self.cfg
        pieces = self.pieces(b)
        h = hidden_in if hidden_in is not None else ops.embedding(b.token_ids, self.w.embed, cfg.embed_scale)
        for li, lw in enumerate(self.w.layers):
            x = ops.rmsnorm(h, lw.norm, cfg.rms_norm_eps, 0.0)
            h = ops.linear(self._mixer(li, lw, x, pieces), lw.out_proj, residual=h)
        return h

    def logits(self, h: torch.Tensor, rows: torch.Tensor | None) -> torch.Tensor:
        if rows is not None:
            h = h.index_select(0, rows)
        x = ops.rmsnorm(h, self.w.final_norm, self.cfg.rms_norm_eps, 0.0)
        return ops.linear(x, self.w.lm_head)

    def forward(self, b: StepBatch, kv_layers=None) -> torch.Tensor:
        return self.logits(self.forward_hidden(b, kv_layers), b.logits_rows)
