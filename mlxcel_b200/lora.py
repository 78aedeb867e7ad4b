"""LoRA adapters: fuse at load, or keep several adapters live with adjustable scales.

Reference behaviour (src/lora/*, src/lib/mlxcel-core/src/layers/runtime_lora.rs, route
``/lora-adapters``): an adapter is a directory with ``adapter_config.json`` (rank ``r``, ``alpha`` /
``scale``, target modules) and ``adapters.safetensors`` holding, per adapted linear,
``<module>.lora_a`` ``[in, r]`` and ``<module>.lora_b`` ``[r, out]`` (MLX layout; the PEFT layout
``lora_A.weight`` ``[r, in]`` / ``lora_B.weight`` ``[out, r]`` is accepted too). Adapters are either
fused into the weights at load time or attached at run time with a per-adapter scale that
``POST /lora-adapters`` changes while the server runs.

Here both modes are ONE mechanism: the weight delta ``scale * (B A)`` is added to the (sharded,
possibly norm-folded) projection weight in place, and a live scale change adds
``(new - old) * (B A)`` — a few GEMMs of rank ``r`` per adapted matrix, after which decode runs
at full speed with no per-token adapter work. Per-request adapter selection (different adapters
inside one batch) is not supported by this scheme.
"""
from __future__ import annotations

import json
import re
from dataclasses import dataclass, field
from pathlib import Path

import torch

from .models.weights import ModelWeights, QuantizedTensor

# adapter module name -> (LayerWeights attribute, row slice selector inside the fused tensor)
_TARGETS = {
    "q_proj": ("wqkv", "q"), "k_proj": ("wqkv", "k"), "v_proj": ("wqkv", "v"), "qkv_proj": ("wqkv", "all"),
    "o_proj": ("wo", "all"), "gate_proj": ("w_gate_up", "gate"), "up_proj": ("w_gate_up", "up"),
    "down_proj": ("w_down", "all"),
}
_KEY = re.compile(r"(?:^|\.)layers\.(\d+)\.(?:self_attn|attention|mlp|feed_forward)\.(\w+)\.lora_([abAB])(?:\.weight)?$")


@dataclass
class Adapter:
    id: int
    path: str
    scale: float                      # currently applied multiplier (0 = detached)
    alpha_over_r: float               # the adapter's own alpha / r
    mats: dict = field(default_factory=dict)   # (layer, module) -> (A [r, in], B [out, r]) fp32 on CPU


def load_adapter(path: str | Path, adapter_id: int = 0) -> Adapter:
    path = Path(path)
    cfg = {}
    for name in ("adapter_config.json", "config.json"):
        if (path / name).exists():
            cfg = json.loads((path / name).read_text())
            break
    lp = cfg.get("lora_parameters", cfg)
    r = int(lp.get("rank", lp.get("r", 8)))
    if "scale" in lp:
        aor = float(lp["scale"])
    else:
        aor = float(lp.get("alpha", lp.get("lora_alpha", r))) / r
    tensors: dict[str, torch.Tensor] = {}
    files = sorted(path.glob("*.safetensors"))
    if not files:
        raise FileNotFoundError(f"no adapter safetensors under {path}")
    from safetensors.torch import load_file

    for f in files:
        tensors.update(load_file(str(f)))
    halves: dict[tuple[int, str], dict[str, torch.Tensor]] = {}
    for k, v in tensors.items():
        m = _KEY.search(k)
        if not m:
            continue
        peft = m.group(3).isupper() or k.endswith(".weight")
        halves.setdefault((int(m.group(1)), m.group(2)), {})[m.group(3).lower()] = (v.float(), peft)
    ad = Adapter(adapter_id, str(path), 0.0, aor)
    for key, ab in halves.items():
        if "a" not in ab or "b" not in ab:
            continue
        (a, peft), (b, _) = ab["a"], ab["b"]
        if not peft:                                                  # MLX layout [in, r] / [r, out]
            a, b = a.t().contiguous(), b.t().contiguous()
        ad.mats[key] = (a, b)                                         # A [r, in], B [out, r]
    if not ad.mats:
        raise ValueError(f"{path}: no lora_a / lora_b pairs recognised")
    return ad


class LoraManager:
    """Owns the adapters of one executor's weights (one per tensor-parallel rank)."""

    def __init__(self, cfg, weights: ModelWeights, tp_rank: int = 0, tp_size: int = 1):
        self.cfg, self.w = cfg, weights
        self.tp_rank, self.tp_size = tp_rank, tp_size
        self.adapters: dict[int, Adapter] = {}

    # ------------------------------------------------------------------ public
    def add(self, path: str | Path, scale: float = 1.0, adapter_id: int | None = None) -> Adapter:
        aid = adapter_id if adapter_id is not None else (max(self.adapters, default=-1) + 1)
        ad = load_adapter(path, aid)
        self.adapters[aid] = ad
        self.set_scale(aid, scale)
        return ad

    def set_scale(self, adapter_id: int, scale: float) -> None:
        ad = self.adapters[adapter_id]
        delta = float(scale) - ad.scale
        if delta != 0.0:
            self._apply(ad, delta)
            ad.scale = float(scale)

    def listing(self) -> list[dict]:
        return [{"id": a.id, "path": a.path, "scale": a.scale} for a in self.adapters.values()]

    # ------------------------------------------------------------------ internals
    def _rows(self, attr: str, sel: str, lw) -> slice:
        cfg, tp = self.cfg, self.tp_size
        D = cfg.head_dim
        hq, hkv = cfg.num_attention_heads // tp, max(1, cfg.num_key_value_heads // tp)
        if attr == "wqkv":
            q, k = hq * D, hkv * D
            return {"q": slice(0, q), "k": slice(q, q + k), "v": slice(q + k, q + 2 * k),
                    "all": slice(0, q + 2 * k)}[sel]
        if attr == "w_gate_up":
            inter = lw.w_gate_up.shape[0] // 2
            return {"gate": slice(0, inter), "up": slice(inter, 2 * inter)}[sel]
        return slice(None)

    def _shard(self, attr: str, sel: str, a: torch.Tensor, b: torch.Tensor):
        """The part of (A [r, in], B [out, r]) that lands on this rank's shard of the weight."""
        tp, rk = self.tp_size, self.tp_rank
        if tp == 1:
            return a, b
        if attr in ("wo", "w_down"):            # row-parallel: input dimension is split
            n = a.shape[1] // tp
            return a[:, rk * n:(rk + 1) * n], b
        n = b.shape[0] // tp                    # column-parallel: output rows are split
        return a, b[rk * n:(rk + 1) * n]

    @torch.no_grad()
    def _apply(self, ad: Adapter, delta_scale: float) -> None:
        for (li, module), (a, b) in ad.mats.items():
            if module not in _TARGETS or li >= len(self.w.layers):
                continue
            attr, sel = _TARGETS[module]
            lw = self.w.layers[li]
            w = getattr(lw, attr, None)
            if w is None:
                continue
            if isinstance(w, QuantizedTensor):
                raise ValueError("LoRA adapters need dense (bf16) projection weights; load with dequantize=True")
            a_s, b_s = self._shard(attr, sel, a, b)
            upd = (b_s.to(w.device) @ a_s.to(w.device)) * (delta_scale * ad.alpha_over_r)   # [out, in] fp32
            gain = getattr(w, "_norm_gain", None)          # RMSNorm weight folded into this projection
            if gain is not None:
                upd = upd * gain.to(upd.device).unsqueeze(0)
            rows = self._rows(attr, sel, lw)
            w[rows] = (w[rows].float() + upd).to(w.dtype)
            if hasattr(w, "_gemm_tiles"):
                del w._gemm_tiles
