"""MLX / HF safetensors checkpoints → :class:`ModelWeights`.

Covers what the reference's loader does for decoder LMs (src/loading/mod.rs:788,
src/models/sanitize.rs:2148, src/lib/mlxcel-core/src/weights.rs:79-955):

* shard index (``model.safetensors.index.json``) with a glob fallback,
* weight-name sanitising (HF ``model.layers.N.self_attn.q_proj`` …, fused ``qkv_proj`` /
  ``gate_up_proj`` of Phi-3, GPT-OSS ``mlp.experts.{gate_up_proj,down_proj}`` with interleaved
  gate/up, Mixtral ``block_sparse_moe.experts.N.w1/w2/w3``, Qwen-MoE ``mlp.experts.N.*_proj``,
  MLX ``switch_mlp`` stacks),
* MLX quantized triplets (``.weight`` uint32 + ``.scales`` + ``.biases``) kept packed as
  :class:`QuantizedTensor` (or dequantized on request), with the mode inferred the way the
  reference does (biases ⇒ affine, bits 8 ⇒ mxfp8, else mxfp4; layers.rs:2322-2332),
* fusing q/k/v → ``wqkv`` and gate/up → ``w_gate_up`` rows, tied embeddings,
* tensor / expert / pipeline sharding at load time (:mod:`mlxcel_b200.loading.shard`).
"""
from __future__ import annotations

import glob
import json
import os
import re
from pathlib import Path

import torch

from ..config import ModelConfig, QuantConfig
from ..models.weights import LayerWeights, ModelWeights, QuantizedTensor
from .shard import shard_weights


class TensorSource:
    """Lazy name → tensor access over one or more safetensors shards."""

    def __init__(self, path: str | Path):
        from safetensors import safe_open

        self.dir = Path(path)
        self._open = safe_open
        self.index: dict[str, str] = {}
        idx = self.dir / "model.safetensors.index.json"
        if idx.exists():
            self.index = dict(json.loads(idx.read_text())["weight_map"])
        else:
            files = sorted(glob.glob(str(self.dir / "*.safetensors")))
            if not files:
                raise FileNotFoundError(f"no safetensors files under {self.dir}")
            for f in files:
                with safe_open(f, framework="pt") as h:
                    for k in h.keys():
                        self.index[k] = os.path.basename(f)
        self._handles: dict[str, object] = {}

    def keys(self):
        return self.index.keys()

    def has(self, name: str) -> bool:
        return name in self.index

    def get(self, name: str) -> torch.Tensor:
        f = self.index[name]
        h = self._handles.get(f)
        if h is None:
            real = (self.dir / f).resolve()
            if not str(real).startswith(str(self.dir.resolve())) and not real.exists():
                raise FileNotFoundError(f)
            h = self._open(str(self.dir / f), framework="pt")
            self._handles[f] = h
        return h.get_tensor(name)

    def footprint(self) -> int:
        """Bytes of all tensors (header-only would need the raw header; sizes via slices)."""
        total = 0
        for name in self.index:
            sl = self._handle(name).get_slice(name)
            n = 1
            for d in sl.get_shape():
                n *= d
            total += n * {"BF16": 2, "F16": 2, "F32": 4, "U32": 4, "I32": 4, "U8": 1, "I8": 1,
                          "F8_E4M3": 1, "I64": 8}.get(sl.get_dtype(), 2)
        return total

    def _handle(self, name):
        self.get  # noqa: B018 - ensure attribute exists
        f = self.index[name]
        if f not in self._handles:
            self._handles[f] = self._open(str(self.dir / f), framework="pt")
        return self._handles[f]


def _infer_quant(packed: torch.Tensor, scales: torch.Tensor, biases, qc: QuantConfig | None) -> QuantizedTensor:
    """Mode / bits / group of one quantized matrix, verified against the tensor shapes
    (packed_in * 32 == bits * in, in == groups * group_size)."""
    groups = scales.shape[-1]
    words = packed.shape[-1]
    if biases is not None:
        mode = "affine"
    elif qc is not None and qc.mode in ("mxfp4", "mxfp8"):
        mode = qc.mode
    elif qc is not None and qc.bits == 8:
        mode = "mxfp8"
    else:
        mode = "mxfp4"
    cands = [(qc.bits, qc.group_size)] if qc is not None and qc.mode != "none" else []
    cands += [(b, g) for g in (64, 32, 128, 16) for b in (4, 8, 2, 3, 5, 6)]
    for bits, g in cands:
        inn = groups * g
        if words * 32 == bits * inn:
            if mode == "mxfp4" and bits != 4:
                continue
            if mode == "mxfp8" and bits != 8:
                continue
            return QuantizedTensor(packed.view(torch.int32) if packed.dtype != torch.int32 else packed,
                                   scales, biases, bits, g, mode)
    raise ValueError(f"cannot reconcile quantized shapes packed={tuple(packed.shape)} scales={tuple(scales.shape)}")


class _Getter:
    def __init__(self, src: TensorSource, cfg: ModelConfig, dtype, dequantize: bool):
        self.src, self.cfg, self.dtype, self.deq = src, cfg, dtype, dequantize

    def has(self, base: str) -> bool:
        return self.src.has(base + ".weight") or self.src.has(base)

    def vec(self, name: str):
        if not self.src.has(name):
            return None
        return self.src.get(name).to(self.dtype)

    def mat(self, base: str):
        """Linear weight ``base.weight`` as bf16 tensor or QuantizedTensor."""
        name = base + ".weight" if self.src.has(base + ".weight") else base
        if not self.src.has(name):
            return None
        w = self.src.get(name)
        sname = base + ".scales"
        if self.src.has(sname) and w.dtype in (torch.uint32, torch.int32, torch.uint8):
            scales = self.src.get(sname)
            biases = self.src.get(base + ".biases") if self.src.has(base + ".biases") else None
            qt = _infer_quant(w, scales, biases, self.cfg.quantization.for_module(base))
            if self.deq:
                from ..ops.quant import dequantize_ref
                return dequantize_ref(qt, self.dtype)
            if qt.mode == "affine":
                qt.scales, qt.biases = qt.scales.to(self.dtype), qt.biases.to(self.dtype)
            return qt
        return w.to(self.dtype)


def _cat_rows(parts):
    parts = [p for p in parts if p is not None]
    if not parts:
        return None
    if isinstance(parts[0], QuantizedTensor):
        q = parts[0]
        same = all(isinstance(p, QuantizedTensor) and (p.bits, p.group_size, p.mode) == (q.bits, q.group_size, q.mode)
                   for p in parts)
        if not same:
            from ..ops.quant import dequantize_ref
            return torch.cat([dequantize_ref(p, torch.bfloat16) if isinstance(p, QuantizedTensor) else p
                              for p in parts], dim=-2)
        return QuantizedTensor(torch.cat([p.packed for p in parts], dim=-2),
                               torch.cat([p.scales for p in parts], dim=-2),
                               None if q.biases is None else torch.cat([p.biases for p in parts], dim=-2),
                               q.bits, q.group_size, q.mode)
    return torch.cat(parts, dim=0)


def _stack(parts):
    if isinstance(parts[0], QuantizedTensor):
        q = parts[0]
        return QuantizedTensor(torch.stack([p.packed for p in parts]), torch.stack([p.scales for p in parts]),
                               None if q.biases is None else torch.stack([p.biases for p in parts]),
                               q.bits, q.group_size, q.mode)
    return torch.stack(parts)
