"""BERT-family text encoders for embeddings (bidirectional attention, post-LayerNorm blocks).

``h = LN(word + position + token_type)``; per layer ``h = LN(h + W_o attn(h))``,
``h = LN(h + W_2 gelu(W_1 h))``; the sentence vector is the [CLS] state or the mean over tokens,
L2-normalised. Reference: src/embeddings/ (BERT / sentence-transformers style embedders) and
src/models/bert.rs.

Projections run through the package's GEMM (``ops.linear``), LayerNorm and GELU through its kernels;
the attention itself is one non-causal softmax(QK^T)V per text through PyTorch's
``scaled_dot_product_attention`` (texts are short and the path is not a serving hot loop).
"""
from __future__ import annotations

import json
from dataclasses import dataclass
from pathlib import Path

import torch
import torch.nn.functional as F

from .. import ops
from ..ops import recurrent as rops


@dataclass
class EncoderLayer:
    wqkv: torch.Tensor
    bqkv: torch.Tensor
    wo: torch.Tensor
    bo: torch.Tensor
    ln1_w: torch.Tensor
    ln1_b: torch.Tensor
    w1: torch.Tensor
    b1: torch.Tensor
    w2: torch.Tensor
    b2: torch.Tensor
    ln2_w: torch.Tensor
    ln2_b: torch.Tensor


class BertEncoder:
    def __init__(self, cfg: dict, tensors: dict, dtype=torch.bfloat16, device="cpu"):
        self.heads = int(cfg["num_attention_heads"])
        self.hidden = int(cfg["hidden_size"])
        self.eps = float(cfg.get("layer_norm_eps", 1e-12))
        self.act = {"gelu": "gelu", "gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh", "relu": None}.get(
            cfg.get("hidden_act", "gelu"), "gelu")
        self.max_len = int(cfg.get("max_position_embeddings", 512))
        self.device = torch.device(device)
        pre = "bert." if any(k.startswith("bert.") for k in tensors) else ""

        def t(name):
            return tensors[pre + name].to(dtype).to(self.device).contiguous()

        e = "embeddings."
        self.word, self.pos = t(e + "word_embeddings.weight"), t(e + "position_embeddings.weight")
        self.type0 = t(e + "token_type_embeddings.weight")[0] if pre + e + "token_type_embeddings.weight" in tensors else None
        self.emb_ln = (t(e + "LayerNorm.weight"), t(e + "LayerNorm.bias"))
        self.layers = []
        for i in range(int(cfg["num_hidden_layers"])):
            p = f"encoder.layer.{i}."
            a = p + "attention."
            self.layers.append(EncoderLayer(
                wqkv=torch.cat([t(a + f"self.{n}.weight") for n in ("query", "key", "value")], 0).contiguous(),
                bqkv=torch.cat([t(a + f"self.{n}.bias") for n in ("query", "key", "value")]).contiguous(),
                wo=t(a + "output.dense.weight"), bo=t(a + "output.dense.bias"),
                ln1_w=t(a + "output.LayerNorm.weight"), ln1_b=t(a + "output.LayerNorm.bias"),
                w1=t(p + "intermediate.dense.weight"), b1=t(p + "intermediate.dense.bias"),
                w2=t(p + "output.dense.weight"), b2=t(p + "output.dense.bias"),
                ln2_w=t(p + "output.LayerNorm.weight"), ln2_b=t(p + "output.LayerNorm.bias")))

    @staticmethod
    def from_pretrained(path, dtype=torch.bfloat16, device="cpu") -> "BertEncoder":
        from ..loading.checkpoint import TensorSource

        cfg = json.loads((Path(path) / "config.json").read_text())
        src = TensorSource(path)
        return BertEncoder(cfg, {k: src.get(k) for k in src.keys()}, dtype, device)

    @torch.inference_mode()
    def hidden_states(self, ids: list[int]) -> torch.Tensor:
        """Final hidden states [T, H] of one text (no padding: one text per call)."""
        ids = ids[: self.max_len]
        T, H, nh = len(ids), self.hidden, self.heads
        tok = torch.tensor(ids, dtype=torch.long, device=self.device)
        h = self.word[tok].float() + self.pos[:T].float()
        if self.type0 is not None:
            h = h + self.type0.float()
        h = rops.layernorm(h.to(self.word.dtype), *self.emb_ln, self.eps)
        for lw in self.layers:
            qkv = ops.linear(h, lw.wqkv, bias=lw.bqkv).view(T, 3, nh, H // nh)
            q, k, v = (qkv[:, j].transpose(0, 1).unsqueeze(0) for j in range(3))          # [1, nh, T, D]
            a = F.scaled_dot_product_attention(q, k, v).squeeze(0).transpose(0, 1).reshape(T, H).contiguous()
            h = rops.layernorm(ops.linear(a, lw.wo, bias=lw.bo, residual=h), lw.ln1_w, lw.ln1_b, self.eps)
            u = ops.linear(h, lw.w1, bias=lw.b1)
            u = torch.relu(u) if self.act is None else rops.activation(u, self.act)
            h = rops.layernorm(ops.linear(u, lw.w2, bias=lw.b2, residual=h), lw.ln2_w, lw.ln2_b, self.eps)
        return h

    def embed(self, ids: list[int], pooling: str = "mean", normalize: bool = True) -> torch.Tensor:
        h = self.hidden_states(ids).float()
        v = h[0] if pooling == "cls" else h.mean(0)
        return v / v.norm().clamp_min(1e-12) if normalize else v
