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
        self.type_emb = t(e + "token_type_embeddings.weight") if pre + e + "token_type_embeddings.weight" in tensors else None
        self.type0 = None if self.type_emb is None else self.type_emb[0]
        # optional heads: tanh pooler over [CLS] and a linear classifier (sequence- or token-level)
        head = lambda n: tensors[n].to(dtype).to(self.device).contiguous() if n in tensors else None  # noqa: E731
        self.pooler = (head(pre + "pooler.dense.weight"), head(pre + "pooler.dense.bias"))
        self.classifier = (head("classifier.weight"), head("classifier.bias"))
        self.token_head = any("TokenClassification" in a for a in cfg.get("architectures") or [])
        self.id2label = {int(k): v for k, v in (cfg.get("id2label") or {}).items()}
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
    def hidden_states(self, ids: list[int], type_ids: list[int] | None = None) -> torch.Tensor:
        """Final hidden states [T, H] of one text (no padding: one text per call). ``type_ids`` marks the
        segments of a sentence pair (0 / 1); all zeros when absent."""
        ids = ids[: self.max_len]
        T, H, nh = len(ids), self.hidden, self.heads
        tok = torch.tensor(ids, dtype=torch.long, device=self.device)
        h = self.word[tok].float() + self.pos[:T].float()
        if self.type_emb is not None and type_ids is not None:
            h = h + self.type_emb[torch.tensor(type_ids[:T], dtype=torch.long, device=self.device)].float()
        elif self.type0 is not None:
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
        v = h[0] if pooling == "cls" else h[-1] if pooling == "last" else h.mean(0)
        return v / v.norm().clamp_min(1e-12) if normalize else v

    @torch.inference_mode()
    def sequence_logits(self, ids: list[int], type_ids: list[int] | None = None) -> torch.Tensor:
        """Cross-encoder head: ``classifier(tanh(pooler([CLS])))`` -> [num_labels] fp32 (a reranker's
        relevance score is logit 0 of a one-label head)."""
        if self.classifier[0] is None or self.token_head:
            raise ValueError("checkpoint has no sequence-classification head")
        v = self.hidden_states(ids, type_ids)[:1]
        if self.pooler[0] is not None:
            v = torch.tanh(ops.linear(v, self.pooler[0], bias=self.pooler[1]).float()).to(v.dtype)
        return ops.linear(v, self.classifier[0], bias=self.classifier[1])[0].float()

    @torch.inference_mode()
    def token_logits(self, ids: list[int]) -> torch.Tensor:
        """Token-classification head: one row of label logits per token, [T, num_labels] fp32."""
        if self.classifier[0] is None or not self.token_head:
            raise ValueError("checkpoint has no token-classification head")
        return ops.linear(self.hidden_states(ids), self.classifier[0], bias=self.classifier[1]).float()


def bio_spans(labels: list[str]) -> list[tuple[int, int, str]]:
    """Merge per-token BIO / BIOES labels into ``(first token, one past last token, entity)`` spans:
    ``B-X`` / ``S-X`` opens a span, ``I-X`` / ``E-X`` of the same entity extends it, anything else closes it."""
    out, start, ent = [], None, None
    for i, lab in enumerate(list(labels) + ["O"]):
        tag, _, name = lab.partition("-")
        if start is not None and not (tag in ("I", "E") and name == ent):
            out.append((start, i, ent))
            start = ent = None
        if start is None and lab != "O" and name:
            start, ent = i, name                    # a stray I-X also opens a span, as taggers commonly emit
    return out


def bio_viterbi(log_probs: torch.Tensor, labels: list[str]) -> list[int]:
    """Best label path under the BIO / BIOES grammar: ``I-X`` / ``E-X`` may only follow ``B-X`` or ``I-X``
    of the same entity, ``B-X`` / ``I-X`` of a BIOES scheme may not be followed by ``O`` when the scheme
    has ``E-`` tags, and a path may not start inside an entity. ``log_probs`` is [T, num_labels]
    (reference src/token_classification/, viterbi decoding; ``--argmax`` turns it off)."""
    T, L = log_probs.shape
    parts = [lab.partition("-") for lab in labels]
    tag, ent = [p[0] if p[1] else "O" for p in parts], [p[2] for p in parts]
    bioes = any(t == "E" for t in tag)
    neg = float("-inf")
    trans = torch.zeros(L, L)
    for a in range(L):
        for b in range(L):
            inside_a = tag[a] in ("B", "I")
            if tag[b] in ("I", "E") and not (inside_a and ent[a] == ent[b]):
                trans[a, b] = neg                    # continuing an entity that is not open
            elif bioes and inside_a and not (tag[b] in ("I", "E") and ent[a] == ent[b]):
                trans[a, b] = neg                    # BIOES: an open entity must be closed by its E tag
    start = torch.tensor([neg if t in ("I", "E") else 0.0 for t in tag])
    lp = log_probs.float().cpu()
    score = start + lp[0]
    back = []
    for t in range(1, T):
        cand = score[:, None] + trans                # [from, to]
        best, arg = cand.max(dim=0)
        back.append(arg)
        score = best + lp[t]
    if bioes:                                        # a path may not end inside an entity
        score = score + torch.tensor([neg if t in ("B", "I") else 0.0 for t in tag])
    path = [int(score.argmax())]
    for arg in reversed(back):
        path.append(int(arg[path[-1]]))
    return path[::-1]


class ModernBertEncoder:
    """ModernBERT: pre-norm blocks with bias-free LayerNorm, fused Wqkv, rotary embedding (one base for
    the global layers, another for the local ones), bidirectional attention that is windowed
    (``|i - j| <= local_attention // 2``) on all but every ``global_attn_every_n_layers``-th layer, and a
    GeGLU MLP ``Wo(act(a) * b)`` with ``[a | b] = Wi(x)`` (reference src/embeddings/, src/models/modernbert.rs)."""

    def __init__(self, cfg: dict, tensors: dict, dtype=torch.bfloat16, device="cpu"):
        from ..ops.reference import rope_inv_freq

        self.heads, self.hidden = int(cfg["num_attention_heads"]), int(cfg["hidden_size"])
        self.eps = float(cfg.get("norm_eps", 1e-5))
        self.act = {"gelu": "gelu", "gelu_new": "gelu_tanh", "gelu_pytorch_tanh": "gelu_tanh", "silu": "silu"}.get(
            cfg.get("hidden_activation", "gelu"), "gelu")
        self.max_len = int(cfg.get("max_position_embeddings", 8192))
        self.device = torch.device(device)
        n = int(cfg["num_hidden_layers"])
        every = int(cfg.get("global_attn_every_n_layers", 3))
        types = cfg.get("layer_types") or ["full_attention" if i % every == 0 else "sliding_attention" for i in range(n)]
        self.local = [t != "full_attention" for t in types]
        self.window = int(cfg.get("local_attention", 128)) // 2
        rp = cfg.get("rope_parameters") or {}
        g_theta = float((rp.get("full_attention") or {}).get("rope_theta", cfg.get("global_rope_theta", 160000.0)))
        l_theta = float((rp.get("sliding_attention") or {}).get("rope_theta", cfg.get("local_rope_theta", 10000.0)))
        D = self.hidden // self.heads
        self.inv_global = rope_inv_freq(D, g_theta, None)[0].to(self.device)
        self.inv_local = rope_inv_freq(D, l_theta, None)[0].to(self.device)
        pre = "model." if any(k.startswith("model.") for k in tensors) else ""

        def t(name):
            return tensors[pre + name].to(dtype).to(self.device).contiguous()

        def opt(name):
            return t(name) if pre + name in tensors else None

        self.word, self.emb_norm = t("embeddings.tok_embeddings.weight"), t("embeddings.norm.weight")
        self.final_norm = t("final_norm.weight")
        self.layers = [dict(attn_norm=opt(f"layers.{i}.attn_norm.weight"), wqkv=t(f"layers.{i}.attn.Wqkv.weight"),
                            wo=t(f"layers.{i}.attn.Wo.weight"), mlp_norm=t(f"layers.{i}.mlp_norm.weight"),
                            wi=t(f"layers.{i}.mlp.Wi.weight"), wo2=t(f"layers.{i}.mlp.Wo.weight")) for i in range(n)]

    @staticmethod
    def from_pretrained(path, dtype=torch.bfloat16, device="cpu") -> "ModernBertEncoder":
        from ..loading.checkpoint import TensorSource

        cfg = json.loads((Path(path) / "config.json").read_text())
        src = TensorSource(path)
        return ModernBertEncoder(cfg, {k: src.get(k) for k in src.keys()}, dtype, device)

    @torch.inference_mode()
    def hidden_states(self, ids: list[int]) -> torch.Tensor:
        from ..ops.reference import apply_rope

        ids = ids[: self.max_len]
        T, H, nh = len(ids), self.hidden, self.heads
        D = H // nh
        tok = torch.tensor(ids, dtype=torch.long, device=self.device)
        pos = torch.arange(T, device=self.device)
        far = (pos[:, None] - pos[None, :]).abs() > self.window            # True = masked out on local layers
        h = rops.layernorm(self.word[tok], self.emb_norm, None, self.eps)
        for lw, local in zip(self.layers, self.local):
            x = h if lw["attn_norm"] is None else rops.layernorm(h, lw["attn_norm"], None, self.eps)
            qkv = ops.linear(x, lw["wqkv"]).view(T, 3, nh, D)
            inv = self.inv_local if local else self.inv_global
            q = apply_rope(qkv[:, 0], pos, inv, D, False).to(h.dtype)
            k = apply_rope(qkv[:, 1], pos, inv, D, False).to(h.dtype)
            q, k, v = (t.transpose(0, 1).unsqueeze(0) for t in (q, k, qkv[:, 2]))
            mask = (~far)[None, None] if local else None
            a = F.scaled_dot_product_attention(q, k, v, attn_mask=mask).squeeze(0).transpose(0, 1).reshape(T, H)
            h = ops.linear(a.contiguous(), lw["wo"], residual=h)
            u = ops.linear(rops.layernorm(h, lw["mlp_norm"], None, self.eps), lw["wi"])
            half = u.shape[1] // 2
            g = rops.activation(u[:, :half].contiguous(), self.act)
            h = ops.linear((g.float() * u[:, half:].float()).to(h.dtype), lw["wo2"], residual=h)
        return rops.layernorm(h, self.final_norm, None, self.eps)

    def embed(self, ids: list[int], pooling: str = "mean", normalize: bool = True) -> torch.Tensor:
        h = self.hidden_states(ids).float()
        v = h[0] if pooling == "cls" else h.mean(0)
        return v / v.norm().clamp_min(1e-12) if normalize else v


class SiglipTextEncoder:
    """SigLIP text tower: token + learned position embeddings, pre-LayerNorm blocks with biased
    projections and tanh-GELU MLPs, bidirectional attention, a final LayerNorm, and the sentence vector
    ``head(last token)`` that is compared with the image tower's pooled output
    (reference src/models/siglip_text.rs). Loads a text-only checkpoint (``siglip_text_model``) or the
    text half of a full SigLIP checkpoint."""

    def __init__(self, cfg: dict, tensors: dict, dtype=torch.bfloat16, device="cpu"):
        cfg = cfg.get("text_config") or cfg
        self.device, self.dtype = torch.device(device), dtype
        self.hidden, self.heads = int(cfg.get("hidden_size", 768)), int(cfg.get("num_attention_heads", 12))
        self.eps = float(cfg.get("layer_norm_eps", 1e-6))
        self.max_len = int(cfg.get("max_position_embeddings", 64))
        act = cfg.get("hidden_act", "gelu_pytorch_tanh")
        self.act = "gelu_tanh" if "tanh" in act else "gelu"
        root = next((r for r in ("text_model.", "model.text_model.", "") if r + "embeddings.token_embedding.weight" in tensors), None)
        if root is None:
            raise KeyError("no SigLIP text tower in this checkpoint")

        def t(name):
            return tensors[root + name].to(dtype).to(self.device).contiguous()
        self.word, self.pos = t("embeddings.token_embedding.weight"), t("embeddings.position_embedding.weight")
        self.layers = []
        for i in range(int(cfg.get("num_hidden_layers", 12))):
            p, a = f"encoder.layers.{i}.", f"encoder.layers.{i}.self_attn."
            self.layers.append(EncoderLayer(
                wqkv=torch.cat([t(a + f"{n}_proj.weight") for n in "qkv"]).contiguous(),
                bqkv=torch.cat([t(a + f"{n}_proj.bias") for n in "qkv"]).contiguous(),
                wo=t(a + "out_proj.weight"), bo=t(a + "out_proj.bias"),
                ln1_w=t(p + "layer_norm1.weight"), ln1_b=t(p + "layer_norm1.bias"),
                w1=t(p + "mlp.fc1.weight"), b1=t(p + "mlp.fc1.bias"), w2=t(p + "mlp.fc2.weight"), b2=t(p + "mlp.fc2.bias"),
                ln2_w=t(p + "layer_norm2.weight"), ln2_b=t(p + "layer_norm2.bias")))
        self.final_ln = (t("final_layer_norm.weight"), t("final_layer_norm.bias"))
        self.head = (t("head.weight"), t("head.bias")) if root + "head.weight" in tensors else None

    @staticmethod
    def from_pretrained(path, dtype=torch.bfloat16, device="cpu") -> "SiglipTextEncoder":
        from ..loading.checkpoint import TensorSource

        cfg = json.loads((Path(path) / "config.json").read_text())
        src = TensorSource(path)
        return SiglipTextEncoder(cfg, {k: src.get(k) for k in src.keys() if "vision_model" not in k}, dtype, device)

    @torch.inference_mode()
    def hidden_states(self, ids: list[int]) -> torch.Tensor:
        ids = ids[: self.max_len]
        T, H, nh = len(ids), self.hidden, self.heads
        tok = torch.tensor(ids, dtype=torch.long, device=self.device)
        h = (self.word[tok].float() + self.pos[:T].float()).to(self.dtype)
        for lw in self.layers:
            y = rops.layernorm(h, lw.ln1_w, lw.ln1_b, self.eps)
            qkv = ops.linear(y, lw.wqkv, bias=lw.bqkv).view(T, 3, nh, H // nh)
            q, k, v = (qkv[:, j].transpose(0, 1).unsqueeze(0) for j in range(3))
            a = F.scaled_dot_product_attention(q, k, v).squeeze(0).transpose(0, 1).reshape(T, H).contiguous()
            h = ops.linear(a, lw.wo, bias=lw.bo, residual=h)
            y = rops.layernorm(h, lw.ln2_w, lw.ln2_b, self.eps)
            h = ops.linear(rops.activation(ops.linear(y, lw.w1, bias=lw.b1), self.act), lw.w2, bias=lw.b2, residual=h)
        return rops.layernorm(h, *self.final_ln, self.eps)

    def embed(self, ids: list[int], pooling: str = "last", normalize: bool = True) -> torch.Tensor:
        """``pooling="last"`` (the model's own sentence vector: the head over the last token), ``"mean"`` or
        ``"cls"`` over the final hidden states."""
        h = self.hidden_states(ids)
        if pooling == "last":
            v = h[-1:]
            v = (ops.linear(v, self.head[0], bias=self.head[1]) if self.head is not None else v)[0].float()
        else:
            v = h.float()[0] if pooling == "cls" else h.float().mean(0)
        return v / v.norm().clamp_min(1e-12) if normalize else v


def load_encoder(path, dtype=torch.bfloat16, device="cpu"):
    """The encoder class for a checkpoint's ``model_type`` (bert, modernbert, deberta-v2, siglip text)."""
    mt = json.loads((Path(path) / "config.json").read_text()).get("model_type")
    from .deberta import DebertaV2Encoder
    cls = {"bert": BertEncoder, "modernbert": ModernBertEncoder, "deberta-v2": DebertaV2Encoder,
           "siglip_text_model": SiglipTextEncoder, "siglip": SiglipTextEncoder}.get(mt)
    if cls is None:
        raise ValueError(f"unsupported encoder model_type {mt!r}")
    enc = cls.from_pretrained(path, dtype, device)
    enc.default_pooling, enc.default_normalize = sentence_transformers_defaults(path)
    if cls is SiglipTextEncoder and not (Path(path) / "1_Pooling" / "config.json").is_file():
        enc.default_pooling = "last"
    return enc


def sentence_transformers_defaults(path) -> tuple[str, bool]:
    """Pooling and normalisation a sentence-transformers checkpoint declares: ``1_Pooling/config.json``
    (``pooling_mode_cls_token`` / ``pooling_mode_mean_tokens`` / ``pooling_mode_lasttoken``) and a
    ``Normalize`` entry in ``modules.json``. Without those files: mean pooling, normalised (reference
    src/embeddings/, pooling read the same way)."""
    root = Path(path)
    pooling, normalize = "mean", True
    pc = root / "1_Pooling" / "config.json"
    if pc.is_file():
        c = json.loads(pc.read_text())
        pooling = ("cls" if c.get("pooling_mode_cls_token") else "last" if c.get("pooling_mode_lasttoken") else "mean")
    mj = root / "modules.json"
    if mj.is_file():
        normalize = any("Normalize" in str(m.get("type", "")) for m in json.loads(mj.read_text()))
    return pooling, normalize


def maxsim(query_vectors: torch.Tensor, doc_vectors: torch.Tensor) -> float:
    """Late-interaction (ColBERT) relevance: for every query token the best cosine match among the document
    tokens, summed over the query tokens. Inputs are per-token vectors [Tq, H] and [Td, H]."""
    q = F.normalize(query_vectors.float(), dim=-1)
    d = F.normalize(doc_vectors.float(), dim=-1)
    return float((q @ d.T).max(dim=1).values.sum())
