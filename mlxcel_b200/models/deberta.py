"""DeBERTa-v2 / v3 encoder: BERT-style post-LayerNorm blocks with *disentangled* attention.

Besides content-to-content scores every head adds content-to-position and position-to-content
terms computed against one shared table of relative-position embeddings (log-bucketed distances):

    score[i, j] = (q_i . k_j  +  q_i . pk[d(i, j)]  +  k_j . pq[d(j, i)]) / sqrt(D * 3)

where ``pk`` / ``pq`` are the relative embeddings pushed through the layer's key / query projections
(``share_att_key``) or through dedicated ones. The positional terms are gathered into a [heads, T, T]
bias and handed to ``scaled_dot_product_attention`` together with the content product
(reference: src/models/deberta_v2.rs, src/embeddings/ and the cross-encoder rerankers built on it).
Projections run through ``ops.linear``; LayerNorm and GELU through the package's kernels.
"""
from __future__ import annotations

import json
import math
from pathlib import Path

import torch
import torch.nn.functional as F

from .. import ops
from ..ops import recurrent as rops


def _log_bucket(rel: torch.Tensor, bucket: int, max_pos: int) -> torch.Tensor:
    sign = torch.sign(rel)
    mid = bucket // 2
    abs_pos = torch.where((rel < mid) & (rel > -mid), torch.tensor(mid - 1, dtype=rel.dtype), rel.abs())
    log_pos = torch.ceil(torch.log(abs_pos / mid) / math.log((max_pos - 1) / mid) * (mid - 1)) + mid
    return torch.where(abs_pos <= mid, rel.to(log_pos.dtype), log_pos * sign)


def relative_positions(T: int, bucket: int, max_pos: int) -> torch.Tensor:
    """[T, T] relative position ids (query index minus key index), log-bucketed when buckets are set."""
    q = torch.arange(T)
    rel = q[:, None] - q[None, :]
    if bucket > 0 and max_pos > 0:
        rel = _log_bucket(rel.float(), bucket, max_pos).long()
    return rel


class DebertaV2Encoder:
    def __init__(self, cfg: dict, tensors: dict, dtype=torch.bfloat16, device="cpu"):
        self.heads, self.hidden = int(cfg["num_attention_heads"]), int(cfg["hidden_size"])
        self.eps = float(cfg.get("layer_norm_eps", 1e-7))
        self.max_len = int(cfg.get("max_position_embeddings", 512))
        self.device = torch.device(device)
        self.word = None
        if int(cfg.get("conv_kernel_size", 0) or 0) > 0:
            raise ValueError("DeBERTa checkpoints with the convolution branch (conv_kernel_size > 0) are not supported")
        self.relative = bool(cfg.get("relative_attention", False))
        self.pos_types = [x.lower() for x in (cfg.get("pos_att_type") or [])] if self.relative else []
        self.share_key = bool(cfg.get("share_att_key", False))
        self.buckets = int(cfg.get("position_buckets", -1))
        mrp = int(cfg.get("max_relative_positions", -1))
        self.max_rel = mrp if mrp >= 1 else self.max_len
        self.span = self.buckets if self.buckets > 0 else self.max_rel
        self.position_biased = bool(cfg.get("position_biased_input", True))
        self.act = {"gelu": "gelu", "gelu_new": "gelu_tanh"}.get(cfg.get("hidden_act", "gelu"), "gelu")
        pre = "deberta." if any(k.startswith("deberta.") for k in tensors) else ""

        def t(n, required=True):
            if pre + n not in tensors:
                if required:
                    raise KeyError(f"DeBERTa tensor {pre + n!r} is missing")
                return None
            return tensors[pre + n].to(dtype).to(self.device).contiguous()

        e = "embeddings."
        self.word = t(e + "word_embeddings.weight")
        self.pos = t(e + "position_embeddings.weight", False) if self.position_biased else None
        self.emb_ln = (t(e + "LayerNorm.weight"), t(e + "LayerNorm.bias"))
        self.emb_proj = t(e + "embed_proj.weight", False)
        self.rel = t("encoder.rel_embeddings.weight", False) if self.relative else None
        self.rel_ln = (t("encoder.LayerNorm.weight", False), t("encoder.LayerNorm.bias", False))
        self.layers = []
        for i in range(int(cfg["num_hidden_layers"])):
            p = f"encoder.layer.{i}."
            a = p + "attention.self."
            L = dict(wq=t(a + "query_proj.weight"), bq=t(a + "query_proj.bias"), wk=t(a + "key_proj.weight"),
                     bk=t(a + "key_proj.bias"), wv=t(a + "value_proj.weight"), bv=t(a + "value_proj.bias"),
                     wo=t(p + "attention.output.dense.weight"), bo=t(p + "attention.output.dense.bias"),
                     ln1=(t(p + "attention.output.LayerNorm.weight"), t(p + "attention.output.LayerNorm.bias")),
                     w1=t(p + "intermediate.dense.weight"), b1=t(p + "intermediate.dense.bias"),
                     w2=t(p + "output.dense.weight"), b2=t(p + "output.dense.bias"),
                     ln2=(t(p + "output.LayerNorm.weight"), t(p + "output.LayerNorm.bias")))
            L["wqkv"] = torch.cat([L["wq"], L["wk"], L["wv"]]).contiguous()
            L["bqkv"] = torch.cat([L["bq"], L["bk"], L["bv"]]).contiguous()
            if self.relative and not self.share_key:
                L["wpk"], L["bpk"] = t(a + "pos_key_proj.weight", False), t(a + "pos_key_proj.bias", False)
                L["wpq"], L["bpq"] = t(a + "pos_query_proj.weight", False), t(a + "pos_query_proj.bias", False)
            self.layers.append(L)
        head = lambda n: tensors[n].to(dtype).to(self.device).contiguous() if n in tensors else None  # noqa: E731
        self.pooler = (head("pooler.dense.weight"), head("pooler.dense.bias"))
        self.classifier = (head("classifier.weight"), head("classifier.bias"))
        self.id2label = {int(k): v for k, v in (cfg.get("id2label") or {}).items()}
        self.default_pooling, self.default_normalize = "cls", True

    @staticmethod
    def from_pretrained(path, dtype=torch.bfloat16, device="cpu") -> "DebertaV2Encoder":
        from ..loading.checkpoint import TensorSource
        src = TensorSource(path)
        return DebertaV2Encoder(json.loads((Path(path) / "config.json").read_text()),
                                {k: src.get(k) for k in src.keys()}, dtype, device)

    @torch.no_grad()
    def hidden_states(self, ids: list[int]) -> torch.Tensor:
        """Token states [T, hidden] of one text (no padding, so no mask)."""
        ids = ids[: self.max_len]
        T, H, nh = len(ids), self.hidden, self.heads
        D = H // nh
        tok = torch.tensor(ids, dtype=torch.long, device=self.device)
        h = self.word[tok]
        if self.pos is not None:
            h = (h.float() + self.pos[:T].float()).to(h.dtype)
        if self.emb_proj is not None:
            h = ops.linear(h.contiguous(), self.emb_proj)
        h = rops.layernorm(h.contiguous(), *self.emb_ln, self.eps)
        rel_emb = idx_c2p = idx_p2c = None
        if self.relative:
            rel_emb = self.rel[: 2 * self.span]
            if self.rel_ln[0] is not None:
                rel_emb = rops.layernorm(rel_emb.contiguous(), *self.rel_ln, self.eps)
            rel = relative_positions(T, self.buckets, self.max_rel).to(self.device)
            idx_c2p = (rel + self.span).clamp(0, 2 * self.span - 1)
            idx_p2c = (-rel + self.span).clamp(0, 2 * self.span - 1)
        scale = math.sqrt(D * (1 + len(self.pos_types)))
        for L in self.layers:
            qkv = ops.linear(h, L["wqkv"], bias=L["bqkv"]).view(T, 3, nh, D)
            q, k, v = (qkv[:, j].transpose(0, 1) for j in range(3))                # [nh, T, D]
            bias = None
            if self.relative:
                bias = torch.zeros(nh, T, T, dtype=torch.float32, device=self.device)
                wk, bk, wq, bq = (L["wk"], L["bk"], L["wq"], L["bq"]) if self.share_key else (L["wpk"], L["bpk"], L["wpq"], L["bpq"])
                if "c2p" in self.pos_types:
                    pk = ops.linear(rel_emb.contiguous(), wk, bias=bk).view(-1, nh, D).transpose(0, 1).float()     # [nh, 2S, D]
                    c2p = q.float() @ pk.transpose(1, 2)                                                         # [nh, T, 2S]
                    bias += torch.gather(c2p, 2, idx_c2p[None].expand(nh, T, T))
                if "p2c" in self.pos_types:
                    pq = ops.linear(rel_emb.contiguous(), wq, bias=bq).view(-1, nh, D).transpose(0, 1).float()
                    p2c = k.float() @ pq.transpose(1, 2)                                                         # [nh, T(key), 2S]
                    bias += torch.gather(p2c, 2, idx_p2c[None].expand(nh, T, T)).transpose(1, 2)
                bias = (bias / scale).to(q.dtype)
            a = F.scaled_dot_product_attention(q[None], k[None], v[None], attn_mask=None if bias is None else bias[None],
                                               scale=1.0 / scale)[0]
            a = a.transpose(0, 1).reshape(T, H).contiguous()
            h = rops.layernorm(ops.linear(a, L["wo"], bias=L["bo"], residual=h), *L["ln1"], self.eps)
            u = rops.activation(ops.linear(h, L["w1"], bias=L["b1"]), self.act)
            h = rops.layernorm(ops.linear(u, L["w2"], bias=L["b2"], residual=h), *L["ln2"], self.eps)
        return h

    def embed(self, ids: list[int], pooling: str = "cls", normalize: bool = True) -> torch.Tensor:
        h = self.hidden_states(ids).float()
        v = h[0] if pooling == "cls" else h[-1] if pooling == "last" else h.mean(0)
        return F.normalize(v, dim=0) if normalize else v

    def classify(self, ids: list[int]) -> torch.Tensor:
        """Sequence-classification logits: [CLS] state → pooler dense + GELU → classifier (cross-encoder
        rerankers score a ``query [SEP] document`` pair this way)."""
        if self.classifier[0] is None:
            raise ValueError("checkpoint has no classification head")
        v = self.hidden_states(ids)[:1]
        if self.pooler[0] is not None:
            v = rops.activation(ops.linear(v.contiguous(), self.pooler[0], bias=self.pooler[1]), "gelu")
        return ops.linear(v.contiguous(), self.classifier[0], bias=self.classifier[1])[0].float()

    def token_logits(self, ids: list[int]) -> torch.Tensor:
        if self.classifier[0] is None:
            raise ValueError("checkpoint has no token-classification head")
        return ops.linear(self.hidden_states(ids), self.classifier[0], bias=self.classifier[1]).float()
