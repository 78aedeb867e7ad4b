"""Decoder-only transformer executor over the kernel library.

One class runs every supported family: the per-family differences (q/k norm, biases, sinks,
sliding windows, Gemma norms, MoE routing, gated activation) are flags of
:class:`mlxcel_b200.config.ModelConfig`. A forward pass takes a flat token batch that may mix
decode rows (one token per sequence) and prefill chunks, vLLM-style, because on B200 a 64-row
decode step and a 512-token prefill chunk fit in the same set of GEMM launches.

Reference behaviour being matched: Llama-3 forward (src/models/llama3.rs:685-807,1112-1320),
Qwen3 q/k norm (src/models/qwen3.rs:309-338), GPT-OSS attention sinks / clipped SwiGLU / top-k
softmax routing (src/models/gpt_oss.rs:51-476), MoE switch layers
(src/models/switch_layers.rs:98-220).
"""
from __future__ import annotations

import os

from dataclasses import dataclass, field

import torch

from .. import ops
from ..config import ModelConfig
from ..ops import KVLayer
from ..ops.reference import rope_inv_freq
from .weights import LayerWeights, ModelWeights, QuantizedTensor


@dataclass
class StepBatch:
    """Device-side description of one forward pass.

    Token layout: the first ``num_decode`` rows are decode rows (sequence i ↔ row i); the rest
    are prefill chunks laid back to back (``cu_q`` is relative to the start of that region)."""

    token_ids: torch.Tensor          # [T] int32
    positions: torch.Tensor          # [T] int32
    slot_mapping: torch.Tensor       # [T] int32 (-1 = padding row, nothing appended)
    num_decode: int = 0
    dec_block_tables: torch.Tensor | None = None   # [Bd, max_blocks] int32
    dec_context_lens: torch.Tensor | None = None   # [Bd] int32 (including the new token)
    dec_max_len: int = 0
    num_prefill_seqs: int = 0
    pf_block_tables: torch.Tensor | None = None    # [Sp, max_blocks]
    pf_cu_q: torch.Tensor | None = None            # [Sp+1] int32
    pf_context_lens: torch.Tensor | None = None    # [Sp] int32 (prefix + chunk)
    pf_max_q_len: int = 0
    pf_cu_q_host: list | None = None               # host copy of pf_cu_q (micro-batch splitting)
    logits_rows: torch.Tensor | None = None        # [R] int64 rows of the hidden state to project
    embeds: torch.Tensor | None = None             # optional [T, H] input embeddings (VLM / MTP)
    deepstack: list | None = None                  # [T, H] per early layer: visual features added to the stream after it
    seq_ids: list | None = None                    # host: sequence id per decode row, then per prefill piece
    pf_starts: list | None = None                  # host: first position of every prefill piece
    # Sliding-window layers with their own block pool (blocks behind the window are given back):
    # slots and block tables of that pool. None = every layer uses the tables above.
    slot_mapping_win: torch.Tensor | None = None
    dec_block_tables_win: torch.Tensor | None = None
    pf_block_tables_win: torch.Tensor | None = None
    # Multimodal rotary positions [3, T] (temporal, height, width) when a row's three components
    # differ (image tokens of the Qwen2-VL family); ``positions`` then holds the temporal one.
    positions3: torch.Tensor | None = None

    @property
    def num_tokens(self) -> int:
        return int(self.token_ids.shape[0])


class LocalComm:
    """Single-GPU communication context (world size 1): every collective is the identity."""

    tp_size = 1
    tp_rank = 0
    ep_size = 1
    ep_rank = 0

    def row_parallel_linear(self, x, w, bias, residual, ssq_out=None):
        return _linear_any(x, w, bias=bias, residual=residual, out=residual, ssq_out=ssq_out)

    def gather_logits(self, logits):
        return logits

    def lm_head(self, x, w):
        return _linear_any(x, w)

    def embed(self, ids, table, scale, vocab_start=0):
        return ops.embedding(ids, table, scale)

    def all_reduce(self, x):
        return x


def _linear_any(x, w, bias=None, residual=None, out=None, row_norm=None, ssq_out=None):
    if isinstance(w, QuantizedTensor):
        from ..ops import quant
        assert row_norm is None, "deferred RMSNorm needs dense weights"
        y = quant.qlinear(x, w, bias=bias, residual=residual, out=out)
        if ssq_out is not None:
            ops.row_ssq(y, ssq_out)
        return y
    return ops.linear(x, w, bias=bias, residual=residual, out=out, row_norm=row_norm, ssq_out=ssq_out)


def _glu_any(x, w, inter, act, bias, alpha, limit, row_norm=None):
    if isinstance(w, QuantizedTensor):
        from ..ops import quant
        assert row_norm is None, "deferred RMSNorm needs dense weights"
        return quant.qglu_linear(x, w, inter, act, bias=bias, alpha=alpha, limit=limit)
    return ops.glu_linear(x, w, inter, act, bias=bias, alpha=alpha, limit=limit, row_norm=row_norm)


class DecoderModel:
    def __init__(self, cfg: ModelConfig, weights: ModelWeights, comm=None, kv_bits: int = 16,
                 layer_range: range | None = None, first_stage: bool = True,
                 last_stage: bool = True, fold_norms: bool = False):
        self.cfg = cfg
        self.w = weights
        self.comm = comm or LocalComm()
        self.kv_bits = kv_bits
        self.layer_range = layer_range or range(cfg.num_hidden_layers)
        self.first_stage, self.last_stage = first_stage, last_stage
        tp = self.comm.tp_size
        self.Hq = cfg.num_attention_heads // tp
        self.Hkv = max(1, cfg.num_key_value_heads // tp)
        self.D = cfg.head_dim
        self.I = cfg.intermediate_size // tp
        dev = weights.final_norm.device
        # served context (when the front end recorded it): longrope / dynamic-NTK tables depend on it
        inv, ms = rope_inv_freq(cfg.rot_dim, cfg.rope_theta, cfg.rope_scaling, int(cfg.extra.get("served_context", 0) or 0))
        if cfg.extra.get("rope_negate"):
            inv = -inv                       # the pair rotates the other way (x2, -x1 instead of -x2, x1)
        self.inv_freq = inv.to(dev)
        self.mscale = ms
        # sliding-window layers with their own RoPE base (Gemma 3: local 10k, global 1M with scaling)
        self.inv_freq_mla = None
        if cfg.extra.get("mla"):                # rotary part of multi-head latent attention
            inv_m, self.mscale = rope_inv_freq(cfg.extra["mla"]["rope"], cfg.rope_theta, cfg.rope_scaling)
            self.inv_freq_mla = inv_m.to(dev)
        self.inv_freq_local = None
        if cfg.extra.get("rope_local_theta"):
            self.inv_freq_local = rope_inv_freq(cfg.rot_dim, cfg.extra["rope_local_theta"], None)[0].to(dev)
        self.device = dev
        self._ssq = None
        self.fold_attn = self.fold_mlp = False
        self.nope_layers = frozenset(cfg.extra.get("nope_layers", ()))
        self.layernorm = cfg.extra.get("norm") == "layernorm"
        # residual stream after these layers is kept in ``captured`` by every forward (block drafters
        # condition on several depths of the target, see speculative/dflash.py)
        self.capture_layers: tuple = ()
        self.captured: list = []
        self.clip_qkv = float(cfg.extra.get("clip_qkv") or 0.0)
        self.plain_mlp = cfg.extra.get("mlp") == "plain"
        if cfg.extra.get("attn_output_gate") and self.comm.tp_size != 1:
            raise NotImplementedError("the attention output gate is not sharded across tensor-parallel ranks")
        self.sub_norms = bool(cfg.extra.get("sub_norms"))
        if self.sub_norms and self.comm.tp_size != 1:
            raise NotImplementedError("sub-layer norms span the whole projection input: not sharded across tensor-parallel ranks")
        self.general = self.layernorm or self.plain_mlp or bool(cfg.extra.get("parallel_block")) or self.sub_norms
        # Folding rewrites the projection weights in place, so only the owner of the weights asks for
        # it (the LLM front end does; weights shared with another executor must stay untouched).
        if fold_norms and dev.type == "cuda" and os.environ.get("MLXCEL_B200_FOLD_NORMS", "1") != "0":
            self._fold_norms()

    # ------------------------------------------------------------------ deferred RMSNorm
    def _fold_norms(self) -> None:
        """Pre-norm layers with dense projections: multiply the norm weight into the columns of the
        projection that consumes the normalised stream. The forward pass then feeds the residual
        stream itself to that GEMM, whose epilogue applies the per-token 1/rms from the sums of
        squares the previous GEMM's epilogue (or ``row_ssq``) left — the RMSNorm kernels between
        the projections disappear (2 per layer). Same math as norm-then-project up to bf16
        rounding of the folded weight."""
        cfg = self.cfg
        if (cfg.post_norms or cfg.extra.get("residual_multiplier", 1.0) != 1.0 or cfg.extra.get("post_norm_only")
                or self.general):
            return
        H = cfg.hidden_size
        if H % 128 or H // 128 > 64:
            return
        layers = self.w.layers
        if not layers or any(isinstance(lw.wqkv, QuantizedTensor) or lw.wqkv.dtype != torch.bfloat16 for lw in layers):
            return
        fold_mlp = not cfg.is_moe and all(
            lw.w_gate_up is not None and not isinstance(lw.w_gate_up, QuantizedTensor)
            and lw.w_gate_up.dtype == torch.bfloat16 for lw in layers)
        wb = cfg.norm_weight_bias

        def fold(w, ln):
            if getattr(w, "_norm_folded", False):      # shared between two executors of one model
                return
            g = (ln.float() + wb).unsqueeze(0)
            for r0 in range(0, w.shape[0], 8192):      # bounded fp32 temporaries
                w[r0:r0 + 8192] = (w[r0:r0 + 8192].float() * g).to(w.dtype)
            w._norm_folded = True
            w._norm_gain = g.squeeze(0)     # weight deltas applied later (LoRA) must be folded the same way

        with torch.no_grad():
            for lw in layers:
                fold(lw.wqkv, lw.ln1)
                if fold_mlp:
                    fold(lw.w_gate_up, lw.ln2)
        self.fold_attn, self.fold_mlp = True, fold_mlp
        self._ssq = ops.SsqBuffer(16384, H // 128, self.device)

    # ------------------------------------------------------------------ blocks
    def _attention(self, li: int, lw: LayerWeights, x: torch.Tensor, b: StepBatch,
                   kv: KVLayer, row_norm=None) -> torch.Tensor:
        cfg = self.cfg
        if lw.mla is not None:
            if cfg.extra.get("mla_latent"):
                return self._attention_mla_latent(li, lw, x, b, kv)
            return self._attention_mla(li, lw, x, b, kv)
        qkv = _linear_any(x, lw.wqkv, bias=lw.bqkv, row_norm=row_norm)
        if self.clip_qkv:                                   # DBRX: symmetric clamp of the fused projection
            qkv = qkv.clamp_(-self.clip_qkv, self.clip_qkv)
        q_norm, k_norm = lw.q_norm, lw.k_norm
        if q_norm is not None and cfg.extra.get("qk_norm_full"):
            # OLMo-2 / OLMoE: RMSNorm over the whole q and k projections (not per head), before RoPE
            if self.comm.tp_size != 1:
                raise NotImplementedError("whole-projection q/k norm is not sharded across tensor-parallel ranks")
            nq, nk = self.Hq * self.D, self.Hkv * self.D
            qn = ops.rmsnorm(qkv[:, :nq].contiguous(), q_norm, cfg.rms_norm_eps, 0.0)
            kn = ops.rmsnorm(qkv[:, nq:nq + nk].contiguous(), k_norm, cfg.rms_norm_eps, 0.0)
            qkv = torch.cat([qn, kn, qkv[:, nq + nk:]], dim=1)
            q_norm = k_norm = None
        if cfg.extra.get("llama4_attn_scale"):
            # queries grow with the logarithm of their position block (a scalar per row commutes with
            # the rotation, so it is applied before the fused RoPE + append kernel)
            beta, orig = cfg.extra["llama4_attn_scale"]
            sc = 1.0 + beta * torch.log1p(torch.floor(b.positions.float() / orig))
            nq = self.Hq * self.D
            qkv = torch.cat([(qkv[:, :nq].float() * sc[:, None]).to(qkv.dtype), qkv[:, nq:]], dim=1)
        window = cfg.layer_window(self.layer_range[li] if li < len(self.layer_range) else li)
        local = window > 0 and self.inv_freq_local is not None
        layer_index = self.layer_range[li] if li < len(self.layer_range) else li
        rot_dim = 0 if layer_index in self.nope_layers else cfg.rot_dim    # layers without positional encoding
        if not rot_dim and cfg.extra.get("qk_norm_rope_layers_only"):
            q_norm = k_norm = None                              # Llama 4: q/k norm on the rotary layers only
        if not rot_dim and cfg.extra.get("nope_query_temperature"):
            # Llama 4: queries of the layers without positions grow with the logarithm of their
            # position block, which keeps long-context attention from flattening
            a_s, floor_s = cfg.extra["nope_query_temperature"]
            sc = 1.0 + a_s * torch.log1p(torch.floor((b.positions.float() + 1.0) / floor_s))
            nq = self.Hq * self.D
            qkv = torch.cat([(qkv[:, :nq].float() * sc[:, None]).to(qkv.dtype), qkv[:, nq:]], dim=1)
        if q_norm is not None and cfg.extra.get("qk_norm_after_rope") and rot_dim:
            # Hunyuan: the per-head q/k norms come AFTER the rotation; the fused kernel norms before it, so
            # rotate and normalise here and let the kernel only append
            from ..ops import reference as ref
            T0, nqk = qkv.shape[0], self.Hq + self.Hkv
            x3 = qkv.view(T0, self.Hq + 2 * self.Hkv, self.D)
            rot = ref.apply_rope(x3[:, :nqk], b.positions, self.inv_freq, rot_dim, cfg.rope_traditional, self.mscale)
            qn = ref.head_rmsnorm(rot[:, :self.Hq], q_norm, cfg.rms_norm_eps)
            kn = ref.head_rmsnorm(rot[:, self.Hq:], k_norm, cfg.rms_norm_eps)
            qkv = torch.cat([qn.to(qkv.dtype), kn.to(qkv.dtype), x3[:, nqk:]], dim=1).reshape(T0, -1).contiguous()
            q_norm = k_norm = None
            rot_dim = 0
        if b.positions3 is not None and rot_dim and cfg.extra.get("mrope_section"):
            # rows with three different rotary positions: rotate here (each frequency takes the position
            # of its section), the kernel only appends
            from ..ops import reference as ref
            T0, nqk = qkv.shape[0], self.Hq + self.Hkv
            x3 = qkv.view(T0, self.Hq + 2 * self.Hkv, self.D)
            rot = ref.apply_mrope(x3[:, :nqk], b.positions3, self.inv_freq, cfg.extra["mrope_section"], self.mscale,
                                  interleaved=bool(cfg.extra.get("mrope_interleaved")), rot_dim=rot_dim,
                                  traditional=cfg.rope_traditional)
            qkv = torch.cat([rot.to(qkv.dtype), x3[:, nqk:]], dim=1).reshape(T0, -1).contiguous()
            rot_dim = 0
        use_win = window > 0 and b.slot_mapping_win is not None     # this layer's KV lives in the window pool
        ops.rope_append(qkv, b.positions, b.slot_mapping_win if use_win else b.slot_mapping,
                        self.inv_freq_local if local else self.inv_freq, kv,
                        Hq=self.Hq, Hkv=self.Hkv, D=self.D, rot_dim=rot_dim,
                        traditional=cfg.rope_traditional, mscale=1.0 if local else self.mscale,
                        q_norm_w=q_norm, k_norm_w=k_norm, norm_eps=cfg.rms_norm_eps)
        return self._attend(qkv, b, kv, window, lw.sinks, use_win)

    def _attend(self, qkv: torch.Tensor, b: StepBatch, kv: KVLayer, window: int, sinks,
                use_win: bool = False) -> torch.Tensor:
        """Paged attention of the step's rows (decode rows first, then the prefill pieces) over the
        keys / values just appended; ``qkv`` carries the (rotated) queries in its first Hq * D columns."""
        cfg = self.cfg
        T = qkv.shape[0]
        attn = torch.empty(T, self.Hq * self.D, dtype=qkv.dtype, device=qkv.device)
        q = qkv[:, : self.Hq * self.D]
        nd = b.num_decode
        common = dict(Hq=self.Hq, Hkv=self.Hkv, D=self.D, scale=cfg.attn_scale, window=window,
                      sinks=sinks, softcap=cfg.attn_logit_softcap)
        dec_tables = b.dec_block_tables_win if use_win else b.dec_block_tables
        pf_tables = b.pf_block_tables_win if use_win else b.pf_block_tables
        if nd > 0:
            o = ops.paged_decode(q[:nd], kv, dec_tables, b.dec_context_lens,
                                 max_len=b.dec_max_len, out=attn[:nd] if attn.is_cuda else None,
                                 **common)
            if not attn.is_cuda:
                attn[:nd] = o
        if b.num_prefill_seqs > 0:
            o = ops.paged_prefill(q[nd:], kv, pf_tables, b.pf_cu_q, b.pf_context_lens,
                                  max_q_len=b.pf_max_q_len, out=attn[nd:] if attn.is_cuda else None,
                                  **common)
            if not attn.is_cuda:
                attn[nd:] = o
        return attn

    def _attention_mla(self, li: int, lw: LayerWeights, x: torch.Tensor, b: StepBatch, kv: KVLayer) -> torch.Tensor:
        """Multi-head latent attention (DeepSeek-V2 / V3; reference src/models/deepseek_v3.rs, mla/*) in
        its expanded form: q from the (optionally low-rank) query path, per-head k_nope and v from the
        normalised latent through kv_b, one rotary key part shared by all heads. Keys [k_nope | k_rot]
        and values are zero-padded to the pool's head size and stored per head, so the ordinary paged
        kernels serve it; the attention output is cut back to v_head_dim. The absorbed form over a
        latent cache (one 576-wide entry per token instead of 2 * heads * D) is `_attention_mla_latent`."""
        from ..ops import reference as ref

        cfg, m, w = self.cfg, self.cfg.extra["mla"], lw.mla
        Hq, Dp = self.Hq, self.D
        nope, r, vd, lat = m["nope"], m["rope"], m["v"], m["kv_lora_rank"]
        T = x.shape[0]
        if w.get("q_a") is not None:
            q = _linear_any(ops.rmsnorm(_linear_any(x, w["q_a"], bias=w.get("q_a_b")), w["q_a_norm"], 1e-6, 0.0), w["q_b"])
        else:
            q = _linear_any(x, w["q"])
        q = q.view(T, Hq, nope + r)
        ckv = _linear_any(x, w["kv_a"], bias=w.get("kv_a_b"))
        kvb = _linear_any(ops.rmsnorm(ckv[:, :lat].contiguous(), w["kv_a_norm"], 1e-6, 0.0), w["kv_b"]).view(T, Hq, nope + vd)
        q_rot = ref.apply_rope(q[..., nope:], b.positions, self.inv_freq_mla, r, m["interleave"], self.mscale)
        k_rot = ref.apply_rope(ckv[:, lat:].view(T, 1, r), b.positions, self.inv_freq_mla, r, m["interleave"], self.mscale)
        if cfg.extra.get("llama4_attn_scale"):           # Mistral 4: queries grow with the log of their position block
            beta, orig = cfg.extra["llama4_attn_scale"]
            sc = (1.0 + beta * torch.log1p(torch.floor(b.positions.float() / orig)))[:, None, None]
            q, q_rot = (q.float() * sc).to(q.dtype), (q_rot.float() * sc).to(q_rot.dtype)
        qkv = torch.zeros(T, 3 * Hq, Dp, dtype=x.dtype, device=x.device)
        qkv[:, :Hq, :nope] = q[..., :nope]
        qkv[:, :Hq, nope:nope + r] = q_rot.to(x.dtype)
        qkv[:, Hq:2 * Hq, :nope] = kvb[..., :nope]
        qkv[:, Hq:2 * Hq, nope:nope + r] = k_rot.to(x.dtype).expand(T, Hq, r)
        qkv[:, 2 * Hq:, :vd] = kvb[..., nope:]
        qkv = qkv.view(T, 3 * Hq * Dp)
        ops.rope_append(qkv, b.positions, b.slot_mapping, self.inv_freq, kv, Hq=Hq, Hkv=self.Hkv, D=Dp, rot_dim=0,
                        traditional=False, mscale=1.0, q_norm_w=None, k_norm_w=None, norm_eps=cfg.rms_norm_eps)
        attn = self._attend(qkv, b, kv, 0, None)
        return attn.view(T, Hq, Dp)[..., :vd].reshape(T, Hq * vd)

    def _attention_mla_latent(self, li: int, lw: LayerWeights, x: torch.Tensor, b: StepBatch, kv: KVLayer) -> torch.Tensor:
        """Multi-head latent attention in its absorbed form over a latent cache (the reference's
        src/lib/mlxcel-core/src/mla/cache.rs:253 and its absorbed decode kernel): the pool keeps one entry
        ``[normalised latent | rotary key]`` per token; the per-head key up-projection is folded into the
        query (``q_lat = q_nope W_uk``) and the value up-projection is applied to the attention output
        (``out = (P latent) W_uv``), so neither per-head keys nor values are ever materialised for the
        context. Scores are ``q_lat . latent + q_rot . k_rot`` — the same numbers as the expanded form.
        The attention itself is batched matrix products over the gathered pages (library GEMMs; a
        hand-written absorbed-decode kernel is not built): decode rows gather their whole block table
        and mask beyond the context length, prefill pieces are walked one by one under a causal mask."""
        from ..ops import reference as ref

        cfg, m, w = self.cfg, self.cfg.extra["mla"], lw.mla
        Hq = self.Hq
        nope, r, vd, lat = m["nope"], m["rope"], m["v"], m["kv_lora_rank"]
        T, dev = x.shape[0], x.device
        if w.get("q_a") is not None:
            q = _linear_any(ops.rmsnorm(_linear_any(x, w["q_a"], bias=w.get("q_a_b")), w["q_a_norm"], 1e-6, 0.0), w["q_b"])
        else:
            q = _linear_any(x, w["q"])
        q = q.view(T, Hq, nope + r)
        ckv = _linear_any(x, w["kv_a"], bias=w.get("kv_a_b"))
        c = ops.rmsnorm(ckv[:, :lat].contiguous(), w["kv_a_norm"], 1e-6, 0.0)
        q_rot = ref.apply_rope(q[..., nope:], b.positions, self.inv_freq_mla, r, m["interleave"], self.mscale)
        k_rot = ref.apply_rope(ckv[:, lat:].view(T, 1, r), b.positions, self.inv_freq_mla, r, m["interleave"], self.mscale)
        q_nope = q[..., :nope]
        if cfg.extra.get("llama4_attn_scale"):
            beta, orig = cfg.extra["llama4_attn_scale"]
            sc = (1.0 + beta * torch.log1p(torch.floor(b.positions.float() / orig)))[:, None, None]
            q_nope, q_rot = (q_nope.float() * sc).to(q.dtype), (q_rot.float() * sc).to(q_rot.dtype)
        wkv = w.get("kv_b_split")
        if wkv is None:
            dense = w["kv_b"]
            if not isinstance(dense, torch.Tensor) or dense.dim() != 2 or dense.shape[1] != lat:
                raise NotImplementedError("the latent MLA cache needs a dense kv_b projection (quantized kv_b is not absorbed)")
            dense = dense.view(Hq, nope + vd, lat)
            wkv = w["kv_b_split"] = (dense[:, :nope].contiguous(), dense[:, nope:].contiguous())     # W_uk, W_uv
        w_uk, w_uv = wkv
        # entry of the new tokens → their slots (padding rows carry slot -1 and are dropped)
        entry = torch.cat([c, k_rot.view(T, r).to(c.dtype)], dim=1)
        W = lat + r
        flat = kv.k.view(-1, W)
        ok = b.slot_mapping >= 0
        flat.index_copy_(0, b.slot_mapping[ok].long(), entry[ok].to(flat.dtype))
        # queries in latent space: [T, Hq, lat + r]
        q_lat = torch.einsum("thn,hnl->thl", q_nope.float(), w_uk.float())
        qq = torch.cat([q_lat, q_rot.float()], dim=-1)
        scale = float(cfg.attn_scale)
        out_lat = torch.zeros(T, Hq, lat, dtype=torch.float32, device=dev)
        bs = kv.block_size
        nd = b.num_decode
        if nd > 0:
            tab = b.dec_block_tables[:nd].clamp(min=0).long()
            ctx = kv.k[tab].view(nd, -1, W).float()                              # [nd, blocks * bs, W]
            s = torch.einsum("nhw,nsw->nhs", qq[:nd], ctx) * scale
            live = torch.arange(ctx.shape[1], device=dev)[None, :] < b.dec_context_lens[:nd, None]
            s = s.masked_fill(~live[:, None, :], float("-inf"))
            p = torch.softmax(s, dim=-1).nan_to_num(0.0)                        # a padding row has no live key
            out_lat[:nd] = torch.einsum("nhs,nsl->nhl", p, ctx[..., :lat])
        if b.num_prefill_seqs > 0:
            cu = b.pf_cu_q_host if b.pf_cu_q_host is not None else b.pf_cu_q.tolist()
            lens = b.pf_context_lens.tolist()
            for i in range(b.num_prefill_seqs):
                r0, r1, L = nd + int(cu[i]), nd + int(cu[i + 1]), int(lens[i])
                n = r1 - r0
                if n <= 0:
                    continue
                nb = (L + bs - 1) // bs
                ctx = kv.k[b.pf_block_tables[i, :nb].long()].view(-1, W)[:L].float()
                s = torch.einsum("thw,sw->ths", qq[r0:r1], ctx) * scale
                qpos = torch.arange(L - n, L, device=dev)
                s = s.masked_fill((torch.arange(L, device=dev)[None, :] > qpos[:, None])[:, None, :], float("-inf"))
                out_lat[r0:r1] = torch.einsum("ths,sl->thl", torch.softmax(s, dim=-1), ctx[:, :lat])
        out = torch.einsum("thl,hvl->thv", out_lat, w_uv.float())
        return out.reshape(T, Hq * vd).to(x.dtype)

    def _norm(self, x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None = None) -> torch.Tensor:
        """The model's normalisation: RMSNorm (with Gemma's +1) or LayerNorm (bias optional)."""
        if self.layernorm:
            from ..ops import recurrent as rops
            return rops.layernorm(x, w, b, self.cfg.rms_norm_eps)
        return ops.rmsnorm(x, w, self.cfg.rms_norm_eps, self.cfg.norm_weight_bias)

    def _mlp(self, lw: LayerWeights, x: torch.Tensor, row_norm=None) -> torch.Tensor:
        cfg = self.cfg
        if self.plain_mlp:                      # fc -> activation -> (proj by the caller)
            from ..ops import recurrent as rops
            u = _linear_any(x, lw.w_gate_up, bias=lw.b_gate_up)
            if cfg.hidden_act == "xielu":
                ap, an, beta, eps_x = lw.act_params or (0.8, 0.8, 0.5, -1e-6)
                return rops.xielu(u, ap, an, beta, eps_x)
            return rops.activation(u, cfg.hidden_act)
        if cfg.hidden_act == "relu2":           # BitNet: relu(gate)^2 * up, then its own norm
            from ..ops import recurrent as rops
            gu = _linear_any(x, lw.w_gate_up, bias=lw.b_gate_up)
            inter = gu.shape[1] // 2
            m = (rops.activation(gu[:, :inter].contiguous(), "relu2").float() * gu[:, inter:].float()).to(gu.dtype)
            return ops.rmsnorm(m, lw.ffn_sub_norm, cfg.rms_norm_eps, 0.0) if lw.ffn_sub_norm is not None else m
        return _glu_any(x, lw.w_gate_up, self.I, cfg.hidden_act, lw.b_gate_up, cfg.swiglu_alpha,
                        cfg.swiglu_limit, row_norm=row_norm)

    def _moe(self, lw: LayerWeights, x: torch.Tensor, h: torch.Tensor) -> torch.Tensor:
        from .moe import moe_forward
        return moe_forward(self.cfg, lw, x, h, self.comm)

    def forward_null(self) -> None:
        """A forward pass without tokens (token-sharded expert parallelism): only the exchanges of the
        MoE layers run, so that the other ranks' rows are served."""
        from .moe import moe_null
        dev, dt = self.w.final_norm.device, self.w.final_norm.dtype
        for lw in self.w.layers:
            if lw.router_w is not None:
                moe_null(self.cfg, lw, self.comm, dt, dev)

    # ------------------------------------------------------------------ forward
    def forward_hidden(self, b: StepBatch, kv_layers: list[KVLayer],
                       hidden_in: torch.Tensor | None = None) -> torch.Tensor:
        """Runs this stage's layers. Returns the residual stream [T, H] (before the final norm)."""
        cfg, w = self.cfg, self.w
        if hidden_in is not None:
            h = hidden_in
        elif b.embeds is not None:
            h = b.embeds
        else:
            h = self.comm.embed(b.token_ids, w.embed, cfg.embed_scale)
            if w.extra.get("pos_embed") is not None:          # learned absolute positions (GPT-2 family)
                h = (h.float() + w.extra["pos_embed"].index_select(0, b.positions.long()).float()).to(h.dtype)
            if cfg.extra.get("embed_norm"):                   # a (gain-free) norm between embedding and blocks
                h = ops.rmsnorm(h, torch.ones_like(w.final_norm), cfg.rms_norm_eps, 0.0)
        eps, wb = cfg.rms_norm_eps, cfg.norm_weight_bias
        res_mult = cfg.extra.get("residual_multiplier", 1.0)
        self.captured = []
        if self.fold_attn and h.is_cuda and h.shape[0] <= self._ssq.max_tokens and h.dtype == torch.bfloat16:
            return self._forward_folded(h, b, kv_layers)
        if self.fold_attn:
            raise RuntimeError("norm weights are folded into the projections: this batch cannot take the "
                               "unfolded path (too many tokens or a non-bf16 stream)")
        if self.general:
            return self._forward_general(h, b, kv_layers)
        if cfg.extra.get("post_norm_only"):
            # OLMo-2: no norm before the blocks; h += norm(attn(h)); h += norm(mlp(h))
            for li, lw in enumerate(w.layers):
                a = self._attention(li, lw, h, b, kv_layers[li])
                o = self.comm.row_parallel_linear(a, lw.wo, lw.bo, None)
                h = (h.float() + ops.rmsnorm(o, lw.post_attn_norm, eps, wb).float()).to(h.dtype)
                if cfg.is_moe:
                    raise NotImplementedError("post-norm-only MoE blocks")
                o = self.comm.row_parallel_linear(self._mlp(lw, h), lw.w_down, lw.b_down, None)
                h = (h.float() + ops.rmsnorm(o, lw.post_mlp_norm, eps, wb).float()).to(h.dtype)
            return h
        for li, lw in enumerate(w.layers):
            kv = kv_layers[li]
            x = ops.rmsnorm(h, lw.ln1, eps, wb)
            a = self._attention(li, lw, x, b, kv)
            if lw.attn_gate is not None:                    # AFMoE: sigmoid gate from the layer input
                a = (a.float() * torch.sigmoid(_linear_any(x, lw.attn_gate).float())).to(a.dtype)
            if cfg.post_norms or res_mult != 1.0:
                o = self.comm.row_parallel_linear(a, lw.wo, lw.bo, None)
                if cfg.post_norms:
                    o = ops.rmsnorm(o, lw.post_attn_norm, eps, wb)
                if res_mult != 1.0:
                    o = (o.float() * res_mult).to(o.dtype)
                x, h = ops.add_rmsnorm(o, h, lw.ln2, eps, wb)
            else:
                h = self.comm.row_parallel_linear(a, lw.wo, lw.bo, h)
                x = ops.rmsnorm(h, lw.ln2, eps, wb)
            if cfg.is_moe and lw.router_w is not None and res_mult != 1.0:              # GraniteMoE: scaled expert branch
                o = self._moe(lw, x, torch.zeros_like(h))
                h = (h.float() + o.float() * res_mult).to(h.dtype)
            elif cfg.is_moe and lw.router_w is not None and cfg.post_norms:     # AFMoE: a norm after the MoE block
                o = ops.rmsnorm(self._moe(lw, x, torch.zeros_like(h)), lw.post_mlp_norm, eps, wb)
                h = (h.float() + o.float()).to(h.dtype)
            elif cfg.is_moe and lw.router_w is not None:
                h = self._moe(lw, x, h)
            else:
                m = self._mlp(lw, x)
                if cfg.post_norms or res_mult != 1.0:
                    o = self.comm.row_parallel_linear(m, lw.w_down, lw.b_down, None)
                    if cfg.post_norms:
                        o = ops.rmsnorm(o, lw.post_mlp_norm, eps, wb)
                    if res_mult != 1.0:
                        o = (o.float() * res_mult).to(o.dtype)
                    h = (h.float() + o.float()).to(h.dtype) if not h.is_cuda else h.add_(o)
                else:
                    h = self.comm.row_parallel_linear(m, lw.w_down, lw.b_down, h)
            h = self._deepstack(li, h, b)
            self._capture(li, h)
        return h

    def _deepstack(self, li: int, h: torch.Tensor, b: StepBatch) -> torch.Tensor:
        """Qwen3-VL DeepStack: the image rows of the first few layers' outputs get visual features of
        intermediate vision-tower depths added (zero rows elsewhere)."""
        ds = b.deepstack
        if ds is None:
            return h
        g = self.layer_range[li] if li < len(self.layer_range) else li
        return (h.float() + ds[g].float()).to(h.dtype) if g < len(ds) else h

    def _capture(self, li: int, h: torch.Tensor) -> None:
        if self.capture_layers and (self.layer_range[li] if li < len(self.layer_range) else li) in self.capture_layers:
            self.captured.append(h.clone())       # (later layers may add into h in place)

    def _forward_general(self, h: torch.Tensor, b: StepBatch, kv_layers: list[KVLayer]) -> torch.Tensor:
        """Layer loop of the less common layouts, without the fusions of the main path: LayerNorm
        instead of RMSNorm (StarCoder2, StableLM, Cohere), a plain fc -> act -> proj MLP
        (StarCoder2), attention and MLP in parallel from one normed input (Cohere, StableLM's
        parallel residual)."""
        cfg = self.cfg
        parallel = bool(cfg.extra.get("parallel_block"))
        for li, lw in enumerate(self.w.layers):
            x = self._norm(h, lw.ln1, lw.ln1_b)
            a = self._attention(li, lw, x, b, kv_layers[li])
            if lw.attn_sub_norm is not None:                 # BitNet: norm between attention and o_proj
                a = ops.rmsnorm(a, lw.attn_sub_norm, cfg.rms_norm_eps, 0.0)
            if parallel:
                # one norm feeds both branches (Cohere, Phi) unless the layer has a second one (GPT-NeoX)
                xm = x if lw.ln2 is lw.ln1 else self._norm(h, lw.ln2, lw.ln2_b)
                o = self.comm.row_parallel_linear(a, lw.wo, lw.bo, None)
                m = self.comm.row_parallel_linear(self._mlp(lw, xm), lw.w_down, lw.b_down, None)
                h = (h.float() + o.float() + m.float()).to(h.dtype)
            else:
                h = self.comm.row_parallel_linear(a, lw.wo, lw.bo, h)
                x = self._norm(h, lw.ln2, lw.ln2_b)
                if cfg.is_moe and lw.router_w is not None:
                    h = self._moe(lw, x, h)
                else:
                    h = self.comm.row_parallel_linear(self._mlp(lw, x), lw.w_down, lw.b_down, h)
            h = self._deepstack(li, h, b)
            self._capture(li, h)
        return h

    def _forward_folded(self, h: torch.Tensor, b: StepBatch, kv_layers: list[KVLayer]) -> torch.Tensor:
        """Layer loop with deferred RMSNorms (see ``_fold_norms``): ``ssq`` always describes the
        current residual stream ``h``."""
        cfg, ssq = self.cfg, self._ssq
        eps, wb = cfg.rms_norm_eps, cfg.norm_weight_bias
        rn = ops.RowNorm(ssq, eps, cfg.hidden_size)
        ops.row_ssq(h, ssq)
        for li, lw in enumerate(self.w.layers):
            a = self._attention(li, lw, h, b, kv_layers[li], row_norm=rn)
            h = self.comm.row_parallel_linear(a, lw.wo, lw.bo, h, ssq_out=ssq)
            if self.fold_mlp:
                m = self._mlp(lw, h, row_norm=rn)
                h = self.comm.row_parallel_linear(m, lw.w_down, lw.b_down, h, ssq_out=ssq)
            else:
                x = ops.rmsnorm(h, lw.ln2, eps, wb)
                if cfg.is_moe and lw.router_w is not None:
                    h = self._moe(lw, x, h)
                else:
                    h = self.comm.row_parallel_linear(self._mlp(lw, x), lw.w_down, lw.b_down, h)
                if li + 1 < len(self.w.layers):
                    ops.row_ssq(h, ssq)
            h2 = self._deepstack(li, h, b)
            if h2 is not h:                          # the stream changed behind the kernels that keep its sums of squares
                h = h2
                ops.row_ssq(h, ssq)
            self._capture(li, h)
        return h

    def logits(self, h: torch.Tensor, rows: torch.Tensor | None) -> torch.Tensor:
        """Final norm + LM head on the selected rows → fp32-comparable logits [R, V]."""
        cfg, w = self.cfg, self.w
        if rows is not None:
            h = h.index_select(0, rows)
        x = self._norm(h, w.final_norm, w.extra.get("final_norm_b"))
        if isinstance(w.lm_head, QuantizedTensor):
            lg = self.comm.gather_logits(_linear_any(x, w.lm_head))
        else:
            lg = self.comm.lm_head(x, w.lm_head)
        if w.extra.get("lm_head_b") is not None:
            if self.comm.tp_size != 1:
                raise NotImplementedError("LM-head bias with a vocabulary-parallel head")
            lg = (lg.float() + w.extra["lm_head_b"].float()).to(lg.dtype)
        ls = cfg.extra.get("logits_scaling", 1.0)
        if ls != 1.0:
            lg = (lg.float() / ls).to(lg.dtype)
        if cfg.final_logit_softcap > 0:
            c = cfg.final_logit_softcap
            lg = (torch.tanh(lg.float() / c) * c).to(lg.dtype)
        return lg

    def forward(self, b: StepBatch, kv_layers: list[KVLayer]) -> torch.Tensor:
        h = self.forward_hidden(b, kv_layers)
        return self.logits(h, b.logits_rows)
