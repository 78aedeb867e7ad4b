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

    def set_aliases(self, aliases: dict) -> None:
        """``{canonical: (actual, transform | None)}`` (see ``loading/aliases.py``): the canonical names
        become resolvable, reading the actual tensor and fixing its layout on the way."""
        self.aliases = dict(aliases)
        for canon, (actual, _) in self.aliases.items():
            self.index[canon] = self.index[actual]

    def set_edits(self, edits: list[dict]) -> None:
        """Load-time weight surgery (see ``loading/surgery.py``): applied to every tensor fetched."""
        self.edits = list(edits)

    def get(self, name: str) -> torch.Tensor:
        t = self._get_raw(name)
        edits = getattr(self, "edits", None)
        if edits and t.is_floating_point():
            from .surgery import apply_edits
            t = apply_edits(edits, name, t, lambda n: self._get_raw(n) if n in self.index else None)
        return t

    def _get_raw(self, name: str) -> torch.Tensor:
        alias = getattr(self, "aliases", {}).get(name)
        if alias is not None:
            t = self._get_raw(alias[0])
            return alias[1](t) if alias[1] is not None else t
        return self._handle(name).get_tensor(name)

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

    def _shard_path(self, f: str) -> Path:
        """A shard named by the index must be a file inside the checkpoint directory: an entry such
        as ``../../x.safetensors`` (or a symlink leading elsewhere) is refused, whether or not the
        target exists."""
        root = self.dir.resolve()
        real = (self.dir / f).resolve()
        if not real.is_relative_to(root):
            raise ValueError(f"weight_map entry {f!r} points outside the checkpoint directory")
        if not real.is_file():
            raise FileNotFoundError(str(self.dir / f))
        return real

    def _handle(self, name):
        f = self.index[name]
        if f not in self._handles:
            self._handles[f] = self._open(str(self._shard_path(f)), framework="pt")
        return self._handles[f]


def _infer_quant(packed: torch.Tensor, scales: torch.Tensor, biases, qc: QuantConfig | None) -> QuantizedTensor:
    """Mode / bits / group of one quantized matrix, verified against the tensor shapes
    (packed_in * 32 == bits * in, in == groups * group_size)."""
    groups = scales.shape[-1]
    words = packed.shape[-1]
    if biases is not None:
        mode = "affine"
    elif qc is not None and qc.mode in ("mxfp4", "mxfp8", "nvfp4"):
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
            if mode in ("mxfp4", "nvfp4") and bits != 4:
                continue
            if mode == "mxfp8" and bits != 8:
                continue
            if mode == "mxfp4" and g == 16:
                mode = "nvfp4"                   # 4-bit floats in groups of 16 carry e4m3 scales
            if mode == "nvfp4" and g != 16:
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
        if w.dtype == torch.uint8 and self.src.has(base + ".weight_scale"):
            return self._unpack_bitlinear(base, w)
        sname = base + ".scales"
        if self.src.has(sname) and w.dtype in (torch.uint32, torch.int32, torch.uint8):
            scales = self.src.get(sname)
            biases = self.src.get(base + ".biases") if self.src.has(base + ".biases") else None
            qt = _infer_quant(w, scales, biases, self.cfg.quantization.for_module(base))
            if self.deq or qt.mode == "nvfp4":
                # (nvfp4: no kernel reads e4m3 group scales; the matrix is expanded once at load)
                from ..ops.quant import dequantize_ref
                return dequantize_ref(qt, self.dtype)
            if qt.mode == "affine":
                qt.scales, qt.biases = qt.scales.to(self.dtype), qt.biases.to(self.dtype)
            return qt
        if w.dtype in (torch.float8_e4m3fn, torch.float8_e5m2):
            return self._dequant_fp8(base, w)
        return w.to(self.dtype)

    def _unpack_bitlinear(self, base: str, packed: torch.Tensor) -> torch.Tensor:
        """BitLinear storage: ternary weights {-1, 0, +1} as 2-bit codes (value + 1), four OUTPUT rows to a
        byte (bits 2i..2i+1 of packed row r hold output row r + i * N / 4), and one scale that divides
        (or, for ``autobitlinear`` checkpoints, multiplies) the output. Expanded to a dense matrix with
        the scale folded in."""
        rows = [((packed >> (2 * i)) & 3).to(torch.int8) - 1 for i in range(4)]
        w = torch.cat(rows, 0).float()
        scale = self.src.get(base + ".weight_scale").float().reshape(-1)[0]
        w = w / scale if self.cfg.extra.get("bitlinear_invert_scale", True) else w * scale
        return w.to(self.dtype)

    def _dequant_fp8(self, base: str, w: torch.Tensor) -> torch.Tensor:
        """FP8 checkpoints are widened at load (reference src/models/fp8_block.rs, fp8_ct.rs): block-scaled
        weights carry ``weight_scale_inv`` with one fp32 factor per ``weight_block_size`` tile (DeepSeek-V3
        style, 128 x 128 unless the config says otherwise); compressed-tensors style weights carry
        ``weight_scale`` per tensor or per output channel. Either way ``w = fp8 * scale``."""
        wf = w.float()
        if self.src.has(base + ".weight_scale_inv"):
            sc = self.src.get(base + ".weight_scale_inv").float()
            bs = getattr(self.cfg.quantization, "block_size", None) or self.cfg.extra.get("fp8_block_size") or (128, 128)
            if sc.dim() == 2 and wf.dim() == 2:
                sc = sc.repeat_interleave(int(bs[0]), 0)[: wf.shape[0]].repeat_interleave(int(bs[1]), 1)[:, : wf.shape[1]]
            wf = wf * sc
        elif self.src.has(base + ".weight_scale"):
            sc = self.src.get(base + ".weight_scale").float()
            wf = wf * (sc.reshape(-1, 1) if sc.numel() == wf.shape[0] and wf.dim() == 2 else sc)
        return wf.to(self.dtype)


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
    # rows are the second-to-last axis (stacked expert tensors carry the expert axis in front)
    return torch.cat(parts, dim=0 if parts[0].dim() < 2 else -2)


def _stack(parts):
    if isinstance(parts[0], QuantizedTensor):
        q = parts[0]
        return QuantizedTensor(torch.stack([p.packed for p in parts]), torch.stack([p.scales for p in parts]),
                               None if q.biases is None else torch.stack([p.biases for p in parts]),
                               q.bits, q.group_size, q.mode)
    return torch.stack(parts)


# ----------------------------------------------------------------------------- assembly
def _first(g: _Getter, *bases):
    for b in bases:
        if g.has(b):
            return b
    return None


def _load_attention(g: _Getter, cfg: ModelConfig, p: str, lw_kwargs: dict) -> None:
    a = p + ".self_attn"
    if cfg.extra.get("mla"):
        # DeepSeek multi-head latent attention: low-rank query path (optional), latent + rotary key
        # projection, per-head expansion of the latent
        mla = dict(kv_a=g.mat(a + ".kv_a_proj_with_mqa"), kv_a_b=g.vec(a + ".kv_a_proj_with_mqa.bias"),
                   kv_a_norm=g.vec(a + ".kv_a_layernorm.weight"), kv_b=g.mat(a + ".kv_b_proj"))
        if g.has(a + ".q_a_proj"):
            mla.update(q_a=g.mat(a + ".q_a_proj"), q_a_b=g.vec(a + ".q_a_proj.bias"),
                       q_a_norm=g.vec(a + ".q_a_layernorm.weight"), q_b=g.mat(a + ".q_b_proj"))
        else:
            mla["q"] = g.mat(a + ".q_proj")
        from ..models.weights import QuantizedTensor as _QT
        for k_, v_ in list(mla.items()):
            if isinstance(v_, _QT):
                from ..ops.quant import dequantize_ref
                mla[k_] = dequantize_ref(v_, g.dtype)
        lw_kwargs.update(mla=mla, wqkv=None, bqkv=None, wo=g.mat(a + ".o_proj"), bo=g.vec(a + ".o_proj.bias"),
                         q_norm=None, k_norm=None, sinks=None)
        return
    if g.has(a + ".qkv_proj"):                       # Phi-3 style fused projection
        lw_kwargs["wqkv"] = g.mat(a + ".qkv_proj")
        lw_kwargs["bqkv"] = g.vec(a + ".qkv_proj.bias")
    else:
        lw_kwargs["wqkv"] = _cat_rows([g.mat(a + ".q_proj"), g.mat(a + ".k_proj"), g.mat(a + ".v_proj")])
        bs = [g.vec(a + f".{n}_proj.bias") for n in "qkv"]
        lw_kwargs["bqkv"] = torch.cat(bs) if all(b is not None for b in bs) else None
    ob = a + (".o_proj" if g.has(a + ".o_proj") else ".dense")      # Phi names the output projection "dense"
    lw_kwargs["wo"] = g.mat(ob)
    lw_kwargs["bo"] = g.vec(ob + ".bias")
    lw_kwargs["q_norm"] = g.vec(_first_name(g.src, a + ".q_norm.weight", a + ".query_layernorm.weight"))
    lw_kwargs["k_norm"] = g.vec(_first_name(g.src, a + ".k_norm.weight", a + ".key_layernorm.weight"))
    if lw_kwargs["q_norm"] is None and cfg.extra.get("qk_norm_no_params"):
        lw_kwargs["q_norm"] = torch.ones(cfg.head_dim, dtype=g.dtype)       # norms without gains
        lw_kwargs["k_norm"] = torch.ones(cfg.head_dim, dtype=g.dtype)
    if cfg.norm_weight_bias and lw_kwargs["q_norm"] is not None:
        # Gemma 3 stores the per-head norms as (weight - 1) like its other norms; the fused
        # q/k-norm + RoPE kernel takes plain gains
        lw_kwargs["q_norm"] = (lw_kwargs["q_norm"].float() + cfg.norm_weight_bias).to(lw_kwargs["q_norm"].dtype)
        lw_kwargs["k_norm"] = (lw_kwargs["k_norm"].float() + cfg.norm_weight_bias).to(lw_kwargs["k_norm"].dtype)
    sinks = g.src.get(a + ".sinks").float() if g.src.has(a + ".sinks") else None
    lw_kwargs["sinks"] = sinks


def _load_dense_mlp(g: _Getter, p: str, lw: LayerWeights) -> None:
    m = p + ".mlp"
    plain = next(((a, b) for a, b in ((".c_fc", ".c_proj"), (".fc1", ".fc2"), (".up_proj", ".down_proj"))
                  if g.has(m + a) and not g.has(m + ".gate_proj") and not g.has(m + ".gate_up_proj")), None)
    if plain is not None:                                   # non-gated MLP: fc -> act -> proj
        lw.w_gate_up, lw.b_gate_up = g.mat(m + plain[0]), g.vec(m + plain[0] + ".bias")
        lw.w_down, lw.b_down = g.mat(m + plain[1]), g.vec(m + plain[1] + ".bias")
        return
    if g.has(m + ".gate_up_proj"):
        lw.w_gate_up = g.mat(m + ".gate_up_proj")
    else:
        lw.w_gate_up = _cat_rows([g.mat(m + ".gate_proj"), g.mat(m + ".up_proj")])
        bg, bu = g.vec(m + ".gate_proj.bias"), g.vec(m + ".up_proj.bias")
        lw.b_gate_up = torch.cat([bg, bu]) if bg is not None and bu is not None else None
    lw.w_down = g.mat(m + ".down_proj")
    lw.b_down = g.vec(m + ".down_proj.bias")


def _load_moe(g: _Getter, cfg: ModelConfig, p: str, lw: LayerWeights) -> None:
    E = cfg.num_experts
    # router
    rb = _first(g, p + ".mlp.router.gate", p + ".mlp.router", p + ".mlp.gate.wg", p + ".mlp.gate", p + ".block_sparse_moe.gate",
                p + ".block_sparse_moe.router.layer")
    r = g.mat(rb)
    if isinstance(r, QuantizedTensor):   # routers are small: keep them dense
        from ..ops.quant import dequantize_ref
        r = dequantize_ref(r, g.dtype)
    lw.router_w = r
    lw.router_b = g.vec(rb + ".bias")
    for bias_name in (rb + ".e_score_correction_bias", p + ".mlp.expert_bias", p + ".mlp.moe_statics.e_score_correction_bias",
                      p + ".mlp.e_score_correction_bias", p + ".block_sparse_moe.e_score_correction_bias"):
        if g.src.has(bias_name):                               # DeepSeek-V3 / ERNIE routing: selection bias (fp32)
            lw.router_b = g.src.get(bias_name).float().reshape(-1)
    # experts: stacked MLX switch layers, GPT-OSS fused tensors, or per-expert HF modules
    sw = _first(g, p + ".mlp.switch_mlp.gate_proj", p + ".block_sparse_moe.switch_mlp.gate_proj",
                p + ".mlp.experts.gate_proj")
    if sw is not None:
        root = sw[: -len(".gate_proj")]
        gate, up, down = g.mat(root + ".gate_proj"), g.mat(root + ".up_proj"), g.mat(root + ".down_proj")
        lw.experts_gate_up = _cat_rows([gate, up])
        lw.experts_down = down
        bg, bu, bd = g.vec(root + ".gate_proj.bias"), g.vec(root + ".up_proj.bias"), g.vec(root + ".down_proj.bias")
        if bg is not None and bu is not None:
            lw.experts_gate_up_b = torch.cat([bg, bu], dim=-1)
        lw.experts_down_b = bd
    elif g.src.has(p + ".block_sparse_moe.input_linear.weight"):
        # GraniteMoE: fused [E, 2I, H] (gate rows first) and [E, H, I]
        lw.experts_gate_up = g.src.get(p + ".block_sparse_moe.input_linear.weight").to(g.dtype).contiguous()
        lw.experts_down = g.src.get(p + ".block_sparse_moe.output_linear.weight").to(g.dtype).contiguous()
    elif g.src.has(p + ".mlp.experts.gate_up_proj") and cfg.model_type != "gpt_oss":
        # fused expert tensors already in Linear orientation: [E, 2I, H] (gate rows, then up rows), [E, H, I]
        lw.experts_gate_up = g.src.get(p + ".mlp.experts.gate_up_proj").to(g.dtype).contiguous()
        lw.experts_down = g.src.get(p + ".mlp.experts.down_proj").to(g.dtype).contiguous()
    elif g.src.has(p + ".mlp.experts.gate_up_proj"):
        # GPT-OSS HF layout: [E, H, 2I] with gate/up interleaved along the last dim
        gu = g.src.get(p + ".mlp.experts.gate_up_proj").to(g.dtype)
        gate, up = gu[..., 0::2], gu[..., 1::2]
        lw.experts_gate_up = torch.cat([gate, up], dim=-1).transpose(1, 2).contiguous()
        lw.experts_down = g.src.get(p + ".mlp.experts.down_proj").to(g.dtype).transpose(1, 2).contiguous()
        if g.src.has(p + ".mlp.experts.gate_up_proj_bias"):
            b = g.src.get(p + ".mlp.experts.gate_up_proj_bias").to(g.dtype)
            lw.experts_gate_up_b = torch.cat([b[..., 0::2], b[..., 1::2]], dim=-1).contiguous()
            lw.experts_down_b = g.src.get(p + ".mlp.experts.down_proj_bias").to(g.dtype)
    else:
        names = (("w1", "w3", "w2") if g.has(p + ".block_sparse_moe.experts.0.w1")
                 else ("gate_proj", "up_proj", "down_proj"))
        root = p + (".block_sparse_moe.experts" if names[0] == "w1" else ".mlp.experts")
        gus, downs = [], []
        for e in range(E):
            gus.append(_cat_rows([g.mat(f"{root}.{e}.{names[0]}"), g.mat(f"{root}.{e}.{names[1]}")]))
            downs.append(g.mat(f"{root}.{e}.{names[2]}"))
        lw.experts_gate_up, lw.experts_down = _stack(gus), _stack(downs)
    sh = next((p + n for n in (".mlp.shared_experts", ".mlp.shared_mlp") if g.has(p + n + ".gate_proj")),
              p + ".mlp.shared_expert")
    if g.src.has(p + ".shared_mlp.input_linear.weight"):
        # GraniteMoE-shared: an always-on gated MLP stored fused ([2S, H], gate rows first)
        lw.shared_gate_up = g.mat(p + ".shared_mlp.input_linear")
        lw.shared_down = g.mat(p + ".shared_mlp.output_linear")
    elif g.has(sh + ".gate_proj"):
        lw.shared_gate_up = _cat_rows([g.mat(sh + ".gate_proj"), g.mat(sh + ".up_proj")])
        lw.shared_down = g.mat(sh + ".down_proj")
        sg = g.mat(p + ".mlp.shared_expert_gate")
        lw.shared_gate = sg if not isinstance(sg, QuantizedTensor) else None


def load_full_weights(path: str | Path, cfg: ModelConfig, dtype=torch.bfloat16, dequantize: bool = False,
                      layers: range | None = None, surgery: str | None = None) -> ModelWeights:
    """Read a checkpoint directory into host memory in the executor's fused layout.
    ``surgery``: YAML file of load-time weight edits (``loading/surgery.py``)."""
    src = TensorSource(path)
    if surgery:
        from .surgery import load_edits
        src.set_edits(load_edits(surgery))
    from .aliases import aliases_for
    al = aliases_for(cfg, list(src.keys()))
    if al:
        src.set_aliases(al)
    g = _Getter(src, cfg, dtype, dequantize)
    pre = "model." if any(k.startswith("model.") for k in src.keys()) else ""
    if any(k.startswith("language_model.model.") for k in src.keys()):
        pre = "language_model.model."
    else:
        # vision-language wrappers nest the language model (``model.language_model.``,
        # ``model.language_model.model.``, ...): take the prefix of its embedding table
        nested = [k for k in src.keys() if k.endswith(".embed_tokens.weight") and ("language_model" in k or "text_model" in k)]
        if len(nested) == 1:
            pre = nested[0][: -len("embed_tokens.weight")]
    emb = g.mat(pre + "embed_tokens")
    if isinstance(emb, QuantizedTensor):
        from ..ops.quant import dequantize_ref
        emb_q, emb = emb, dequantize_ref(emb, dtype)
    else:
        emb_q = None
    lws = []
    for i in (layers if layers is not None else range(cfg.num_hidden_layers)):
        p = f"{pre}layers.{i}"
        kw: dict = {}
        _load_attention(g, cfg, p, kw)
        ln1 = g.vec(_first_name(src, p + ".input_layernorm.weight", p + ".attention_layernorm.weight"))
        ln2 = g.vec(_first_name(src, p + ".post_attention_layernorm.weight", p + ".pre_feedforward_layernorm.weight",
                                p + ".feedforward_layernorm.weight"))
        if cfg.extra.get("norm_no_params"):                     # OLMo-1: LayerNorm without gain or bias
            ln1 = ln2 = torch.ones(cfg.hidden_size, dtype=dtype)
        elif ln2 is None and cfg.extra.get("parallel_block"):
            ln2 = ln1                                           # one norm feeds both branches
        lw = LayerWeights(ln1=ln1, ln2=ln2, **kw)
        lw.ln1_b = g.vec(p + ".input_layernorm.bias")
        lw.ln2_b = g.vec(p + ".post_attention_layernorm.bias")
        if cfg.extra.get("post_norm_only"):
            lw.post_attn_norm = g.vec(p + ".post_attention_layernorm.weight")
            lw.post_mlp_norm = g.vec(p + ".post_feedforward_layernorm.weight")
            lw.ln1 = lw.ln2 = lw.post_attn_norm          # placeholders: this layout has no pre-norms
        if cfg.post_norms:
            names = cfg.extra.get("post_norm_names",
                                  ("post_attention_layernorm", "pre_feedforward_layernorm", "post_feedforward_layernorm"))
            lw.post_attn_norm = g.vec(f"{p}.{names[0]}.weight")
            lw.ln2 = g.vec(f"{p}.{names[1]}.weight")
            lw.post_mlp_norm = g.vec(f"{p}.{names[2]}.weight")
        if cfg.is_moe and _first(g, p + ".mlp.router.gate", p + ".mlp.router", p + ".mlp.gate.wg", p + ".mlp.gate", p + ".block_sparse_moe.gate",
                                 p + ".block_sparse_moe.router.layer"):
            _load_moe(g, cfg, p, lw)
        else:
            _load_dense_mlp(g, p, lw)
        if cfg.extra.get("norm_plus_one"):                      # LayerNorm1P: stored as (weight - 1)
            lw.ln1, lw.ln2 = lw.ln1 + 1.0, lw.ln2 + 1.0
        if cfg.extra.get("attn_output_gate"):
            lw.attn_gate = g.mat(p + ".self_attn.gate_proj")
        lw.attn_sub_norm = g.vec(p + ".self_attn.attn_sub_norm.weight")
        lw.ffn_sub_norm = g.vec(p + ".mlp.ffn_sub_norm.weight")
        if src.has(p + ".mlp.act_fn.alpha_p"):                 # xIELU (Apertus): stored before softplus
            sp = torch.nn.functional.softplus
            beta = float(src.get(p + ".mlp.act_fn.beta")) if src.has(p + ".mlp.act_fn.beta") else 0.5
            eps_x = float(src.get(p + ".mlp.act_fn.eps")) if src.has(p + ".mlp.act_fn.eps") else -1e-6
            lw.act_params = (float(sp(src.get(p + ".mlp.act_fn.alpha_p").float())),
                             beta + float(sp(src.get(p + ".mlp.act_fn.alpha_n").float())), beta, eps_x)
        lws.append(lw)
    final_norm = g.vec(_first_name(src, pre + "norm.weight", pre + "final_layernorm.weight"))
    if cfg.extra.get("norm_no_params"):
        final_norm = torch.ones(cfg.hidden_size, dtype=dtype)
    if cfg.extra.get("norm_plus_one"):
        final_norm = final_norm + 1.0
    head_base = "lm_head" if g.has("lm_head") else ("language_model.lm_head" if g.has("language_model.lm_head") else None)
    if head_base is not None and not cfg.tie_word_embeddings:
        lm_head = g.mat(head_base)
    else:
        lm_head = emb_q if (emb_q is not None and not dequantize) else emb
    mw = ModelWeights(embed=emb, layers=lws, final_norm=final_norm, lm_head=lm_head)
    if src.has(pre + "embed_positions.weight"):               # learned absolute positions (GPT-2 family)
        mw.extra["pos_embed"] = g.vec(pre + "embed_positions.weight")
    fb = g.vec(_first_name(src, pre + "norm.bias", pre + "final_layernorm.bias"))
    if fb is not None:
        mw.extra["final_norm_b"] = fb
    if head_base is not None and g.vec(head_base + ".bias") is not None:
        mw.extra["lm_head_b"] = g.vec(head_base + ".bias")
    return mw


def _first_name(src: TensorSource, *names):
    for n in names:
        if src.has(n):
            return n
    return names[0]


def _to_device(w: ModelWeights, device) -> ModelWeights:
    def mv(x):
        if isinstance(x, (torch.Tensor, QuantizedTensor)):
            return x.to(device)
        return x

    tied = w.lm_head is w.embed
    w.embed, w.final_norm = mv(w.embed), mv(w.final_norm)
    w.lm_head = w.embed if tied else mv(w.lm_head)
    for lw in w.layers:
        for k, v in list(vars(lw).items()):
            setattr(lw, k, mv(v))
    return w


def load_model_weights(path: str | Path, cfg: ModelConfig, device="cuda", comm=None, dequantize: bool = False,
                       layers: range | None = None, dtype=torch.bfloat16, surgery: str | None = None) -> ModelWeights:
    """Load, shard for this rank (tensor / expert parallel, pipeline layer range) and upload."""
    full = load_full_weights(path, cfg, dtype=dtype, dequantize=dequantize, layers=layers, surgery=surgery)
    tp = comm.tp_size if comm is not None else 1
    if tp > 1:
        full = shard_weights(cfg, full, comm.tp_rank, tp, ep=getattr(comm, "ep_size", tp))
    return _to_device(full, device)


def save_checkpoint(path: str | Path, cfg_dict: dict, w: ModelWeights, quantization: dict | None = None) -> None:
    """Write an MLX/HF-style checkpoint directory (used by tests, `split-mtp` and the random-init tool)."""
    from safetensors.torch import save_file

    out = Path(path)
    out.mkdir(parents=True, exist_ok=True)
    cfg = ModelConfig.from_dict(cfg_dict)
    t: dict[str, torch.Tensor] = {}

    def put(base: str, v):
        if v is None:
            return
        if isinstance(v, QuantizedTensor):
            t[base + ".weight"] = v.packed.contiguous().cpu()
            t[base + ".scales"] = v.scales.contiguous().cpu()
            if v.biases is not None:
                t[base + ".biases"] = v.biases.contiguous().cpu()
        else:
            t[base + ".weight"] = v.contiguous().cpu()

    def rows(v, lo, hi):
        from .shard import _rows
        return _rows(v, lo, hi)

    D, Hq, Hkv = cfg.head_dim, cfg.num_attention_heads, cfg.num_key_value_heads
    put("model.embed_tokens", w.embed)
    t["model.norm.weight"] = w.final_norm.cpu()
    if not cfg.tie_word_embeddings:
        put("lm_head", w.lm_head)
    for i, lw in enumerate(w.layers):
        p = f"model.layers.{i}"
        t[p + ".input_layernorm.weight"] = lw.ln1.cpu()
        t[p + ".post_attention_layernorm.weight"] = lw.ln2.cpu()
        q1, k1 = Hq * D, (Hq + Hkv) * D
        put(p + ".self_attn.q_proj", rows(lw.wqkv, 0, q1))
        put(p + ".self_attn.k_proj", rows(lw.wqkv, q1, k1))
        put(p + ".self_attn.v_proj", rows(lw.wqkv, k1, k1 + Hkv * D))
        put(p + ".self_attn.o_proj", lw.wo)
        if lw.bqkv is not None:
            t[p + ".self_attn.q_proj.bias"] = lw.bqkv[:q1].cpu()
            t[p + ".self_attn.k_proj.bias"] = lw.bqkv[q1:k1].cpu()
            t[p + ".self_attn.v_proj.bias"] = lw.bqkv[k1:].cpu()
        if lw.bo is not None:
            t[p + ".self_attn.o_proj.bias"] = lw.bo.cpu()
        if lw.q_norm is not None:
            t[p + ".self_attn.q_norm.weight"] = lw.q_norm.cpu()
            t[p + ".self_attn.k_norm.weight"] = lw.k_norm.cpu()
        if lw.sinks is not None:
            t[p + ".self_attn.sinks"] = lw.sinks.cpu()
        if lw.w_gate_up is not None:
            I = cfg.intermediate_size
            put(p + ".mlp.gate_proj", rows(lw.w_gate_up, 0, I))
            put(p + ".mlp.up_proj", rows(lw.w_gate_up, I, 2 * I))
            put(p + ".mlp.down_proj", lw.w_down)
        if lw.router_w is not None:
            mi = cfg.moe_intermediate_size
            put(p + ".mlp.router", lw.router_w)
            if lw.router_b is not None:
                t[p + ".mlp.router.bias"] = lw.router_b.cpu()
            put(p + ".mlp.switch_mlp.gate_proj", rows(lw.experts_gate_up, 0, mi))
            put(p + ".mlp.switch_mlp.up_proj", rows(lw.experts_gate_up, mi, 2 * mi))
            put(p + ".mlp.switch_mlp.down_proj", lw.experts_down)
            if lw.experts_gate_up_b is not None:
                t[p + ".mlp.switch_mlp.gate_proj.bias"] = lw.experts_gate_up_b[:, :mi].contiguous().cpu()
                t[p + ".mlp.switch_mlp.up_proj.bias"] = lw.experts_gate_up_b[:, mi:].contiguous().cpu()
                t[p + ".mlp.switch_mlp.down_proj.bias"] = lw.experts_down_b.cpu()
    save_file(t, str(out / "model.safetensors"))
    cd = dict(cfg_dict)
    if quantization:
        cd["quantization"] = quantization
    (out / "config.json").write_text(json.dumps(cd, indent=1))
