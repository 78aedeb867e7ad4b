"""Block drafter conditioned on the target's hidden states (DFlash style).

Where the MTP head drafts K tokens with K small autoregressive forwards, this drafter fills a whole
block in ONE forward: the block is ``[bonus token, mask, mask, ...]`` and every mask position is read
out at once. It is a small transformer (a handful of layers) whose attention has *split projections*:
keys and values come from two inputs, the projected hidden states of the target at several depths
(``fc`` over their concatenation, then a norm: the *context*, one row per token the target has
already processed) and the block itself; queries come from the block only. Context keys / values are
cached (own paged pool, same block tables and positions as the target's), block keys / values are
not: they are written behind the context and overwritten by the next round. Inside the block
attention is bidirectional. Reference: src/lib/mlxcel-core/src/drafter/dflash/ (model.rs,
attention.rs, round_loop.rs) and its engine wiring in src/server/batch/.

On the paged kernels a block's rows are decode rows that share one table and one context length
(context + block), exactly the mask described above; the context rows of a round only append.
Verification and acceptance are the engine's ordinary speculative round, so the output is that of
plain decoding whatever the drafter proposes.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .. import ops
from ..cache.kv_pool import KVPool
from ..config import ModelConfig
from ..models.weights import LayerWeights


@dataclass
class DFlashWeights:
    fc: torch.Tensor                 # [H, n_features * H]: concatenated target hidden states -> H
    hidden_norm: torch.Tensor        # [H]
    layers: list                     # LayerWeights: ln1, ln2, wqkv, wo, q_norm, k_norm, w_gate_up, w_down
    final_norm: torch.Tensor         # [H]
    lm_head: torch.Tensor | None = None   # None: the target's head
    embed: torch.Tensor | None = None     # None: the target's embedding table


def random_dflash_weights(dcfg: ModelConfig, n_features: int, seed: int = 0, dtype=torch.bfloat16, device="cpu",
                          std: float = 0.05) -> DFlashWeights:
    g = torch.Generator().manual_seed(seed)
    H, Hq, Hkv, D, I = dcfg.hidden_size, dcfg.num_attention_heads, dcfg.num_key_value_heads, dcfg.head_dim, dcfg.intermediate_size
    r = lambda *s: (torch.randn(*s, generator=g) * std).to(dtype).to(device)  # noqa: E731
    one = lambda n: (1 + torch.randn(n, generator=g) * 0.05).to(dtype).to(device)  # noqa: E731
    layers = [LayerWeights(ln1=one(H), ln2=one(H), wqkv=r((Hq + 2 * Hkv) * D, H), wo=r(H, Hq * D), q_norm=one(D), k_norm=one(D),
                           w_gate_up=r(2 * I, H), w_down=r(H, I)) for _ in range(dcfg.num_hidden_layers)]
    return DFlashWeights(fc=r(H, n_features * H), hidden_norm=one(H), layers=layers, final_norm=one(H))


class DFlashDrafter:
    """``dcfg``: the drafter's own geometry (hidden size = the target's); ``target_layers``: indices of
    the target layers whose output feeds the drafter; ``block``: tokens per block (bonus + drafts)."""

    needs_hidden = True

    def __init__(self, target, dcfg: ModelConfig, weights: DFlashWeights, target_layers: list[int], mask_token_id: int,
                 num_blocks: int, block: int = 16, block_size: int = 16):
        if dcfg.hidden_size != target.cfg.hidden_size:
            raise ValueError("the block drafter works in the target's hidden size")
        self.target, self.dcfg, self.w = target, dcfg, weights
        self.dev = target.device
        self.block, self.mask_id = int(block), int(mask_token_id)
        self.target_layers = tuple(int(i) for i in target_layers)
        target.capture_layers = self.target_layers
        self.Hq, self.Hkv, self.D = dcfg.num_attention_heads, dcfg.num_key_value_heads, dcfg.head_dim
        self.pool = KVPool(dcfg, num_blocks, block_size, device=self.dev, num_layers=len(weights.layers),
                           dtype=weights.final_norm.dtype)
        from ..ops.reference import rope_inv_freq
        inv, self.mscale = rope_inv_freq(dcfg.rot_dim, dcfg.rope_theta, dcfg.rope_scaling)
        self.inv_freq = inv.to(self.dev)
        self.pending: dict[int, tuple[int, torch.Tensor]] = {}   # seq -> (first position, context rows not in the pool yet)
        self.ctx_len: dict[int, int] = {}                        # seq -> context rows in the pool
        self.stale: set[int] = set()
        self.stats = dict(rounds=0, blocks=0)

    # ------------------------------------------------------------------ features
    def _features(self, rows: slice | None = None) -> torch.Tensor:
        """Context rows from what the target's last forward left in ``captured``."""
        caps = self.target.captured
        if len(caps) != len(self.target_layers):
            raise RuntimeError("the target did not capture the drafter's layers in its last forward")
        cat = torch.cat([c if rows is None else c[rows] for c in caps], dim=-1).contiguous()
        return ops.rmsnorm(ops.linear(cat, self.w.fc), self.w.hidden_norm, self.dcfg.rms_norm_eps, 0.0)

    # ------------------------------------------------------------------ one drafting forward
    @torch.inference_mode()
    def _draft(self, engine, items):
        """items: (seq, context rows [S, H] to append at ctx_len, bonus token). Returns the argmax of the
        block's mask positions per item, [len(items), block - 1]."""
        d, cfg, L = self.dev, self.dcfg, self.block
        n = len(items)
        mb = engine.max_blocks_per_seq
        tables = np.zeros((n, mb), dtype=np.int32)
        ctx_rows = sum(c.shape[0] for _, c, _ in items)
        slots = np.zeros(ctx_rows + n * L, dtype=np.int32)
        pos, toks, lens = [], [], []
        off = 0
        for s, c, _ in items:                         # context rows first ...
            start, S = self.ctx_len.get(s.seq_id, 0), c.shape[0]
            engine.bm.reserve(s.seq_id, start + S + L)
            engine.bm.fill_slots(s.seq_id, start, S, slots, off)
            pos += list(range(start, start + S))
            off += S
        for s, c, bonus in items:                     # ... then the blocks, behind their context
            start = self.ctx_len.get(s.seq_id, 0) + c.shape[0]
            engine.bm.fill_slots(s.seq_id, start, L, slots, off)
            pos += list(range(start, start + L))
            toks += [int(bonus)] + [self.mask_id] * (L - 1)
            lens += [start + L] * L
            off += L
        engine.bm.fill_tables([s.seq_id for s, _, _ in items], tables)
        row_tables = torch.from_numpy(np.repeat(tables, L, axis=0)).to(d)
        positions = torch.tensor(pos, dtype=torch.int32, device=d)
        slot_t = torch.from_numpy(slots).to(d)
        lens_t = torch.tensor(lens, dtype=torch.int32, device=d)
        emb = self.w.embed if self.w.embed is not None else self.target.w.embed
        x = ops.embedding(torch.tensor(toks, dtype=torch.int32, device=d), emb, cfg.embed_scale)
        xc = torch.cat([c for _, c, _ in items], dim=0).to(x.dtype).contiguous() if ctx_rows else x[:0]
        Hq, Hkv, D = self.Hq, self.Hkv, self.D
        nq = Hq * D
        eps = cfg.rms_norm_eps
        for lw, kv in zip(self.w.layers, self.pool.layers):
            qkv_b = ops.linear(ops.rmsnorm(x, lw.ln1, eps, 0.0), lw.wqkv)                 # block rows: q, k, v
            kv_c = ops.linear(xc, lw.wqkv[nq:].contiguous()) if ctx_rows else qkv_b[:0, nq:]   # context rows: k, v only
            qkv = torch.cat([torch.cat([kv_c.new_zeros(ctx_rows, nq), kv_c], dim=1), qkv_b], dim=0).contiguous()
            ops.rope_append(qkv, positions, slot_t, self.inv_freq, kv, Hq=Hq, Hkv=Hkv, D=D, rot_dim=cfg.rot_dim,
                            traditional=cfg.rope_traditional, mscale=self.mscale, q_norm_w=lw.q_norm, k_norm_w=lw.k_norm,
                            norm_eps=eps)
            a = ops.paged_decode(qkv[ctx_rows:, :nq], kv, row_tables, lens_t, Hq=Hq, Hkv=Hkv, D=D, scale=D ** -0.5,
                                 max_len=max(lens))
            x = ops.linear(a, lw.wo, residual=x)
            m = ops.glu_linear(ops.rmsnorm(x, lw.ln2, eps, 0.0), lw.w_gate_up, lw.w_gate_up.shape[0] // 2, cfg.hidden_act)
            x = ops.linear(m, lw.w_down, residual=x)
        head = self.w.lm_head if self.w.lm_head is not None else self.target.w.lm_head
        h = ops.rmsnorm(x, self.w.final_norm, eps, 0.0).view(n, L, -1)[:, 1:].reshape(n * (L - 1), -1).contiguous()
        from ..models.weights import QuantizedTensor
        if isinstance(head, QuantizedTensor):
            from ..ops import quant
            logits = quant.qlinear(h, head)
        else:
            logits = ops.linear(h, head)
        for s, c, _ in items:
            self.ctx_len[s.seq_id] = self.ctx_len.get(s.seq_id, 0) + c.shape[0]
        self.stats["blocks"] += n
        return ops.argmax(logits).view(n, L - 1).cpu().tolist()

    # ------------------------------------------------------------------ engine hooks
    def _queue(self, seq_id: int, start: int, rows: torch.Tensor) -> None:
        p = self.pending.get(seq_id)
        have = self.ctx_len.get(seq_id, 0) + (p[1].shape[0] if p is not None else 0)
        if seq_id in self.stale:
            return
        if start != have:
            self.stale.add(seq_id)
            self.pending.pop(seq_id, None)
            return
        first = p[0] if p is not None else start
        self.pending[seq_id] = (first, rows.clone() if p is None else torch.cat([p[1], rows], dim=0))

    def on_forward(self, engine, decode, pieces, hidden) -> None:
        """After an ordinary forward: every row that went through the target becomes a context row."""
        feats = self._features()
        row = 0
        for s in decode:
            self._queue(s.seq_id, s.total_len - 1, feats[row:row + 1])
            row += 1
        for s, start, cnt in pieces:
            if s.seq_id not in self.ctx_len and s.seq_id not in self.pending and start > 0:
                self.stale.add(s.seq_id)             # a prefix adopted from the cache never passed through here
            self._queue(s.seq_id, start, feats[row:row + cnt])
            row += cnt

    def on_verify(self, engine, accepted_info, hidden) -> None:
        feats = self._features()
        for s, row0, kept in accepted_info:
            if s.status.value == "finished":
                continue
            self._queue(s.seq_id, s.num_computed - kept - 1, feats[row0:row0 + kept + 1])

    def propose(self, engine, seqs, max_draft: int) -> list[list[int]]:
        out: list[list[int]] = [[] for _ in seqs]
        if max_draft <= 0:
            return out
        items, idx = [], []
        for i, s in enumerate(seqs):
            p = self.pending.pop(s.seq_id, None)
            if s.seq_id in self.stale:
                continue
            have = self.ctx_len.get(s.seq_id, 0)
            rows = p[1] if p is not None else None
            if (rows.shape[0] if rows is not None else 0) + have != s.total_len - 1:
                self.stale.add(s.seq_id)
                continue
            if rows is None:
                rows = torch.empty(0, self.dcfg.hidden_size, dtype=self.w.final_norm.dtype, device=self.dev)
            items.append((s, rows, s.tokens[-1]))
            idx.append(i)
        if not items:
            return out
        self.stats["rounds"] += 1
        props = self._draft(engine, items)
        for j, i in enumerate(idx):
            out[i] = props[j][:max_draft]
        return out

    def release(self, seq_id: int) -> None:
        self.pending.pop(seq_id, None)
        self.ctx_len.pop(seq_id, None)
        self.stale.discard(seq_id)


# ----------------------------------------------------------------------------- checkpoints
def is_dflash_dir(path) -> bool:
    """A drafter directory of this kind: its config names the target layers it conditions on."""
    import json
    from pathlib import Path
    f = Path(path) / "config.json"
    if not f.is_file():
        return False
    c = json.loads(f.read_text())
    return "target_layer_ids" in c and "mask_token_id" in c


def load_dflash(path, dtype=torch.bfloat16, device="cpu"):
    """Reads a block-drafter checkpoint: ``config.json`` (geometry, ``block_size``, ``mask_token_id``,
    ``target_layer_ids``, ``rope_is_neox_style``) and tensors ``fc.weight``, ``hidden_norm.weight``,
    ``layers.N.{input_layernorm, self_attn.{q,k,v,o}_proj, self_attn.{q,k}_norm, post_attention_layernorm,
    mlp.{gate,up,down}_proj}``, ``norm.weight`` and optionally ``embed_tokens.weight`` / ``lm_head.weight``
    (absent: the target's tables are used; names may carry a ``model.`` prefix).
    Returns (drafter config, weights, dict(block, mask_token_id, target_layers))."""
    import json
    from pathlib import Path

    from ..loading.checkpoint import TensorSource

    raw = json.loads((Path(path) / "config.json").read_text())
    dcfg = ModelConfig.from_dict(dict(
        model_type="qwen3", hidden_size=raw["hidden_size"], intermediate_size=raw["intermediate_size"],
        num_hidden_layers=raw["num_hidden_layers"], num_attention_heads=raw["num_attention_heads"],
        num_key_value_heads=raw.get("num_key_value_heads", raw["num_attention_heads"]),
        head_dim=raw.get("head_dim") or raw["hidden_size"] // raw["num_attention_heads"], vocab_size=raw["vocab_size"],
        rms_norm_eps=raw.get("rms_norm_eps", 1e-6), rope_theta=raw.get("rope_theta", 10000.0),
        max_position_embeddings=raw.get("max_position_embeddings", 32768)))
    dcfg.rope_traditional = not bool(raw.get("rope_is_neox_style", True))
    src = TensorSource(path)
    pre = "model." if any(k.startswith("model.") for k in src.keys()) else ""

    def t(name, required=True):
        for n in (pre + name, name):
            if src.has(n):
                return src.get(n).to(dtype).to(device).contiguous()
        if required:
            raise KeyError(f"{path}: missing tensor {name}")
        return None

    layers = []
    for i in range(dcfg.num_hidden_layers):
        p = f"layers.{i}."
        layers.append(LayerWeights(
            ln1=t(p + "input_layernorm.weight"), ln2=t(p + "post_attention_layernorm.weight"),
            wqkv=torch.cat([t(p + f"self_attn.{n}_proj.weight") for n in "qkv"]).contiguous(), wo=t(p + "self_attn.o_proj.weight"),
            q_norm=t(p + "self_attn.q_norm.weight"), k_norm=t(p + "self_attn.k_norm.weight"),
            w_gate_up=torch.cat([t(p + "mlp.gate_proj.weight"), t(p + "mlp.up_proj.weight")]).contiguous(),
            w_down=t(p + "mlp.down_proj.weight")))
    w = DFlashWeights(fc=t("fc.weight"), hidden_norm=t("hidden_norm.weight"), layers=layers, final_norm=t("norm.weight"),
                      lm_head=t("lm_head.weight", False), embed=t("embed_tokens.weight", False))
    if w.lm_head is None and raw.get("tie_word_embeddings") and w.embed is not None:
        w.lm_head = w.embed
    info = dict(block=int(raw.get("runtime_block_size") or raw.get("block_size", 16)), mask_token_id=int(raw["mask_token_id"]),
                target_layers=[int(i) for i in raw["target_layer_ids"]])
    return dcfg, w, info


def save_dflash(path, dcfg: ModelConfig, w: DFlashWeights, block: int, mask_token_id: int, target_layers: list[int]) -> None:
    """Writes a drafter directory that :func:`load_dflash` reads (tests, random-init drafters)."""
    import json
    from pathlib import Path

    from safetensors.torch import save_file

    Path(path).mkdir(parents=True, exist_ok=True)
    Hq, Hkv, D, I = dcfg.num_attention_heads, dcfg.num_key_value_heads, dcfg.head_dim, dcfg.intermediate_size
    tens = {"fc.weight": w.fc, "hidden_norm.weight": w.hidden_norm, "norm.weight": w.final_norm}
    for i, lw in enumerate(w.layers):
        p = f"layers.{i}."
        q, k, v = lw.wqkv[:Hq * D], lw.wqkv[Hq * D:(Hq + Hkv) * D], lw.wqkv[(Hq + Hkv) * D:]
        tens.update({p + "input_layernorm.weight": lw.ln1, p + "post_attention_layernorm.weight": lw.ln2,
                     p + "self_attn.q_proj.weight": q, p + "self_attn.k_proj.weight": k, p + "self_attn.v_proj.weight": v,
                     p + "self_attn.o_proj.weight": lw.wo, p + "self_attn.q_norm.weight": lw.q_norm,
                     p + "self_attn.k_norm.weight": lw.k_norm, p + "mlp.gate_proj.weight": lw.w_gate_up[:I],
                     p + "mlp.up_proj.weight": lw.w_gate_up[I:], p + "mlp.down_proj.weight": lw.w_down})
    if w.embed is not None:
        tens["embed_tokens.weight"] = w.embed
    if w.lm_head is not None and w.lm_head is not w.embed:
        tens["lm_head.weight"] = w.lm_head
    save_file({k: v.detach().cpu().contiguous() for k, v in tens.items()}, str(Path(path) / "model.safetensors"))
    (Path(path) / "config.json").write_text(json.dumps(dict(
        architectures=["DFlashDraftModel"], hidden_size=dcfg.hidden_size, intermediate_size=I,
        num_hidden_layers=dcfg.num_hidden_layers, num_attention_heads=Hq, num_key_value_heads=Hkv, head_dim=D,
        vocab_size=dcfg.vocab_size, rms_norm_eps=dcfg.rms_norm_eps, rope_theta=dcfg.rope_theta,
        rope_is_neox_style=not dcfg.rope_traditional, block_size=block, mask_token_id=mask_token_id,
        target_layer_ids=list(target_layers), num_target_layers=len(target_layers),
        tie_word_embeddings=w.lm_head is w.embed and w.embed is not None), indent=1))
