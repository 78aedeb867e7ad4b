"""Memory estimator (`mlxcel inspect`, serve preflight): weights, KV pool, activations per GPU.
Counterpart of the reference's byte-exact estimator (src/execution/memory_estimate.rs)."""
from __future__ import annotations

from ..config import ModelConfig


def _block_kinds(cfg: ModelConfig) -> list[str] | None:
    """Pattern characters of a state-space or hybrid model (one per block), None for attention-only models."""
    if cfg.model_type == "mamba2":
        return ["M"] * cfg.num_hidden_layers
    if cfg.model_type == "mamba":
        return ["m"] * cfg.num_hidden_layers
    pat = cfg.extra.get("hybrid_pattern")
    return list(pat) if pat else None


def _recurrent_block(cfg: ModelConfig, kind: str) -> tuple[int, int]:
    """(parameters, fp32 state bytes per sequence) of one block of a state-space / hybrid model."""
    h, x = cfg.hidden_size, cfg.extra
    attn = h * (cfg.q_size + 2 * cfg.kv_size) + cfg.q_size * h
    if kind in ("M", "P"):
        m = x["mamba"]
        di = m.get("d_inner", m.get("expand", 2) * h)
        P, G, N, K = m.get("head_dim", 64), m.get("n_groups", 1), m.get("d_state", 128), m.get("d_conv", 4)
        heads, conv = di // P, di + 2 * G * N
        par = h * (2 * di + 2 * G * N + heads) + conv * K + di * h + 3 * heads + di + h
        st = 4 * ((K - 1) * conv + heads * P * N)
        return (par + attn, st) if kind == "P" else (par, st)
    if kind == "m":
        m = x["mamba1"]
        di, N, K, R = m["d_inner"], m["d_state"], m["d_conv"], m["dt_rank"]
        return 2 * di * h + di * K + (R + 2 * N) * di + di * R + di * N + 2 * di + di * h + h, 4 * ((K - 1) * di + di * N)
    if kind == "L":
        m = x["gdn"]
        kd, vd = m["k_heads"] * m["k_dim"], m["v_heads"] * m["v_dim"]
        conv = 2 * kd + vd
        return (h * (2 * kd + 2 * vd) + 2 * m["v_heads"] * h + conv * m["d_conv"] + vd * h + h,
                4 * ((m["d_conv"] - 1) * conv + m["v_heads"] * m["k_dim"] * m["v_dim"]))
    if kind == "C":
        K = x["shortconv"]["d_conv"]
        return 4 * h * h + h * K + h, 4 * (K - 1) * h
    if kind in ("*", "A"):
        return attn + (cfg.q_size * h if kind == "A" else 0) + h, 0
    if kind == "-":
        return 2 * h * cfg.intermediate_size + h, 0
    if kind == "G":
        return 3 * h * int(x.get("mlp_size", cfg.intermediate_size)) + h, 0
    if kind == "E":
        mi = cfg.moe_intermediate_size or cfg.intermediate_size
        shared = cfg.shared_expert_intermediate_size or int(x.get("mlp_size", 0) or 0)
        return cfg.num_experts * 3 * h * mi + h * cfg.num_experts + 3 * h * shared + h, 0
    return 0, 0


def estimate_memory(cfg: ModelConfig, ctx: int = 8192, parallel: int = 4, kv_bits: int = 16, tp: int = 1,
                    max_batch_tokens: int = 8192, block_size: int = 16) -> dict:
    q = cfg.quantization
    bpp = 2.0 if q.mode == "none" else q.bits / 8.0 + (4.0 if q.mode == "affine" else 1.0) / q.group_size
    emb = cfg.vocab_size * cfg.hidden_size * (1 if cfg.tie_word_embeddings else 2)
    kinds = _block_kinds(cfg)
    state_seq = 0
    if kinds is None:
        params = cfg.param_count()
        kv_tok = cfg.kv_bytes_per_token(kv_bits) / min(tp, cfg.num_key_value_heads)
    else:
        # state-space / hybrid models: parameters and per-sequence recurrent state block by block; only
        # the attention blocks have KV; state slots are allocated for 2 x parallel sequences in fp32
        per = [_recurrent_block(cfg, k) for k in kinds]
        params = sum(p for p, _ in per) + emb + cfg.hidden_size
        state_seq = sum(s for _, s in per)
        n_attn = sum(k in ("*", "A", "P") for k in kinds)
        kv_tok = cfg.kv_bytes_per_token(kv_bits) / max(cfg.num_hidden_layers, 1) * n_attn
    weights = (params - emb) * bpp / tp + emb * 2 / (1 if tp == 1 else 1)  # embedding replicated, head sharded
    blocks = (ctx + block_size - 1) // block_size * parallel
    kv = blocks * block_size * kv_tok
    act = max_batch_tokens * (cfg.hidden_size * 6 + (cfg.q_size + 2 * cfg.kv_size) // tp +
                              3 * max(cfg.intermediate_size, cfg.moe_intermediate_size) // tp) * 2
    logits = parallel * cfg.vocab_size * 2
    state = 2 * parallel * state_seq
    total = weights + kv + state + act + logits + (64 << 20)
    return dict(model_type=cfg.model_type, parameters=params, recurrent_state_bytes_per_seq=int(state_seq),
                recurrent_state_bytes=int(state), bytes_per_param=round(bpp, 4),
                weights_bytes=int(weights), kv_bytes_per_token=int(kv_tok), kv_pool_blocks=blocks,
                kv_pool_bytes=int(kv), activation_bytes=int(act), logits_bytes=int(logits),
                total_bytes=int(total), total_gib=round(total / 2 ** 30, 3), fits_b200=total < 170 * 2 ** 30)
