"""Memory estimator (`mlxcel inspect`, serve preflight): weights, KV pool, activations per GPU.
Counterpart of the reference's byte-exact estimator (src/execution/memory_estimate.rs)."""
from __future__ import annotations

from ..config import ModelConfig


def estimate_memory(cfg: ModelConfig, ctx: int = 8192, parallel: int = 4, kv_bits: int = 16, tp: int = 1,
                    max_batch_tokens: int = 8192, block_size: int = 16) -> dict:
    q = cfg.quantization
    bpp = 2.0 if q.mode == "none" else q.bits / 8.0 + (4.0 if q.mode == "affine" else 1.0) / q.group_size
    params = cfg.param_count()
    emb = cfg.vocab_size * cfg.hidden_size * (1 if cfg.tie_word_embeddings else 2)
    weights = (params - emb) * bpp / tp + emb * 2 / (1 if tp == 1 else 1)  # embedding replicated, head sharded
    kv_tok = cfg.kv_bytes_per_token(kv_bits) / min(tp, cfg.num_key_value_heads)
    blocks = (ctx + block_size - 1) // block_size * parallel
    kv = blocks * block_size * kv_tok
    act = max_batch_tokens * (cfg.hidden_size * 6 + (cfg.q_size + 2 * cfg.kv_size) // tp +
                              3 * max(cfg.intermediate_size, cfg.moe_intermediate_size) // tp) * 2
    logits = parallel * cfg.vocab_size * 2
    total = weights + kv + act + logits + (64 << 20)
    return dict(model_type=cfg.model_type, parameters=params, bytes_per_param=round(bpp, 4),
                weights_bytes=int(weights), kv_bytes_per_token=int(kv_tok), kv_pool_blocks=blocks,
                kv_pool_bytes=int(kv), activation_bytes=int(act), logits_bytes=int(logits),
                total_bytes=int(total), total_gib=round(total / 2 ** 30, 3), fits_b200=total < 170 * 2 ** 30)
