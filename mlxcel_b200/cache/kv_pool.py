"""Paged KV pool: one slab per layer, ``[num_blocks, Hkv, block_size, D]``.

A block id addresses the same slot in every layer, so a sequence has one block table for the
whole model. ``kv_bits=8`` stores uint8 values plus a bf16 (scale, bias) pair per 64 elements
(``--kv-bits 8 --kv-group-size 64`` of the reference, src/cli/batch_quant_args.rs:33-80), written
by the fused RoPE+append kernel and dequantized inside the attention kernels. ``kv_bits=4`` is the
same affine scheme with 16 levels, two codes per byte (``[..., D / 2]`` bytes per row); the
reference rejects uniform 4-bit KV (its 4-bit mode is TurboQuant), so this mode has no counterpart.

Multi-head latent attention with ``cfg.extra["mla_latent"]`` keeps ONE entry per token and layer,
``[normalised latent (kv_lora_rank) | rotary key (qk_rope_head_dim)]`` (576 values for DeepSeek-V3
instead of 2 * heads * head_dim), in the K slab with a single head; the V slab is empty
(the reference's MLA cache, src/lib/mlxcel-core/src/mla/cache.rs:253).
"""
from __future__ import annotations

import torch

from ..config import ModelConfig
from ..ops import KVLayer


class KVPool:
    def __init__(self, cfg: ModelConfig, num_blocks: int, block_size: int = 16, *, kv_bits: int = 16,
                 device="cpu", dtype=torch.bfloat16, tp_size: int = 1, num_layers: int | None = None):
        if kv_bits not in (16, 8, 4):
            raise ValueError("kv_bits must be 16, 8 or 4")
        self.cfg, self.num_blocks, self.block_size, self.kv_bits = cfg, num_blocks, block_size, kv_bits
        self.Hkv = max(1, cfg.num_key_value_heads // tp_size)
        self.D = cfg.head_dim
        L = cfg.num_hidden_layers if num_layers is None else num_layers
        shape = (num_blocks, self.Hkv, block_size, self.D)
        self.layers: list[KVLayer] = []
        self.latent = bool(cfg.extra.get("mla_latent"))
        if self.latent:
            if kv_bits != 16:
                raise ValueError("the latent MLA cache stores 16-bit entries (kv_bits must be 16)")
            self.Hkv, self.D = 1, self.latent_width(cfg)
        for _ in range(L):
            if self.latent:
                k = torch.zeros((num_blocks, 1, block_size, self.D), dtype=dtype, device=device)
                v = torch.zeros((num_blocks, 1, block_size, 0), dtype=dtype, device=device)
                km = vm = None
            elif kv_bits == 16:
                k = torch.zeros(shape, dtype=dtype, device=device)
                v = torch.zeros(shape, dtype=dtype, device=device)
                km = vm = None
            else:
                if self.D % 64:
                    raise ValueError("quantized KV needs head_dim % 64 == 0")
                qshape = shape if kv_bits == 8 else (num_blocks, self.Hkv, block_size, self.D // 2)
                k = torch.zeros(qshape, dtype=torch.uint8, device=device)
                v = torch.zeros(qshape, dtype=torch.uint8, device=device)
                mshape = (num_blocks, self.Hkv, block_size, self.D // 64, 2)
                km = torch.zeros(mshape, dtype=torch.bfloat16, device=device)
                vm = torch.zeros(mshape, dtype=torch.bfloat16, device=device)
            self.layers.append(KVLayer(k, v, km, vm, block_size, kv_bits))

    @staticmethod
    def latent_width(cfg: ModelConfig) -> int:
        m = cfg.extra["mla"]
        return int(m["kv_lora_rank"]) + int(m["rope"])

    @staticmethod
    def bytes_per_block(cfg: ModelConfig, block_size: int, kv_bits: int = 16, tp_size: int = 1,
                        num_layers: int | None = None) -> int:
        Hkv = max(1, cfg.num_key_value_heads // tp_size)
        L = cfg.num_hidden_layers if num_layers is None else num_layers
        if cfg.extra.get("mla_latent"):
            return KVPool.latent_width(cfg) * 2 * block_size * L
        per_tok = Hkv * cfg.head_dim * kv_bits // 8
        if kv_bits != 16:
            per_tok += Hkv * (cfg.head_dim // 64) * 4
        return 2 * per_tok * block_size * L

    def copy_blocks(self, pairs: list[tuple[int, int]]) -> None:
        """Copy-on-write support: duplicate block contents ``src -> dst`` in every layer."""
        if not pairs:
            return
        src = torch.tensor([p[0] for p in pairs], device=self.layers[0].k.device)
        dst = torch.tensor([p[1] for p in pairs], device=self.layers[0].k.device)
        for l in self.layers:
            for t in (l.k, l.v, l.k_meta, l.v_meta):
                if t is not None:
                    t[dst] = t[src]

    def extract_blocks(self, block_ids: list[int]) -> list[dict]:
        """Host copies of blocks (KV handoff / snapshot)."""
        idx = torch.tensor(block_ids, device=self.layers[0].k.device)
        out = []
        for l in self.layers:
            out.append({n: getattr(l, n)[idx].cpu() for n in ("k", "v", "k_meta", "v_meta")
                        if getattr(l, n) is not None})
        return out

    def restore_blocks(self, block_ids: list[int], data: list[dict]) -> None:
        idx = torch.tensor(block_ids, device=self.layers[0].k.device)
        for l, d in zip(self.layers, data):
            for n, t in d.items():
                getattr(l, n)[idx] = t.to(getattr(l, n).device)
