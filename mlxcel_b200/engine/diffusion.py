"""Block-unmasking generation for masked-diffusion language models (LLaDA-style).

The sequence is a canvas: the prompt followed by generation blocks of ``block_length`` mask tokens.
Attention is *block-causal*: a token sees every earlier block and all of its own block. The prompt
is committed to the paged KV cache block by block; each generation block is then denoised by
forwarding the block against the frozen prefix, choosing a token for every still-masked position
and revealing the positions whose chosen-token probability clears a threshold that decays linearly
over the block's steps (at least one position per step, so every block finishes); a finished block
is committed to the cache and its tokens are streamed. Generation stops at an end-of-sequence token
(reference: src/models/llada2_moe/generate.rs, src/models/diffusion_gemma/generate.rs — block
length 32, 32 steps, threshold 0.95 by default).

How a block runs on the paged kernels: the B rows of a block are submitted as B *decode rows* that
share one block table and one context length (prefix + B). The fused RoPE + append kernel writes all
B keys / values first, and the decode attention kernel gives every row the whole context, which is
exactly the bidirectional-inside-the-block, causal-across-blocks mask. Re-forwarding a block
overwrites its own B cache slots, so nothing is rolled back between denoising steps.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..cache.kv_pool import KVPool
from ..models.decoder import StepBatch


@dataclass
class DiffusionOptions:
    max_new_tokens: int = 256
    block_length: int = 32
    steps: int = 32                 # denoising steps per block (at most block_length are ever needed)
    threshold: float = 0.95         # confidence needed at a block's first step
    min_threshold: float = 0.95     # ... and at its last step (linear in between)
    temperature: float = 0.0        # <= 0: argmax
    eos_token_ids: list = field(default_factory=list)
    seed: int = 0


def block_threshold(step: int, steps: int, hi: float, lo: float) -> float:
    """Confidence threshold of denoising step ``step`` (0-based) of ``steps``: linear from hi to lo."""
    if steps <= 1:
        return lo
    return hi + (lo - hi) * (step / (steps - 1))


def transfer_mask(conf: torch.Tensor, masked: torch.Tensor, threshold: float) -> torch.Tensor:
    """Which masked positions are revealed this step: every one whose confidence reaches the
    threshold, and always the most confident one (progress is guaranteed)."""
    take = masked & (conf >= threshold)
    if masked.any() and not take.any():
        c = torch.where(masked, conf, torch.full_like(conf, float("-inf")))
        take = torch.zeros_like(masked)
        take[int(c.argmax())] = True
    return take


def truncate_at_eos(tokens: list[int], eos: set[int]) -> tuple[list[int], bool]:
    for i, t in enumerate(tokens):
        if t in eos:
            return tokens[:i], True
    return tokens, False


class DiffusionGenerator:
    """One sequence at a time over a `DecoderModel` (any decoder checkpoint trained as a masked-diffusion
    model; ``mask_token_id`` names its mask token)."""

    def __init__(self, model, cfg, mask_token_id: int, max_len: int = 4096, block_size: int = 16):
        self.model, self.cfg, self.mask_id = model, cfg, int(mask_token_id)
        self.device = model.device
        self.bs = block_size
        self.nblocks = (max_len + block_size - 1) // block_size + 1
        self.pool = KVPool(cfg, self.nblocks, block_size, device=self.device, dtype=model.w.final_norm.dtype,
                           num_layers=len(model.w.layers), tp_size=model.comm.tp_size)
        self.max_len = max_len
        self.stats = dict(forwards=0, blocks=0, revealed=0)

    def _forward_block(self, tokens: list[int], start: int) -> torch.Tensor:
        """Logits [B, V] of ``tokens`` placed at positions start .. start+B with block-causal attention."""
        B, dev = len(tokens), self.device
        pos = torch.arange(start, start + B, dtype=torch.int32, device=dev)
        table = torch.arange(self.nblocks, dtype=torch.int32, device=dev)[None].expand(B, -1).contiguous()
        b = StepBatch(token_ids=torch.tensor(tokens, dtype=torch.int32, device=dev), positions=pos, slot_mapping=pos.clone(),
                      num_decode=B, dec_block_tables=table,
                      dec_context_lens=torch.full((B,), start + B, dtype=torch.int32, device=dev), dec_max_len=start + B,
                      logits_rows=torch.arange(B, device=dev))
        b.seq_ids, b.pf_starts = [0] * B, []
        self.stats["forwards"] += 1
        return self.model.forward(b, self.pool.layers).float()

    @torch.no_grad()
    def generate(self, prompt: list[int], opts: DiffusionOptions | None = None, on_block=None) -> list[int]:
        o = opts or DiffusionOptions()
        L = o.block_length
        if len(prompt) + o.max_new_tokens + L > self.max_len:
            raise ValueError("prompt + max_new_tokens exceeds the generator's max_len")
        eos = set(o.eos_token_ids)
        gen = torch.Generator(device="cpu").manual_seed(o.seed)
        # commit the prompt block by block (a last partial block joins the first generation block)
        done = 0
        while len(prompt) - done >= L:
            self._forward_block(prompt[done:done + L], done)
            done += L
        tail = prompt[done:]
        out: list[int] = []
        while len(out) < o.max_new_tokens:
            n_new = min(L - len(tail), o.max_new_tokens - len(out))
            canvas = list(tail) + [self.mask_id] * n_new
            masked = torch.tensor([False] * len(tail) + [True] * n_new)
            steps = max(1, min(o.steps, n_new))
            step = 0
            while masked.any():
                logits = self._forward_block(canvas, done).cpu()
                if o.temperature > 0:
                    probs = torch.softmax(logits / o.temperature, dim=-1)
                    choice = torch.multinomial(probs, 1, generator=gen)[:, 0]
                    conf = torch.softmax(logits, dim=-1).gather(1, choice[:, None])[:, 0]
                else:
                    probs = torch.softmax(logits, dim=-1)
                    conf, choice = probs.max(dim=-1)
                thr = block_threshold(min(step, steps - 1), steps, o.threshold, o.min_threshold)
                take = transfer_mask(conf, masked, thr)
                for i in take.nonzero().flatten().tolist():
                    canvas[i] = int(choice[i])
                masked &= ~take
                self.stats["revealed"] += int(take.sum())
                step += 1
            self._forward_block(canvas, done)            # commit the finished block's keys / values
            new = canvas[len(tail):]
            new, hit = truncate_at_eos(new, eos)
            out += new
            self.stats["blocks"] += 1
            if on_block is not None:
                on_block(new)
            if hit:
                break
            done += len(canvas)
            tail = []
        return out[: o.max_new_tokens]
