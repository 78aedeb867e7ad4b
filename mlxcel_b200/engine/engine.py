"""Engine: continuous batching over the paged KV pool.

The engine owns the model executor, the KV pool and the C++ block manager and is the only
path to a model forward (the role of ``Engine<M>`` in the reference,
src/lib/mlxcel-core/src/engine/mod.rs:148-540). One :meth:`Engine.step` forms a batch (all
decoding rows + prefill chunks under a token budget, admission under the block watermark,
preemption by recompute under block pressure), runs one forward pass, samples, and applies the
shared finish step (EOS / stop ids / max tokens / loop detection,
src/lib/mlxcel-core/src/decode_finish.rs).

Pure decode steps replay CUDA graphs captured per padded batch size; every buffer a captured
kernel reads is a persistent device tensor that the host refreshes from pinned memory.
"""
from __future__ import annotations

import os
import time
from collections import deque
from dataclasses import dataclass, field
from typing import Callable

import numpy as np
import torch

from .. import ops
from ..cache.kv_pool import KVPool
from ..config import ModelConfig
from ..host_runtime import BlockManager, TickAction, TickState, decide_tick, prefill_piece
from ..models.decoder import DecoderModel, StepBatch
from .params import FinishReason, SamplingParams, SeqStatus
from .sampler import Sampler


@dataclass
class Sequence:
    seq_id: int
    prompt: list[int]
    params: SamplingParams
    output: list[int] = field(default_factory=list)
    logprobs: list[float] = field(default_factory=list)
    num_computed: int = 0          # tokens whose KV is in the pool
    num_cached: int = 0            # prompt tokens adopted from the prefix cache
    status: SeqStatus = SeqStatus.QUEUED
    finish_reason: FinishReason | None = None
    arrival: float = 0.0
    first_token_time: float | None = None
    finish_time: float | None = None
    preemptions: int = 0
    on_token: Callable | None = None
    mask_fn: Callable | None = None   # structured output: fn(seq) -> bool mask [V] or None
    user_data: object = None
    think_open: bool = False          # inside a reasoning block (thinking budget bookkeeping)
    think_count: int = 0              # tokens generated inside the current block
    think_forced: int = 0             # end-of-thinking tokens this engine forced
    draft_n: int = 0                  # speculative decoding: drafted / accepted tokens of this request
    draft_n_accepted: int = 0
    mm_embeds: list | None = None     # [(start, rows)] media rows replacing placeholder embeddings
    prompt_keys: list | None = None   # prompt ids with media placeholders salted (prefix-cache keys)
    rope_pos: object = None           # int32 [3, len(prompt)]: (t, h, w) rotary positions of the prompt
    rope_delta: int = 0               # rotary position minus token index for tokens after the prompt

    @property
    def tokens(self) -> list[int]:
        return self.prompt + self.output

    def key_tokens(self) -> list[int]:
        return self.tokens if self.prompt_keys is None else self.prompt_keys + self.output

    @property
    def total_len(self) -> int:
        return len(self.prompt) + len(self.output)


@dataclass
class EngineConfig:
    max_batch: int = 64                  # concurrent decoding rows (--parallel)
    max_num_batched_tokens: int = 8192   # token budget of one forward pass
    prefill_chunk_alone: int = 2048      # DEFAULT_PREFILL_CHUNK (prefill_plan.rs:65)
    prefill_chunk_contended: int = 512   # CONTENDED_PREFILL_CHUNK (prefill_plan.rs:72)
    max_prefill_seqs: int = 8            # prefill cohort size per step
    block_size: int = 16
    num_blocks: int = 0                  # 0 = size from free memory
    kv_bits: int = 16
    gpu_memory_utilization: float = 0.90
    watermark: float = 0.01
    prefix_cache: bool = True
    max_queue_depth: int = 4096
    max_model_len: int = 8192
    # KV window bound of one sequence (0 = max_model_len). Without context_shift a sequence ends with
    # finish reason "length" when prompt + generated + 1 reaches it; with context_shift the oldest
    # blocks behind the first n_keep tokens are dropped instead and generation goes on (the keys that
    # stay keep their rotary positions; reference --max-kv-size / --context-shift / --keep,
    # src/server/batch/finish.rs:37-65, cache.rs trim_front_keep_sink)
    max_kv_size: int = 0
    mla_latent_cache: bool = False       # MLA models: one [latent | rotary key] entry per token instead of per-head K / V
    context_shift: bool = False
    n_keep: int = 0
    cuda_graphs: bool = True
    prefill_grant_interval: int = 16
    mixed_steps: bool = True
    preemption: bool = True
    lookahead: bool = True               # submit decode step n+1 before reading step n (greedy rows)
    window_release: bool = True          # sliding-window layers get their own block pool and give back
    #                                      the blocks that fell out of the window (RotatingKVCache role)
    status_check_interval: int = 64      # steps between reads of the device status word (0 = never)


class Engine:
    def __init__(self, model: DecoderModel, cfg: ModelConfig, ecfg: EngineConfig | None = None):
        self.model, self.cfg = model, cfg
        self.ecfg = ecfg or EngineConfig()
        e = self.ecfg
        self.device = model.device
        self.is_cuda = self.device.type == "cuda"
        tp = model.comm.tp_size
        nl = getattr(model, "num_kv_layers", len(model.w.layers))
        self.recurrent = bool(getattr(model, "recurrent", False))
        if self.recurrent:
            # per-sequence recurrent state lives in the model, not in the block pool: a cached prefix has
            # no state to resume from, and the state slot indices change from step to step
            e.prefix_cache = e.cuda_graphs = e.lookahead = False
        self.pipeline = getattr(model, "ctx", None) is not None
        # token-sharded expert parallelism (parallel/dp_ep.py): ticks are taken in lockstep with the
        # other ranks; the lookahead pipeline (two forwards in flight) does not fit that
        self.dp_lockstep = getattr(getattr(model, "comm", None), "a2a", None) is not None
        self.dp_active = True
        if self.dp_lockstep:
            e.lookahead = False
        if self.pipeline:
            # stages exchange activations with send / recv inside the forward pass: no graph capture,
            # and the token ids come back from the last stage, so nothing can be fed back on the device
            e.cuda_graphs = e.lookahead = False
        if e.mla_latent_cache:
            if not cfg.extra.get("mla"):
                raise ValueError("mla_latent_cache is for multi-head latent attention models (DeepSeek-V2 / V3 layout)")
            # the absorbed attention is composed of batched matrix products with data-dependent shapes
            cfg.extra["mla_latent"] = True
            e.cuda_graphs = e.lookahead = False
        if e.num_blocks <= 0:
            e.num_blocks = self._auto_num_blocks(tp, nl)
        # fp32 models (CPU oracles) keep fp32 keys / values; everything else stores bf16 (or 8-bit)
        wdt = getattr(getattr(model.w, "final_norm", None), "dtype", torch.bfloat16)
        kv_dtype = torch.float32 if wdt == torch.float32 else torch.bfloat16
        # Sliding-window layers (gpt-oss alternates 128-token windows with full layers, Mistral / Gemma
        # have them too) never attend beyond their window: they get a pool of their own whose blocks
        # are returned once every token in them is out of reach, instead of holding the whole
        # context (the reference's RotatingKVCache, src/lib/mlxcel-core/src/cache.rs:4397). The
        # window pool has no prefix index (a released block cannot be shared), so prefix caching
        # is off for such models — the reference does the same for its model-owned mixed caches.
        self.win_layers = self._window_layers() if e.window_release else None
        self.bm_win = self.pool_win = None
        self.window = 0
        if self.win_layers is not None:
            e.prefix_cache = False
            self.window = max(self.win_layers)
            n_win = sum(1 for w in self.win_layers if w > 0)
            per_pf = (self.window + max(e.prefill_chunk_alone, e.prefill_chunk_contended) + e.block_size - 1) // e.block_size + 2
            per_dec = (self.window + self.spec_k_max + e.block_size - 1) // e.block_size + 3
            self.win_blocks_prefill = per_pf
            nb_win = min(e.num_blocks, e.max_prefill_seqs * per_pf + e.max_batch * per_dec + 8)
            self.pool_win = KVPool(cfg, nb_win, e.block_size, kv_bits=e.kv_bits, device=self.device, dtype=kv_dtype,
                                   tp_size=tp, num_layers=n_win)
            self.bm_win = BlockManager(nb_win, e.block_size, False, 0.0)
            nl = nl - n_win
        self.pool = KVPool(cfg, e.num_blocks, e.block_size, kv_bits=e.kv_bits, device=self.device,
                           dtype=kv_dtype, tp_size=tp, num_layers=nl)
        self.bm = BlockManager(e.num_blocks, e.block_size, e.prefix_cache, e.watermark)
        if self.win_layers is None:
            self.kv_layers = self.pool.layers
        else:
            full, win = iter(self.pool.layers), iter(self.pool_win.layers)
            self.kv_layers = [next(win) if w > 0 else next(full) for w in self.win_layers]
        self.sampler = Sampler(cfg.vocab_size, self.device)
        self.max_blocks_per_seq = (e.max_model_len + e.block_size - 1) // e.block_size
        self._ctx_shift = bool(e.context_shift) and not self.recurrent
        if self._ctx_shift:
            if self.bm_win is not None:
                raise ValueError("context shift is not available for models with a sliding-window KV pool "
                                 "(their window layers already drop old blocks)")
            if getattr(self, "pipeline", None):
                raise ValueError("context shift is not available under pipeline parallelism")
            cap = e.max_model_len - e.block_size
            e.max_kv_size = min(e.max_kv_size, cap) if e.max_kv_size > 0 else cap
            if e.max_kv_size < 4 * e.block_size + e.n_keep:
                raise ValueError("max_kv_size is too small for context shifting (needs n_keep + 4 blocks)")
            e.lookahead = False          # a step in flight holds the table it was launched with
        self.waiting: deque[Sequence] = deque()
        self.running: list[Sequence] = []      # PREFILLING or DECODING, in admission order
        self.seqs: dict[int, Sequence] = {}
        self._next_id = 0
        self._decode_ticks_since_grant = 0
        self._graphs: dict[tuple, tuple] = {}
        self.drafter = None          # speculative drafter (see mlxcel_b200.speculative)
        self.d_drafts = self.h_drafts = None
        self.spec_k = 4              # block size K: K-1 draft tokens + 1 bonus token per round
        self._last_spec = self._spec_now = False
        self.spec_policy = None      # optional speculative.policy.SpecPolicy (adaptive on / off)
        self._evicted: list[Sequence] = []   # rows the scheduler had to end (pool exhausted), reported by step()
        self._alloc_buffers()
        # MLXCEL_B200_STEP_TIMING=1: CUDA events around every non-pipelined step; the sums land in stats
        # as {decode,mixed}_{gpu_ms,wall_ms,timed_steps} (the gap between the two is host time)
        self._step_timing = self.is_cuda and os.environ.get("MLXCEL_B200_STEP_TIMING", "0") == "1"
        self.stats = dict(steps=0, decode_steps=0, prefill_tokens=0, decode_tokens=0, preemptions=0,
                          graph_replays=0, prefix_hit_tokens=0, h2d_bytes=0, d2h_bytes=0,
                          graph_kernel_launches=0, spec_rounds=0, spec_drafted=0, spec_accepted=0)

    # ------------------------------------------------------------------ setup
    spec_k_max = 16          # most tokens a verify round may append beyond the current one

    def _window_layers(self) -> list[int] | None:
        """Window size per layer of this executor (0 = full attention), or None when no layer has one
        or the executor does not take per-pool tables."""
        m = self.model
        if self.recurrent or not hasattr(m, "layer_range") or not hasattr(m, "_attend") or self.pipeline:
            return None
        ws = [int(self.cfg.layer_window(i)) for i in m.layer_range]
        return ws if any(w > 0 for w in ws) else None

    # The window pool mirrors the main block manager: same sequences, same token counts.
    def _kv_create(self, seq_id: int) -> None:
        self.bm.create(seq_id, 0)
        if self.bm_win is not None:
            self.bm_win.create(seq_id, 0)

    def _kv_free(self, seq_id: int) -> None:
        self.bm.free_seq(seq_id)
        if self.bm_win is not None:
            self.bm_win.free_seq(seq_id)

    def _kv_reserve(self, seq_id: int, total: int) -> bool:
        if not self.bm.reserve(seq_id, total):
            return False
        return self.bm_win is None or self.bm_win.reserve(seq_id, total)

    def _kv_truncate(self, seq_id: int, n: int) -> None:
        self.bm.truncate(seq_id, n)
        if self.bm_win is not None:
            self.bm_win.truncate(seq_id, n)

    def _release_window(self, seqs) -> None:
        """After a step: blocks of the window pool whose tokens no later query can reach go back; with
        context shifting, sequences that reached the KV bound drop their oldest blocks behind n_keep."""
        if self._ctx_shift:
            e = self.ecfg
            for s in seqs:
                if s.status == SeqStatus.DECODING and self.bm.has_seq(s.seq_id) \
                        and s.total_len - self.bm.shifted(s.seq_id) + 1 >= e.max_kv_size:
                    # one block of headroom more than needed, so that this happens once per block
                    cut = self.bm.shift_front(s.seq_id, e.n_keep, e.max_kv_size - 2 * e.block_size)
                    if cut:
                        self.stats["context_shifts"] = self.stats.get("context_shifts", 0) + 1
                        self.stats["context_shift_tokens"] = self.stats.get("context_shift_tokens", 0) + cut
        if self.bm_win is None:
            return
        for s in seqs:
            if s.status != SeqStatus.FINISHED and self.bm_win.has_seq(s.seq_id):
                self.bm_win.release_front(s.seq_id, s.num_computed - self.window)

    def _auto_num_blocks(self, tp: int, nl: int) -> int:
        e = self.ecfg
        per_block = KVPool.bytes_per_block(self.cfg, e.block_size, e.kv_bits, tp, nl)
        if self.is_cuda:
            free, total = torch.cuda.mem_get_info(self.device)
            budget = free - (1.0 - e.gpu_memory_utilization) * total - (6 << 30)
            n = int(max(budget, 1 << 30) // per_block)
        else:
            n = 2048
        need = (e.max_model_len // e.block_size + 2) * e.max_batch * 2
        n = max(64, min(n, need))
        if tp > 1 or getattr(self.model, "ctx", None) is not None:
            # every rank sizes the pool from its own free memory; schedulers in lockstep need one size
            from ..parallel.control import agree_min
            n = agree_min(n)
        return n

    def _alloc_buffers(self) -> None:
        e = self.ecfg
        T, B, MB = e.max_num_batched_tokens, e.max_batch, self.max_blocks_per_seq
        S = e.max_prefill_seqs
        pin = self.is_cuda

        def host(shape, dtype):
            t = torch.zeros(shape, dtype=dtype)
            return t.pin_memory() if pin else t

        def dev(shape, dtype):
            return torch.zeros(shape, dtype=dtype, device=self.device)

        self.h_tokens, self.d_tokens = host(T, torch.int32), dev(T, torch.int32)
        self.h_pos, self.d_pos = host(T, torch.int32), dev(T, torch.int32)
        self.h_slots, self.d_slots = host(T, torch.int32), dev(T, torch.int32)
        if self.bm_win is not None:      # the window pool's slots and tables travel beside the main ones
            self.h_slots_w, self.d_slots_w = host(T, torch.int32), dev(T, torch.int32)
            self.h_dec_tables_w, self.d_dec_tables_w = host((B, MB), torch.int32), dev((B, MB), torch.int32)
            self.h_pf_tables_w, self.d_pf_tables_w = host((S, MB), torch.int32), dev((S, MB), torch.int32)
            self.np_slots_w = self.h_slots_w.numpy()
            self.np_dec_tables_w, self.np_pf_tables_w = self.h_dec_tables_w.numpy(), self.h_pf_tables_w.numpy()
        self.h_dec_tables, self.d_dec_tables = host((B, MB), torch.int32), dev((B, MB), torch.int32)
        self.h_dec_lens, self.d_dec_lens = host(B, torch.int32), dev(B, torch.int32)
        self.h_pf_tables, self.d_pf_tables = host((S, MB), torch.int32), dev((S, MB), torch.int32)
        self.h_pf_lens, self.d_pf_lens = host(S, torch.int32), dev(S, torch.int32)
        self.h_cu, self.d_cu = host(S + 1, torch.int32), dev(S + 1, torch.int32)
        self.h_rows, self.d_rows = host(B * 9 + S, torch.int64), dev(B * 9 + S, torch.int64)
        self.h_out, self.d_out = host(B + S, torch.int32), dev(B + S, torch.int32)
        # second staging set + token read-back buffers for the lookahead pipeline
        self.la_host = [dict(pos=host(B, torch.int32), slots=host(B, torch.int32), lens=host(B, torch.int32),
                             tables=host((B, MB), torch.int32), out=host(B, torch.int32),
                             slots_w=host(B, torch.int32), tables_w=host((B, MB), torch.int32)) for _ in range(2)]
        self._inflight = None
        self._la_parity = 0
        self.np_dec_tables = self.h_dec_tables.numpy()
        self.np_pf_tables = self.h_pf_tables.numpy()
        self.np_slots = self.h_slots.numpy()

    # ------------------------------------------------------------------ request API
    def add_request(self, prompt: list[int], params: SamplingParams | None = None,
                    on_token: Callable | None = None, mask_fn: Callable | None = None,
                    user_data=None, mm_embeds: list | None = None, key_tokens: list[int] | None = None,
                    rope_pos=None, rope_delta: int = 0) -> int:
        """``mm_embeds``: ``[(start, rows[n, hidden])]`` — rows that replace the token embeddings of
        prompt positions ``start .. start+n`` (image / audio placeholders). ``key_tokens``: what the
        prefix cache hashes instead of the prompt ids (placeholders salted by media content).
        ``rope_pos`` ([3, len(prompt)] ints) / ``rope_delta``: multimodal rotary positions (temporal,
        height, width) of the prompt tokens and the offset ``rotary position - token index`` of every
        later token (Qwen2-VL family; text-only prompts need neither)."""
        if not prompt:
            raise ValueError("empty prompt")
        if mm_embeds and (self.recurrent or self.pipeline):
            raise ValueError("media inputs need the attention executor on one pipeline stage")
        if key_tokens is not None and len(key_tokens) != len(prompt):
            raise ValueError("key_tokens must have one entry per prompt token")
        params = params or SamplingParams()
        if len(prompt) + 1 > self.ecfg.max_model_len:
            raise ValueError(f"prompt of {len(prompt)} tokens exceeds max_model_len {self.ecfg.max_model_len}")
        if len(self.waiting) >= self.ecfg.max_queue_depth:
            raise RuntimeError("queue full")
        # a prompt that cannot fit the KV pool even when it runs alone would park forever
        bs = self.ecfg.block_size
        usable = self.ecfg.num_blocks - int(self.ecfg.num_blocks * self.ecfg.watermark) - 1
        if (len(prompt) + 1 + bs - 1) // bs > usable:
            raise ValueError(f"prompt of {len(prompt)} tokens needs {(len(prompt) + bs) // bs} KV blocks; "
                             f"the pool has {usable} usable blocks of {bs} tokens")
        sid = self._next_id
        self._next_id += 1
        s = Sequence(sid, list(prompt), params, arrival=time.perf_counter(), on_token=on_token,
                     mask_fn=mask_fn, user_data=user_data)
        if mm_embeds:
            s.mm_embeds = [(int(st), rows.to(self.device)) for st, rows in mm_embeds]
            s.prompt_keys = list(key_tokens) if key_tokens is not None else None
        if rope_pos is not None:
            s.rope_pos = np.asarray(rope_pos, dtype=np.int32).reshape(3, len(prompt))
            s.rope_delta = int(rope_delta)
        if params.thinking_cap is not None and params.think_start_id is not None:
            # a generation prompt may already have opened the reasoning block
            for t in reversed(prompt):
                if t == params.think_end_id:
                    break
                if t == params.think_start_id:
                    s.think_open = True
                    break
        self.seqs[sid] = s
        if params.priority > 0:
            # priority lanes: insert before the first lower-priority request
            idx = next((i for i, w in enumerate(self.waiting) if w.params.priority < params.priority),
                       len(self.waiting))
            self.waiting.insert(idx, s)
        else:
            self.waiting.append(s)
        return sid

    def abort(self, seq_id: int) -> None:
        s = self.seqs.get(seq_id)
        if s is None or s.status == SeqStatus.FINISHED:
            return
        self._finish(s, FinishReason.CANCELLED)
        if s in self.waiting:
            self.waiting.remove(s)

    def has_work(self) -> bool:
        return bool(self.waiting or self.running or self._inflight is not None)

    def release(self, seq_id: int) -> Sequence | None:
        """Forget a finished sequence (its blocks were already returned to the pool)."""
        return self.seqs.pop(seq_id, None)

    # ------------------------------------------------------------------ scheduling
    def _finish(self, s: Sequence, reason: FinishReason) -> None:
        if s.status == SeqStatus.FINISHED:
            return
        s.status, s.finish_reason, s.finish_time = SeqStatus.FINISHED, reason, time.perf_counter()
        if self.bm.has_seq(s.seq_id):
            # donate computed full blocks to the prefix cache, then drop our references
            toks = np.asarray(s.key_tokens()[: s.num_computed], dtype=np.int32)
            self.bm.commit(s.seq_id, toks, s.num_computed)
            self._kv_free(s.seq_id)
        if s in self.running:
            self.running.remove(s)
        if self.recurrent:
            self.model.release_seq(s.seq_id)
        if self.spec_policy is not None and reason != FinishReason.CANCELLED:
            self.spec_policy.on_request_finished()

    def _preempt_one(self) -> bool:
        """Reclaim blocks by recompute-preempting the least progressed running row
        (reclaim order of the reference: cached prefixes are evicted first by the block manager
        itself, docs/CONTINUOUS_BATCHING.md:358-363)."""
        cands = [s for s in self.running]
        if len(cands) <= 1:
            return False
        if self._ctx_shift:
            # a sequence whose context was shifted cannot be recomputed from its tokens (part of its
            # history is gone from the cache on purpose): it is never the victim
            cands = [s for s in cands if not (self.bm.has_seq(s.seq_id) and self.bm.shifted(s.seq_id))]
            if not cands:
                return False
        victim = min(cands, key=lambda s: (len(s.output), -s.seq_id))
        self.running.remove(victim)
        self._kv_free(victim.seq_id)
        if self.recurrent:
            self.model.release_seq(victim.seq_id)
        victim.num_computed = 0
        victim.status = SeqStatus.PREEMPTED
        victim.preemptions += 1
        self.stats["preemptions"] += 1
        self.waiting.appendleft(victim)
        return True

    def _schedule(self):
        """Returns (decode_seqs, [(seq, start, count)] prefill pieces)."""
        e = self.ecfg
        decode = [s for s in self.running if s.status == SeqStatus.DECODING]
        # reserve the next slot of every decoding row; preempt under pressure
        i = 0
        while i < len(decode):
            s = decode[i]
            if self._kv_reserve(s.seq_id, s.total_len):
                i += 1
                continue
            if not (e.preemption and self._preempt_one()):
                # nothing left to reclaim: the row has reached what the pool can hold
                self._finish(s, FinishReason.LENGTH)
                self._evicted.append(s)
            decode = [s for s in self.running if s.status == SeqStatus.DECODING]
            i = 0
        parked = [s for s in self.running if s.status == SeqStatus.PREFILLING]
        st = TickState()
        st.active_rows = len(decode)
        st.max_batch = e.max_batch
        st.queued = len(self.waiting)
        st.parked_prefill = bool(parked)
        st.decode_ticks_since_prefill_grant = self._decode_ticks_since_grant
        st.prefill_grant_interval = e.prefill_grant_interval
        st.mixed_steps = e.mixed_steps
        # A verify round alternates with classic work (admission, a parked prefill): the tick policy
        # never grants two rounds in a row while classic work waits (tick_policy.rs:284-356).
        st.speculative_ready = (self.drafter is not None and bool(decode) and not self._ctx_shift
                                and all(self._spec_row_ok(s) for s in decode)
                                and (not self.pipeline or all(s.params.greedy for s in decode))
                                and (self.spec_policy is None or self.spec_policy.allow()))
        st.last_was_speculative = self._last_spec
        if self.waiting:
            nxt = self.waiting[0]
            st.blocks_available = self.bm.can_allocate(
                self.bm.blocks_needed(nxt.seq_id, nxt.total_len + 1) if self.bm.has_seq(nxt.seq_id)
                else (nxt.total_len + e.block_size) // e.block_size, True)
        d = decide_tick(st)
        self._last_spec = self._spec_now = d.action == TickAction.SpeculativeRound
        if self._spec_now:
            return decode, []
        pieces: list[tuple[Sequence, int, int]] = []
        run_decode = d.action in (TickAction.Decode, TickAction.MixedStep)
        run_prefill = d.action in (TickAction.Prefill, TickAction.MixedStep)
        if not run_decode:
            decode_rows = []
        else:
            decode_rows = decode
        if run_prefill:
            budget = e.max_num_batched_tokens - len(decode_rows)
            n_dec = len(decode_rows)
            # continue parked prefills first, then admit from the queue
            cands = list(parked)
            while (self.waiting and len(cands) < e.max_prefill_seqs and
                   len(self.running) + (len(cands) - len(parked)) < e.max_batch):
                s = self.waiting[0]
                need_blocks = (s.total_len + e.block_size) // e.block_size
                if not self.bm.can_allocate(need_blocks, True) and (self.running or cands):
                    break
                if (self.bm_win is not None and (self.running or cands)
                        and not self.bm_win.can_allocate(min(need_blocks, self.win_blocks_prefill), False)):
                    break
                self.waiting.popleft()
                if not self.bm.has_seq(s.seq_id):
                    self._kv_create(s.seq_id)
                    toks = np.asarray(s.key_tokens(), dtype=np.int32)
                    hit = self.bm.match_prefix(s.seq_id, toks)
                    s.num_computed = s.num_cached = hit
                    self.stats["prefix_hit_tokens"] += hit
                s.status = SeqStatus.PREFILLING
                cands.append(s)
            for s in cands:
                if budget <= 0:
                    break
                remaining = s.total_len - s.num_computed
                piece = prefill_piece(budget + n_dec, n_dec, max(e.prefill_chunk_alone, 1),
                                      max(e.prefill_chunk_contended, 1), remaining)
                piece = min(piece, budget)
                if piece <= 0:
                    break
                if not self._kv_reserve(s.seq_id, s.num_computed + piece):
                    if s not in self.running:
                        # could not get blocks after all: back to the queue
                        self._kv_free(s.seq_id)
                        s.status, s.num_computed = SeqStatus.QUEUED, 0
                        self.waiting.appendleft(s)
                    elif len(self.running) == 1 and not decode_rows:
                        # a lone parked prefill that cannot get its next blocks would park forever
                        self._finish(s, FinishReason.ERROR)
                        self._evicted.append(s)
                    break
                if s not in self.running:
                    self.running.append(s)
                pieces.append((s, s.num_computed, piece))
                budget -= piece
            # admitted but unscheduled candidates stay parked in `running`
            for s in cands:
                if s.status == SeqStatus.PREFILLING and s not in self.running and self.bm.has_seq(s.seq_id):
                    self.running.append(s)
            self._decode_ticks_since_grant = 0
        elif run_decode:
            self._decode_ticks_since_grant += 1
        return decode_rows, pieces

    # ------------------------------------------------------------------ batch building
    def _build_batch(self, decode: list[Sequence], pieces, drafts: dict | None = None,
                     all_rows: bool = False) -> tuple[StepBatch, int]:
        """``drafts`` maps seq_id → speculative tokens appended after the sequence's own tokens (verify
        rounds); ``all_rows`` asks for logits of every row of every piece."""
        nd = len(decode)
        t = 0
        tok, pos = self.h_tokens.numpy(), self.h_pos.numpy()
        for i, s in enumerate(decode):
            L = s.total_len
            tok[i] = s.output[-1] if s.output else s.prompt[-1]
            pos[i] = L - 1 + s.rope_delta
            self.bm.fill_slots(s.seq_id, L - 1, 1, self.np_slots, i)
            if self.bm_win is not None:
                self.bm_win.fill_slots(s.seq_id, L - 1, 1, self.np_slots_w, i)
            # (after a context shift the table holds fewer tokens than the sequence has seen)
            self.h_dec_lens[i] = L - (self.bm.shifted(s.seq_id) if self._ctx_shift else 0)
        max_len = int(self.h_dec_lens[:nd].max()) if nd else 0
        if nd:
            self.bm.fill_tables([s.seq_id for s in decode], self.np_dec_tables)
            if self.bm_win is not None:
                self.bm_win.fill_tables([s.seq_id for s in decode], self.np_dec_tables_w)
        t = nd
        cu = [0]
        max_q = 0
        pos3 = None                      # [3, T] rotary positions when a piece carries multimodal ones
        rows: list[int] = list(range(nd))
        for j, (s, start, count) in enumerate(pieces):
            toks = s.tokens + drafts[s.seq_id] if (drafts and s.seq_id in drafts) else s.tokens
            tok[t:t + count] = toks[start:start + count]
            pos[t:t + count] = np.arange(start, start + count, dtype=np.int32)
            if s.rope_pos is not None:
                if pos3 is None:
                    pos3 = np.zeros((3, self.h_pos.shape[0]), dtype=np.int32)
                    pos3[:, :t] = pos[None, :t]
                n_in = max(0, min(start + count, len(s.prompt)) - start)       # rows still inside the prompt
                pos3[:, t:t + n_in] = s.rope_pos[:, start:start + n_in]
                pos3[:, t + n_in:t + count] = pos[None, t + n_in:t + count] + s.rope_delta
                pos[t:t + count] = pos3[0, t:t + count]
            elif pos3 is not None:
                pos3[:, t:t + count] = pos[None, t:t + count]
            self.bm.fill_slots(s.seq_id, start, count, self.np_slots, t)
            if self.bm_win is not None:
                self.bm_win.fill_slots(s.seq_id, start, count, self.np_slots_w, t)
            self.h_pf_lens[j] = start + count
            t += count
            cu.append(t - nd)
            max_q = max(max_q, count)
            if all_rows:
                rows.extend(range(t - count, t))
            elif start + count >= s.total_len:
                rows.append(t - 1)
        if pieces:
            self.bm.fill_tables([p[0].seq_id for p in pieces], self.np_pf_tables)
            if self.bm_win is not None:
                self.bm_win.fill_tables([p[0].seq_id for p in pieces], self.np_pf_tables_w)
            self.h_cu[: len(cu)] = torch.tensor(cu, dtype=torch.int32)
        R = len(rows)
        self.h_rows[:R] = torch.tensor(rows, dtype=torch.int64)
        nb = self.is_cuda
        sp = len(pieces)
        self.d_tokens[:t].copy_(self.h_tokens[:t], non_blocking=nb)
        self.d_pos[:t].copy_(self.h_pos[:t], non_blocking=nb)
        self.d_slots[:t].copy_(self.h_slots[:t], non_blocking=nb)
        if nd:
            self.d_dec_tables[:nd].copy_(self.h_dec_tables[:nd], non_blocking=nb)
            self.d_dec_lens[:nd].copy_(self.h_dec_lens[:nd], non_blocking=nb)
        if sp:
            self.d_pf_tables[:sp].copy_(self.h_pf_tables[:sp], non_blocking=nb)
            self.d_pf_lens[:sp].copy_(self.h_pf_lens[:sp], non_blocking=nb)
            self.d_cu[: sp + 1].copy_(self.h_cu[: sp + 1], non_blocking=nb)
        self.d_rows[:R].copy_(self.h_rows[:R], non_blocking=nb)
        win = self.bm_win is not None
        if win:
            self.d_slots_w[:t].copy_(self.h_slots_w[:t], non_blocking=nb)
            if nd:
                self.d_dec_tables_w[:nd].copy_(self.h_dec_tables_w[:nd], non_blocking=nb)
            if sp:
                self.d_pf_tables_w[:sp].copy_(self.h_pf_tables_w[:sp], non_blocking=nb)
            self.stats["h2d_bytes"] += 4 * t + (nd + sp) * self.max_blocks_per_seq * 4
        mb4 = self.max_blocks_per_seq * 4 + 4
        self.stats["h2d_bytes"] += 12 * t + nd * mb4 + sp * mb4 + (sp + 1) * 4 + R * 8
        self.stats["d2h_bytes"] += R * 4
        b = StepBatch(token_ids=self.d_tokens[:t], positions=self.d_pos[:t],
                      slot_mapping=self.d_slots[:t], num_decode=nd,
                      dec_block_tables=self.d_dec_tables[:nd] if nd else None,
                      dec_context_lens=self.d_dec_lens[:nd] if nd else None, dec_max_len=max_len,
                      num_prefill_seqs=sp, pf_block_tables=self.d_pf_tables[:sp] if sp else None,
                      pf_cu_q=self.d_cu[: sp + 1] if sp else None,
                      pf_context_lens=self.d_pf_lens[:sp] if sp else None, pf_max_q_len=max_q,
                      pf_cu_q_host=cu if sp else None, logits_rows=self.d_rows[:R],
                      slot_mapping_win=self.d_slots_w[:t] if win else None,
                      dec_block_tables_win=self.d_dec_tables_w[:nd] if (win and nd) else None,
                      pf_block_tables_win=self.d_pf_tables_w[:sp] if (win and sp) else None)
        b.logits_rows_host = rows
        if any(p[0].mm_embeds for p in pieces):
            b.embeds = self._media_embeds(b, nd, pieces)
        if pos3 is not None:
            b.positions3 = torch.from_numpy(pos3[:, :t].copy()).to(self.device)
        b.seq_ids = [s.seq_id for s in decode] + [p[0].seq_id for p in pieces]
        b.pf_starts = [p[1] for p in pieces]
        return b, R

    def _media_embeds(self, b: StepBatch, nd: int, pieces) -> torch.Tensor:
        """Input embeddings of a step that covers media placeholders: the token embeddings with the
        rows of every placeholder position replaced by the connector's output."""
        m = self.model
        h = m.comm.embed(b.token_ids, m.w.embed, self.cfg.embed_scale).clone()
        H = h.shape[1]
        t = nd
        deep = None
        for s, start, count in pieces:
            for st, rows in s.mm_embeds or ():
                lo, hi = max(st, start), min(st + rows.shape[0], start + count)
                if lo < hi:
                    h[t + lo - start: t + hi - start] = rows[lo - st: hi - st, :H].to(h.dtype)
                    # rows wider than the hidden size carry features for the first layers' outputs (DeepStack)
                    extra = rows.shape[1] // H - 1
                    if extra > 0:
                        if deep is None:
                            deep = [torch.zeros_like(h) for _ in range(extra)]
                        for j in range(min(extra, len(deep))):
                            deep[j][t + lo - start: t + hi - start] = rows[lo - st: hi - st, (j + 1) * H:(j + 2) * H].to(h.dtype)
            t += count
        b.deepstack = deep
        return h

    # ------------------------------------------------------------------ cuda graphs
    def _decode_graph(self, nd: int, max_len: int) -> torch.Tensor | None:
        """Replay (capturing on first use) the decode graph for the padded batch size.
        Returns the logits tensor [Bpad, V] owned by the graph, or None when graphs are off."""
        e = self.ecfg
        if not (self.is_cuda and e.cuda_graphs):
            return None
        bp = 1
        while bp < nd:
            bp *= 2
        bp = min(bp, e.max_batch) if e.max_batch >= nd else nd
        if bp < nd:
            return None
        splits = ops.decode_splits(bp, self.model.Hkv, max(max_len, 1))
        key = (bp, splits)
        # padding rows: no KV append, zero context
        if bp > nd:
            self.d_tokens[nd:bp].zero_()
            self.d_pos[nd:bp].zero_()
            self.d_slots[nd:bp].fill_(-1)
            self.d_dec_lens[nd:bp].zero_()
            self.d_dec_tables[nd:bp].zero_()
            if self.bm_win is not None:
                self.d_slots_w[nd:bp].fill_(-1)
                self.d_dec_tables_w[nd:bp].zero_()
        ent = self._graphs.get(key)
        if ent is None:
            b = StepBatch(token_ids=self.d_tokens[:bp], positions=self.d_pos[:bp],
                          slot_mapping=self.d_slots[:bp], num_decode=bp,
                          dec_block_tables=self.d_dec_tables[:bp], dec_context_lens=self.d_dec_lens[:bp],
                          dec_max_len=max_len, logits_rows=None,
                          slot_mapping_win=self.d_slots_w[:bp] if self.bm_win is not None else None,
                          dec_block_tables_win=self.d_dec_tables_w[:bp] if self.bm_win is not None else None)
            fwd = lambda: self.model.forward(b, self.kv_layers)  # noqa: E731
            # warm-up outside capture (sets function attributes, fills descriptor caches). With
            # token-sharded experts this pass is this rank's alone, so it runs "dry": no exchange
            # with the other ranks (the capture below records kernels without running them, and the
            # replay is the tick's one real forward).
            a2a = getattr(self.model.comm, "a2a", None)
            s = torch.cuda.Stream(device=self.device)
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                if a2a is not None:
                    a2a.dry = True
                try:
                    fwd()
                finally:
                    if a2a is not None:
                        a2a.dry = False
            torch.cuda.current_stream().wait_stream(s)
            from ..ops import _lib
            n0 = _lib.launches()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                logits = fwd()
                # Greedy token feedback on the device: the step's argmax lands in the token buffer
                # the next replay reads, so a following step can be submitted before the host has
                # seen these tokens.
                ops.argmax(logits, out=self.d_tokens[:bp])
            ent = (g, logits, _lib.launches() - n0)
            self._graphs[key] = ent
        ent[0].replay()
        self.stats["graph_replays"] += 1
        self.stats["graph_kernel_launches"] += ent[2]
        return ent[1]

    # ------------------------------------------------------------------ lookahead pipeline
    # Decode step n+1 is submitted before step n's tokens are read (the reference's lookahead
    # pipeline, src/server/batch/scheduler/decode_tick.rs:386-485 and :686-794): the host prepares
    # positions / slots / page tables from what it already knows, the token ids come from the
    # device (the graph's argmax feeds the token buffer), and reading tokens lags one step.
    # Eligibility mirrors the reference: every row greedy without history penalties, masks,
    # logprobs or stop strings to watch mid-step, nothing queued, no prefill parked, no drafter.
    def _lookahead_eligible(self, decode, pieces) -> bool:
        e = self.ecfg
        if not (e.lookahead and self.is_cuda and e.cuda_graphs and decode and not pieces):
            return False
        if self.drafter is not None or self.waiting or len(decode) > e.max_batch:
            return False
        if any(s.status != SeqStatus.DECODING for s in self.running):
            return False
        for s in decode:
            p = s.params
            if not (p.greedy and not p.needs_history and not p.logit_bias and s.mask_fn is None
                    and not p.logprobs and p.thinking_cap is None):
                return False       # (a forced end-of-thinking token cannot be fed back on the device)
        return True

    def _can_pipeline(self, inf) -> bool:
        seqs = inf["seqs"]
        if not self._lookahead_eligible(seqs, []):
            return False
        if len(seqs) != len(self.running) or any(a is not b for a, b in zip(seqs, self.running)):
            return False
        for s in seqs:
            if s.status != SeqStatus.DECODING:
                return False
            # the token in flight must not be the one that ends the row by length
            if len(s.output) + 2 > s.params.max_tokens or s.total_len + 3 > self.ecfg.max_model_len:
                return False
        return True

    def _launch_lookahead(self, seqs, from_device: bool):
        nd = len(seqs)
        extra = 1 if from_device else 0
        for s in seqs:
            if not self._kv_reserve(s.seq_id, s.total_len + extra):
                return None
        par = self._la_parity
        self._la_parity ^= 1
        hb = self.la_host[par]
        pos, lens, slots = hb["pos"].numpy(), hb["lens"].numpy(), hb["slots"].numpy()
        max_len = 0
        for i, s in enumerate(seqs):
            L = s.total_len + extra
            pos[i] = L - 1
            lens[i] = L
            self.bm.fill_slots(s.seq_id, L - 1, 1, slots, i)
            if self.bm_win is not None:
                self.bm_win.fill_slots(s.seq_id, L - 1, 1, hb["slots_w"].numpy(), i)
            max_len = max(max_len, L)
        self.bm.fill_tables([s.seq_id for s in seqs], hb["tables"].numpy())
        if self.bm_win is not None:
            self.bm_win.fill_tables([s.seq_id for s in seqs], hb["tables_w"].numpy())
            self.d_slots_w[:nd].copy_(hb["slots_w"][:nd], non_blocking=True)
            self.d_dec_tables_w[:nd].copy_(hb["tables_w"][:nd], non_blocking=True)
        if not from_device:
            tok = self.h_tokens.numpy()
            for i, s in enumerate(seqs):
                tok[i] = s.output[-1] if s.output else s.prompt[-1]
            self.d_tokens[:nd].copy_(self.h_tokens[:nd], non_blocking=True)
        self.d_pos[:nd].copy_(hb["pos"][:nd], non_blocking=True)
        self.d_slots[:nd].copy_(hb["slots"][:nd], non_blocking=True)
        self.d_dec_lens[:nd].copy_(hb["lens"][:nd], non_blocking=True)
        self.d_dec_tables[:nd].copy_(hb["tables"][:nd], non_blocking=True)
        mb4 = self.max_blocks_per_seq * 4 + 4
        self.stats["h2d_bytes"] += nd * (8 + mb4) + (0 if from_device else 4 * nd)
        self.stats["d2h_bytes"] += 4 * nd
        if self._decode_graph(nd, max_len) is None:
            return None
        hb["out"][:nd].copy_(self.d_tokens[:nd], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.stats["decode_steps"] += 1
        return dict(seqs=list(seqs), nd=nd, buf=hb["out"], event=ev)

    def _collect_lookahead(self, inf) -> list[Sequence]:
        inf["event"].synchronize()
        toks = inf["buf"][: inf["nd"]].tolist()
        self.stats["steps"] += 1
        finished: list[Sequence] = []
        now = time.perf_counter()
        for s, tok in zip(inf["seqs"], toks):
            if s.status != SeqStatus.DECODING:
                continue            # ended while this step was in flight: its row is discarded
            self.stats["decode_tokens"] += 1
            s.num_computed = s.total_len
            if s.first_token_time is None:
                s.first_token_time = now
            reason = self._finish_step(s, tok, None)
            if s.on_token is not None and (reason is None or reason == FinishReason.LENGTH):
                s.on_token(s, tok)
                if s.status == SeqStatus.FINISHED:
                    continue
            if reason is not None:
                self._finish(s, reason)
                finished.append(s)
        self._release_window(inf["seqs"])
        return finished

    # ------------------------------------------------------------------ step
    @torch.inference_mode()
    def _check_device_status(self) -> None:
        """Every ``status_check_interval`` steps: read the device status word (bounded waits in the
        kernels record a code there instead of hanging) and fail the step loudly. One 4-byte
        read-back per interval, so a lost peer or a broken pipeline surfaces within that many steps."""
        iv = getattr(self.ecfg, "status_check_interval", 64)
        if not self.is_cuda or iv <= 0:
            return
        self._steps_since_check = getattr(self, "_steps_since_check", 0) + 1
        if self._steps_since_check < iv:
            return
        self._steps_since_check = 0
        from ..ops import _lib
        code = _lib.read_status(self.device)
        if code != 0:
            raise RuntimeError(f"a kernel reported failure code {code} (bounded wait ran out: 1xx GEMM pipeline, "
                               f"2xx peer flag, 4xx attention pipeline); the step's results are not valid")

    def step(self) -> list[Sequence]:
        """One scheduling tick + forward + sample. Returns the sequences that finished."""
        self._check_device_status()
        from ..utils.tracing import TRACER
        if TRACER.active:
            with TRACER.span("engine.step", running=len(self.running), waiting=len(self.waiting)):
                return self._step()
        return self._step()

    def _dp_step(self) -> list[Sequence]:
        """One tick of a data-parallel rank whose MoE layers exchange rows with the other ranks: all
        ranks run exactly one forward pass per tick in which anyone has work (a null forward here when
        this rank has nothing scheduled), none when everybody is idle."""
        decode, pieces = self._schedule() if self.has_work() else ([], [])
        tokens = len(decode) + sum(p[2] for p in pieces)
        t0 = time.perf_counter()
        self.dp_active = self.model.comm.any_work(self.has_work(), tokens) > 0
        self.stats["tick_sync_ms"] = self.stats.get("tick_sync_ms", 0.0) + (time.perf_counter() - t0) * 1e3
        ended, self._evicted = self._evicted, []
        if not self.dp_active:
            return ended
        if not decode and not pieces:
            self.model.forward_null()
            self.stats["null_forwards"] = self.stats.get("null_forwards", 0) + 1
            return ended
        return ended + self._run_scheduled(decode, pieces)

    def _step(self) -> list[Sequence]:
        if self.dp_lockstep:
            return self._dp_step()
        if self._inflight is not None:
            inf = self._inflight
            nxt = self._launch_lookahead(inf["seqs"], from_device=True) if self._can_pipeline(inf) else None
            fin = self._collect_lookahead(inf)
            self._inflight = nxt
            return fin
        decode, pieces = self._schedule()
        if self._evicted:
            ended, self._evicted = self._evicted, []
            if not decode and not pieces:
                return ended
            return ended + self._run_scheduled(decode, pieces)
        return self._run_scheduled(decode, pieces)

    def _run_scheduled(self, decode, pieces) -> list[Sequence]:
        if not decode and not pieces:
            return []
        if self._lookahead_eligible(decode, pieces):
            self._inflight = self._launch_lookahead(decode, from_device=False)
            if self._inflight is not None:
                return []
        if self._spec_now:
            self._spec_now = False
            return self._spec_step(decode)
        t_step = time.perf_counter()
        b, R = self._build_batch(decode, pieces)
        nd = len(decode)
        logits = None
        timing = self._step_timing
        if timing:
            ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            ev0.record()
        # a decode graph holds the expert kernels chosen for decode-sized groups; in a tick in which
        # another data-parallel rank prefills, this rank's experts get that rank's rows too
        if not pieces and nd and not (self.dp_lockstep and getattr(self.model.comm, "heavy", False)):
            gl = self._decode_graph(nd, b.dec_max_len)
            if gl is not None:
                logits = gl[:nd]
                self.stats["decode_steps"] += 1
        if logits is None:
            if self.drafter is not None and getattr(self.drafter, "needs_hidden", False):
                if self.pipeline:
                    # the residual stream exists on the last stage only, and so does the drafter
                    h = self.model.pipeline_hidden(b, self.kv_layers)
                    logits = self.model.logits(h, b.logits_rows) if h is not None else None
                else:
                    h = self.model.forward_hidden(b, self.kv_layers)
                    logits = self.model.logits(h, b.logits_rows)
                if h is not None:
                    self.drafter.on_forward(self, decode, pieces, h)
            else:
                logits = self.model.forward(b, self.kv_layers)
        # rows: decode rows first, then prefill rows that completed their prompt
        sample_seqs = list(decode) + [s for (s, start, cnt) in pieces if start + cnt >= s.total_len]
        if self.pipeline:
            toks, lps = self.model.sample_and_share(logits, sample_seqs, self.sampler)
        else:
            toks, lps = self.sampler.sample(logits, sample_seqs)
        if timing:
            # device time of the forward pass + sampling against the wall time of the whole step
            ev1.record()
            ev1.synchronize()
            kind = "decode" if not pieces else "mixed"
            st = self.stats
            st[f"{kind}_timed_steps"] = st.get(f"{kind}_timed_steps", 0) + 1
            st[f"{kind}_gpu_ms"] = st.get(f"{kind}_gpu_ms", 0.0) + ev0.elapsed_time(ev1)
            st[f"{kind}_wall_ms"] = st.get(f"{kind}_wall_ms", 0.0) + (time.perf_counter() - t_step) * 1e3
        self.stats["steps"] += 1
        self.stats["decode_tokens"] += nd
        self.stats["prefill_tokens"] += sum(p[2] for p in pieces)
        if self.spec_policy is not None and self.drafter is not None and nd and not pieces:
            self.spec_policy.record_classic((time.perf_counter() - t_step) * 1e3, nd)
        finished: list[Sequence] = []
        for s, _, cnt in pieces:
            s.num_computed += cnt
        for s in decode:
            s.num_computed = s.total_len
        self._release_window([p[0] for p in pieces] + list(decode))
        now = time.perf_counter()
        for i, s in enumerate(sample_seqs):
            tok = self._thinking_override(s, int(toks[i]))
            if s.status == SeqStatus.PREFILLING:
                s.status = SeqStatus.DECODING
            if s.first_token_time is None:
                s.first_token_time = now
            reason = self._finish_step(s, tok, lps[i] if lps is not None else None)
            if s.on_token is not None and (reason is None or reason == FinishReason.LENGTH):
                s.on_token(s, tok)
                if s.status == SeqStatus.FINISHED:
                    continue  # the callback ended the sequence (stop string)
            if reason is not None:
                self._finish(s, reason)
                finished.append(s)
        return finished

    def _thinking_override(self, s: Sequence, tok: int) -> int:
        """Thinking-budget enforcement on the sampled token (the reference's scheduler hook,
        src/server/batch/scheduler/run_loop.rs:58-71 with the rules of src/server/thinking_budget.rs):
        inside a reasoning block the tokens are counted, and once the cap is reached the next token
        is replaced by the end-of-thinking token. The forced token is an ordinary generated token
        afterwards (streamed, counted, part of the history)."""
        p = s.params
        cap = p.thinking_cap
        if cap is None:
            return tok
        if s.think_open:
            if tok == p.think_end_id:
                s.think_open = False
            elif s.think_count >= cap:
                s.think_open = False
                s.think_forced += 1
                self.stats["thinking_forced"] = self.stats.get("thinking_forced", 0) + 1
                return p.think_end_id
            else:
                s.think_count += 1
        elif p.think_start_id is not None and tok == p.think_start_id:
            s.think_open, s.think_count = True, 0
        return tok

    def _finish_step(self, s: Sequence, tok: int, lp) -> FinishReason | None:
        """Shared finish rule: an EOS / stop token is not pushed to the output
        (src/lib/mlxcel-core/src/engine/mod.rs:441-450)."""
        p = s.params
        n_out = len(s.output)
        if not p.ignore_eos and n_out >= p.min_tokens:
            if tok in self.cfg.eos_ids() or tok in p.stop_token_ids:
                return FinishReason.STOP
        s.output.append(tok)
        if lp is not None and p.logprobs:
            s.logprobs.append(float(lp))
        if len(s.output) >= p.max_tokens:
            return FinishReason.LENGTH
        if not self._ctx_shift:
            if s.total_len + 1 > self.ecfg.max_model_len:
                return FinishReason.LENGTH
            if self.ecfg.max_kv_size > 0 and s.total_len + 1 >= self.ecfg.max_kv_size and not s.mm_embeds:
                return FinishReason.LENGTH
        if p.loop_max_pattern > 0 and _tail_loop(s.output, p.loop_min_pattern, p.loop_max_pattern,
                                                 p.loop_min_count):
            return FinishReason.REPETITION_LOOP
        return None

    # ------------------------------------------------------------------ speculative decoding
    @staticmethod
    def _spec_row_ok(s: Sequence) -> bool:
        """Rows a verify round is exact for. Greedy rows: a draft is accepted when it equals the
        target's argmax. Sampled rows whose chain the fused sampler expresses (temperature, top-k,
        top-p, min-p, typical-p, top-n-sigma): *sampler-match* acceptance — every verify position
        is drawn with the row's own seed and step counter, and a draft is accepted when it equals
        that draw, so the emitted tokens are exactly the ones classic decoding would have drawn
        (docs/speculative-acceptance.md:18-35). Rows with per-step logit edits (penalties over the
        history, masks, bias) or per-step state (mirostat) are not eligible."""
        p = s.params
        return ((p.greedy or p.fused_eligible) and s.mask_fn is None and not p.needs_history and not p.logit_bias
                and not p.logprobs and p.thinking_cap is None)

    def _spec_step(self, decode: list[Sequence]) -> list[Sequence]:
        """One verify round for every decoding row (the reference's verify_round,
        src/lib/mlxcel-core/src/engine/verify_round.rs:170-305 and mtp/walk.rs:15-95): forward
        ``[pending, d0 .. d(K-2)]``, accept drafts while they equal the target argmax, emit the
        accepted drafts plus the target token at the first mismatch, roll the KV back."""
        K = self.spec_k
        t_round = time.perf_counter()
        props = self.drafter.propose(self, decode, K - 1)
        if self.pipeline:
            # proposals come from the stage that holds the drafter; every scheduler needs them
            flat = [[len(d)] + list(d) + [0] * (K - 1 - len(d)) for d in props]
            flat = self.model.share_ints(flat, (len(decode), K))
            props = [row[1:1 + row[0]] for row in flat]
        drafts, pieces = {}, []
        for s, d in zip(decode, props):
            room = min(s.params.max_tokens - len(s.output) - 1, self.ecfg.max_model_len - s.total_len - 1)
            d = list(d[: max(0, room)])
            if not self._kv_reserve(s.seq_id, s.total_len + len(d)):
                d = []
            drafts[s.seq_id] = d
            pieces.append((s, s.total_len - 1, 1 + len(d)))
        b, R = self._build_batch([], pieces, drafts=drafts, all_rows=True)
        need_h = getattr(self.drafter, "needs_hidden", False)
        walk = None
        all_greedy = all(s.params.greedy for s in decode)
        full = K > 1 and all(len(drafts[s.seq_id]) == K - 1 for s in decode)
        if self.pipeline:
            h = self.model.pipeline_hidden(b, self.kv_layers)
            logits = self.model.logits(h, b.logits_rows) if h is not None else None
            # argmax of every verify row on the last stage, shared with the other stages (R ints)
            target = self.model.share_ints(ops.argmax(logits).cpu().tolist() if logits is not None else None, (R,))
        elif self.is_cuda and all_greedy and full:
            # every row carries a full block: argmax + accept walk on the device, and the host reads
            # back two ints per row (accepted length, token at the first mismatch) instead of the
            # K target tokens of every row. The whole verify pass (forward, LM head, walk) is one
            # CUDA graph per (rows, K).
            nd = len(decode)
            if self.d_drafts is None or self.d_drafts.shape[1] != K - 1:
                self.d_drafts = torch.zeros(self.ecfg.max_batch, K - 1, dtype=torch.int32, device=self.device)
                self.h_drafts = torch.zeros(self.ecfg.max_batch, K - 1, dtype=torch.int32,
                                            pin_memory=True)
            self.h_drafts[:nd] = torch.tensor([drafts[s.seq_id] for s in decode], dtype=torch.int32)
            self.d_drafts[:nd].copy_(self.h_drafts[:nd], non_blocking=True)
            h, acc, nxt = self._verify_pass(b, nd, K)
            walk = torch.stack([acc, nxt]).cpu().tolist()
            self.stats["d2h_bytes"] += 8 * nd
        else:
            h = self.model.forward_hidden(b, self.kv_layers)
            logits = self.model.logits(h, b.logits_rows)
            if not all_greedy:
                # sampler-match: one draw per verify row with the owner's seed and the step it stands for
                owners, offs = [], []
                for s, _, cnt in pieces:
                    owners += [s] * cnt
                    offs += list(range(cnt))
                target, _ = self.sampler.sample(logits, owners, step_offsets=offs)
                self.stats["spec_sampled_rounds"] = self.stats.get("spec_sampled_rounds", 0) + 1
            else:
                target = ops.argmax(logits).cpu().tolist()
        self.stats["steps"] += 1
        self.stats["spec_rounds"] += 1
        finished, now, row0 = [], time.perf_counter(), 0
        accepted_info = []
        for i, (s, start, cnt) in enumerate(pieces):
            d = drafts[s.seq_id]
            if walk is not None:
                a = int(walk[0][i])
                emitted = d[:a] + [int(walk[1][i])]
            else:
                tgt = target[row0:row0 + cnt]
                a = 0
                while a < len(d) and d[a] == tgt[a]:
                    a += 1
                emitted = d[:a] + [tgt[a]]
            self.stats["spec_drafted"] += len(d)
            self.stats["spec_accepted"] += a
            s.draft_n += len(d)
            s.draft_n_accepted += a
            if hasattr(self.drafter, "record"):
                self.drafter.record(s.seq_id, len(d), a)
            L = s.total_len
            reason = None
            n_emit = 0
            if s.first_token_time is None:
                s.first_token_time = now
            for tok in emitted:
                reason = self._finish_step(s, tok, None)
                n_emit += 1
                if s.on_token is not None and (reason is None or reason == FinishReason.LENGTH):
                    s.on_token(s, tok)
                    if s.status == SeqStatus.FINISHED:
                        break
                if reason is not None:
                    break
            # KV is valid for the pending token and the accepted drafts actually kept
            kept = min(a, max(0, n_emit - 1)) if n_emit else 0
            s.num_computed = L + kept
            accepted_info.append((s, row0, kept))
            if s.status != SeqStatus.FINISHED:
                self._kv_truncate(s.seq_id, L + kept)
                if reason is not None:
                    self._finish(s, reason)
                    finished.append(s)
            elif s not in finished:
                finished.append(s)
            row0 += cnt
        self.stats["decode_tokens"] += sum(k + 1 for _, _, k in accepted_info)
        self._release_window(decode)
        if self.spec_policy is not None:
            self.spec_policy.record_spec((time.perf_counter() - t_round) * 1e3, sum(k + 1 for _, _, k in accepted_info))
        if need_h and h is not None:
            self.drafter.on_verify(self, accepted_info, h)
        for s in finished:
            self.drafter.release(s.seq_id)
        return finished

    def _verify_pass(self, b: StepBatch, nd: int, K: int):
        """Forward of ``nd`` verify blocks of ``K`` rows, LM head over every row and the accept walk
        against ``d_drafts``; replayed from a CUDA graph per (nd, K) when graphs are on (the batch
        lives in the engine's fixed device buffers, so a replay sees the current step's contents).
        Returns (hidden [nd * K, H], accepted [nd], next token [nd])."""
        V = None

        def run():
            h = self.model.forward_hidden(b, self.kv_layers)
            logits = self.model.logits(h, b.logits_rows)
            _, acc, nxt = ops.spec_verify(logits.view(nd, K, logits.shape[-1]), self.d_drafts[:nd])
            return h, acc, nxt
        if not self.ecfg.cuda_graphs or b.embeds is not None or b.positions3 is not None:
            return run()
        key = ("verify", nd, K)
        ent = self._graphs.get(key)
        if ent is None:
            side = torch.cuda.Stream(device=self.device)
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                run()                       # warm-up outside capture (descriptor caches, lazy buffers)
            torch.cuda.current_stream().wait_stream(side)
            from ..ops import _lib
            n0 = _lib.launches()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                out = run()
            # hidden states a drafter asked the executor to keep live in the graph's buffers too
            ent = (g, out, _lib.launches() - n0, list(getattr(self.model, "captured", ())))
            self._graphs[key] = ent
        ent[0].replay()
        if ent[3]:
            self.model.captured = list(ent[3])
        self.stats["graph_replays"] += 1
        self.stats["verify_graph_replays"] = self.stats.get("verify_graph_replays", 0) + 1
        self.stats["graph_kernel_launches"] += ent[2]
        return ent[1]

    # ------------------------------------------------------------------ convenience
    def generate(self, prompts: list[list[int]], params: SamplingParams | list[SamplingParams] | None = None,
                 media: list | None = None) -> list[Sequence]:
        """Run the given prompts to completion (continuous batching) and return them in order.
        ``media[i]``: ``dict(mm_embeds=..., key_tokens=...)`` of prompt i, or None."""
        if not isinstance(params, list):
            params = [params or SamplingParams()] * len(prompts)
        media = media or [None] * len(prompts)
        ids = [self.add_request(p, sp, **(mm or {})) for p, sp, mm in zip(prompts, params, media)]
        if self.dp_lockstep:
            # ticks are collective: keep stepping (null forwards once this rank is done) until every
            # rank has finished its own requests
            while True:
                self.step()
                if not self.dp_active:
                    break
        while self.has_work():
            self.step()
        return [self.seqs[i] for i in ids]


def _tail_loop(out: list[int], min_pat: int, max_pat: int, min_count: int) -> bool:
    n = len(out)
    for pat in range(max(1, min_pat), max_pat + 1):
        if pat * min_count > n:
            break
        tail = out[n - pat:]
        ok = True
        for r in range(2, min_count + 1):
            if out[n - r * pat: n - (r - 1) * pat] != tail:
                ok = False
                break
        if ok:
            return True
    return False
