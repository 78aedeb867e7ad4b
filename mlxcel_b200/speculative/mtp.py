"""Multi-token-prediction (MTP) drafter.

A one-layer head in the style of the Qwen3.5 / DeepSeek MTP modules the reference drives
(src/lib/mlxcel-core/src/drafter/qwen3_5_mtp/model.rs:15-140): at position p it fuses the target's
last hidden state h_p with the embedding of token p+1,

    x_p = fc([rmsnorm(embed(tok_{p+1})), rmsnorm(h_p)]),

runs one full-attention decoder layer with its own KV cache, and projects through the target's LM
head to predict token p+2. The head borrows the target's embedding table and LM head, and its KV
lives in a one-layer pool addressed by the TARGET's block tables (position p of the head sits in
the same slot as position p of the target), so no second block manager is needed.

Round structure (MTP block size K ⇒ K-1 drafts, mtp/walk.rs:15-95): one catch-up forward over the
positions the target verified last round (their real hidden states) yields d0; K-2 single-token
steps chained on the head's own hidden state yield d1…; the target verifies ``[pending, d0…]``.
Positions adopted from the prefix cache were never seen by the head (their KV slots hold zeros):
that only lowers acceptance, verification keeps the output exact.
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from .. import ops
from ..cache.kv_pool import KVPool
from ..models.decoder import DecoderModel, StepBatch
from ..models.weights import LayerWeights, ModelWeights, random_weights


@dataclass
class MTPWeights:
    enorm: torch.Tensor        # [H]
    hnorm: torch.Tensor        # [H]
    fc: torch.Tensor           # [H, 2H]
    layer: LayerWeights
    final_norm: torch.Tensor   # [H]


def random_mtp_weights(cfg, *, seed: int = 1, dtype=torch.bfloat16, device="cpu", tp_rank: int = 0,
                       tp_size: int = 1, std: float = 0.02) -> MTPWeights:
    one = random_weights(cfg, seed=seed + 7919, dtype=dtype, device=device, tp_rank=tp_rank, tp_size=tp_size,
                         layers=range(1), std=std)
    g = torch.Generator(device=torch.device(device)).manual_seed(seed + 104729)
    H = cfg.hidden_size
    fc = torch.empty(H, 2 * H, dtype=dtype, device=device).normal_(0.0, std, generator=g)
    ones = torch.ones(H, dtype=dtype, device=device) - cfg.norm_weight_bias
    return MTPWeights(enorm=ones.clone(), hnorm=ones.clone(), fc=fc, layer=one.layers[0], final_norm=ones.clone())


class MTPDrafter:
    needs_hidden = True

    def __init__(self, target: DecoderModel, cfg, weights: MTPWeights, num_blocks: int, block_size: int = 16):
        self.cfg, self.w, self.target = cfg, weights, target
        self.dev = target.device
        mw = ModelWeights(embed=target.w.embed, layers=[weights.layer], final_norm=weights.final_norm,
                          lm_head=target.w.lm_head)
        # the head's layer is a full-attention layer regardless of the target's layer pattern
        self.head = DecoderModel(cfg, mw, comm=target.comm, layer_range=range(cfg.num_hidden_layers - 1,
                                                                              cfg.num_hidden_layers))
        if cfg.layer_types:
            self.head.layer_range = range(next(i for i, t in enumerate(cfg.layer_types) if t == "full_attention"),
                                          cfg.num_hidden_layers)
        self.pool = KVPool(cfg, num_blocks, block_size, device=self.dev, tp_size=target.comm.tp_size, num_layers=1,
                           dtype=weights.final_norm.dtype)
        self.pending: dict[int, tuple[int, torch.Tensor]] = {}   # seq → (first position, hidden rows)
        self.mtp_len: dict[int, int] = {}                        # positions with head KV from real hidden
        self.stale: set[int] = set()

    # ------------------------------------------------------------------ head forward
    @torch.inference_mode()
    def _forward(self, engine, items):
        """items: (seq, start position, next-token ids, hidden rows [n, H]).
        Returns (argmax of the last row per item, head hidden of the last row per item [S, H])."""
        cfg, d = self.cfg, self.dev
        S = len(items)
        mb = engine.max_blocks_per_seq
        tables = np.zeros((S, mb), dtype=np.int32)
        total = sum(len(t) for _, _, t, _ in items)
        slots = np.zeros(total, dtype=np.int32)
        toks, pos, cu, lens, hs = [], [], [0], [], []
        off = 0
        for s, start, t, h in items:
            engine.bm.reserve(s.seq_id, start + len(t))
            engine.bm.fill_slots(s.seq_id, start, len(t), slots, off)
            toks += t
            pos += list(range(start, start + len(t)))
            off += len(t)
            cu.append(off)
            lens.append(start + len(t))
            hs.append(h)
        engine.bm.fill_tables([i[0].seq_id for i in items], tables)
        tok_t = torch.tensor(toks, dtype=torch.int32, device=d)
        e = self.target.comm.embed(tok_t, self.target.w.embed, cfg.embed_scale)
        hcat = torch.cat(hs, dim=0).to(e.dtype)
        x = torch.cat([ops.rmsnorm(e, self.w.enorm, cfg.rms_norm_eps, cfg.norm_weight_bias),
                       ops.rmsnorm(hcat, self.w.hnorm, cfg.rms_norm_eps, cfg.norm_weight_bias)], dim=-1)
        x = ops.linear(x.contiguous(), self.w.fc)
        b = StepBatch(token_ids=tok_t, positions=torch.tensor(pos, dtype=torch.int32, device=d),
                      slot_mapping=torch.from_numpy(slots).to(d), num_prefill_seqs=S,
                      pf_block_tables=torch.from_numpy(tables).to(d),
                      pf_cu_q=torch.tensor(cu, dtype=torch.int32, device=d),
                      pf_context_lens=torch.tensor(lens, dtype=torch.int32, device=d),
                      pf_max_q_len=max(len(t) for _, _, t, _ in items))
        g = self.head.forward_hidden(b, self.pool.layers, hidden_in=x)
        rows = torch.tensor([c - 1 for c in cu[1:]], device=d)
        logits = self.head.logits(g, rows)
        return ops.argmax(logits).cpu().tolist(), g.index_select(0, rows)

    # ------------------------------------------------------------------ engine hooks
    def on_forward(self, engine, decode, pieces, hidden) -> None:
        """Called after an ordinary forward (prefill pieces and/or decode rows), before sampling."""
        row = 0
        for s in decode:
            # A decode row outside a verify round (mixed step, sampled row): its hidden state is the
            # one of the pending token; queue it behind whatever the last verify left.
            pos = s.total_len - 1
            p = self.pending.get(s.seq_id)
            if s.seq_id in self.stale:
                pass
            elif p is not None and p[0] + p[1].shape[0] == pos:
                self.pending[s.seq_id] = (p[0], torch.cat([p[1], hidden[row:row + 1]], dim=0))
            elif p is None and self.mtp_len.get(s.seq_id, -1) == pos:
                self.pending[s.seq_id] = (pos, hidden[row:row + 1].clone())
            else:
                self.stale.add(s.seq_id)
            row += 1
        items = []
        for (s, start, cnt) in pieces:
            if s.seq_id in self.stale:
                row += cnt
                continue
            have = self.mtp_len.get(s.seq_id, 0)
            if s.seq_id not in self.mtp_len and start > 0:
                have = start                       # prefix adopted from the cache: nothing to replay
            if start != have:
                self.stale.add(s.seq_id)
                row += cnt
                continue
            toks = s.tokens
            known = min(cnt, max(0, len(toks) - 1 - start))   # rows whose next token already exists
            if known > 0:
                items.append((s, start, toks[start + 1:start + 1 + known], hidden[row:row + known]))
            if known < cnt:                         # last prompt row: its next token is sampled now
                self.pending[s.seq_id] = (start + known, hidden[row + known:row + cnt].clone())
            self.mtp_len[s.seq_id] = start + known
            row += cnt
        if items:
            self._forward(engine, items)

    def on_verify(self, engine, accepted_info, hidden) -> None:
        for s, row0, kept in accepted_info:
            if s.seq_id in self.stale or s.status.value == "finished":
                continue
            start = s.num_computed - kept - 1      # position of the pending token that was verified
            self.pending[s.seq_id] = (start, hidden[row0:row0 + kept + 1].clone())

    def propose(self, engine, seqs, max_draft: int) -> list[list[int]]:
        out: list[list[int]] = [[] for _ in seqs]
        if max_draft <= 0:
            return out
        items, idx = [], []
        for i, s in enumerate(seqs):
            p = self.pending.pop(s.seq_id, None)
            if p is None or s.seq_id in self.stale:
                continue
            start, h = p
            if start != self.mtp_len.get(s.seq_id, -1) or start + h.shape[0] != s.total_len - 1:
                self.stale.add(s.seq_id)
                continue
            toks = s.tokens
            items.append((s, start, toks[start + 1:start + 1 + h.shape[0]], h))
            idx.append(i)
        if not items:
            return out
        nxt, g = self._forward(engine, items)
        for (s, start, t, h) in items:
            self.mtp_len[s.seq_id] = start + len(t)
        for j, i in enumerate(idx):
            out[i].append(nxt[j])
        for k in range(1, max_draft):
            step = [(seqs[i], seqs[i].total_len - 1 + k - 1, [out[i][-1]], g[j:j + 1]) for j, i in enumerate(idx)]
            nxt, g = self._forward(engine, step)
            for j, i in enumerate(idx):
                out[i].append(nxt[j])
        return out

    def release(self, seq_id: int) -> None:
        self.pending.pop(seq_id, None)
        self.mtp_len.pop(seq_id, None)
        self.stale.discard(seq_id)
