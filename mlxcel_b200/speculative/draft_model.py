"""Full-model drafter: an ordinary small checkpoint with its own KV pool proposes greedy tokens
(the reference's src/lib/mlxcel-core/src/speculative/full_model_drafter.rs). The drafter mirrors
every target sequence in its own block manager: before proposing it prefills whatever the target
has accepted since the last round, decodes ``max_draft`` tokens for all rows in lockstep, then
truncates its mirror back to the accepted length."""
from __future__ import annotations

import numpy as np
import torch

from .. import ops
from ..cache.kv_pool import KVPool
from ..host_runtime import BlockManager
from ..models.decoder import DecoderModel, StepBatch


class DraftModelDrafter:
    needs_hidden = False

    def __init__(self, model: DecoderModel, cfg, num_blocks: int = 4096, block_size: int = 16,
                 max_model_len: int = 8192):
        self.model, self.cfg = model, cfg
        self.dev = model.device
        self.bs = block_size
        self.pool = KVPool(cfg, num_blocks, block_size, device=self.dev, tp_size=model.comm.tp_size,
                           num_layers=len(model.w.layers), dtype=model.w.final_norm.dtype)
        self.bm = BlockManager(num_blocks, block_size, False, 0.0)
        self.max_blocks = (max_model_len + block_size - 1) // block_size
        self.computed: dict[int, int] = {}

    @torch.inference_mode()
    def _forward(self, items: list[tuple[int, list[int], int]]) -> torch.Tensor:
        """items: (seq_id, tokens, start position). Returns the last-row logits argmax per item."""
        toks, pos, cu, lens = [], [], [0], []
        S = len(items)
        tables = np.zeros((S, self.max_blocks), dtype=np.int32)
        total = sum(len(t) for _, t, _ in items)
        slots = np.zeros(total, dtype=np.int32)
        off = 0
        for sid, t, start in items:
            if not self.bm.reserve(sid, start + len(t)):
                raise RuntimeError("draft KV pool exhausted")
            self.bm.fill_slots(sid, start, len(t), slots, off)
            toks += t
            pos += list(range(start, start + len(t)))
            off += len(t)
            cu.append(off)
            lens.append(start + len(t))
        self.bm.fill_tables([i[0] for i in items], tables)
        d = self.dev
        b = StepBatch(token_ids=torch.tensor(toks, dtype=torch.int32, device=d),
                      positions=torch.tensor(pos, dtype=torch.int32, device=d),
                      slot_mapping=torch.from_numpy(slots).to(d), num_prefill_seqs=S,
                      pf_block_tables=torch.from_numpy(tables).to(d),
                      pf_cu_q=torch.tensor(cu, dtype=torch.int32, device=d),
                      pf_context_lens=torch.tensor(lens, dtype=torch.int32, device=d),
                      pf_max_q_len=max(len(t) for _, t, _ in items),
                      logits_rows=torch.tensor([c - 1 for c in cu[1:]], device=d))
        return ops.argmax(self.model.forward(b, self.pool.layers)).cpu().tolist()

    def propose(self, engine, seqs, max_draft: int) -> list[list[int]]:
        if max_draft <= 0:
            return [[] for _ in seqs]
        items = []
        for s in seqs:
            if not self.bm.has_seq(s.seq_id):
                self.bm.create(s.seq_id, 0)
                self.computed[s.seq_id] = 0
            c = self.computed[s.seq_id]
            toks = s.tokens
            items.append((s.seq_id, toks[c:], c))
        nxt = self._forward(items)                      # catch-up prefill, yields d0
        drafts = [[t] for t in nxt]
        base = [s.total_len for s in seqs]
        for k in range(1, max_draft):
            nxt = self._forward([(s.seq_id, [drafts[i][-1]], base[i] + k - 1) for i, s in enumerate(seqs)])
            for i, t in enumerate(nxt):
                drafts[i].append(t)
        for i, s in enumerate(seqs):                    # forget the speculative tail
            self.bm.truncate(s.seq_id, base[i])
            self.computed[s.seq_id] = base[i]
        return drafts

    def on_forward(self, engine, decode, pieces, hidden):
        pass

    def on_verify(self, engine, accepted_info, hidden):
        pass

    def release(self, seq_id: int) -> None:
        self.bm.free_seq(seq_id)
        self.computed.pop(seq_id, None)
