"""Pipeline parallelism: contiguous layer ranges per stage, activations over NCCL send/recv.

Every rank runs the same scheduler (SPMD lockstep), so the batch description is already known on
every stage and only the residual stream ``[tokens, hidden]`` moves between stages. A step's
batch is cut into micro-batches along sequences; stage s works on micro-batch i+1 while stage
s+1 works on micro-batch i (GPipe-style fill/drain, the reference's schedule in
src/distributed/pipeline/schedule.rs), sends are issued on a side stream so they overlap the next
micro-batch's compute. The last stage computes the logits, samples, and broadcasts the sampled
token ids so that every rank's scheduler advances identically. Where the reference moves JSON+base64 tensors over TCP
(src/distributed/pipeline/runtime.rs:1081-1207), stages here are GPUs of one NVSwitch domain.

With tensor parallelism inside a stage (TP × PP) rank = stage * tp + tp_rank; a rank exchanges
activations with the rank of the same tp_rank in the neighbouring stage.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.decoder import DecoderModel, StepBatch


class PipelineContext:
    def __init__(self, world_group, stage: int, num_stages: int, tp_size: int = 1, tp_rank: int = 0):
        self.group = world_group
        self.stage, self.num_stages, self.tp_size, self.tp_rank = stage, num_stages, tp_size, tp_rank
        self.prev_rank = (stage - 1) * tp_size + tp_rank if stage > 0 else None
        self.next_rank = (stage + 1) * tp_size + tp_rank if stage < num_stages - 1 else None
        self.last_stage_rank0 = (num_stages - 1) * tp_size
        self.is_first, self.is_last = stage == 0, stage == num_stages - 1
        self.comm_stream = None
        self.stats = dict(sent_bytes=0, recv_bytes=0, microbatches=0)


def split_batch(b: StepBatch, num_micro: int) -> list[tuple[StepBatch, slice]]:
    """Cut a step batch into up to ``num_micro`` micro-batches along sequences (decode rows and
    prefill sequences are split separately). Returns (micro-batch, token slice in the full batch)."""
    nd, sp = b.num_decode, b.num_prefill_seqs
    units = nd + sp
    m = max(1, min(num_micro, units))
    out = []
    cu = b.pf_cu_q_host or [0]
    for i in range(m):
        d0, d1 = nd * i // m, nd * (i + 1) // m
        s0, s1 = sp * i // m, sp * (i + 1) // m
        if d1 == d0 and s1 == s0:
            continue
        t_dec = slice(d0, d1)
        p0, p1 = (cu[s0], cu[s1]) if sp else (0, 0)
        idx = list(range(d0, d1)) + list(range(nd + p0, nd + p1))
        sel = torch.tensor(idx, dtype=torch.long, device=b.token_ids.device)
        mb = StepBatch(token_ids=b.token_ids.index_select(0, sel), positions=b.positions.index_select(0, sel),
                       slot_mapping=b.slot_mapping.index_select(0, sel), num_decode=d1 - d0,
                       dec_block_tables=b.dec_block_tables[t_dec] if d1 > d0 else None,
                       dec_context_lens=b.dec_context_lens[t_dec] if d1 > d0 else None,
                       dec_max_len=b.dec_max_len, num_prefill_seqs=s1 - s0,
                       pf_block_tables=b.pf_block_tables[s0:s1] if s1 > s0 else None,
                       pf_cu_q=(b.pf_cu_q[s0:s1 + 1] - cu[s0]).to(torch.int32) if s1 > s0 else None,
                       pf_context_lens=b.pf_context_lens[s0:s1] if s1 > s0 else None,
                       pf_max_q_len=b.pf_max_q_len, pf_cu_q_host=[c - cu[s0] for c in cu[s0:s1 + 1]] if s1 > s0 else None)
        out.append((mb, sel))
    return out


class PipelineModel(DecoderModel):
    """A DecoderModel holding one stage's layers; ``forward`` runs the micro-batch pipeline."""

    def __init__(self, cfg, weights, ctx: PipelineContext, comm=None, num_micro: int = 2, **kw):
        layer_range = kw.pop("layer_range")
        super().__init__(cfg, weights, comm=comm, layer_range=layer_range, first_stage=ctx.is_first,
                         last_stage=ctx.is_last, **kw)
        self.ctx, self.num_micro = ctx, num_micro

    def _send(self, h: torch.Tensor) -> None:
        ctx = self.ctx
        if h.is_cuda:
            if ctx.comm_stream is None:
                ctx.comm_stream = torch.cuda.Stream(device=h.device)
            ev = torch.cuda.Event()
            ev.record()
            with torch.cuda.stream(ctx.comm_stream):
                ctx.comm_stream.wait_event(ev)
                dist.send(h, ctx.next_rank, group=ctx.group)
                h.record_stream(ctx.comm_stream)
        else:
            dist.send(h.contiguous(), ctx.next_rank, group=ctx.group)
        ctx.stats["sent_bytes"] += h.numel() * h.element_size()

    def _recv(self, tokens: int, like: torch.Tensor) -> torch.Tensor:
        ctx = self.ctx
        h = torch.empty(tokens, self.cfg.hidden_size, dtype=self.w.final_norm.dtype, device=self.device)
        dist.recv(h, ctx.prev_rank, group=ctx.group)
        ctx.stats["recv_bytes"] += h.numel() * h.element_size()
        return h

    def pipeline_hidden(self, b: StepBatch, kv_layers) -> torch.Tensor | None:
        """Runs the step through all stages in micro-batches. The last stage returns the residual
        stream of the whole batch ``[T, H]``; the others return None."""
        ctx = self.ctx
        T = b.num_tokens
        micro = split_batch(b, self.num_micro)
        h_full = torch.empty(T, self.cfg.hidden_size, dtype=self.w.final_norm.dtype, device=self.device) \
            if ctx.is_last else None
        from ..utils.tracing import span
        for i, (mb, sel) in enumerate(micro):
            ctx.stats["microbatches"] += 1
            if ctx.is_first:
                h_in = None
            else:
                with span("pp.recv", cat="pipeline", stage=ctx.stage, micro=i, tokens=mb.num_tokens):
                    h_in = self._recv(mb.num_tokens, mb.token_ids)
            with span("pp.stage", cat="pipeline", stage=ctx.stage, micro=i, tokens=mb.num_tokens):
                h = self.forward_hidden(mb, kv_layers, hidden_in=h_in)
            if ctx.is_last:
                h_full.index_copy_(0, sel, h)
            else:
                with span("pp.send", cat="pipeline", stage=ctx.stage, micro=i):
                    self._send(h)
        if ctx.comm_stream is not None:
            torch.cuda.current_stream().wait_stream(ctx.comm_stream)
        return h_full

    def forward(self, b: StepBatch, kv_layers) -> torch.Tensor | None:
        # only the last stage has logits; the sampled token ids are what travels back
        # (see sample_and_share), not [rows, vocab] logits
        h = self.pipeline_hidden(b, kv_layers)
        return self.logits(h, b.logits_rows).contiguous() if self.ctx.is_last else None

    def share_ints(self, values, shape) -> list:
        """Broadcast a small int tensor (drafts, verify results) from the last stage to every rank."""
        ctx = self.ctx
        if ctx.is_last:
            t = torch.as_tensor(values, dtype=torch.int32).reshape(shape).to(self.device)
        else:
            t = torch.empty(shape, dtype=torch.int32, device=self.device)
        dist.broadcast(t, ctx.last_stage_rank0, group=ctx.group)
        return t.cpu().tolist()

    def sample_and_share(self, logits, seqs, sampler):
        """Sample on the last stage and broadcast the token ids (and log-probabilities when a row
        asks for them) to every rank: R * 4 bytes per step instead of R * vocab logits."""
        ctx = self.ctx
        R = len(seqs)
        want_lp = any(s.params.logprobs for s in seqs)
        if ctx.is_last:
            toks, lps = sampler.sample(logits, seqs)
            t = torch.tensor(toks, dtype=torch.int32, device=self.device)
            lp = torch.tensor([float(x) if x is not None else 0.0 for x in (lps or [0.0] * R)],
                              dtype=torch.float32, device=self.device) if want_lp else None
        else:
            t = torch.empty(R, dtype=torch.int32, device=self.device)
            lp = torch.empty(R, dtype=torch.float32, device=self.device) if want_lp else None
        dist.broadcast(t, ctx.last_stage_rank0, group=ctx.group)
        if lp is not None:
            dist.broadcast(lp, ctx.last_stage_rank0, group=ctx.group)
        ctx.stats["token_bytes"] = ctx.stats.get("token_bytes", 0) + 4 * R
        return t.cpu().tolist(), (lp.cpu().tolist() if lp is not None else None)


class RemoteDrafter:
    """Drafter stand-in on the stages that do not hold the last layers: a hidden-state drafter (MTP
    head) lives on the last stage, which broadcasts its proposals; the other stages only take part
    in that broadcast and keep no drafter state."""

    needs_hidden = True
    remote = True

    def propose(self, engine, seqs, max_draft):
        return [[] for _ in seqs]

    def on_forward(self, engine, decode, pieces, hidden) -> None:
        pass

    def on_verify(self, engine, accepted_info, hidden) -> None:
        pass

    def record(self, *a) -> None:
        pass

    def release(self, seq_id: int) -> None:
        pass
