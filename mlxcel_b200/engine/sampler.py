"""Row sampler: turns a logits matrix into one token per sequence.

Chain order follows the reference (docs/architecture.md:48-51 and
src/lib/mlxcel-core/src/generate.rs:1296-1340): token bias and penalties → top-k / top-p / min-p
evaluated on the untempered distribution → one temperature scale applied only to the final draw.
Rows whose parameters are expressible by the fused kernel (top-k, top-p, min-p, top-n-sigma,
typical-p, temperature) go through ``ops.sample`` in one launch (``fused_eligible``); the rest
(XTC, mirostat, dynamic temperature, DRY, top-logprobs) take the extended chain below, row by
row, on device tensors.
"""
from __future__ import annotations

import math

import torch

from .. import ops


class Sampler:
    def __init__(self, vocab_size: int, device):
        self.V = vocab_size
        self.device = device
        self._mirostat_mu: dict[int, float] = {}

    def sample(self, logits: torch.Tensor, seqs, step_offsets: list[int] | None = None
               ) -> tuple[list[int], list | None]:
        """One token per logits row. ``step_offsets`` (speculative verify blocks) lets one sequence own
        several rows: row i is drawn as that sequence's step ``len(output) + step_offsets[i]``, so the
        draw at each position is the one classic decoding would make there."""
        R = len(seqs)
        if R == 0:
            return [], None
        logits = logits[:R]
        plain_greedy = all(s.params.greedy and not s.params.needs_history and not s.params.logit_bias
                           and s.mask_fn is None and not s.params.logprobs for s in seqs)
        if plain_greedy:
            toks = ops.argmax(logits)
            return toks.cpu().tolist(), None
        work = logits.float() if logits.dtype != torch.float32 else logits.clone()
        # ---- token bias, structured-output masks, penalties
        for i, s in enumerate(seqs):
            p = s.params
            if p.logit_bias:
                idx = torch.tensor(list(p.logit_bias.keys()), device=work.device, dtype=torch.long)
                val = torch.tensor(list(p.logit_bias.values()), device=work.device, dtype=torch.float32)
                work[i].index_add_(0, idx, val)
            if s.mask_fn is not None:
                m = s.mask_fn(s)
                if m is not None:
                    # the tokenizer's vocabulary may be shorter than the (padded) logits row: ids the
                    # matcher does not know are never allowed
                    n = min(m.numel(), work.shape[1])
                    work[i, :n].masked_fill_(~m[:n].to(work.device), float("-inf"))
                    work[i, n:] = float("-inf")
        if any(s.params.needs_history for s in seqs):
            H = max(min(len(s.tokens), s.params.repetition_context_size) for s in seqs
                    if s.params.needs_history)
            H = max(H, 1)
            hist = torch.full((R, H), -1, dtype=torch.int32)
            rep, freq, pres = torch.ones(R), torch.zeros(R), torch.zeros(R)
            for i, s in enumerate(seqs):
                p = s.params
                if not p.needs_history:
                    continue
                tail = s.tokens[-min(len(s.tokens), p.repetition_context_size):]
                hist[i, : len(tail)] = torch.tensor(tail, dtype=torch.int32)
                rep[i], freq[i], pres[i] = p.repetition_penalty, p.frequency_penalty, p.presence_penalty
            work = ops.apply_penalties(work, hist.to(work.device), rep.to(work.device),
                                       freq.to(work.device), pres.to(work.device))
            for i, s in enumerate(seqs):
                if s.params.dry_multiplier > 0:
                    _apply_dry(work[i], s.tokens, s.params)
        toks = [0] * R
        lps: list = [None] * R
        fused = [i for i, s in enumerate(seqs) if s.params.fused_eligible]
        if fused:
            sel = work if len(fused) == R else work[fused]
            temp = torch.tensor([max(seqs[i].params.temperature, 0.0) for i in fused], dtype=torch.float32)
            tk = torch.tensor([seqs[i].params.top_k for i in fused], dtype=torch.int32)
            tp = torch.tensor([seqs[i].params.top_p for i in fused], dtype=torch.float32)
            mp = torch.tensor([seqs[i].params.min_p for i in fused], dtype=torch.float32)
            ty = ns = None
            if any(seqs[i].params.typical_p < 1.0 or seqs[i].params.top_n_sigma > 0.0 for i in fused):
                ty = torch.tensor([seqs[i].params.typical_p for i in fused], dtype=torch.float32)
                ns = torch.tensor([seqs[i].params.top_n_sigma for i in fused], dtype=torch.float32)
            seeds = torch.tensor([_seed_of(seqs[i]) for i in fused], dtype=torch.int64)
            steps = torch.tensor([len(seqs[i].output) + (step_offsets[i] if step_offsets else 0) for i in fused],
                                 dtype=torch.int64)
            d = work.device
            t, lp = ops.sample(sel.contiguous(), temp.to(d), tk.to(d), tp.to(d), mp.to(d), seeds.to(d),
                               steps.to(d), ty.to(d) if ty is not None else None,
                               ns.to(d) if ns is not None else None)
            t, lp = t.cpu().tolist(), lp.cpu().tolist()
            for j, i in enumerate(fused):
                toks[i], lps[i] = t[j], lp[j]
        for i, s in enumerate(seqs):
            if not s.params.fused_eligible:
                toks[i], lps[i] = self._extended(work[i], s)
        return toks, lps

    # ------------------------------------------------------------------ extended chain
    def _extended(self, l: torch.Tensor, s) -> tuple[int, float]:
        p = s.params
        l = torch.nan_to_num(l.float(), nan=float("-inf"))
        logz = torch.logsumexp(l, 0)
        gen = torch.Generator(device=l.device)
        gen.manual_seed((_seed_of(s) * 1000003 + len(s.output)) & 0x7FFFFFFFFFFFFFFF)
        if p.mirostat in (1, 2):
            tok = self._mirostat(l, s, gen)
            return tok, float(l[tok] - logz)
        if p.greedy:
            tok = int(l.argmax())
            return tok, float(l[tok] - logz)
        keep = ops.reference.filter_mask(l, p.top_k, p.top_p, p.min_p)
        if p.top_n_sigma > 0:
            keep &= l >= l.max() - p.top_n_sigma * l[torch.isfinite(l)].std()
        lk = torch.where(keep, l, torch.full_like(l, float("-inf")))
        if p.typical_p < 1.0:
            lk = _typical_filter(lk, p.typical_p)
        if p.xtc_probability > 0 and torch.rand(1, generator=gen, device=l.device).item() < p.xtc_probability:
            probs = torch.softmax(lk, 0)
            above = torch.nonzero(probs >= p.xtc_threshold).flatten()
            if above.numel() > 1:
                # drop every token above the threshold except the least likely of them
                keep_one = above[probs[above].argmin()]
                lk[above] = float("-inf")
                lk[keep_one] = l[keep_one]
        T = p.temperature
        if p.dynatemp_range > 0:
            probs = torch.softmax(lk, 0)
            ent = -(probs * torch.log(probs.clamp_min(1e-30))).sum()
            max_ent = math.log(max(2, int((probs > 0).sum())))
            lo, hi = max(0.0, T - p.dynatemp_range), T + p.dynatemp_range
            T = lo + (hi - lo) * float((ent / max_ent).clamp(0, 1)) ** p.dynatemp_exponent
        T = max(T, 1e-5)
        probs = torch.softmax(lk / T, 0)
        tok = int(torch.multinomial(probs, 1, generator=gen))
        return tok, float(l[tok] - logz)

    def _mirostat(self, l, s, gen) -> int:
        p = s.params
        mu = self._mirostat_mu.get(s.seq_id, 2.0 * p.mirostat_tau)
        probs = torch.softmax(l / max(p.temperature, 1e-5), 0)
        sp, order = torch.sort(probs, descending=True)
        surprise = -torch.log2(sp.clamp_min(1e-30))
        if p.mirostat == 1:
            # estimate the Zipf exponent from the top tokens, then the k that meets the target
            m = min(100, sp.numel() - 1)
            i = torch.arange(1, m + 1, device=l.device, dtype=torch.float32)
            t = torch.log((i + 1) / i)
            b = torch.log(sp[:m] / sp[1:m + 1].clamp_min(1e-30))
            s_hat = float((t * b).sum() / (t * t).sum())
            eps = s_hat - 1.0
            k = ((eps * (2 ** mu)) / (1 - sp.numel() ** (-eps) if eps != 0 else 1.0)) ** (1 / max(s_hat, 1e-6))
            k = int(min(max(1, round(float(k))), sp.numel()))
            cand = sp[:k]
        else:
            k = int(max(1, (surprise <= mu).sum()))
            cand = sp[:k]
        cand = cand / cand.sum()
        j = int(torch.multinomial(cand, 1, generator=gen))
        obs = float(-torch.log2(cand[j].clamp_min(1e-30)))
        self._mirostat_mu[s.seq_id] = mu - p.mirostat_eta * (obs - p.mirostat_tau)
        return int(order[j])


def _seed_of(s) -> int:
    return s.params.seed if s.params.seed is not None else (0x9E3779B9 ^ (s.seq_id * 2654435761)) & 0xFFFFFFFF


def _typical_filter(l: torch.Tensor, typical_p: float) -> torch.Tensor:
    probs = torch.softmax(l, 0)
    logp = torch.log(probs.clamp_min(1e-30))
    ent = -(probs * logp).sum()
    dev = (-logp - ent).abs()
    dev = torch.where(probs > 0, dev, torch.full_like(dev, float("inf")))
    order = torch.argsort(dev)
    cum = torch.cumsum(probs[order], 0)
    last = int((cum < typical_p).sum())
    keep = torch.zeros_like(probs, dtype=torch.bool)
    keep[order[: last + 1]] = True
    return torch.where(keep, l, torch.full_like(l, float("-inf")))


def _apply_dry(l: torch.Tensor, tokens: list[int], p) -> None:
    """DRY ("don't repeat yourself"): penalise tokens that would extend a repeated suffix."""
    n = len(tokens)
    if n < 2:
        return
    breakers = set(p.dry_sequence_breakers)
    best: dict[int, int] = {}
    last = tokens[-1]
    if last in breakers:
        return
    for i in range(n - 2, -1, -1):
        if tokens[i] != last:
            continue
        m = 1
        while i - m >= 0 and m < 64 and tokens[i - m] == tokens[n - 1 - m] and tokens[i - m] not in breakers:
            m += 1
        nxt = tokens[i + 1]
        if m > best.get(nxt, 0):
            best[nxt] = m
    for tok, m in best.items():
        if m >= p.dry_allowed_length and 0 <= tok < l.numel():
            l[tok] -= p.dry_multiplier * (p.dry_base ** (m - p.dry_allowed_length))
