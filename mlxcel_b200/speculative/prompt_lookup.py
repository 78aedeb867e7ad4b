"""Prompt-lookup (n-gram) drafter: propose the continuation of the most recent earlier occurrence
of the sequence's last n tokens (the reference's src/lib/mlxcel-core/src/speculative/prompt_lookup.rs;
server defaults: max draft 7, n-gram sizes 3..1). A break-even governor turns proposals off for a
row whose recent acceptance does not pay for the wider verify forward."""
from __future__ import annotations


class PromptLookupDrafter:
    needs_hidden = False

    def __init__(self, max_ngram: int = 3, min_ngram: int = 1, min_accept_rate: float = 0.15, window: int = 16):
        self.max_ngram, self.min_ngram = max_ngram, min_ngram
        self.min_accept_rate, self.window = min_accept_rate, window
        self.hist: dict[int, list[tuple[int, int]]] = {}

    def _lookup(self, toks: list[int], max_draft: int) -> list[int]:
        n_tok = len(toks)
        for n in range(min(self.max_ngram, n_tok - 1), self.min_ngram - 1, -1):
            pat = toks[n_tok - n:]
            for i in range(n_tok - n - 1, -1, -1):
                if toks[i:i + n] == pat:
                    cont = toks[i + n:i + n + max_draft]
                    if cont:
                        return cont
        return []

    def propose(self, engine, seqs, max_draft: int) -> list[list[int]]:
        out = []
        for s in seqs:
            h = self.hist.get(s.seq_id, [])
            if len(h) >= self.window:
                d = sum(x for x, _ in h[-self.window:])
                a = sum(y for _, y in h[-self.window:])
                if d and a / d < self.min_accept_rate and len(h) % 8:   # re-probe every 8 rounds
                    out.append([])
                    h.append((0, 0))
                    continue
            out.append(self._lookup(s.tokens, max_draft))
        self._last = {s.seq_id: (len(d), s.total_len) for s, d in zip(seqs, out)}
        return out

    def on_forward(self, engine, decode, pieces, hidden):
        pass

    def on_verify(self, engine, accepted_info, hidden):
        pass

    def record(self, seq_id: int, drafted: int, accepted: int) -> None:
        self.hist.setdefault(seq_id, []).append((drafted, accepted))

    def release(self, seq_id: int) -> None:
        self.hist.pop(seq_id, None)
