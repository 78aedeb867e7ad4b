"""Adaptive speculation policy and the exactness probe.

Speculative decoding only pays when the drafts are accepted often enough to beat the wider verify
forward. The policy measures it on the live server instead of assuming it (the reference's adaptive
MTP policy, src/server/batch/mtp_policy.rs and docs/CONTINUOUS_BATCHING.md:684-798): while
*profiling*, the first ``profile_requests`` requests run verify rounds and a few *classic probe*
steps are interleaved; tokens per millisecond of both are compared and the verdict (``enabled`` /
``disabled``) is kept for the process and persisted per (model, drafter, K, device), so the next
start skips the profile. A verdict can be forced or reset through ``/v1/internal/mtp-policy``.

The exactness probe (src/models/speculative_exactness.rs, docs/speculative-acceptance.md:25-60)
checks the property greedy acceptance relies on: forwarding a block ``[cur, d0 .. dK-2]`` in one
pass must give the same argmax tokens as decoding those positions one at a time. Kernels that pick
different tilings for 1-row and K-row batches can differ by rounding; if a near-tie flips, the
"lossless" claim is false for this model / build and speculation stays off.
"""
from __future__ import annotations

import hashlib
import json
import os
import time
from dataclasses import asdict, dataclass, field
from pathlib import Path


@dataclass
class PolicyState:
    mode: str = "profiling"            # profiling | enabled | disabled | forced_on | forced_off
    spec_ms: float = 0.0
    spec_tokens: int = 0
    spec_rounds: int = 0
    classic_ms: float = 0.0
    classic_tokens: int = 0
    classic_steps: int = 0
    requests_seen: int = 0
    verdict_reason: str = ""
    exact: bool | None = None          # result of the exactness probe (None = not run)
    history: list = field(default_factory=list)


class SpecPolicy:
    def __init__(self, key: str = "", profile_requests: int = 4, classic_probes: int = 2, min_gain: float = 1.0,
                 cache_dir: str | None = None, clock=time.perf_counter, persist: bool = True):
        self.key, self.profile_requests, self.classic_probes, self.min_gain = key, profile_requests, classic_probes, min_gain
        self.clock, self.persist = clock, persist
        base = cache_dir or os.environ.get("MLXCEL_B200_CACHE_DIR") or os.path.join(os.path.expanduser("~"), ".cache", "mlxcel_b200")
        self.path = Path(base) / "mtp-policy" / (hashlib.sha256(key.encode()).hexdigest()[:24] + ".json")
        self.state = PolicyState()
        self._probe_due = 0
        self._load()

    # ------------------------------------------------------------------ persistence
    def _load(self) -> None:
        if not (self.persist and self.key and self.path.exists()):
            return
        try:
            d = json.loads(self.path.read_text())
            if d.get("key") == self.key and d.get("mode") in ("enabled", "disabled"):
                self.state.mode = d["mode"]
                self.state.verdict_reason = d.get("reason", "") + " (persisted)"
        except (OSError, ValueError):
            pass

    def _save(self) -> None:
        if not (self.persist and self.key):
            return
        try:
            self.path.parent.mkdir(parents=True, exist_ok=True)
            tmp = self.path.with_suffix(".tmp")
            tmp.write_text(json.dumps(dict(key=self.key, mode=self.state.mode, reason=self.state.verdict_reason,
                                           spec_tok_per_ms=self._rate(True), classic_tok_per_ms=self._rate(False))))
            os.replace(tmp, self.path)
        except OSError:
            pass

    # ------------------------------------------------------------------ decisions
    def allow(self) -> bool:
        """May the next decode tick be a speculative round?"""
        st = self.state
        if st.exact is False:
            return False
        if st.mode in ("enabled", "forced_on"):
            return True
        if st.mode in ("disabled", "forced_off"):
            return False
        # profiling: interleave classic probe steps so that both rates are measured on the same rows
        if st.classic_steps < self.classic_probes and st.spec_rounds >= (st.classic_steps + 1) * 4:
            return False
        return True

    def on_request_finished(self) -> None:
        st = self.state
        st.requests_seen += 1
        if st.mode == "profiling" and st.requests_seen >= self.profile_requests:
            self._decide()

    def record_spec(self, ms: float, tokens: int) -> None:
        st = self.state
        st.spec_ms += ms
        st.spec_tokens += tokens
        st.spec_rounds += 1

    def record_classic(self, ms: float, tokens: int) -> None:
        st = self.state
        if st.mode != "profiling":
            return
        st.classic_ms += ms
        st.classic_tokens += tokens
        st.classic_steps += 1

    def _rate(self, spec: bool) -> float | None:
        st = self.state
        ms, tok = (st.spec_ms, st.spec_tokens) if spec else (st.classic_ms, st.classic_tokens)
        return tok / ms if ms > 0 else None

    def _decide(self) -> None:
        st = self.state
        s, c = self._rate(True), self._rate(False)
        if s is None or c is None:
            return                      # not enough evidence yet: keep profiling
        st.mode = "enabled" if s >= self.min_gain * c else "disabled"
        st.verdict_reason = f"speculative {s:.4f} tok/ms vs classic {c:.4f} tok/ms over {st.requests_seen} requests"
        st.history.append(dict(at=time.time(), mode=st.mode, reason=st.verdict_reason))
        self._save()

    # ------------------------------------------------------------------ control (HTTP)
    def force(self, mode: str) -> None:
        """``on`` / ``off`` pin the decision, ``auto`` starts a new profile, ``reset`` also forgets the
        persisted verdict."""
        st = self.state
        if mode == "on":
            st.mode = "forced_on"
        elif mode == "off":
            st.mode = "forced_off"
        elif mode in ("auto", "reset"):
            keep_exact = st.exact
            self.state = PolicyState(exact=keep_exact)
            if mode == "reset" and self.path.exists():
                try:
                    self.path.unlink()
                except OSError:
                    pass
        else:
            raise ValueError("mode must be on, off, auto or reset")

    def snapshot(self) -> dict:
        d = asdict(self.state)
        d.update(key=self.key, spec_tok_per_ms=self._rate(True), classic_tok_per_ms=self._rate(False),
                 profile_requests=self.profile_requests, classic_probes=self.classic_probes)
        return d


class _ScriptedDrafter:
    """Proposes a fixed continuation (the exactness probe feeds the chain-decoded tokens back as drafts)."""

    needs_hidden = False

    def __init__(self, script: list[int]):
        self.script = script

    def propose(self, engine, seqs, max_draft):
        out = []
        for s in seqs:
            done = len(s.output)
            out.append(self.script[done:done + max_draft])
        return out

    def on_forward(self, *a):
        pass

    def on_verify(self, *a):
        pass

    def release(self, seq_id):
        pass


def exactness_probe(engine, prompt: list[int], k: int = 4, tokens: int = 12) -> bool:
    """Block-vs-chain check on ``engine`` (no requests may be in flight): decode ``tokens`` tokens one
    at a time, then decode them again through verify rounds whose drafts are exactly those tokens.
    Every draft must be accepted and the outputs must be identical."""
    from ..engine.params import SamplingParams

    if engine.has_work():
        raise RuntimeError("the exactness probe needs an idle engine")
    saved = engine.drafter, engine.spec_k, getattr(engine, "spec_policy", None)
    sp = SamplingParams(max_tokens=tokens, temperature=0.0, ignore_eos=True)
    try:
        engine.drafter, engine.spec_policy = None, None
        chain = engine.generate([list(prompt)], sp)[0]
        want = list(chain.output)
        engine.release(chain.seq_id)
        d0, a0 = engine.stats.get("spec_drafted", 0), engine.stats.get("spec_accepted", 0)
        engine.drafter, engine.spec_k = _ScriptedDrafter(want[1:] + [0] * k), k
        block = engine.generate([list(prompt)], sp)[0]
        got = list(block.output)
        engine.release(block.seq_id)
        accepted = engine.stats.get("spec_accepted", 0) - a0
        # a block-path argmax that differs from the chain rejects that draft and emits its own token,
        # so equal outputs mean every real draft was accepted
        return got == want and accepted > 0 and engine.stats.get("spec_drafted", 0) > d0
    finally:
        engine.drafter, engine.spec_k, engine.spec_policy = saved
