"""Model provider and worker thread.

The HTTP layer (asyncio) never touches the engine: it posts requests to a thread-safe queue and
reads per-request event streams; one OS thread owns the engine and runs the scheduler loop —
the same split as the reference (tokio ⇄ std::mpsc ⇄ model-worker thread,
src/server/model_provider.rs:63-632, src/server/model_worker.rs:247-446). Events follow its
``GenerateEvent`` protocol: Admitted, Token, Done, Error.
"""
from __future__ import annotations

import asyncio
import queue
import threading
import time
import traceback
from dataclasses import dataclass, field

from ..engine import Engine, FinishReason, SamplingParams
from ..tokenizer import IncrementalDetokenizer
from .stop_matcher import StopMatcher

MAX_CONSECUTIVE_STEP_FAILURES = 8   # the reference's MAX_CONSECUTIVE_EVAL_FAILURES


@dataclass
class GenEvent:
    kind: str                 # admitted | token | done | error
    text: str = ""
    token_id: int | None = None
    logprob: float | None = None
    finish_reason: str | None = None
    usage: dict | None = None
    timings: dict | None = None
    error: str | None = None


@dataclass
class GenRequest:
    prompt_ids: list[int]
    params: SamplingParams
    loop: asyncio.AbstractEventLoop | None = None
    out: "asyncio.Queue | queue.Queue | None" = None
    constraint: object = None
    request_id: str = ""
    seq_id: int | None = None
    cancelled: bool = False
    detok: IncrementalDetokenizer | None = None
    stopper: StopMatcher | None = None
    t_submit: float = field(default_factory=time.perf_counter)
    n_emitted: int = 0


class ModelWorker:
    def __init__(self, engine: Engine, tokenizer, model_id: str = "model"):
        self.recent: dict[int, list[int]] = {}    # slot id -> tokens of its last finished sequence
        self.engine, self.tokenizer, self.model_id = engine, tokenizer, model_id
        self.inbox: "queue.Queue[GenRequest | tuple]" = queue.Queue()
        self.by_seq: dict[int, GenRequest] = {}
        self.thread = threading.Thread(target=self._run, name="model-worker", daemon=True)
        self.running = True
        self.failures = 0
        self.healthy = True
        self.counters = dict(requests=0, prompt_tokens=0, generated_tokens=0, errors=0, cancelled=0,
                             prompt_seconds=0.0, decode_seconds=0.0)
        self.thread.start()

    # ------------------------------------------------------------------ client side
    def submit(self, req: GenRequest) -> None:
        self.inbox.put(req)

    def cancel(self, req: GenRequest) -> None:
        req.cancelled = True
        self.inbox.put(("cancel", req))

    def run_exclusive(self, fn):
        """Run ``fn()`` on the worker thread between two engine steps (weight edits, cache resets) and
        return its result; exceptions propagate to the caller."""
        import concurrent.futures

        fut: concurrent.futures.Future = concurrent.futures.Future()
        self.inbox.put(("call", (fn, fut)))
        return fut.result()

    def shutdown(self) -> None:
        self.running = False
        self.inbox.put(("stop", None))
        self.thread.join(timeout=10)

    # ------------------------------------------------------------------ worker side
    def _emit(self, req: GenRequest, ev: GenEvent) -> None:
        if req.out is None:
            return
        if req.loop is not None:
            req.loop.call_soon_threadsafe(req.out.put_nowait, ev)
        else:
            req.out.put(ev)

    def _admit(self, req: GenRequest) -> None:
        if req.cancelled:
            return
        try:
            mask_fn = (lambda s, c=req.constraint: c.mask(s)) if req.constraint is not None else None
            sid = self.engine.add_request(req.prompt_ids, req.params, on_token=self._on_token, mask_fn=mask_fn,
                                          user_data=req)
        except Exception as e:
            self.counters["errors"] += 1
            self._emit(req, GenEvent("error", error=str(e)))
            return
        req.seq_id = sid
        req.detok = IncrementalDetokenizer(self.tokenizer, req.prompt_ids)
        req.stopper = StopMatcher(req.params.stop)
        self.by_seq[sid] = req
        self.counters["requests"] += 1
        self._emit(req, GenEvent("admitted"))

    def _on_token(self, seq, tok: int) -> None:
        req: GenRequest = seq.user_data
        if req is None or req.cancelled:
            return
        text = req.stopper.feed(req.detok.push(tok))
        lp = seq.logprobs[-1] if (seq.params.logprobs and seq.logprobs) else None
        req.n_emitted += 1
        self._emit(req, GenEvent("token", text=text, token_id=tok, logprob=lp))
        if req.stopper.stopped is not None:
            self.engine._finish(seq, FinishReason.STOP_SEQUENCE)
            self._finalize(seq)

    def _finalize(self, seq) -> None:
        req: GenRequest = seq.user_data
        if req is None or seq.seq_id not in self.by_seq:
            return
        del self.by_seq[seq.seq_id]
        tail = ""
        if req.stopper.stopped is None:
            tail = req.stopper.feed(req.detok.flush()) + req.stopper.flush()
        t_first = seq.first_token_time or seq.finish_time or time.perf_counter()
        t_end = seq.finish_time or time.perf_counter()
        n_prompt, n_out = len(seq.prompt), len(seq.output)
        prompt_ms = max(1e-6, (t_first - seq.arrival) * 1e3)
        pred_ms = max(1e-6, (t_end - t_first) * 1e3)
        timings = dict(cache_n=seq.num_cached, prompt_n=n_prompt - seq.num_cached, prompt_ms=prompt_ms,
                       prompt_per_second=(n_prompt - seq.num_cached) / prompt_ms * 1e3, predicted_n=n_out,
                       predicted_ms=pred_ms, predicted_per_second=n_out / pred_ms * 1e3)
        self.counters["prompt_tokens"] += n_prompt
        self.counters["generated_tokens"] += n_out
        self.counters["prompt_seconds"] += prompt_ms / 1e3
        self.counters["decode_seconds"] += pred_ms / 1e3
        reason = seq.finish_reason.value if seq.finish_reason else "stop"
        usage = dict(prompt_tokens=n_prompt, completion_tokens=n_out, total_tokens=n_prompt + n_out,
                     prompt_tokens_details=dict(cached_tokens=seq.num_cached))
        self._emit(req, GenEvent("done", text=tail, finish_reason=reason, usage=usage, timings=timings))
        # token stream of the slot's last occupant (what /slots/{id}?action=save writes out)
        self.recent[seq.seq_id % max(1, self.engine.ecfg.max_batch)] = list(seq.prompt) + list(seq.output)
        self.engine.release(seq.seq_id)

    def _run(self) -> None:
        eng = self.engine
        while self.running:
            block = not eng.has_work()
            try:
                item = self.inbox.get(timeout=0.2) if block else self.inbox.get_nowait()
            except queue.Empty:
                item = None
            while item is not None:
                if isinstance(item, tuple):
                    kind, req = item
                    if kind == "stop":
                        return
                    if kind == "call":
                        fn, fut = req
                        try:
                            fut.set_result(fn())
                        except BaseException as e:      # hand the failure to the waiting caller
                            fut.set_exception(e)
                    if kind == "cancel" and req.seq_id is not None and req.seq_id in self.by_seq:
                        eng.abort(req.seq_id)
                        self.by_seq.pop(req.seq_id, None)
                        eng.release(req.seq_id)
                        self.counters["cancelled"] += 1
                else:
                    self._admit(item)
                try:
                    item = self.inbox.get_nowait()
                except queue.Empty:
                    item = None
            if not eng.has_work():
                continue
            try:
                finished = eng.step()
                self.failures = 0
            except Exception as e:  # per-step failure: fail the affected rows, keep serving
                self.failures += 1
                self.counters["errors"] += 1
                msg = f"{type(e).__name__}: {e}"
                traceback.print_exc()
                for sid, req in list(self.by_seq.items()):
                    self._emit(req, GenEvent("error", error=msg))
                    eng.abort(sid)
                    eng.release(sid)
                self.by_seq.clear()
                if self.failures >= MAX_CONSECUTIVE_STEP_FAILURES:
                    self.healthy = False
                    self.running = False
                continue
            for s in finished:
                self._finalize(s)

    # ------------------------------------------------------------------ introspection
    def slots(self) -> list[dict]:
        out = []
        for i, s in enumerate(self.engine.running):
            out.append(dict(id=i, id_task=s.seq_id, is_processing=True, n_prompt=len(s.prompt),
                            n_decoded=len(s.output), state=s.status.value))
        return out
