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
    media: list | None = None          # decoded images, one per placeholder token of prompt_ids


class ModelWorker:
    def __init__(self, engine: Engine, tokenizer, model_id: str = "model", control=None, start: bool = True,
                 hang_timeout: float = 0.0, failfast: bool = False, engine_factory=None, sleep_idle: float = 0.0):
        """``control``: a :class:`mlxcel_b200.parallel.control.ControlPlane` when several processes run
        the engine together. On the leader the worker thread broadcasts what it drained from its inbox
        before every step; on the other ranks :meth:`follow` replaces the thread and applies the
        leader's descriptors. ``hang_timeout`` > 0: a step that has not returned after that many
        seconds fails the requests in flight and marks the worker unhealthy (the reference's decode
        hang timeout, src/server/model_provider.rs:3002-3036). ``failfast``: an exception that escapes
        the worker loop ends the process instead of leaving a server that accepts requests and never
        answers (src/worker_failfast.rs). ``sleep_idle`` > 0 with an ``engine_factory``: after that
        many seconds without a request the engine (weights, KV pool, graphs) is dropped and its device
        memory returned; the next request builds it again through the factory before it is admitted
        (``--sleep-idle-seconds``, src/server/model_worker.rs:259-288). ``sleeping`` is what `/props`
        reports as ``is_sleeping``."""
        self.vision = None                  # multimodal.VisionLanguage of a vision-language checkpoint
        self.engine_factory, self.sleep_idle = engine_factory, float(sleep_idle)
        self.sleeping = False
        self._wake_lock = threading.Lock()
        self._last_activity = time.monotonic()
        self.sleep_snapshot: dict = {}
        self.recent: dict[int, list[int]] = {}    # slot id -> tokens of its last finished sequence
        self._engine, self.tokenizer, self.model_id = engine, tokenizer, model_id
        self.control = control
        self.hang_timeout, self.failfast = hang_timeout, failfast
        self._step_started: float | None = None
        self._by_request: dict[str, GenRequest] = {}
        self.named_calls = {"cache_reset": self._call_cache_reset}
        self.inbox: "queue.Queue[GenRequest | tuple]" = queue.Queue()
        self.by_seq: dict[int, GenRequest] = {}
        self.thread = threading.Thread(target=self._run, name="model-worker", daemon=True)
        self.running = True
        self.failures = 0
        self.healthy = True
        self.counters = dict(requests=0, prompt_tokens=0, generated_tokens=0, errors=0, cancelled=0,
                             prompt_seconds=0.0, decode_seconds=0.0, hangs=0)
        if hang_timeout > 0:
            threading.Thread(target=self._watchdog, name="step-watchdog", daemon=True).start()
        if start and (control is None or control.is_leader):
            self.thread.start()

    # ------------------------------------------------------------------ idle sleep
    @property
    def engine(self) -> Engine:
        """The live engine; touching it while the worker sleeps loads the model again."""
        if self._engine is None:
            self._wake()
        return self._engine

    @engine.setter
    def engine(self, value) -> None:
        self._engine = value

    def view(self):
        """What read-only routes (`/props`, `/metrics`, cache statistics) look at: the live engine, or
        while the worker sleeps a frozen copy of its last counters so that a scrape does not load the
        model."""
        eng = self._engine
        if eng is not None:
            return eng
        from types import SimpleNamespace
        snap = self.sleep_snapshot
        return SimpleNamespace(bm=SimpleNamespace(stats=lambda: dict(snap["kv"])), stats=snap["stats"], running=[],
                               waiting=[], ecfg=snap["ecfg"], spec_policy=None, drafter=None)

    def _sleep(self) -> None:
        with self._wake_lock:
            if self._engine is None or self._engine.has_work():
                return
            eng = self._engine
            self.sleep_snapshot = dict(kv=dict(eng.bm.stats()), stats=dict(eng.stats), slept_at=time.time(),
                                       ecfg=eng.ecfg)
            self._engine = None
            self.sleeping = True
            self.recent.clear()
            del eng
            import gc
            gc.collect()
            import torch
            if torch.cuda.is_available():
                torch.cuda.empty_cache()
            self.counters["sleeps"] = self.counters.get("sleeps", 0) + 1

    def _wake(self) -> None:
        with self._wake_lock:
            if self._engine is not None:
                return
            t0 = time.monotonic()
            self._engine = self.engine_factory()
            self.sleeping = False
            self._last_activity = time.monotonic()
            self.counters["wakes"] = self.counters.get("wakes", 0) + 1
            self.counters["wake_seconds"] = self.counters.get("wake_seconds", 0.0) + (time.monotonic() - t0)

    # ------------------------------------------------------------------ client side
    def submit(self, req: GenRequest) -> None:
        self.inbox.put(req)

    def cancel(self, req: GenRequest) -> None:
        # With several processes the flag flips when the cancellation's descriptor is applied, on every
        # rank at the same step: flipping it here would let this rank skip stop matching for tokens
        # the other ranks still process.
        if self.control is None:
            req.cancelled = True
        self.inbox.put(("cancel", req))

    def run_exclusive(self, fn, name: str | None = None, args: tuple = ()):
        """Run ``fn()`` on the worker thread between two engine steps (weight edits, cache resets) and
        return its result; exceptions propagate to the caller. With a control plane only calls
        registered by ``name`` in ``named_calls`` can run (every rank has to make the same call)."""
        import concurrent.futures

        fut: concurrent.futures.Future = concurrent.futures.Future()
        self.inbox.put(("call", (fn, fut, name, tuple(args))))
        return fut.result()

    def _call_cache_reset(self):
        return self.engine.bm.reset_prefix_cache()

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
            mm = {}
            if req.media:
                # tower + connector run here, on the engine's thread and stream, between two steps
                if self.vision is None:
                    raise ValueError("this model takes no image input")
                if self.control is not None:
                    raise ValueError("image input needs a single-process server")
                req.prompt_ids, mm = self.vision.prepare(req.prompt_ids, req.media)
                req.media = None
            sid = self.engine.add_request(req.prompt_ids, req.params, on_token=self._on_token, mask_fn=mask_fn,
                                          user_data=req, **mm)
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
        self._by_request.pop(req.request_id, None)
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
        if self.engine.drafter is not None:
            # llama-server's speculative fields (docs/speculative-acceptance.md:189-238)
            timings.update(draft_n=seq.draft_n, draft_n_accepted=seq.draft_n_accepted,
                           draft_kind=type(self.engine.drafter).__name__)
        if seq.think_forced:
            timings["thinking_forced"] = seq.think_forced
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

    # ------------------------------------------------------------------ loop
    def _drain(self, block: bool) -> list:
        items = []
        try:
            items.append(self.inbox.get(timeout=0.2) if block else self.inbox.get_nowait())
            while True:
                items.append(self.inbox.get_nowait())
        except queue.Empty:
            pass
        return items

    def _cancel(self, req: GenRequest) -> None:
        eng = self.engine
        if req.seq_id is not None and req.seq_id in self.by_seq:
            eng.abort(req.seq_id)
            self.by_seq.pop(req.seq_id, None)
            eng.release(req.seq_id)
            self.counters["cancelled"] += 1
        self._by_request.pop(req.request_id, None)

    def _apply_local(self, items: list) -> bool:
        """Single-process path: apply inbox items directly. Returns False on a stop request."""
        for item in items:
            if isinstance(item, tuple):
                kind, req = item
                if kind == "stop":
                    return False
                if kind == "call":
                    fn, fut = req[0], req[1]
                    try:
                        fut.set_result(fn())
                    except BaseException as e:      # hand the failure to the waiting caller
                        fut.set_exception(e)
                if kind == "cancel":
                    self._cancel(req)
            else:
                self._admit(item)
        return True

    def _lead(self, items: list) -> bool:
        """Leader of a multi-process engine: what was drained becomes this step's descriptor; every
        rank (this one included) then applies the descriptor, so all engines see the same events in
        the same order."""
        from ..parallel.control import StepDescriptor, engine_digest, params_to_wire

        d = StepDescriptor(digest=engine_digest(self.engine))
        futures = []
        for item in items:
            if isinstance(item, tuple):
                kind, req = item
                if kind == "stop":
                    d.stop = True
                elif kind == "cancel":
                    d.cancels.append(req.request_id)
                elif kind == "call":
                    fn, fut, name, args = req
                    if name is None or name not in self.named_calls:
                        fut.set_exception(RuntimeError("this operation is not available while several processes "
                                                       "serve the model together"))
                    else:
                        d.calls.append((name, args))
                        futures.append(fut)
            else:
                if item.cancelled:
                    continue
                self._by_request[item.request_id] = item
                spec = getattr(item.constraint, "spec", None) if item.constraint is not None else None
                d.requests.append(dict(request_id=item.request_id, prompt_ids=list(item.prompt_ids),
                                       params=params_to_wire(item.params), constraint=spec))
        d = self.control.exchange(d)
        return self._apply_descriptor(d, futures)

    def _apply_descriptor(self, d, futures=()) -> bool:
        for r in d.requests:
            req = self._by_request.get(r["request_id"])
            if req is None:                        # follower: a request without a client side
                from ..parallel.control import params_from_wire
                c = None
                if r.get("constraint"):
                    from .structured import Constraint
                    c = Constraint(self.tokenizer, **r["constraint"])
                req = GenRequest(prompt_ids=r["prompt_ids"], params=params_from_wire(r["params"]),
                                 constraint=c, request_id=r["request_id"])
                self._by_request[req.request_id] = req
            self._admit(req)
        for rid in d.cancels:
            req = self._by_request.get(rid)
            if req is not None:
                req.cancelled = True
                self._cancel(req)
        results = []
        for name, args in d.calls:
            try:
                results.append((True, self.named_calls[name](*args)))
            except BaseException as e:
                results.append((False, e))
        for fut, (ok, val) in zip(futures, results):
            fut.set_result(val) if ok else fut.set_exception(val)
        return not d.stop

    def _step_once(self) -> None:
        eng = self.engine
        try:
            self._step_started = time.monotonic()
            finished = eng.step()
            self._step_started = None
            self.failures = 0
        except Exception as e:  # per-step failure: fail the affected rows, keep serving
            self._step_started = None
            self.failures += 1
            self.counters["errors"] += 1
            msg = f"{type(e).__name__}: {e}"
            traceback.print_exc()
            self._fail_all(msg)
            if self.failures >= MAX_CONSECUTIVE_STEP_FAILURES:
                self.healthy = False
                self.running = False
            return
        for s in finished:
            self._finalize(s)

    def _fail_all(self, msg: str) -> None:
        eng = self.engine
        for sid, req in list(self.by_seq.items()):
            self._emit(req, GenEvent("error", error=msg))
            self._by_request.pop(req.request_id, None)
            try:
                eng.abort(sid)
                eng.release(sid)
            except Exception:
                pass
        self.by_seq.clear()

    def _watchdog(self) -> None:
        """Decode-hang timeout: a step that does not return cannot be interrupted from here, but the
        clients waiting on it can be answered and the server can report itself unhealthy."""
        while self.running:
            time.sleep(min(1.0, self.hang_timeout / 4))
            t0 = self._step_started
            if t0 is not None and time.monotonic() - t0 > self.hang_timeout and self.healthy:
                self.healthy = False
                self.counters["hangs"] += 1
                for req in list(self.by_seq.values()):
                    self._emit(req, GenEvent("error", error=f"engine step exceeded {self.hang_timeout:.0f} s"))

    def _run(self) -> None:
        try:
            self._loop()
        except BaseException:
            traceback.print_exc()
            self.healthy = False
            if self.failfast:
                import os
                os._exit(70)
            raise

    def _loop(self) -> None:
        can_sleep = self.sleep_idle > 0 and self.engine_factory is not None and self.control is None
        # data-parallel ranks that share experts tick together: this worker steps even without work of
        # its own (its engine then runs a null forward for the others), and idles briefly when no rank
        # has any
        dp = self._engine is not None and getattr(self._engine, "dp_lockstep", False)
        can_sleep = can_sleep and not dp
        while self.running:
            eng = self._engine
            items = self._drain(block=not dp and (eng is None or not eng.has_work()))
            if items:
                self._last_activity = time.monotonic()
                if eng is None and not all(isinstance(i, tuple) and i[0] == "stop" for i in items):
                    self._wake()
            elif can_sleep and eng is not None and not eng.has_work() and \
                    time.monotonic() - self._last_activity > self.sleep_idle:
                self._sleep()
                continue
            if self.control is not None:
                if not self._lead(items):
                    return
            elif not self._apply_local(items):
                return
            eng = self._engine
            if dp:
                self._step_once()
                if not eng.dp_active:
                    time.sleep(0.002)
            elif eng is not None and eng.has_work():
                self._step_once()
                self._last_activity = time.monotonic()

    def follow(self) -> None:
        """Executor loop of a non-leader rank: apply the leader's descriptors, check lockstep, step.
        Returns when the leader broadcasts a stop (or raises when lockstep is lost)."""
        eng = self.engine
        while self.running:
            d = self.control.exchange(None)
            self.control.check_digest(d, eng)
            if not self._apply_descriptor(d):
                return
            if eng.has_work():
                self._step_once()

    # ------------------------------------------------------------------ introspection
    def slots(self) -> list[dict]:
        out = []
        if self._engine is None:
            return out
        for i, s in enumerate(self.engine.running):
            out.append(dict(id=i, id_task=s.seq_id, is_processing=True, n_prompt=len(s.prompt),
                            n_decoded=len(s.output), state=s.status.value))
        return out
