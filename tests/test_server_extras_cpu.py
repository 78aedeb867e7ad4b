"""Server features around the core routes, on a tiny random model on CPU: CORS preflights, the
X-Priority lane, thinking budgets from requests and live settings, the Responses store (TTL,
background, cancel, compaction), resumable stream sessions, in-flight control, histograms."""
import json
import time

import pytest
import torch
from fastapi.testclient import TestClient

from mlxcel_b200.config import preset
from mlxcel_b200.engine import Engine, EngineConfig
from mlxcel_b200.models.decoder import DecoderModel
from mlxcel_b200.models.weights import random_weights
from mlxcel_b200.server.app import ServerState, create_app
from mlxcel_b200.server.extras import ResponsesStore, compact_messages
from mlxcel_b200.server.worker import ModelWorker
from mlxcel_b200.tokenizer import ByteTokenizer


class ThinkTokenizer(ByteTokenizer):
    """Byte tokenizer that declares two of its ids as the reasoning-block markers."""
    think_open, think_close = 300, 301


@pytest.fixture(scope="module")
def server():
    cfg = preset("tiny-llama")
    w = random_weights(cfg, seed=0, dtype=torch.float32, std=0.05)
    eng = Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=4, max_num_batched_tokens=256, num_blocks=128,
                                                         max_model_len=512, cuda_graphs=False))
    tk = ThinkTokenizer(cfg.vocab_size)
    worker = ModelWorker(eng, tk, "tiny")
    state = ServerState(worker, tk, "tiny", api_keys={"k1"})
    state.settings_enabled = True
    state.cors_origins = ["https://app.example"]
    with TestClient(create_app(state)) as c:
        c.headers.update({"Authorization": "Bearer k1"})
        yield c, state
    worker.shutdown()


def test_cors_preflight_is_answered_before_authentication(server):
    c, state = server
    r = c.options("/v1/chat/completions", headers={"Origin": "https://app.example", "Authorization": "",
                                                   "Access-Control-Request-Method": "POST",
                                                   "Access-Control-Request-Headers": "content-type, authorization"})
    assert r.status_code == 204 and r.headers["access-control-allow-origin"] == "https://app.example"
    assert "authorization" in r.headers["access-control-allow-headers"]
    r = c.options("/v1/chat/completions", headers={"Origin": "https://evil.example",
                                                   "Access-Control-Request-Method": "POST"})
    assert r.status_code == 403 and "access-control-allow-origin" not in r.headers
    ok = c.get("/v1/models", headers={"Origin": "https://app.example"})
    assert ok.headers["access-control-allow-origin"] == "https://app.example"
    other = c.get("/v1/models", headers={"Origin": "https://evil.example"})
    assert other.status_code == 200 and "access-control-allow-origin" not in other.headers


def test_thinking_budget_request_validation_and_enforcement(server):
    c, state = server
    body = {"prompt": [65, 66, 300], "max_tokens": 8, "temperature": 0, "ignore_eos": True}
    assert c.post("/v1/completions", json={**body, "thinking_budget_tokens": -2}).status_code == 400
    assert c.post("/v1/completions", json={**body, "thinking_budget_tokens": 50}).status_code == 400   # > max_tokens
    free = c.post("/completion", json={"prompt": [65, 66, 300], "n_predict": 8, "temperature": 0, "ignore_eos": True}).json()
    capped = c.post("/completion", json={"prompt": [65, 66, 300], "n_predict": 8, "temperature": 0, "ignore_eos": True,
                                         "thinking_budget_tokens": 3}).json()
    assert capped["tokens_predicted"] == 8 and capped["timings"]["thinking_forced"] == 1
    assert "thinking_forced" not in free["timings"]
    # a live default applies to requests that give none; -1 on the request switches it off again
    assert c.post("/v1/settings", json={"thinking_budget": 2}).json()["thinking_budget"] == 2
    d = c.post("/completion", json={"prompt": [65, 66, 300], "n_predict": 8, "temperature": 0, "ignore_eos": True}).json()
    assert d["timings"]["thinking_forced"] == 1
    off = c.post("/completion", json={"prompt": [65, 66, 300], "n_predict": 8, "temperature": 0, "ignore_eos": True,
                                      "thinking_budget_tokens": -1}).json()
    assert "thinking_forced" not in off["timings"]
    c.post("/v1/settings", json={"thinking_budget": None})


def test_live_settings_need_opt_in_and_reject_unknown_keys(server):
    c, state = server
    s = c.get("/v1/settings").json()
    assert s["max_queue_depth"] == 4096 and s["log_redact"] is True
    assert c.post("/v1/settings", json={"nonsense": 1}).status_code == 400
    r = c.post("/v1/settings", json={"default_max_tokens": 3, "log_verbosity": 2, "log_format": "json"}).json()
    assert r["default_max_tokens"] == 3 and r["log_format"] == "json"
    out = c.post("/v1/completions", json={"prompt": "hello", "temperature": 0, "ignore_eos": True}).json()
    assert out["usage"]["completion_tokens"] == 3          # the live default replaced the route's
    c.post("/v1/settings", json={"default_max_tokens": None, "log_verbosity": 1, "log_format": "text"})
    state.settings_enabled = False
    assert c.get("/v1/settings").status_code == 404
    state.settings_enabled = True


def test_priority_header_reaches_the_engine_queue(server):
    c, state = server
    seen = []
    eng = state.worker.engine
    orig = eng.add_request

    def spy(prompt, params=None, **kw):
        seen.append(params.priority)
        return orig(prompt, params, **kw)
    eng.add_request = spy
    try:
        c.post("/v1/completions", json={"prompt": "a", "max_tokens": 1}, headers={"X-Priority": "5"})
        c.post("/v1/completions", json={"prompt": "a", "max_tokens": 1})
    finally:
        eng.add_request = orig
    assert seen == [5, 0]


def test_responses_background_cancel_ttl_and_compaction(server):
    c, state = server
    r = c.post("/v1/responses", json={"input": "hello", "max_output_tokens": 4, "temperature": 0}).json()
    assert r["status"] == "completed" and c.get(f"/v1/responses/{r['id']}").json()["id"] == r["id"]
    bg = c.post("/v1/responses", json={"input": "tell me more", "max_output_tokens": 400, "temperature": 0,
                                       "background": True, "ignore_eos": True}).json()
    assert bg["status"] in ("queued", "in_progress") and bg["background"] is True
    cancelled = c.post(f"/v1/responses/{bg['id']}/cancel").json()
    assert cancelled["status"] == "cancelled"
    for _ in range(100):                       # the engine row is gone shortly after
        if not state.worker.by_seq:
            break
        time.sleep(0.05)
    assert not state.worker.by_seq
    assert c.get(f"/v1/responses/{bg['id']}").json()["status"] == "cancelled"
    done = c.post("/v1/responses", json={"input": "short", "max_output_tokens": 3, "temperature": 0,
                                         "background": True}).json()
    for _ in range(200):
        cur = c.get(f"/v1/responses/{done['id']}").json()
        if cur["status"] == "completed":
            break
        time.sleep(0.05)
    assert cur["status"] == "completed" and cur["usage"]["output_tokens"] <= 3
    assert c.post("/v1/responses/nope/cancel").status_code == 404
    # compaction keeps the system message and the latest turns
    msgs = [{"role": "system", "content": "s"}] + [{"role": "user" if i % 2 == 0 else "assistant", "content": "x" * 40}
                                                      for i in range(10)]
    out = c.post("/v1/responses/compact", json={"input": msgs, "max_input_tokens": 150, "keep_last": 2}).json()
    assert out["dropped_messages"] > 0 and out["input"][0]["role"] == "system" and len(out["input"]) >= 3
    assert out["input_tokens_after"] <= max(150, out["input_tokens_before"] - 1)
    # the store itself: TTL and LRU with an injected clock
    t = [0.0]
    st = ResponsesStore(capacity=2, ttl_s=10, clock=lambda: t[0])
    st["a"], st["b"] = {"v": 1}, {"v": 2}
    assert st.get("a")["v"] == 1
    st["c"] = {"v": 3}                          # evicts the least recently used ("b")
    assert st.get("b") is None and st.get("a") is not None
    t[0] = 11.0
    assert st.get("a") is None and st.stats["expired"] >= 1
    kept, dropped = compact_messages([{"role": "user", "content": "a"}] * 5, lambda ms: 10 * len(ms), 25, keep_last=1)
    assert dropped == 3 and len(kept) == 2


def test_stream_session_can_be_resumed_and_controlled(server):
    c, state = server
    body = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 0, "stream": True,
            "ignore_eos": True}
    with c.stream("POST", "/v1/chat/completions", json=body, headers={"X-Conversation-Id": "conv-1"}) as r:
        assert r.headers["x-conversation-id"] == "conv-1"
        raw = list(r.iter_lines())
    ids = [int(l[4:]) for l in raw if l.startswith("id: ")]
    data = [l for l in raw if l.startswith("data: ")]
    assert ids == list(range(len(ids))) and len(ids) == len(data) and data[-1] == "data: [DONE]"
    info = c.get("/v1/streams/lookup", params={"conversation_id": "conv-1"}).json()
    assert info["done"] is True and info["next_event_id"] >= len(ids)
    with c.stream("GET", "/v1/stream", params={"conversation_id": "conv-1", "last_event_id": ids[2]}) as r:
        again = list(r.iter_lines())
    assert [l for l in again if l.startswith("data: ")] == data[3:]
    assert c.get("/v1/stream", params={"conversation_id": "nope"}).status_code == 404
    assert c.post("/v1/chat/completions/control", json={"id": "chatcmpl-none", "action": "cancel"}).status_code == 404
    assert c.post("/v1/chat/completions/control", json={"id": "x", "action": "explode"}).status_code == 400


def test_metrics_have_histograms(server):
    c, state = server
    c.post("/v1/completions", json={"prompt": "hello", "max_tokens": 4, "temperature": 0})
    text = c.get("/metrics").text
    assert 'mlxcel_request_ttft_seconds_bucket{le="+Inf"}' in text and "mlxcel_request_ttft_seconds_count" in text
    assert "mlxcel_spec_decode_rounds_total" in text and "mlxcel_responses_store_entries" in text


def test_idle_worker_unloads_the_model_and_the_next_request_loads_it_again():
    """--sleep-idle-seconds: the engine is dropped after the idle window, read-only routes answer from
    the frozen counters without waking it, and the next request gets the same greedy text."""
    import queue as _q
    import time as _t

    import torch as _torch

    from mlxcel_b200.config import preset
    from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams
    from mlxcel_b200.models.decoder import DecoderModel
    from mlxcel_b200.models.weights import random_weights
    from mlxcel_b200.server.metrics import render_metrics
    from mlxcel_b200.server.worker import GenRequest, ModelWorker
    from mlxcel_b200.tokenizer import ByteTokenizer
    cfg = preset("tiny-llama")
    built = []

    def factory():
        w = random_weights(cfg, seed=0, dtype=_torch.float32, std=0.05)
        built.append(1)
        return Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=2, max_num_batched_tokens=64, num_blocks=32,
                                                              max_model_len=128, cuda_graphs=False))
    tk = ByteTokenizer(cfg.vocab_size)
    worker = ModelWorker(factory(), tk, "tiny", engine_factory=factory, sleep_idle=0.4)

    def ask():
        out = _q.Queue()
        worker.submit(GenRequest(prompt_ids=[5, 6, 7, 8], params=SamplingParams(max_tokens=5, ignore_eos=True), out=out))
        text = ""
        while True:
            ev = out.get(timeout=60)
            if ev.kind == "token":
                text += ev.text
            if ev.kind in ("done", "error"):
                assert ev.kind == "done"
                return text + (ev.text or "")
    try:
        first = ask()
        deadline = _t.monotonic() + 20
        while not worker.sleeping and _t.monotonic() < deadline:
            _t.sleep(0.05)
        assert worker.sleeping and worker._engine is None
        v = worker.view()
        assert v.ecfg.max_batch == 2 and v.bm.stats()["num_blocks"] == 32 and worker.slots() == []
        from types import SimpleNamespace
        assert "mlxcel_model_sleeping 1" in render_metrics(SimpleNamespace(worker=worker, hist=None))
        assert worker.sleeping and len(built) == 1                 # looking did not wake it
        assert ask() == first
        assert not worker.sleeping and len(built) == 2 and worker.counters["wakes"] == 1
    finally:
        worker.shutdown()
