"""The replica front over real listening servers (tiny random models on CPU): least-loaded routing
with sticky conversations, streaming pass-through, failover, and the prefill -> decode KV hand-off."""
import json
import socket
import threading
import time

import pytest
import torch

from mlxcel_b200.server.front import Backend, Balancer, create_front_app


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _serve(app, port):
    import uvicorn
    cfg = uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error")
    srv = uvicorn.Server(cfg)
    t = threading.Thread(target=srv.run, daemon=True)
    t.start()
    for _ in range(200):
        if srv.started:
            break
        time.sleep(0.05)
    return srv


def _model_server():
    from mlxcel_b200.config import preset
    from mlxcel_b200.engine import Engine, EngineConfig
    from mlxcel_b200.models.decoder import DecoderModel
    from mlxcel_b200.models.weights import random_weights
    from mlxcel_b200.server.app import ServerState, create_app
    from mlxcel_b200.server.worker import ModelWorker
    from mlxcel_b200.tokenizer import ByteTokenizer
    cfg = preset("tiny-llama")
    w = random_weights(cfg, seed=0, dtype=torch.float32, std=0.05)
    eng = Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=4, max_num_batched_tokens=256, num_blocks=128,
                                                         max_model_len=512, cuda_graphs=False))
    tk = ByteTokenizer(cfg.vocab_size)
    worker = ModelWorker(eng, tk, "tiny")
    port = _free_port()
    srv = _serve(create_app(ServerState(worker, tk, "tiny")), port)
    return srv, worker, f"http://127.0.0.1:{port}"


def test_balancer_prefers_idle_backends_and_keeps_conversations():
    t = [0.0]
    a, b = Backend("a"), Backend("b")
    lb = Balancer([a, b], cooldown_s=5.0, clock=lambda: t[0])
    first = lb.pick("replica", "conv")
    first.in_flight = 3
    assert lb.pick("replica") is (b if first is a else a)          # least loaded
    assert lb.pick("replica", "conv") is first                     # sticky
    lb.failed(first, "refused")
    other = b if first is a else a
    assert lb.pick("replica", "conv") is other                     # failed backend leaves the rotation
    t[0] = 6.0
    first.in_flight = 0
    other.in_flight = 1
    assert lb.pick("replica") is first                             # and returns after the cool-down
    with pytest.raises(LookupError):
        lb.pick("prefill")


def test_front_routes_streams_and_fails_over():
    import urllib.request
    s1, w1, u1 = _model_server()
    s2, w2, u2 = _model_server()
    dead = f"http://127.0.0.1:{_free_port()}"
    fport = _free_port()
    front = _serve(create_front_app(replicas=[u1, u2, dead], cooldown_s=60.0), fport)
    base = f"http://127.0.0.1:{fport}"
    try:
        def post(path, body, headers=None):
            req = urllib.request.Request(base + path, data=json.dumps(body).encode(),
                                         headers={"Content-Type": "application/json", **(headers or {})})
            return urllib.request.urlopen(req, timeout=120)

        served = set()
        for i in range(6):          # the dead backend is skipped after its first refusal
            with post("/v1/completions", {"prompt": "hello", "max_tokens": 3, "temperature": 0, "ignore_eos": True}) as r:
                assert json.loads(r.read())["usage"]["completion_tokens"] == 3
                served.add(r.headers["x-served-by"])
        assert served == {u1, u2}
        sticky = set()
        for i in range(4):
            with post("/v1/completions", {"prompt": "abc", "max_tokens": 2, "temperature": 0},
                      {"X-Conversation-Id": "c-9"}) as r:
                r.read()
                sticky.add(r.headers["x-served-by"])
        assert len(sticky) == 1
        with post("/v1/chat/completions", {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 4, "stream": True,
                                           "temperature": 0, "ignore_eos": True}) as r:
            lines = [l.decode().strip() for l in r if l.strip()]
        assert lines[-1] == "data: [DONE]" and len(lines) >= 3
        with urllib.request.urlopen(base + "/health", timeout=30) as r:
            h = json.loads(r.read())
        assert h["status"] == "ok" and [b["ok"] for b in h["backends"]].count(True) == 2
        with urllib.request.urlopen(base + "/front/stats", timeout=30) as r:
            st = json.loads(r.read())
        assert st["requests"] >= 11 and st["retries"] >= 1
    finally:
        for s in (front, s1, s2):
            s.should_exit = True
        w1.shutdown()
        w2.shutdown()


def test_front_hands_prompts_from_prefill_to_decode_servers():
    import urllib.request
    sp, wp, up = _model_server()
    sd, wd, ud = _model_server()
    fport = _free_port()
    front = _serve(create_front_app(prefill=[up], decode=[ud]), fport)
    base = f"http://127.0.0.1:{fport}"
    try:
        prompt = "the quick brown fox jumps over the lazy dog " * 2          # > 5 blocks of 16 byte-tokens
        body = {"prompt": prompt, "max_tokens": 6, "temperature": 0, "ignore_eos": True}
        req = urllib.request.Request(base + "/v1/completions", data=json.dumps(body).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=120) as r:
            out = json.loads(r.read())
            assert r.headers["x-served-by"] == ud
        # the decode server started from the imported blocks; the prefill server generated nothing for the client
        assert out["usage"]["prompt_tokens_details"]["cached_tokens"] >= 64
        direct = urllib.request.Request(ud + "/v1/completions", data=json.dumps(body).encode(),
                                        headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(direct, timeout=120) as r:
            assert json.loads(r.read())["choices"][0]["text"] == out["choices"][0]["text"]
        with urllib.request.urlopen(base + "/front/stats", timeout=30) as r:
            st = json.loads(r.read())
        assert st["handoffs"] == 1 and st["handoff_bytes"] > 0
    finally:
        for s in (front, sp, sd):
            s.should_exit = True
        wp.shutdown()
        wd.shutdown()


def test_front_verb_starts_and_stops_its_replicas():
    """`front --dp 2 -- -m preset:tiny-llama …` starts two CPU replicas, serves through them and takes
    them down with itself."""
    import os
    import signal
    import subprocess
    import sys
    import urllib.request
    fport, bport = _free_port(), _free_port()
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    proc = subprocess.Popen([sys.executable, "-m", "mlxcel_b200.cli", "front", "--dp", "2", "--no-pin-gpus",
                             "--base-port", str(bport), "--port", str(fport), "--start-timeout", "300", "--",
                             "-m", "preset:tiny-llama", "--device", "cpu", "--no-warmup", "-c", "256"], env=env)
    try:
        base = f"http://127.0.0.1:{fport}"
        ok = False
        for _ in range(600):
            if proc.poll() is not None:
                break
            try:
                with urllib.request.urlopen(base + "/health", timeout=2) as r:
                    ok = json.loads(r.read())["status"] == "ok"
                    break
            except OSError:
                time.sleep(0.5)
        assert ok, "front did not come up"
        served = set()
        for _ in range(4):
            req = urllib.request.Request(base + "/v1/completions", data=json.dumps({"prompt": "hi", "max_tokens": 2}).encode(),
                                         headers={"Content-Type": "application/json"})
            with urllib.request.urlopen(req, timeout=120) as r:
                r.read()
                served.add(r.headers["x-served-by"])
        assert len(served) == 2
    finally:
        proc.send_signal(signal.SIGTERM)
        try:
            proc.wait(timeout=60)
        except subprocess.TimeoutExpired:
            proc.kill()
    # the replicas went down with the front
    for i in range(2):
        with pytest.raises(OSError):
            urllib.request.urlopen(f"http://127.0.0.1:{bport + i}/health", timeout=2)
