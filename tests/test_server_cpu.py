"""HTTP API over a tiny random model on CPU with the byte tokenizer (no network, in-process client)."""
import json

import pytest
import torch
from fastapi.testclient import TestClient

from mlxcel_b200.config import preset
from mlxcel_b200.engine import Engine, EngineConfig
from mlxcel_b200.models.decoder import DecoderModel
from mlxcel_b200.models.weights import random_weights
from mlxcel_b200.server.app import ServerState, create_app
from mlxcel_b200.server.stop_matcher import StopMatcher
from mlxcel_b200.server.tool_calls import ToolCallStreamFilter, parse_tool_calls
from mlxcel_b200.server.worker import ModelWorker
from mlxcel_b200.tokenizer import ByteTokenizer


@pytest.fixture(scope="module")
def client():
    cfg = preset("tiny-llama")
    w = random_weights(cfg, seed=0, dtype=torch.float32, std=0.05)
    eng = Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=4, max_num_batched_tokens=256, num_blocks=128,
                                                         max_model_len=512, cuda_graphs=False))
    tk = ByteTokenizer(cfg.vocab_size)
    worker = ModelWorker(eng, tk, "tiny")
    with TestClient(create_app(ServerState(worker, tk, "tiny"))) as c:
        yield c
    worker.shutdown()


def test_health_models_props(client):
    assert client.get("/health").json()["status"] == "ok"
    assert client.get("/v1/models").json()["data"][0]["id"] == "tiny"
    assert client.get("/props").json()["total_slots"] == 4
    assert "llamacpp:prompt_tokens_total" in client.get("/metrics").text


def test_completion_and_determinism(client):
    body = {"prompt": "hello", "max_tokens": 8, "temperature": 0, "ignore_eos": True}
    a = client.post("/v1/completions", json=body).json()
    b = client.post("/v1/completions", json=body).json()
    assert a["usage"]["completion_tokens"] == 8 and a["choices"][0]["text"] == b["choices"][0]["text"]
    assert a["choices"][0]["finish_reason"] == "length"
    n = client.post("/completion", json={"prompt": "hello", "n_predict": 5, "temperature": 0, "ignore_eos": True}).json()
    assert n["tokens_predicted"] == 5 and n["stop_type"] == "limit" and "predicted_per_second" in n["timings"]


def test_chat_stream_and_usage(client):
    body = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 0, "stream": True,
            "ignore_eos": True, "stream_options": {"include_usage": True}}
    with client.stream("POST", "/v1/chat/completions", json=body) as r:
        lines = [l for l in r.iter_lines() if l.startswith("data: ")]
    assert lines[-1] == "data: [DONE]"
    chunks = [json.loads(l[6:]) for l in lines[:-1]]
    assert chunks[0]["choices"][0]["delta"]["role"] == "assistant"
    assert chunks[-1]["usage"]["completion_tokens"] == 6
    assert any(c["choices"] and c["choices"][0]["finish_reason"] == "length" for c in chunks)


def test_chat_nonstream_seeded_sampling(client):
    body = {"messages": [{"role": "system", "content": "s"}, {"role": "user", "content": "hi"}], "max_tokens": 6,
            "temperature": 1.0, "top_p": 0.9, "seed": 7, "ignore_eos": True}
    a = client.post("/v1/chat/completions", json=body).json()
    b = client.post("/v1/chat/completions", json=body).json()
    assert a["choices"][0]["message"]["content"] == b["choices"][0]["message"]["content"]
    assert a["usage"]["prompt_tokens_details"]["cached_tokens"] >= 0


def test_tokenize_template_messages_responses_embeddings(client):
    t = client.post("/tokenize", json={"content": "abc"}).json()["tokens"]
    assert client.post("/detokenize", json={"tokens": t}).json()["content"] == "abc"
    p = client.post("/apply-template", json={"messages": [{"role": "user", "content": "x"}]}).json()["prompt"]
    assert "<|im_start|>user" in p
    m = client.post("/v1/messages", json={"messages": [{"role": "user", "content": "x"}], "max_tokens": 4,
                                          "temperature": 0}).json()
    assert m["type"] == "message" and m["usage"]["output_tokens"] <= 4
    r = client.post("/v1/responses", json={"input": "x", "max_output_tokens": 4, "temperature": 0}).json()
    assert r["status"] == "completed" and client.get("/v1/responses/" + r["id"]).json()["id"] == r["id"]
    e = client.post("/v1/embeddings", json={"input": ["a", "bb"]}).json()
    assert len(e["data"]) == 2 and abs(sum(x * x for x in e["data"][0]["embedding"]) - 1.0) < 1e-3
    assert client.get("/v1/cache/stats").json()["num_blocks"] == 128


def test_stop_matcher_and_tool_parsing():
    sm = StopMatcher(["END", "\n\n"])
    out = sm.feed("abc E") + sm.feed("N") + sm.feed("D tail")
    assert out == "abc " and sm.stopped == "END"
    content, calls = parse_tool_calls('ok <tool_call>{"name": "f", "arguments": {"a": 1}}</tool_call>')
    assert content == "ok" and calls[0].name == "f" and json.loads(calls[0].arguments) == {"a": 1}
    _, calls = parse_tool_calls('{"name": "g", "parameters": {"x": 2}}')
    assert calls[0].name == "g"
    _, calls = parse_tool_calls('[TOOL_CALLS] [{"name": "h", "arguments": {}}]')
    assert calls[0].name == "h"
    f = ToolCallStreamFilter()
    vis, got = "", []
    for piece in ["he", "llo <tool", "_call>{\"name\": \"f\", \"argum", "ents\": {}}</tool_call> bye"]:
        v, c = f.feed(piece)
        vis += v
        got += c
    v, c = f.flush()
    assert (vis + v).replace("  ", " ").strip() == "hello bye" and got[0].name == "f"
