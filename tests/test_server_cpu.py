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


def test_extra_routes_webui_rerank_lora_stubs(client, tmp_path):
    r = client.get("/")
    assert r.status_code == 200 and "<title>mlxcel_b200</title>" in r.text and "/v1/chat/completions" in r.text
    assert client.get("/ui").status_code == 200
    assert client.get("/tools").status_code == 403 and client.post("/cors-proxy").status_code == 403
    pol = client.get("/v1/internal/mtp-policy").json()
    assert pol["drafter"] is None and pol["drafted"] == 0
    rr = client.post("/v1/rerank", json={"query": "abc", "documents": ["abc", "zzzzzz", "abd"], "top_n": 2,
                                         "return_documents": True}).json()
    assert len(rr["results"]) == 2 and rr["results"][0]["index"] == 0        # identical text ranks first
    assert rr["results"][0]["relevance_score"] > rr["results"][1]["relevance_score"]
    assert rr["results"][0]["document"]["text"] == "abc"
    assert client.post("/v1/rerank", json={"query": "", "documents": []}).status_code == 400
    # LoRA: not enabled on this app -> 400; enabled -> attach, rescale, list
    assert client.get("/lora-adapters").json() == []
    assert client.post("/lora-adapters", json=[{"id": 0, "scale": 1.0}]).status_code == 400


def test_lora_routes_change_weights_between_steps(tmp_path):
    import json as _json

    from safetensors.torch import save_file

    from mlxcel_b200.lora import LoraManager
    cfg = preset("tiny-llama")
    cfg.vocab_size = 300
    w = random_weights(cfg, seed=5, dtype=torch.float32)
    tk = ByteTokenizer(cfg.vocab_size)
    eng = Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=2, num_blocks=64, max_model_len=128, cuda_graphs=False))
    worker = ModelWorker(eng, tk, "tiny")
    state = ServerState(worker, tk, "tiny")
    state.lora = LoraManager(cfg, w)
    d = tmp_path / "ad"
    d.mkdir()
    g = torch.Generator().manual_seed(3)
    save_file({"model.layers.0.self_attn.o_proj.lora_a": torch.randn(cfg.num_attention_heads * cfg.head_dim, 2, generator=g),
               "model.layers.0.self_attn.o_proj.lora_b": torch.randn(2, cfg.hidden_size, generator=g)},
              str(d / "adapters.safetensors"))
    (d / "adapter_config.json").write_text(_json.dumps({"lora_parameters": {"rank": 2, "scale": 1.0}}))
    before = w.layers[0].wo.clone()
    with TestClient(create_app(state)) as c:
        out = c.post("/lora-adapters", json=[{"id": 0, "path": str(d), "scale": 0.5}]).json()
        assert out == [{"id": 0, "path": str(d), "scale": 0.5}]
        assert not torch.allclose(w.layers[0].wo, before)
        assert c.get("/lora-adapters").json()[0]["scale"] == 0.5
        c.post("/lora-adapters", json=[{"id": 0, "scale": 0.0}])
        assert torch.allclose(w.layers[0].wo, before, atol=1e-5)
        assert c.post("/lora-adapters", json=[{"id": 9, "scale": 1.0}]).status_code == 400
    worker.shutdown()


def test_slot_save_restore_erase(tmp_path):
    """POST /slots/{id}?action=save|restore|erase: the token stream of a finished request is written
    out, read back (its blocks return to the prefix cache: the same prompt then hits it) and dropped."""
    cfg = preset("tiny-llama")
    w = random_weights(cfg, seed=0, dtype=torch.float32, std=0.05)
    eng = Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=4, max_num_batched_tokens=256, num_blocks=128,
                                                         max_model_len=512, cuda_graphs=False))
    tk = ByteTokenizer(cfg.vocab_size)
    worker = ModelWorker(eng, tk, "tiny")
    state = ServerState(worker, tk, "tiny")
    with TestClient(create_app(state)) as c:
        prompt = "The quick brown fox jumps over the lazy dog, again and again and again."
        r = c.post("/completion", json=dict(prompt=prompt, n_predict=4, temperature=0)).json()
        slot = next(iter(worker.recent))
        assert c.post(f"/slots/{slot}?action=save", json=dict(filename="a.bin")).status_code == 501
        state.slot_save_path = str(tmp_path)
        assert c.post(f"/slots/{slot}?action=save", json=dict(filename="../a.bin")).status_code == 400
        sv = c.post(f"/slots/{slot}?action=save", json=dict(filename="a.bin")).json()
        assert sv["n_saved"] == r["tokens_evaluated"] + r["tokens_predicted"] and (tmp_path / "a.bin").exists()
        er = c.post(f"/slots/{slot}?action=erase").json()
        assert er["n_erased"] > 0
        cold = c.post("/completion", json=dict(prompt=prompt, n_predict=1, temperature=0)).json()
        assert cold["timings"]["cache_n"] == 0
        c.post(f"/slots/{slot}?action=erase")
        rs = c.post(f"/slots/{slot}?action=restore", json=dict(filename="a.bin")).json()
        assert rs["n_restored"] == sv["n_saved"]
        warm = c.post("/completion", json=dict(prompt=prompt, n_predict=1, temperature=0)).json()
        assert warm["timings"]["cache_n"] >= 64
        assert c.post(f"/slots/{slot}?action=restore", json=dict(filename="missing.bin")).status_code == 404
        assert c.post(f"/slots/{slot}?action=bogus").status_code == 400
    worker.shutdown()


def test_kv_handoff_routes_between_two_servers():
    """A prefill-role server exports a prompt's KV blocks, a decode-role server imports them and then
    answers the same prompt from its cache with the same text."""
    cfg = preset("tiny-llama")
    w = random_weights(cfg, seed=0, dtype=torch.float32, std=0.05)
    tk = ByteTokenizer(cfg.vocab_size)

    def server():
        eng = Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=4, max_num_batched_tokens=256, num_blocks=128,
                                                             max_model_len=512, cuda_graphs=False))
        worker = ModelWorker(eng, tk, "tiny")
        return worker, TestClient(create_app(ServerState(worker, tk, "tiny")))

    (wa, ca), (wb, cb) = server(), server()
    prompt = "In a hole in the ground there lived a hobbit. Not a nasty, dirty, wet hole."
    with ca, cb:
        want = ca.post("/completion", json=dict(prompt=prompt, n_predict=5, temperature=0)).json()["content"]
        r = ca.post("/v1/internal/kv/export", json=dict(prompt=prompt))
        assert r.status_code == 200 and r.content[:5] == b"MXKV1"
        assert cb.post("/v1/internal/kv/import", content=r.content).json()["cached_tokens"] >= 64
        got = cb.post("/completion", json=dict(prompt=prompt, n_predict=5, temperature=0)).json()
        assert got["content"] == want and got["timings"]["cache_n"] >= 64
        assert cb.post("/v1/internal/kv/import", content=b"garbage").status_code == 400
    wa.shutdown()
    wb.shutdown()


def test_secondary_routes(client):
    """Routes beside the main completion paths: token counting, stored responses, cache reset, alias
    paths, fill-in-the-middle on a tokenizer without FIM tokens."""
    msgs = [{"role": "user", "content": "count me"}]
    n = client.post("/v1/messages/count_tokens", json={"messages": msgs}).json()["input_tokens"]
    assert n > len("count me")
    m = client.post("/v1/responses/input_tokens", json={"input": "count me"}).json()["input_tokens"]
    assert m > 0
    r = client.post("/v1/responses", json={"input": "hi", "max_output_tokens": 4, "temperature": 0}).json()
    got = client.get(f"/v1/responses/{r['id']}")
    assert got.status_code == 200 and got.json()["id"] == r["id"] and not any(k.startswith("_") for k in got.json())
    assert client.get("/v1/responses/resp_missing").status_code == 404
    client.post("/v1/completions", json={"prompt": "x" * 64, "max_tokens": 2, "temperature": 0, "ignore_eos": True})
    assert client.get("/v1/cache/stats").status_code == 200
    assert client.post("/v1/cache/reset").json()["dropped_blocks"] >= 0
    body = {"messages": msgs, "max_tokens": 3, "temperature": 0, "ignore_eos": True}
    a, b = client.post("/chat/completions", json=body).json(), client.post("/v1/chat/completions", json=body).json()
    assert a["choices"][0]["message"]["content"] == b["choices"][0]["message"]["content"]
    c = client.post("/completions", json={"prompt": "hello", "n_predict": 3, "temperature": 0, "ignore_eos": True}).json()
    assert c["tokens_predicted"] == 3
    assert client.post("/infill", json={"input_prefix": "def f(", "input_suffix": "return x"}).status_code == 501
    e = client.post("/embeddings", json={"input": ["a", "bb"]})
    assert e.status_code == 200 and len(e.json()["data"]) == 2
    n = client.post("/embedding", json={"content": ["a", "bb"]}).json()
    assert [x["index"] for x in n] == [0, 1] and len(n[0]["embedding"]) == len(e.json()["data"][0]["embedding"])
    rr = client.post("/rerank", json={"query": "a", "documents": ["a", "zzz"]}).json()
    assert len(rr["results"]) == 2 and client.post("/v1/reranking", json={"query": "a", "documents": ["a"]}).status_code == 200


def test_completions_echo_scores_the_prompt(client):
    """``echo`` + ``max_tokens: 0``: per-token prompt log-probabilities (the evaluation-harness request);
    with generation, the greedy continuation's first token is the argmax the prompt scores imply."""
    r = client.post("/v1/completions", json={"prompt": "hello world", "echo": True, "max_tokens": 0, "logprobs": 1}).json()
    ch = r["choices"][0]
    lp = ch["logprobs"]
    n = r["usage"]["prompt_tokens"]
    assert ch["text"].endswith("hello world") and len(lp["tokens"]) == n == len(lp["token_logprobs"]) == len(lp["text_offset"])
    assert lp["token_logprobs"][0] is None and all(x <= 0.0 for x in lp["token_logprobs"][1:])
    assert r["usage"]["completion_tokens"] == 0
    longer = client.post("/v1/completions", json={"prompt": "hello world!", "echo": True, "max_tokens": 0}).json()
    a, b = lp["token_logprobs"][1:], longer["choices"][0]["logprobs"]["token_logprobs"][1:n]
    assert all(abs(x - y) < 1e-4 for x, y in zip(a, b))          # causal: a longer prompt scores its prefix the same
    g = client.post("/v1/completions", json={"prompt": "hello world", "echo": True, "max_tokens": 3, "temperature": 0,
                                             "ignore_eos": True, "logprobs": 1}).json()["choices"][0]
    assert len(g["logprobs"]["tokens"]) == n + 3 and g["logprobs"]["token_logprobs"][n] is not None


def test_n_choices(client):
    """``n``: several samples of one prompt in one request; greedy samples coincide, seeded ones are
    reproducible and use seed + index."""
    g = client.post("/v1/completions", json={"prompt": "hello", "max_tokens": 5, "temperature": 0, "ignore_eos": True, "n": 3}).json()
    assert [c["index"] for c in g["choices"]] == [0, 1, 2] and len({c["text"] for c in g["choices"]}) == 1
    assert g["usage"]["completion_tokens"] == 15
    body = {"messages": [{"role": "user", "content": "hi"}], "max_tokens": 6, "temperature": 1.0, "seed": 11, "ignore_eos": True,
            "n": 2}
    a, b = client.post("/v1/chat/completions", json=body).json(), client.post("/v1/chat/completions", json=body).json()
    ta, tb = [c["message"]["content"] for c in a["choices"]], [c["message"]["content"] for c in b["choices"]]
    assert ta == tb and len(ta) == 2
    one = client.post("/v1/chat/completions", json=dict(body, n=1, seed=12)).json()["choices"][0]["message"]["content"]
    assert one == ta[1]                                           # sample 1 of seed 11 is sample 0 of seed 12
