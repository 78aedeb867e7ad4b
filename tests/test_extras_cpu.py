"""LoRA adapters, load-time weight surgery, the Python client and the extra server routes (CPU)."""
import json

import pytest
import torch

from mlxcel_b200.config import preset
from mlxcel_b200.models.weights import random_weights


def _write_adapter(tmp_path, cfg, r=4, alpha=8.0, layers=(0, 1)):
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(7)
    H, D = cfg.hidden_size, cfg.head_dim
    t = {}
    for li in layers:
        base = f"model.layers.{li}.self_attn.q_proj"
        t[base + ".lora_a"] = torch.randn(H, r, generator=g) * 0.1                      # MLX layout [in, r]
        t[base + ".lora_b"] = torch.randn(r, cfg.num_attention_heads * D, generator=g) * 0.1
        base = f"model.layers.{li}.mlp.down_proj"
        t[base + ".lora_A.weight"] = torch.randn(r, cfg.intermediate_size, generator=g) * 0.1   # PEFT layout
        t[base + ".lora_B.weight"] = torch.randn(H, r, generator=g) * 0.1
    d = tmp_path / "adapter"
    d.mkdir()
    save_file(t, str(d / "adapters.safetensors"))
    (d / "adapter_config.json").write_text(json.dumps({"lora_parameters": {"rank": r, "alpha": alpha}}))
    return d, t


def test_lora_fuse_scale_and_detach(tmp_path):
    from mlxcel_b200.lora import LoraManager
    cfg = preset("tiny-llama")
    w = random_weights(cfg, seed=1, dtype=torch.float32)
    q0 = w.layers[0].wqkv.clone()
    d0 = w.layers[1].w_down.clone()
    path, t = _write_adapter(tmp_path, cfg)
    mgr = LoraManager(cfg, w)
    ad = mgr.add(path, scale=1.0)
    nq = cfg.num_attention_heads * cfg.head_dim
    a, b = t["model.layers.0.self_attn.q_proj.lora_a"], t["model.layers.0.self_attn.q_proj.lora_b"]
    want = q0.clone()
    want[:nq] += (b.t() @ a.t()) * (8.0 / 4)
    assert torch.allclose(w.layers[0].wqkv, want, atol=1e-5)
    assert torch.equal(w.layers[0].wqkv[nq:], q0[nq:])            # k / v rows untouched
    A, B = t["model.layers.1.mlp.down_proj.lora_A.weight"], t["model.layers.1.mlp.down_proj.lora_B.weight"]
    assert torch.allclose(w.layers[1].w_down, d0 + (B @ A) * 2.0, atol=1e-5)
    mgr.set_scale(ad.id, 0.25)
    assert torch.allclose(w.layers[1].w_down, d0 + (B @ A) * 0.5, atol=1e-5)
    mgr.set_scale(ad.id, 0.0)                                       # detached: original weights back
    assert torch.allclose(w.layers[0].wqkv, q0, atol=1e-5) and torch.allclose(w.layers[1].w_down, d0, atol=1e-5)
    assert mgr.listing() == [{"id": 0, "path": str(path), "scale": 0.0}]


def test_lora_tensor_parallel_shards_sum_to_full(tmp_path):
    from mlxcel_b200.loading.shard import shard_weights
    from mlxcel_b200.lora import LoraManager
    cfg = preset("tiny-llama")
    full = random_weights(cfg, seed=2, dtype=torch.float32)
    path, _ = _write_adapter(tmp_path, cfg)
    shards = [shard_weights(cfg, random_weights(cfg, seed=2, dtype=torch.float32), r, 2) for r in range(2)]
    LoraManager(cfg, full).add(path, 1.0)
    for r in range(2):
        LoraManager(cfg, shards[r], tp_rank=r, tp_size=2).add(path, 1.0)
    ref = [shard_weights(cfg, full, r, 2) for r in range(2)]
    for r in range(2):
        assert torch.allclose(shards[r].layers[0].wqkv, ref[r].layers[0].wqkv, atol=1e-5)
        assert torch.allclose(shards[r].layers[1].w_down, ref[r].layers[1].w_down, atol=1e-5)


def test_weight_surgery(tmp_path):
    from mlxcel_b200.loading.surgery import apply_edits, load_edits
    y = tmp_path / "edits.yaml"
    y.write_text("""
- op: scale
  match: "model.layers.(0|1).mlp.down_proj.weight"
  factor: 0.5
- op: interpolate
  match: "model.layers.1.(.*)"
  source: "model.layers.0.\\\\1"
  t: 0.25
- op: prune
  match: "lm_head.weight"
  threshold: 0.5
- op: replace
  match: "model.norm.weight"
  value: 1.0
""")
    edits = load_edits(str(y))
    store = {"model.layers.0.mlp.down_proj.weight": torch.full((2, 2), 4.0),
             "model.layers.1.mlp.down_proj.weight": torch.full((2, 2), 8.0),
             "lm_head.weight": torch.tensor([[0.1, -0.7], [0.6, -0.2]]), "model.norm.weight": torch.zeros(3)}
    get = lambda n: apply_edits(edits, n, store[n], lambda k: store.get(k))
    assert torch.equal(get("model.layers.0.mlp.down_proj.weight"), torch.full((2, 2), 2.0))
    # layer 1: scaled to 4.0, then 0.75 * 4.0 + 0.25 * (raw layer 0 = 4.0) = 4.0
    assert torch.allclose(get("model.layers.1.mlp.down_proj.weight"), torch.full((2, 2), 4.0))
    assert torch.equal(get("lm_head.weight"), torch.tensor([[0.0, -0.7], [0.6, 0.0]]))
    assert torch.equal(get("model.norm.weight"), torch.ones(3))
    with pytest.raises(ValueError):
        (tmp_path / "bad.yaml").write_text("- op: explode\n  match: x\n")
        load_edits(str(tmp_path / "bad.yaml"))


class _FakeResp:
    def __init__(self, payload, status=200, lines=None):
        self._p, self.status_code, self._lines, self.text = payload, status, lines or [], json.dumps(payload)

    def json(self):
        return self._p

    def iter_lines(self):
        return iter(self._lines)


class _FakeSession:
    def __init__(self):
        self.calls = []

    def post(self, url, json=None, headers=None, timeout=None, stream=False):
        self.calls.append(("POST", url, json, headers))
        if url.endswith("/v1/chat/completions") and json.get("stream"):
            ev = lambda c: ("data: " + __import__("json").dumps({"choices": [{"delta": {"content": c}}]})).encode()
            return _FakeResp({}, lines=[ev("Hel"), b"", ev("lo"), b"data: [DONE]"])
        if url.endswith("/v1/chat/completions"):
            return _FakeResp({"choices": [{"message": {"content": "hi"}}]})
        if url.endswith("/v1/embeddings"):
            return _FakeResp({"data": [{"embedding": [1.0, 0.0]}]})
        if url.endswith("/tokenize"):
            return _FakeResp({"tokens": [1, 2, 3]})
        return _FakeResp({"error": "nope"}, status=404)

    def get(self, url, headers=None, timeout=None):
        self.calls.append(("GET", url, None, headers))
        if url.endswith("/health"):
            return _FakeResp({"status": "ok"})
        return _FakeResp({"data": [{"id": "m"}]})


def test_python_client_against_fake_transport():
    from mlxcel_b200.client import Client, MlxcelError
    s = _FakeSession()
    c = Client("http://x:1/", api_key="k", session=s)
    assert c.health() and c.models() == ["m"]
    assert c.chat([{"role": "user", "content": "yo"}], max_tokens=4) == "hi"
    assert "".join(c.chat_stream([{"role": "user", "content": "yo"}])) == "Hello"
    assert c.embed("a") == [[1.0, 0.0]] and c.tokenize("abc") == [1, 2, 3]
    assert s.calls[0][3] == {"Authorization": "Bearer k"} and s.calls[2][2]["max_tokens"] == 4
    with pytest.raises(MlxcelError):
        c.detokenize([1])


def test_llama_server_flag_spellings_map_onto_native_options(capsys):
    """-md / --draft / -b / -ub / -ctk / --no-cache-prompt fold into the native options; CPU-thread, mmap and
    GPU-offload flags are accepted and reported as having no effect."""
    import argparse

    from mlxcel_b200 import cli

    ap = argparse.ArgumentParser()
    cli._add_model_args(ap)
    a = ap.parse_args(["-m", "x", "-md", "drafter", "--draft", "3", "-b", "512", "-ub", "128", "-ctk", "q8_0", "-ctv", "f16",
                       "--no-cache-prompt", "-ngl", "99", "-fa", "--mlock", "-t", "8"])
    ignored = cli._apply_compat(a)
    assert (a.draft_model, a.draft_max, a.max_batch_tokens, a.prefill_chunk_size, a.kv_bits, a.no_prompt_cache) == \
        ("drafter", 3, 512, 128, 8, True)
    assert ignored == ["--flash-attn", "--gpu-layers", "--mlock", "--threads"]
    b = ap.parse_args(["-m", "x", "--draft-model", "native", "-md", "compat", "--kv-bits", "16", "-ctk", "q8_0"])
    cli._apply_compat(b)
    assert b.draft_model == "native" and b.kv_bits == 16          # the native spelling wins
    import pytest
    with pytest.raises(SystemExit):
        cli._apply_compat(ap.parse_args(["-m", "x", "-ctk", "q5_1"]))
    c4 = ap.parse_args(["-m", "x", "-ctk", "q4_0"])
    cli._apply_compat(c4)
    assert c4.kv_bits == 4


def test_rope_and_kv_overrides_change_the_built_config(tmp_path):
    import argparse
    import json

    from mlxcel_b200 import cli
    from mlxcel_b200.config import ModelConfig

    base = dict(model_type="llama", hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                num_key_value_heads=2, vocab_size=300, max_position_embeddings=256, rope_theta=10000.0,
                rope_scaling=dict(rope_type="llama3", factor=8.0, low_freq_factor=1.0, high_freq_factor=4.0,
                                  original_max_position_embeddings=64))
    (tmp_path / "config.json").write_text(json.dumps(base))
    ap = argparse.ArgumentParser()
    cli._add_model_args(ap)
    a = ap.parse_args(["-m", "x", "--rope-freq-base", "500000", "--rope-scaling", "yarn", "--rope-scale", "4",
                       "--yarn-orig-ctx", "64", "--override-kv", "rms_norm_eps=1e-4", "--override-kv", "sliding_window=null"])
    ov = cli.config_overrides(a)
    cfg = ModelConfig.from_path(tmp_path, ov)
    assert cfg.rope_theta == 500000.0 and cfg.rope_scaling["rope_type"] == "yarn" and cfg.rope_scaling["factor"] == 4.0
    assert cfg.rope_scaling["original_max_position_embeddings"] == 64 and cfg.rms_norm_eps == 1e-4
    none = ModelConfig.from_path(tmp_path, cli.config_overrides(ap.parse_args(["-m", "x", "--rope-scaling", "none"])))
    assert not none.rope_scaling and ModelConfig.from_path(tmp_path).rope_scaling["rope_type"] == "llama3"
    # the rope_parameters spelling of newer checkpoints is rewritten as well
    new = dict(base, rope_parameters=dict(rope_type="llama3", rope_theta=10000.0, factor=8.0, low_freq_factor=1.0,
                                          high_freq_factor=4.0, original_max_position_embeddings=64))
    new.pop("rope_theta"), new.pop("rope_scaling")
    (tmp_path / "config.json").write_text(json.dumps(new))
    cfg2 = ModelConfig.from_path(tmp_path, ov)
    assert cfg2.rope_theta == 500000.0 and cfg2.rope_scaling["rope_type"] == "yarn" and cfg2.rope_scaling["factor"] == 4.0
    assert cli.config_overrides(ap.parse_args(["-m", "x"])) is None


def test_repl_grammar_slash_commands_and_multiline():
    from mlxcel_b200.cli import repl_turns

    lines = ["hello", "/help", "/nope", '"""first', "second", 'third"""', "/clear", "again", "/system be brief", "x", "/bye",
             "never read"]
    seen = []
    for kind, payload in repl_turns(lines, system="sys"):
        if kind == "send":
            seen.append(("send", [dict(m) for m in payload]))
            payload.append({"role": "assistant", "content": "ok"})
        else:
            seen.append((kind, payload))
    sends = [p for k, p in seen if k == "send"]
    assert [m["content"] for m in sends[0]] == ["sys", "hello"]
    assert sends[1][-1]["content"] == "first\nsecond\nthird" and len(sends[1]) == 4      # sys, hello, ok, multiline
    assert [m["content"] for m in sends[2]] == ["sys", "again"]                          # /clear kept the system prompt
    assert [m["content"] for m in sends[3]] == ["be brief", "x"] and len(sends) == 4
    prints = [p for k, p in seen if k == "print"]
    assert prints[0].startswith("Available commands") and "Unknown command: /nope" in prints[1]
    assert list(repl_turns(["", "ignored"])) == []


def test_memory_estimate_of_recurrent_models_matches_the_built_model():
    """State-space / hybrid presets: estimated parameters within 1 % of the tensors the model holds, the
    per-sequence recurrent state equal to the executor's state slots, KV only for attention blocks."""
    import torch

    from mlxcel_b200.config import preset
    from mlxcel_b200.models.hybrid import HybridModel, random_hybrid_weights
    from mlxcel_b200.models.mamba1 import Mamba1Model, random_mamba1_weights
    from mlxcel_b200.models.mamba2 import Mamba2Model, random_mamba2_weights
    from mlxcel_b200.utils.memory import estimate_memory

    def count(o, seen):
        if isinstance(o, torch.Tensor):
            if o.data_ptr() in seen:
                return 0
            seen.add(o.data_ptr())
            return o.numel()
        if isinstance(o, (list, tuple)):
            return sum(count(x, seen) for x in o)
        return sum(count(v, seen) for v in vars(o).values()) if hasattr(o, "__dict__") else 0

    for name, make, cls in (("tiny-mamba2", random_mamba2_weights, Mamba2Model), ("tiny-mamba", random_mamba1_weights, Mamba1Model),
                            ("tiny-nemotron-h", random_hybrid_weights, HybridModel)):
        cfg = preset(name)
        w = make(cfg, dtype=torch.float32)
        est = estimate_memory(cfg, ctx=256, parallel=2)
        real = count(w, set())
        assert abs(est["parameters"] - real) < 0.01 * real, (name, est["parameters"], real)
        m = cls(cfg, w, max_seqs=4)
        ssm = getattr(m, "ssm", m)
        per_seq = 4 * (ssm.conv_state[:, 0].numel() + ssm.ssm_state[:, 0].numel())
        assert est["recurrent_state_bytes_per_seq"] == per_seq, name
        assert est["recurrent_state_bytes"] == 2 * 2 * per_seq
        assert (est["kv_bytes_per_token"] > 0) == (name == "tiny-nemotron-h")
    assert estimate_memory(preset("tiny-llama"))["recurrent_state_bytes"] == 0


def test_serve_preflight(capsys):
    import json

    import pytest

    from mlxcel_b200 import cli

    cli.main(["serve", "-m", "preset:llama-3.1-8b", "--estimate-memory", "-c", "8192", "--parallel", "8"])
    est = json.loads(capsys.readouterr().out)
    assert est["fits_b200"] and est["kv_pool_blocks"] == 8 * 512
    with pytest.raises(SystemExit, match="does not fit"):
        cli.main(["serve", "-m", "preset:llama-3.1-8b", "-c", "4000000", "--parallel", "1"])


def test_llama_server_compat_manifest_matches_the_parser_and_the_routes():
    """compat/llama_server.json lists every option spelling with its treatment and the served routes; it
    must agree with what the argument parser accepts and what the application registers."""
    import argparse
    import json
    from pathlib import Path

    from mlxcel_b200 import cli
    from mlxcel_b200.server import app as app_mod

    doc = json.loads((Path(__file__).resolve().parent.parent / "compat" / "llama_server.json").read_text())
    ap = argparse.ArgumentParser()
    cli._add_model_args(ap)
    cli._add_sampling_args(ap)
    known = {s: a for a in ap._actions for s in a.option_strings}
    listed = {f for o in doc["options"] if o["status"] != "unsupported" for f in o["flags"]}
    assert listed == set(known) - {"-h", "--help"}
    for o in doc["options"]:
        if o["status"] == "accepted-no-effect":
            assert all(known[f].dest.startswith("compat_noop_") for f in o["flags"])
        elif o["status"] == "unsupported":
            assert o["flags"][0].split()[0] not in known and o["why"]
    src = Path(app_mod.__file__).read_text() + (Path(app_mod.__file__).parent / "extras.py").read_text()
    for r in doc["routes"]:
        path = r.split("?")[0].replace("{id}", "{slot_id}")
        assert f'"{path}"' in src, r


def test_arch_catalog_lists_every_family(capsys):
    import json

    from mlxcel_b200 import cli
    from mlxcel_b200.config import FAMILIES

    cli.main(["arch", "--json"])
    cat = json.loads(capsys.readouterr().out)
    names = {f["name"]: f for f in cat["families"]}
    assert set(names) == set(FAMILIES) and names["jamba"]["executor"] == "hybrid" and names["mamba2"]["executor"] == "state-space"
    assert names["llama"]["checked_against"] == "transformers logits" and "modernbert" in cat["encoders"]
    cli.main(["supported"])
    out = capsys.readouterr().out
    assert out.splitlines()[0].startswith("FAMILY") and "qwen3_next" in out


def test_tiktoken_vocabulary_files_load_and_round_trip(tmp_path):
    """A tiktoken-format vocabulary (base64 token + rank per line) with control tokens from
    tokenizer_config.json: merges follow the ranks (lowest first), control literals map to their ids,
    decoding restores the text, and the incremental detokenizer streams it."""
    import base64
    import json

    from mlxcel_b200.tokenizer import IncrementalDetokenizer, TiktokenTokenizer, load_tokenizer

    toks = [bytes([i]) for i in range(256)] + [b"he", b"ll", b"hell", b"hello", b" w", b"or", b" wor", b"ld", b" world", "é".encode()]
    (tmp_path / "tiktoken.model").write_text("\n".join(f"{base64.b64encode(t).decode()} {r}" for r, t in enumerate(toks)))
    (tmp_path / "tokenizer_config.json").write_text(json.dumps(dict(
        added_tokens_decoder={"266": dict(content="<|im_end|>"), "267": dict(content="<|bos|>"), "268": dict(content="<think>")},
        bos_token="<|bos|>", eos_token=dict(content="<|im_end|>"))))
    tk = load_tokenizer(tmp_path)
    assert isinstance(tk, TiktokenTokenizer) and tk.vocab_size == 269
    assert tk.encode("hello world") == [259, 264]
    assert tk.encode("hell") == [258] and tk.encode("hel") == [256, ord("l")]
    assert tk.encode("hello<|im_end|>", add_special_tokens=True) == [267, 259, 266]
    assert tk.eos_ids() == [266] and tk.think_open == 268 and tk.control_id("<|bos|>") == 267
    text = "hello world, héllo\n\n  wörld 12345!"
    ids = tk.encode(text)
    assert tk.decode(ids) == text and all(0 <= i < 266 for i in ids)
    assert tk.decode([259, 266]) == "hello" and tk.decode([259, 266], skip_special_tokens=False) == "hello<|im_end|>"
    det = IncrementalDetokenizer(tk)
    assert "".join(det.push(i) for i in ids) + det.flush() == text
    assert len(tk.fingerprint()) == 16


def test_host_tensors_are_refused_as_kernel_operands():
    """An optional kernel operand that lives in pageable host memory is refused before any launch (the
    kernel would fault on it and take the CUDA context down)."""
    import pytest as _pytest
    import torch

    from mlxcel_b200.ops import _lib

    assert _lib.ptr(None) is None
    with _pytest.raises(ValueError, match="host tensor"):
        _lib.ptr(torch.zeros(4))
