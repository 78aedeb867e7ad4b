"""Structured output end to end on CPU: a random tiny model under a JSON schema, a GBNF grammar and a
regex must emit text of that shape and then stop; the tokenizer's vocabulary is shorter than the logits."""
import json
import re
import tempfile
from pathlib import Path

import pytest

pytest.importorskip("llguidance")
tokenizers = pytest.importorskip("tokenizers")

from mlxcel_b200 import cli  # noqa: E402
from mlxcel_b200.server.structured import gbnf_to_lark  # noqa: E402

SCHEMA = {"type": "object", "properties": {"a": {"type": "integer"}, "ok": {"type": "boolean"}},
          "required": ["a", "ok"], "additionalProperties": False}


@pytest.fixture(scope="module")
def model_dir():
    """tiny-llama random weights (vocabulary 1024) with a byte-level tokenizer of 260 entries."""
    from tokenizers import Tokenizer, decoders, models, pre_tokenizers

    d = Path(tempfile.mkdtemp(prefix="structured_"))
    cli.main(["random-init", "tiny-llama", str(d)])
    vocab = {ch: i for i, ch in enumerate(sorted(pre_tokenizers.ByteLevel.alphabet()))}
    vocab["<eos>"] = 256
    for i, name in enumerate(("<fim_prefix>", "<fim_suffix>", "<fim_middle>")):      # StarCoder spelling
        vocab[name] = 257 + i
    tok = Tokenizer(models.BPE(vocab=vocab, merges=[]))
    tok.pre_tokenizer = pre_tokenizers.ByteLevel(add_prefix_space=False, use_regex=False)
    tok.decoder = decoders.ByteLevel()
    tok.add_special_tokens(["<eos>", "<fim_prefix>", "<fim_suffix>", "<fim_middle>"])
    tok.save(str(d / "tokenizer.json"))
    (d / "tokenizer_config.json").write_text(json.dumps(dict(eos_token="<eos>", tokenizer_class="PreTrainedTokenizerFast")))
    return d


def _gen(capsys, model_dir, *extra):
    capsys.readouterr()
    cli.main(["generate", "-m", str(model_dir), "--device", "cpu", "-n", "96", "--temp", "0.8", "--seed", "3", "-p", "out:",
              *extra])
    cap = capsys.readouterr()
    return cap.out.rstrip("\n"), cap.err


def test_json_schema_constrains_and_ends_generation(model_dir, capsys):
    text, err = _gen(capsys, model_dir, "--json-schema", json.dumps(SCHEMA))
    doc = json.loads(text)
    assert set(doc) == {"a", "ok"} and isinstance(doc["a"], int) and isinstance(doc["ok"], bool)
    assert "finish: stop" in err                                   # the grammar completed, nothing ran on after it


def test_gbnf_and_regex(model_dir, capsys, tmp_path):
    g = tmp_path / "g.gbnf"
    g.write_text('root ::= "yes" | "no" ("!" | "?")\n')
    text, _ = _gen(capsys, model_dir, "--grammar-file", str(g))
    assert text in ("yes", "no!", "no?")
    text, _ = _gen(capsys, model_dir, "--regex", "[a-c]{3}-[0-9]{2}")
    assert re.fullmatch(r"[a-c]{3}-[0-9]{2}", text)
    with pytest.raises(SystemExit):
        _gen(capsys, model_dir, "--grammar", "root ::= (")


def test_gbnf_lowering():
    lark = gbnf_to_lark('root ::= item+\nitem ::= [a-z] "x"? # comment\n')
    assert "start" in lark and "item" in lark and "comment" not in lark


def test_server_response_format(model_dir):
    from fastapi.testclient import TestClient

    from mlxcel_b200.engine.engine import EngineConfig
    from mlxcel_b200.llm import LLM
    from mlxcel_b200.server.app import ServerState, create_app
    from mlxcel_b200.server.worker import ModelWorker

    llm = LLM.from_pretrained(str(model_dir), device="cpu",
                              engine_config=EngineConfig(num_blocks=64, block_size=16, max_batch=4, max_model_len=256))
    worker = ModelWorker(llm.engine, llm.tokenizer, "m")
    try:
        c = TestClient(create_app(ServerState(worker, llm.tokenizer, "m")))
        r = c.post("/v1/completions", json=dict(prompt="out:", max_tokens=96, temperature=0.8, seed=5,
                                                response_format=dict(type="json_schema", json_schema=dict(schema=SCHEMA))))
        assert r.status_code == 200, r.text
        doc = json.loads(r.json()["choices"][0]["text"])
        assert set(doc) == {"a", "ok"}
        fim = c.post("/infill", json=dict(input_prefix="def f(x):\n    ", input_suffix="\n    return y", n_predict=6,
                                          temperature=0, ignore_eos=True))
        assert fim.status_code == 200 and fim.json()["tokens_predicted"] == 6
        assert llm.tokenizer.fim == dict(prefix=257, suffix=258, middle=259)
        r = c.post("/completion", json=dict(prompt="out:", n_predict=32, temperature=0.8, seed=5,
                                            grammar='root ::= "a" [0-9] [0-9]'))
        assert r.status_code == 200 and re.fullmatch(r"a[0-9]{2}", r.json()["content"])
    finally:
        worker.shutdown()
