"""Log-likelihood scoring and perplexity against transformers' cross-entropy (CPU, fp32)."""
import json
import math
import tempfile

import pytest
import torch

transformers = pytest.importorskip("transformers")

from mlxcel_b200 import cli  # noqa: E402
from mlxcel_b200.engine.engine import EngineConfig  # noqa: E402
from mlxcel_b200.engine.scoring import perplexity  # noqa: E402
from mlxcel_b200.llm import LLM  # noqa: E402


def _tiny(name, **kw):
    from transformers import AutoConfig, AutoModelForCausalLM
    torch.manual_seed(0)
    base = dict(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
                vocab_size=300, max_position_embeddings=256)
    base.update(kw)
    m = AutoModelForCausalLM.from_config(AutoConfig.for_model(name, **base)).float().eval()
    with torch.no_grad():
        for p in m.parameters():
            if p.dim() >= 2:
                p.normal_(0, 0.08)
    d = tempfile.mkdtemp(prefix=f"score_{name}_")
    m.save_pretrained(d, safe_serialization=True)
    return m, d


@pytest.mark.parametrize("name,kw", [("llama", {}), ("mamba2", dict(num_heads=8, head_dim=16, state_size=16, n_groups=1, expand=2,
                                                                     conv_kernel=4, chunk_size=8))])
def test_loglikelihoods_match_transformers(name, kw):
    if name == "mamba2":
        kw = dict(kw, intermediate_size=None, num_attention_heads=None, num_key_value_heads=None)
        kw = {k: v for k, v in kw.items() if v is not None}
    try:
        m, d = _tiny(name, **kw)
    except (KeyError, ValueError, ImportError, TypeError) as e:
        pytest.skip(f"transformers cannot build {name}: {e}")
    ids = torch.randint(0, 300, (57,), generator=torch.Generator().manual_seed(1))
    with torch.no_grad():
        want = torch.log_softmax(m(ids[None]).logits[0, :-1].float(), -1).gather(1, ids[1:, None])[:, 0]
    llm = LLM.from_pretrained(d, device="cpu", engine_config=EngineConfig(num_blocks=32, block_size=16, max_batch=2,
                                                                          max_model_len=128))
    got = llm.loglikelihoods(ids.tolist())
    assert got.shape == want.shape and (got - want).abs().max().item() < 4e-2     # the front end loads bf16 weights
    again = llm.loglikelihoods(ids.tolist())                    # scratch state released: same answer twice
    assert torch.equal(got, again)
    res = perplexity(llm.model, llm.cfg, ids.tolist(), window=57)
    assert res["tokens"] == 56 and abs(res["perplexity"] - math.exp(-want.mean().item())) < 2e-2 * res["perplexity"]
    win = perplexity(llm.model, llm.cfg, ids.tolist(), window=32, stride=16)
    assert win["tokens"] == 56 and win["perplexity"] > 1.0       # every token scored once under the strided windows


def test_perplexity_cli(capsys, tmp_path):
    f = tmp_path / "t.txt"
    f.write_text("the quick brown fox jumps over the lazy dog. " * 6)
    cli.main(["perplexity", "-m", "preset:tiny-llama", "--device", "cpu", "-f", str(f), "--window", "64", "--json"])
    res = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert res["tokens"] > 200 and res["perplexity"] > 1.0 and res["window"] == 64


def test_generative_rerank_scores_and_route(capsys):
    """The yes/no reranker: scores are p(yes) of the judgement prompt (checked against a direct forward),
    through the function, the CLI verb on a decoder preset and the server route."""
    from fastapi.testclient import TestClient

    from mlxcel_b200.engine.scoring import generative_rerank, prefill_hidden, rerank_prompt
    from mlxcel_b200.server.app import ServerState, create_app
    from mlxcel_b200.server.worker import ModelWorker
    from mlxcel_b200.tokenizer import ByteTokenizer

    llm = LLM.from_preset("tiny-llama", device="cpu", dtype=torch.float32,
                          engine_config=EngineConfig(num_blocks=128, block_size=16, max_batch=2, max_model_len=1024))
    tk = ByteTokenizer(llm.cfg.vocab_size)
    docs = ["pandas are bears", "berlin is in germany"]
    scores = generative_rerank(llm.model, llm.cfg, tk, "what is a panda?", docs)
    assert len(scores) == 2 and all(0.0 < s < 1.0 for s in scores)
    ids = tk.encode(rerank_prompt("what is a panda?", docs[0]))
    lg = llm.model.logits(prefill_hidden(llm.model, llm.cfg, ids), torch.tensor([len(ids) - 1])).float()[0]
    y, n = tk.encode("yes")[0], tk.encode("no")[0]
    assert abs(scores[0] - float(torch.sigmoid(lg[y] - lg[n]))) < 1e-5
    worker = ModelWorker(llm.engine, tk, "m")
    try:
        c = TestClient(create_app(ServerState(worker, tk, "m")))
        r = c.post("/v1/rerank", json=dict(query="what is a panda?", documents=docs, mode="generative", top_n=1)).json()
        best = max(range(2), key=lambda i: scores[i])
        assert len(r["results"]) == 1 and r["results"][0]["index"] == best
        assert abs(r["results"][0]["relevance_score"] - scores[best]) < 1e-5
    finally:
        worker.shutdown()
    cli.main(["rerank", "-m", "preset:tiny-llama", "--device", "cpu", "-q", "q", "-d", "a", "-d", "b", "--json"])
    res = json.loads(capsys.readouterr().out.strip().splitlines()[-1])["results"]
    assert sorted(r["index"] for r in res) == [0, 1]
