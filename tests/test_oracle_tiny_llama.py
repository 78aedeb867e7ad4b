"""Benchmark configuration 1: tiny Llama on CPU, world_size 1, greedy decode of 32 tokens must
match the independent PyTorch-CPU oracle token for token."""
import torch

from mlxcel_b200.config import preset
from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams
from mlxcel_b200.models.decoder import DecoderModel
from mlxcel_b200.models.weights import random_weights

from oracle import oracle_greedy


def _engine(cfg, w, **kw):
    model = DecoderModel(cfg, w)
    return Engine(model, cfg, EngineConfig(max_batch=4, max_num_batched_tokens=256, num_blocks=64,
                                           max_model_len=256, cuda_graphs=False, **kw))


def test_tiny_llama_matches_oracle():
    cfg = preset("tiny-llama")
    w = random_weights(cfg, seed=1234, dtype=torch.float32)
    g = torch.Generator().manual_seed(7)
    prompt = torch.randint(0, cfg.vocab_size, (16,), generator=g).tolist()
    want = oracle_greedy(cfg, w, prompt, 32)
    eng = _engine(cfg, w)
    got = eng.generate([prompt], SamplingParams(max_tokens=32, ignore_eos=True))[0].output
    assert got == want


def test_chunked_prefill_and_batching_match_oracle():
    cfg = preset("tiny-llama")
    w = random_weights(cfg, seed=5, dtype=torch.float32)
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 37, 16)]
    want = [oracle_greedy(cfg, w, p, 8) for p in prompts]
    eng = _engine(cfg, w, prefill_chunk_alone=16, prefill_chunk_contended=8)
    outs = eng.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    assert [o.output for o in outs] == want
