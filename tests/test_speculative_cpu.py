"""Speculative decoding is lossless for greedy decoding: every drafter must reproduce plain greedy
output token for token (the reference's byte-equal parity rule, tests/speculative_parity.rs)."""
import pytest
import torch

from mlxcel_b200.config import preset
from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams
from mlxcel_b200.models.decoder import DecoderModel
from mlxcel_b200.models.weights import random_weights
from mlxcel_b200.speculative import DraftModelDrafter, MTPDrafter, PromptLookupDrafter, random_mtp_weights


def _mk(cfg, w, **kw):
    base = dict(max_batch=4, max_num_batched_tokens=128, num_blocks=96, max_model_len=384, cuda_graphs=False)
    base.update(kw)
    return Engine(DecoderModel(cfg, w), cfg, EngineConfig(**base))


def _prompts(cfg, lens=(9, 40, 23)):
    g = torch.Generator().manual_seed(3)
    ps = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    ps.append([5, 6, 7, 8] * 8)   # repetitive prompt: prompt lookup finds matches
    return ps


@pytest.mark.parametrize("kind", ["prompt_lookup", "draft_model", "self_draft", "mtp"])
@pytest.mark.parametrize("name", ["tiny-llama", "tiny-qwen3"])
def test_speculative_is_lossless(kind, name):
    cfg = preset(name)
    w = random_weights(cfg, seed=4, dtype=torch.float32, std=0.05)
    sp = SamplingParams(max_tokens=24, ignore_eos=True)
    prompts = _prompts(cfg)
    want = [s.output for s in _mk(cfg, w).generate(prompts, sp)]
    eng = _mk(cfg, w)
    if kind == "prompt_lookup":
        eng.drafter = PromptLookupDrafter()
    elif kind == "draft_model":
        dcfg = preset("tiny-llama")
        dw = random_weights(dcfg, seed=99, dtype=torch.float32, std=0.05)
        eng.drafter = DraftModelDrafter(DecoderModel(dcfg, dw), dcfg, num_blocks=96, max_model_len=384)
    elif kind == "self_draft":     # the target as its own drafter: every draft must be accepted
        eng.drafter = DraftModelDrafter(DecoderModel(cfg, w), cfg, num_blocks=96, max_model_len=384)
    else:
        eng.drafter = MTPDrafter(eng.model, cfg, random_mtp_weights(cfg, dtype=torch.float32, std=0.05),
                                 num_blocks=96)
    eng.spec_k = 4
    got = [s.output for s in eng.generate(prompts, sp)]
    assert got == want
    assert eng.stats["spec_rounds"] > 0
    if kind == "self_draft":
        assert eng.stats["spec_accepted"] == eng.stats["spec_drafted"] > 0
    if kind == "prompt_lookup":
        assert eng.stats["spec_drafted"] > 0


def test_speculative_respects_max_tokens_and_eos():
    cfg = preset("tiny-llama")
    w = random_weights(cfg, seed=4, dtype=torch.float32, std=0.05)
    prompts = _prompts(cfg)
    base = _mk(cfg, w).generate(prompts, SamplingParams(max_tokens=7, ignore_eos=True))
    stop = base[0].output[3]
    sp = [SamplingParams(max_tokens=7, stop_token_ids=[stop])] + [SamplingParams(max_tokens=7, ignore_eos=True)] * 3
    want = [s.output for s in _mk(cfg, w).generate(prompts, sp)]
    eng = _mk(cfg, w)
    eng.drafter = DraftModelDrafter(DecoderModel(cfg, w), cfg, num_blocks=96, max_model_len=384)
    got = [s.output for s in eng.generate(prompts, sp)]
    assert got == want and all(len(o) <= 7 for o in got)
