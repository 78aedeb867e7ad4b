"""Model-family coverage on CPU (fp32 reference ops): every preset family must generate, and a
sequence decoded alone must equal the same sequence decoded inside a batch with chunked prefill
(continuous batching must not change greedy tokens)."""
import pytest
import torch

from mlxcel_b200.config import ModelConfig, preset
from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams
from mlxcel_b200.models.decoder import DecoderModel
from mlxcel_b200.models.weights import random_weights


def _eng(cfg, w, **kw):
    base = dict(max_batch=4, max_num_batched_tokens=128, num_blocks=64, max_model_len=256, cuda_graphs=False)
    base.update(kw)
    return Engine(DecoderModel(cfg, w), cfg, EngineConfig(**base))


FAMILIES = ["tiny-llama", "tiny-qwen3", "tiny-moe", "tiny-gpt-oss"]


@pytest.mark.parametrize("name", FAMILIES)
def test_family_batch_invariance(name):
    cfg = preset(name)
    w = random_weights(cfg, seed=4, dtype=torch.float32, std=0.05)
    g = torch.Generator().manual_seed(3)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 50, 21)]
    sp = SamplingParams(max_tokens=6, ignore_eos=True)
    alone = [_eng(cfg, w).generate([p], sp)[0].output for p in prompts]
    batched = [s.output for s in _eng(cfg, w, prefill_chunk_alone=16, prefill_chunk_contended=8).generate(prompts, sp)]
    assert alone == batched


def test_gemma_style_config_runs():
    cfg = ModelConfig.from_dict(dict(model_type="gemma2", num_hidden_layers=2, hidden_size=128,
                                     num_attention_heads=4, num_key_value_heads=2, head_dim=32,
                                     intermediate_size=256, vocab_size=512, sliding_window=16,
                                     attn_logit_softcapping=50.0, final_logit_softcapping=30.0,
                                     query_pre_attn_scalar=32))
    assert cfg.post_norms and cfg.norm_weight_bias == 1.0 and cfg.layer_window(0) == 16 and cfg.layer_window(1) == 0
    w = random_weights(cfg, seed=1, dtype=torch.float32, std=0.05)
    out = _eng(cfg, w).generate([[1, 2, 3, 4, 5] * 6], SamplingParams(max_tokens=5, ignore_eos=True))[0].output
    assert len(out) == 5


def test_eos_and_stop_tokens_and_prefix_cache():
    cfg = preset("tiny-llama")
    w = random_weights(cfg, seed=2, dtype=torch.float32, std=0.05)
    eng = _eng(cfg, w)
    prompt = list(range(40))
    first = eng.generate([prompt], SamplingParams(max_tokens=8, ignore_eos=True))[0]
    # the second token as a stop id ends the sequence right before it
    stop = first.output[1]
    s2 = eng.generate([prompt], SamplingParams(max_tokens=8, stop_token_ids=[stop]))[0]
    assert s2.output == first.output[:1] and s2.finish_reason.value == "stop"
    # the second run adopted cached prefix blocks (2 full blocks of 16)
    assert s2.num_cached == 32 and eng.stats["prefix_hit_tokens"] >= 32
    # and a cached prefix must not change the tokens
    s3 = eng.generate([prompt], SamplingParams(max_tokens=8, ignore_eos=True))[0]
    assert s3.output == first.output


def test_preemption_recompute_keeps_tokens():
    cfg = preset("tiny-llama")
    w = random_weights(cfg, seed=6, dtype=torch.float32, std=0.05)
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab_size, (30,), generator=g).tolist() for _ in range(3)]
    sp = SamplingParams(max_tokens=20, ignore_eos=True)
    want = [s.output for s in _eng(cfg, w, prefix_cache=False).generate(prompts, sp)]
    tight = _eng(cfg, w, num_blocks=9, prefix_cache=False, watermark=0.0)   # 144 slots for 150 tokens
    got = [s.output for s in tight.generate(prompts, sp)]
    assert got == want and tight.stats["preemptions"] >= 1
