"""Block-unmasking generation for masked-diffusion language models: the block-causal forward on the
paged kernels against transformers with an explicit block-causal mask, and the schedule / reveal
rules of the denoising loop."""
import tempfile

import pytest
import torch

transformers = pytest.importorskip("transformers")

from mlxcel_b200.config import ModelConfig  # noqa: E402
from mlxcel_b200.engine.diffusion import (DiffusionGenerator, DiffusionOptions, block_threshold, transfer_mask,  # noqa: E402
                                          truncate_at_eos)
from mlxcel_b200.loading.checkpoint import load_full_weights  # noqa: E402
from mlxcel_b200.models.decoder import DecoderModel  # noqa: E402

MASK = 299


def _model():
    from transformers import LlamaConfig, LlamaForCausalLM
    torch.manual_seed(0)
    hc = LlamaConfig(hidden_size=64, intermediate_size=128, num_hidden_layers=2, num_attention_heads=4,
                     num_key_value_heads=2, vocab_size=300, max_position_embeddings=256)
    m = LlamaForCausalLM(hc).eval()
    d = tempfile.mkdtemp(prefix="diffusion_")
    m.save_pretrained(d, safe_serialization=True)
    cfg = ModelConfig.from_path(d)
    return m, DecoderModel(cfg, load_full_weights(d, cfg, dtype=torch.float32)), cfg


def test_block_causal_forward_matches_transformers_with_an_explicit_mask():
    m, ours, cfg = _model()
    L, T = 8, 24
    ids = torch.randint(0, 290, (T,), generator=torch.Generator().manual_seed(1))
    blk = torch.arange(T) // L
    allowed = blk[:, None] >= blk[None, :]                        # own block and every earlier one
    mask = torch.zeros(1, 1, T, T).masked_fill(~allowed, float("-inf"))
    with torch.no_grad():
        want = m(ids[None], attention_mask=mask).logits[0]
    g = DiffusionGenerator(ours, cfg, MASK, max_len=64)
    got = torch.cat([g._forward_block(ids[s:s + L].tolist(), s) for s in range(0, T, L)])
    assert (got - want).abs().max().item() < 2e-4
    # forwarding a block again (other tokens, then the final ones) leaves no trace of the first pass
    g2 = DiffusionGenerator(ours, cfg, MASK, max_len=64)
    g2._forward_block(ids[:L].tolist(), 0)
    g2._forward_block([MASK] * L, L)
    got2 = g2._forward_block(ids[L:2 * L].tolist(), L)
    assert (got2 - want[L:2 * L]).abs().max().item() < 2e-4


def test_schedule_and_reveal_rules():
    assert block_threshold(0, 4, 0.9, 0.3) == pytest.approx(0.9) and block_threshold(3, 4, 0.9, 0.3) == pytest.approx(0.3)
    assert block_threshold(1, 4, 0.9, 0.3) == pytest.approx(0.7) and block_threshold(0, 1, 0.9, 0.3) == 0.3
    conf = torch.tensor([0.99, 0.2, 0.6, 0.97])
    masked = torch.tensor([False, True, True, True])
    assert transfer_mask(conf, masked, 0.95).tolist() == [False, False, False, True]
    assert transfer_mask(conf, masked, 0.999).tolist() == [False, False, False, True]      # forced progress: the best one
    assert transfer_mask(conf, torch.tensor([False] * 4), 0.1).tolist() == [False] * 4
    assert truncate_at_eos([5, 6, 7, 8], {7}) == ([5, 6], True) and truncate_at_eos([5, 6], {7}) == ([5, 6], False)


def test_generation_loop_counts_and_stops():
    m, ours, cfg = _model()
    prompt = torch.randint(0, 290, (13,), generator=torch.Generator().manual_seed(2)).tolist()
    g = DiffusionGenerator(ours, cfg, MASK, max_len=128)
    # threshold 0: every block is revealed in one denoising forward (+ one commit forward per block)
    out = g.generate(prompt, DiffusionOptions(max_new_tokens=20, block_length=8, threshold=0.0, min_threshold=0.0))
    assert len(out) == 20 and MASK not in out
    # 13 prompt tokens: one full block committed, 5 join the first generation block (3 new), then 8, 8, 1
    assert g.stats["blocks"] == 4 and g.stats["forwards"] == 1 + 2 * 4 and g.stats["revealed"] == 20
    # an unreachable threshold reveals exactly one position per step
    g = DiffusionGenerator(ours, cfg, MASK, max_len=128)
    seen = []
    out2 = g.generate(prompt, DiffusionOptions(max_new_tokens=11, block_length=8, threshold=2.0, min_threshold=2.0),
                      on_block=seen.append)
    assert len(out2) == 11 and g.stats["forwards"] == 1 + (3 + 1) + (8 + 1) and [len(b) for b in seen] == [3, 8]
    # deterministic, and an end-of-sequence token ends the text at its block
    g = DiffusionGenerator(ours, cfg, MASK, max_len=128)
    assert g.generate(prompt, DiffusionOptions(max_new_tokens=11, block_length=8, threshold=2.0, min_threshold=2.0)) == out2
    g = DiffusionGenerator(ours, cfg, MASK, max_len=128)
    cut = g.generate(prompt, DiffusionOptions(max_new_tokens=20, block_length=8, threshold=0.0, min_threshold=0.0,
                                              eos_token_ids=[out[5]]))
    assert cut == out[:out.index(out[5])]
    with pytest.raises(ValueError):
        g.generate(prompt, DiffusionOptions(max_new_tokens=500))
