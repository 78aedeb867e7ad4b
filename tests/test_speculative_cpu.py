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


def test_block_drafter_is_lossless_and_matches_a_dense_statement():
    """DFlash-style block drafter: (1) one drafting forward on the paged kernels equals a dense PyTorch
    statement of the same block (context keys from the projected target states, bidirectional
    attention inside the block, block keys not cached); (2) generation with the drafter is
    token-identical to plain greedy decoding, alone and in a batch with chunked prefill."""
    import torch

    from mlxcel_b200.config import ModelConfig, preset
    from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams
    from mlxcel_b200.models.decoder import DecoderModel
    from mlxcel_b200.models.weights import random_weights
    from mlxcel_b200.ops import reference as ref
    from mlxcel_b200.speculative import DFlashDrafter, random_dflash_weights

    cfg = preset("tiny-llama")
    w = random_weights(cfg, seed=3, dtype=torch.float32, std=0.05)
    dcfg = ModelConfig.from_dict(dict(model_type="qwen3", hidden_size=cfg.hidden_size, num_hidden_layers=2, num_attention_heads=4,
                                      num_key_value_heads=2, head_dim=16, intermediate_size=96, vocab_size=cfg.vocab_size,
                                      rms_norm_eps=1e-6))
    layers = [0, cfg.num_hidden_layers - 1]
    dw = random_dflash_weights(dcfg, len(layers), seed=5, dtype=torch.float32)
    L, mask_id = 6, cfg.vocab_size - 1

    def engine(with_drafter: bool, **kw):
        base = dict(max_batch=4, max_num_batched_tokens=32, num_blocks=64, block_size=8, max_model_len=128, cuda_graphs=False,
                    prefix_cache=False)
        base.update(kw)
        e = Engine(DecoderModel(cfg, w), cfg, EngineConfig(**base))
        if with_drafter:
            e.drafter = DFlashDrafter(e.model, dcfg, dw, layers, mask_id, num_blocks=64, block=L, block_size=8)
            e.spec_k = L
        return e

    g = torch.Generator().manual_seed(9)
    p1 = torch.randint(0, cfg.vocab_size - 1, (13,), generator=g).tolist()
    p2 = torch.randint(0, cfg.vocab_size - 1, (40,), generator=g).tolist()
    sp = SamplingParams(max_tokens=24, temperature=0.0, ignore_eos=True)
    plain = [s.output for s in engine(False).generate([p1, p2], sp)]
    e = engine(True)
    spec = [s.output for s in e.generate([p1, p2], sp)]
    assert spec == plain
    assert e.stats["spec_rounds"] > 0 and e.drafter.stats["blocks"] > 0 and not e.drafter.pending and not e.drafter.ctx_len
    alone = engine(True, prefill_chunk_alone=8, prefill_chunk_contended=8).generate([p2], sp)[0].output
    assert alone == plain[1]

    # (1) the drafting forward against a dense statement
    e = engine(True)
    sid = e.add_request(p1, SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))
    while not e.seqs[sid].output:
        e.step()                                        # prefill: context rows for the whole prompt are pending
    s = e.seqs[sid]
    dr = e.drafter
    start, ctx = dr.pending[sid]
    assert start == 0 and ctx.shape[0] == len(p1) and sid not in dr.ctx_len
    bonus = s.tokens[-1]
    got = dr._draft(e, [(s, ctx, bonus)])[0]
    # dense: keys / values of the context rows + the block, queries of the block, no mask inside the block
    emb = w.embed
    x = emb[torch.tensor([bonus] + [mask_id] * (L - 1))].float()
    S = ctx.shape[0]
    pos_c, pos_b = torch.arange(S), torch.arange(S, S + L)
    Hq, Hkv, D = 4, 2, 16
    inv = ref.rope_inv_freq(D, dcfg.rope_theta, None)[0]

    def rms(t, wt):
        t = t.float()
        return t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + 1e-6) * wt.float()

    def heads(t, n, pos, norm_w):
        t = ref.head_rmsnorm(t.view(-1, n, D), norm_w, 1e-6)
        return ref.apply_rope(t, pos.int(), inv, D, False, 1.0).float()
    for lw in dw.layers:
        xn = rms(x, lw.ln1)
        qkv_b = xn @ lw.wqkv.float().t()
        kv_c = ctx.float() @ lw.wqkv[Hq * D:].float().t()
        q = heads(qkv_b[:, :Hq * D], Hq, pos_b, lw.q_norm)
        k = torch.cat([heads(kv_c[:, :Hkv * D], Hkv, pos_c, lw.k_norm), heads(qkv_b[:, Hq * D:(Hq + Hkv) * D], Hkv, pos_b, lw.k_norm)])
        v = torch.cat([kv_c[:, Hkv * D:].view(-1, Hkv, D), qkv_b[:, (Hq + Hkv) * D:].view(-1, Hkv, D)]).float()
        k, v = k.repeat_interleave(Hq // Hkv, 1), v.repeat_interleave(Hq // Hkv, 1)
        att = torch.einsum("qhd,khd->hqk", q, k) / D ** 0.5
        a = torch.einsum("hqk,khd->qhd", att.softmax(-1), v).reshape(L, Hq * D)
        x = x + a @ lw.wo.float().t()
        xm = rms(x, lw.ln2)
        gu = xm @ lw.w_gate_up.float().t()
        I = gu.shape[1] // 2
        x = x + (torch.nn.functional.silu(gu[:, :I]) * gu[:, I:]) @ lw.w_down.float().t()
    want = (rms(x, dw.final_norm) @ w.lm_head.float().t())[1:].argmax(-1).tolist()
    assert got == want


def test_block_drafter_directory_round_trip_and_cli_attach(tmp_path):
    """A block-drafter directory (config with target_layer_ids / mask_token_id / block_size) is
    recognised by ``--draft-model``, loads back to the same weights, and generation stays lossless."""
    import argparse

    import torch

    from mlxcel_b200 import cli
    from mlxcel_b200.config import ModelConfig, preset
    from mlxcel_b200.engine import EngineConfig, SamplingParams
    from mlxcel_b200.llm import LLM
    from mlxcel_b200.models.weights import random_weights
    from mlxcel_b200.speculative.dflash import DFlashDrafter, is_dflash_dir, load_dflash, random_dflash_weights, save_dflash

    cfg = preset("tiny-llama")
    dcfg = ModelConfig.from_dict(dict(model_type="qwen3", hidden_size=cfg.hidden_size, num_hidden_layers=1, num_attention_heads=2,
                                      num_key_value_heads=1, head_dim=32, intermediate_size=64, vocab_size=cfg.vocab_size,
                                      rms_norm_eps=1e-6))
    dw = random_dflash_weights(dcfg, 2, seed=1, dtype=torch.float32)
    d = tmp_path / "drafter"
    save_dflash(d, dcfg, dw, block=5, mask_token_id=7, target_layers=[0, 1])
    assert is_dflash_dir(d) and not is_dflash_dir(tmp_path)
    dcfg2, w2, info = load_dflash(d, dtype=torch.float32)
    assert info == dict(block=5, mask_token_id=7, target_layers=[0, 1]) and dcfg2.head_dim == 32
    assert torch.equal(w2.fc, dw.fc) and torch.equal(w2.layers[0].wqkv, dw.layers[0].wqkv) and w2.embed is None

    def llm():
        w = random_weights(cfg, seed=3, dtype=torch.float32, std=0.05)
        return LLM(cfg, w, EngineConfig(max_batch=2, max_num_batched_tokens=32, num_blocks=64, block_size=8, max_model_len=96,
                                        cuda_graphs=False, prefix_cache=False))
    prompt = list(range(5, 25))
    sp = SamplingParams(max_tokens=16, temperature=0.0, ignore_eos=True)
    plain = llm().generate(prompt_token_ids=[prompt], sampling_params=sp)[0].output
    m = llm()
    cli.attach_drafter(m, argparse.Namespace(draft_model=str(d), prompt_lookup=False, draft_max=4), "cpu")
    assert isinstance(m.engine.drafter, DFlashDrafter) and m.engine.spec_k == 5
    assert m.generate(prompt_token_ids=[prompt], sampling_params=sp)[0].output == plain
    assert m.engine.stats["spec_rounds"] > 0
