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


def test_dbrx_checkpoint_matches_a_plain_statement_of_the_model(tmp_path):
    """DBRX from its original checkpoint layout (MPT names, nested config, experts stacked as
    [E * I, H] with w2 used transposed): logits against a direct PyTorch statement of the model
    written here (bias-free LayerNorm, clamped fused Wqkv, rotary GQA attention, softmax over all
    experts -> top-k -> L1 renormalisation)."""
    import json

    from safetensors.torch import save_file

    from mlxcel_b200.llm import LLM

    torch.manual_seed(0)
    H, Hq, Hkv, D, I, E, k, V, L, clip = 64, 4, 2, 16, 48, 4, 2, 200, 2, 0.6
    cfgd = dict(model_type="dbrx", d_model=H, n_heads=Hq, n_layers=L, max_seq_len=256, vocab_size=V,
                attn_config=dict(kv_n_heads=Hkv, clip_qkv=clip, rope_theta=10000.0),
                ffn_config=dict(ffn_hidden_size=I, moe_num_experts=E, moe_top_k=k, moe_normalize_expert_weights=1.0,
                                ffn_act_fn=dict(name="silu")), tie_word_embeddings=False)
    r = lambda *s, sc=0.15: torch.randn(*s) * sc  # noqa: E731
    t = {"transformer.wte.weight": r(V, H, sc=0.5), "transformer.norm_f.weight": 1 + r(H, sc=0.1), "lm_head.weight": r(V, H)}
    for i in range(L):
        b = f"transformer.blocks.{i}."
        t[b + "norm_attn_norm.norm_1.weight"] = 1 + r(H, sc=0.1)
        t[b + "norm_attn_norm.norm_2.weight"] = 1 + r(H, sc=0.1)
        t[b + "norm_attn_norm.attn.Wqkv.weight"] = r((Hq + 2 * Hkv) * D, H, sc=0.3)
        t[b + "norm_attn_norm.attn.out_proj.weight"] = r(H, Hq * D)
        t[b + "ffn.router.layer.weight"] = r(E, H, sc=0.5)
        for n in ("w1", "v1", "w2"):
            t[b + f"ffn.experts.mlp.{n}"] = r(E * I, H)
    (tmp_path / "config.json").write_text(json.dumps(cfgd))
    save_file({n: v.contiguous() for n, v in t.items()}, str(tmp_path / "model.safetensors"))

    T = 19
    ids = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(2))
    F = torch.nn.functional
    inv = 1.0 / (10000.0 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.arange(T).float()[:, None] * inv[None]
    cos, sin = torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)
    rot = lambda x: x * cos[:, None] + torch.cat([-x[..., D // 2:], x[..., :D // 2]], -1) * sin[:, None]  # noqa: E731
    h = t["transformer.wte.weight"][ids]
    for i in range(L):
        b = f"transformer.blocks.{i}."
        x = F.layer_norm(h, (H,), t[b + "norm_attn_norm.norm_1.weight"], None, 1e-5)
        qkv = (x @ t[b + "norm_attn_norm.attn.Wqkv.weight"].t()).clamp(-clip, clip)
        q, kk, v = qkv.split([Hq * D, Hkv * D, Hkv * D], -1)
        q, kk, v = rot(q.view(T, Hq, D)), rot(kk.view(T, Hkv, D)), v.view(T, Hkv, D)
        kk, v = kk.repeat_interleave(Hq // Hkv, 1), v.repeat_interleave(Hq // Hkv, 1)
        sc = torch.einsum("qhd,khd->hqk", q, kk) / D ** 0.5
        sc = sc.masked_fill(torch.triu(torch.ones(T, T, dtype=torch.bool), 1), float("-inf"))
        a = torch.einsum("hqk,khd->qhd", sc.softmax(-1), v).reshape(T, Hq * D)
        h = h + a @ t[b + "norm_attn_norm.attn.out_proj.weight"].t()
        x = F.layer_norm(h, (H,), t[b + "norm_attn_norm.norm_2.weight"], None, 1e-5)
        p = (x @ t[b + "ffn.router.layer.weight"].t()).softmax(-1)
        w, idx = p.topk(k, -1)
        w = w / w.sum(-1, keepdim=True)
        w1, v1, w2 = (t[b + f"ffn.experts.mlp.{n}"].view(E, I, H) for n in ("w1", "v1", "w2"))
        y = torch.zeros_like(x)
        for tok in range(T):
            for s in range(k):
                e = int(idx[tok, s])
                y[tok] += w[tok, s] * ((F.silu(x[tok] @ w1[e].t()) * (x[tok] @ v1[e].t())) @ w2[e])
        h = h + y
    want = F.layer_norm(h, (H,), t["transformer.norm_f.weight"], None, 1e-5) @ t["lm_head.weight"].t()
    assert (qkv.abs() == clip).any()                      # the clamp is active in this test

    from mlxcel_b200.cache.kv_pool import KVPool
    from mlxcel_b200.loading.checkpoint import load_full_weights
    from mlxcel_b200.models.decoder import StepBatch
    cfg = ModelConfig.from_path(str(tmp_path))
    assert cfg.num_experts == E and cfg.extra["clip_qkv"] == clip and cfg.num_key_value_heads == Hkv
    model = DecoderModel(cfg, load_full_weights(str(tmp_path), cfg, dtype=torch.float32))
    pool = KVPool(cfg, 4, 16, device="cpu", dtype=torch.float32, num_layers=L)
    sb = StepBatch(token_ids=ids.int(), positions=torch.arange(T, dtype=torch.int32), slot_mapping=torch.arange(T, dtype=torch.int32),
                   num_prefill_seqs=1, pf_block_tables=torch.arange(4, dtype=torch.int32)[None],
                   pf_cu_q=torch.tensor([0, T], dtype=torch.int32), pf_context_lens=torch.tensor([T], dtype=torch.int32),
                   pf_max_q_len=T, pf_cu_q_host=[0, T], logits_rows=torch.arange(T))
    got = model.forward(sb, pool.layers).float()
    assert (got - want).abs().max().item() < 2e-3 * max(1.0, want.abs().max().item())
    # and through the public loader + engine (bf16 weights): the first greedy token agrees
    llm = LLM.from_pretrained(str(tmp_path), device="cpu",
                              engine_config=EngineConfig(max_batch=2, max_num_batched_tokens=64, num_blocks=32,
                                                         max_model_len=128, cuda_graphs=False))
    out = llm.generate(prompt_token_ids=[ids.tolist()], sampling_params=SamplingParams(max_tokens=3, temperature=0.0, ignore_eos=True))[0]
    top2 = want[-1].topk(2).values
    if float(top2[0] - top2[1]) > 0.05:
        assert out.output[0] == int(want[-1].argmax())


def test_bitnet_packed_checkpoint_equals_its_dense_expansion(tmp_path):
    """A BitNet checkpoint with BitLinear storage (uint8, four output rows per byte, one scale that
    divides the output) gives the logits of the same model saved with dense ternary / scale weights."""
    import json

    from safetensors.torch import save_file

    from mlxcel_b200.cache.kv_pool import KVPool
    from mlxcel_b200.loading.checkpoint import load_full_weights
    from mlxcel_b200.models.decoder import StepBatch

    torch.manual_seed(0)
    H, Hq, Hkv, D, I, V, L = 64, 4, 2, 16, 96, 200, 2
    cfgd = dict(model_type="bitnet", hidden_size=H, num_attention_heads=Hq, num_key_value_heads=Hkv, num_hidden_layers=L,
                intermediate_size=I, vocab_size=V, max_position_embeddings=128, rms_norm_eps=1e-5, rope_theta=10000.0,
                hidden_act="relu2", tie_word_embeddings=True)
    dense, packed = {}, {}

    def put_linear(name, n, k):
        tern = torch.randint(-1, 2, (n, k))
        scale = torch.rand(1) * 20 + 5
        dense[name + ".weight"] = tern.float() / scale
        codes = (tern + 1).to(torch.uint8).view(4, n // 4, k)            # output row r + i * n / 4 -> bits 2i of row r
        packed[name + ".weight"] = (codes[0] | (codes[1] << 2) | (codes[2] << 4) | (codes[3] << 6)).contiguous()
        packed[name + ".weight_scale"] = scale

    def put(name, t):
        dense[name] = packed[name] = t

    put("model.embed_tokens.weight", torch.randn(V, H) * 0.5)
    put("model.norm.weight", 1 + torch.randn(H) * 0.1)
    for i in range(L):
        p = f"model.layers.{i}."
        put(p + "input_layernorm.weight", 1 + torch.randn(H) * 0.1)
        put(p + "post_attention_layernorm.weight", 1 + torch.randn(H) * 0.1)
        put(p + "self_attn.attn_sub_norm.weight", 1 + torch.randn(H) * 0.1)
        put(p + "mlp.ffn_sub_norm.weight", 1 + torch.randn(I) * 0.1)
        for n, (rows, cols) in dict(q_proj=(Hq * D, H), k_proj=(Hkv * D, H), v_proj=(Hkv * D, H), o_proj=(H, Hq * D)).items():
            put_linear(p + "self_attn." + n, rows, cols)
        for n, (rows, cols) in dict(gate_proj=(I, H), up_proj=(I, H), down_proj=(H, I)).items():
            put_linear(p + "mlp." + n, rows, cols)
    logits = []
    T = 17
    ids = torch.randint(0, V, (T,), generator=torch.Generator().manual_seed(3))
    for name, tensors in (("dense", dense), ("packed", packed)):
        d = tmp_path / name
        d.mkdir()
        (d / "config.json").write_text(json.dumps(cfgd))
        save_file({k: v.contiguous() for k, v in tensors.items()}, str(d / "model.safetensors"))
        cfg = ModelConfig.from_path(str(d))
        model = DecoderModel(cfg, load_full_weights(str(d), cfg, dtype=torch.float32))
        pool = KVPool(cfg, 4, 16, device="cpu", dtype=torch.float32, num_layers=L)
        sb = StepBatch(token_ids=ids.int(), positions=torch.arange(T, dtype=torch.int32), slot_mapping=torch.arange(T, dtype=torch.int32),
                       num_prefill_seqs=1, pf_block_tables=torch.arange(4, dtype=torch.int32)[None],
                       pf_cu_q=torch.tensor([0, T], dtype=torch.int32), pf_context_lens=torch.tensor([T], dtype=torch.int32),
                       pf_max_q_len=T, pf_cu_q_host=[0, T], logits_rows=torch.arange(T))
        logits.append(model.forward(sb, pool.layers).float())
        assert model.w.layers[0].attn_sub_norm is not None and model.w.layers[0].ffn_sub_norm is not None
    assert torch.isfinite(logits[0]).all() and logits[0].abs().max() > 0.1
    assert (logits[0] - logits[1]).abs().max().item() < 1e-4 * max(1.0, logits[0].abs().max().item())
