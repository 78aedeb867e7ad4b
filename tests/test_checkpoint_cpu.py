"""Checkpoint round trip: save an MLX-style directory (bf16 and affine 4-bit / mxfp4) and load it
back through the name sanitiser; generation from the loaded weights must equal the original."""
import torch

from mlxcel_b200.config import ModelConfig
from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams
from mlxcel_b200.loading.checkpoint import load_full_weights, save_checkpoint
from mlxcel_b200.models.decoder import DecoderModel
from mlxcel_b200.models.weights import QuantizedTensor, random_weights
from mlxcel_b200.ops import quant

LLAMA = dict(model_type="llama", num_hidden_layers=2, hidden_size=128, num_attention_heads=4,
             num_key_value_heads=2, head_dim=32, intermediate_size=256, vocab_size=320, rms_norm_eps=1e-5)
GPTOSS = dict(model_type="gpt_oss", num_hidden_layers=2, hidden_size=128, num_attention_heads=4,
              num_key_value_heads=2, head_dim=32, intermediate_size=128, vocab_size=320,
              num_local_experts=4, num_experts_per_tok=2, sliding_window=16)


def _gen(cfg, w):
    eng = Engine(DecoderModel(cfg, w), cfg, EngineConfig(max_batch=2, max_num_batched_tokens=64, num_blocks=32,
                                                         max_model_len=128, cuda_graphs=False))
    return eng.generate([list(range(3, 30))], SamplingParams(max_tokens=6, ignore_eos=True))[0].output


def test_roundtrip_bf16_and_moe(tmp_path):
    for cd in (LLAMA, GPTOSS):
        cfg = ModelConfig.from_dict(cd)
        w = random_weights(cfg, seed=1, dtype=torch.float32, std=0.05)
        save_checkpoint(tmp_path / cd["model_type"], cd, w)
        w2 = load_full_weights(tmp_path / cd["model_type"], cfg, dtype=torch.float32)
        assert _gen(cfg, w) == _gen(cfg, w2)


def test_roundtrip_quantized(tmp_path):
    cfg = ModelConfig.from_dict(LLAMA)
    w = random_weights(cfg, seed=2, dtype=torch.float32, std=0.05)
    for mode, bits, group in (("affine", 4, 64), ("mxfp4", 4, 32)):
        for lw in w.layers:
            for name in ("wqkv", "wo", "w_gate_up", "w_down"):
                v = getattr(lw, name)
                if not isinstance(v, QuantizedTensor):
                    setattr(lw, name, quant.quantize(v, mode, bits, group, dtype=torch.float32))
        d = tmp_path / mode
        save_checkpoint(d, LLAMA, w, quantization=dict(mode=mode, bits=bits, group_size=group))
        cfg2 = ModelConfig.from_path(d)
        assert cfg2.quantization.mode == mode
        w2 = load_full_weights(d, cfg2, dtype=torch.float32)
        assert isinstance(w2.layers[0].wqkv, QuantizedTensor) and w2.layers[0].wqkv.mode == mode
        assert _gen(cfg, w) == _gen(cfg2, w2)
        # dequantize-at-load gives the same tokens
        w3 = load_full_weights(d, cfg2, dtype=torch.float32, dequantize=True)
        assert _gen(cfg, w) == _gen(cfg2, w3)
        # reset to dense for the next mode
        w = random_weights(cfg, seed=2, dtype=torch.float32, std=0.05)


def test_fp8_block_scaled_and_per_channel_checkpoints_load(tmp_path):
    """DeepSeek-V3 style block-scaled FP8 (``weight_scale_inv`` per 128 x 128 tile, here 32 x 32) and
    compressed-tensors style per-channel FP8 (``weight_scale``) are widened at load: the loaded matrices
    equal fp8 * scale, and the logits equal those of a checkpoint holding the widened weights."""
    import json

    import torch
    from safetensors.torch import load_file, save_file

    from mlxcel_b200.config import ModelConfig, preset
    from mlxcel_b200.loading.checkpoint import load_full_weights, save_checkpoint
    from mlxcel_b200.models.weights import random_weights

    cfg = preset("tiny-llama")
    src = tmp_path / "bf16"
    save_checkpoint(src, cfg.to_dict() | {"model_type": "llama"}, random_weights(cfg, seed=0, dtype=torch.bfloat16, std=0.05))
    t = {k: v.clone() for k, v in load_file(str(src / "model.safetensors")).items()}
    raw = json.loads((src / "config.json").read_text())
    raw.pop("quantization", None)

    def write(name, tensors, qc):
        d = tmp_path / name
        d.mkdir()
        save_file(tensors, str(d / "model.safetensors"), metadata={"format": "pt"})
        (d / "config.json").write_text(json.dumps(raw | {"quantization_config": qc}))
        return d

    B = 32
    block, chan, wide = {}, {}, {}
    for k, v in t.items():
        if k.endswith("_proj.weight") and v.dim() == 2:
            w = v.float()
            n, kk = w.shape
            pad = torch.zeros((n + B - 1) // B * B, (kk + B - 1) // B * B)
            pad[:n, :kk] = w
            tiles = pad.view(pad.shape[0] // B, B, pad.shape[1] // B, B)
            sc = tiles.abs().amax(dim=(1, 3)).clamp_min(1e-8) / 448.0
            q = (tiles / sc[:, None, :, None]).view_as(pad)[:n, :kk].to(torch.float8_e4m3fn)
            block[k], block[k[:-7] + ".weight_scale_inv"] = q, sc
            wide[k] = (q.float() * sc.repeat_interleave(B, 0)[:n].repeat_interleave(B, 1)[:, :kk]).to(torch.bfloat16)
            cs = w.abs().amax(dim=1, keepdim=True).clamp_min(1e-8) / 448.0
            chan[k], chan[k[:-7] + ".weight_scale"] = (w / cs).to(torch.float8_e4m3fn), cs
        else:
            block[k] = chan[k] = wide[k] = v
    d_block = write("fp8_block", block, dict(quant_method="fp8", fmt="e4m3", weight_block_size=[B, B]))
    d_chan = write("fp8_chan", chan, dict(quant_method="compressed-tensors", format="float-quantized"))
    d_wide = write("wide", wide, None)
    c_block = ModelConfig.from_path(d_block)
    assert c_block.quantization.mode == "none" and c_block.extra["fp8_block_size"] == (B, B)
    w_block = load_full_weights(d_block, c_block, dtype=torch.bfloat16)
    w_wide = load_full_weights(d_wide, ModelConfig.from_path(d_wide), dtype=torch.bfloat16)
    for a, b in zip(w_block.layers, w_wide.layers):
        assert torch.equal(a.wqkv, b.wqkv) and torch.equal(a.w_down, b.w_down) and a.wqkv.dtype == torch.bfloat16
    w_chan = load_full_weights(d_chan, ModelConfig.from_path(d_chan), dtype=torch.bfloat16)
    ref = load_full_weights(src, ModelConfig.from_path(src), dtype=torch.bfloat16)
    for a, b in zip(w_chan.layers, ref.layers):
        err = (a.wo.float() - b.wo.float()).abs().max().item()
        assert err < 0.07 * b.wo.float().abs().max().item()          # e4m3 keeps 3 mantissa bits


def test_internlm2_and_baichuan_layouts_load_like_their_llama_form(tmp_path):
    """The same weights written in InternLM2's layout (grouped wqkv, w1/w3/w2, tok_embeddings / output) and
    in Baichuan's (W_pack) load into the executor layout of the plain Llama checkpoint they came from."""
    import json

    import torch
    from safetensors.torch import load_file, save_file

    from mlxcel_b200.config import ModelConfig, preset
    from mlxcel_b200.loading.checkpoint import load_full_weights, save_checkpoint
    from mlxcel_b200.models.weights import random_weights

    cfg = preset("tiny-llama")
    src = tmp_path / "llama"
    save_checkpoint(src, cfg.to_dict() | {"model_type": "llama", "tie_word_embeddings": False},
                    random_weights(ModelConfig.from_dict(cfg.to_dict() | {"tie_word_embeddings": False}), seed=0,
                                   dtype=torch.bfloat16, std=0.05))
    t = {k: v.clone() for k, v in load_file(str(src / "model.safetensors")).items()}
    raw = json.loads((src / "config.json").read_text())
    Hq, Hkv, D, L = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.num_hidden_layers
    g = Hq // Hkv
    il = {"model.tok_embeddings.weight": t["model.embed_tokens.weight"], "model.norm.weight": t["model.norm.weight"],
          "output.weight": t["lm_head.weight"]}
    for i in range(L):
        p, o = f"model.layers.{i}.", f"model.layers.{i}."
        q = t[p + "self_attn.q_proj.weight"].view(Hkv, g, D, -1)
        k = t[p + "self_attn.k_proj.weight"].view(Hkv, 1, D, -1)
        v = t[p + "self_attn.v_proj.weight"].view(Hkv, 1, D, -1)
        il[o + "attention.wqkv.weight"] = torch.cat([q, k, v], 1).reshape((Hq + 2 * Hkv) * D, -1).contiguous()
        il[o + "attention.wo.weight"] = t[p + "self_attn.o_proj.weight"]
        il[o + "attention_norm.weight"], il[o + "ffn_norm.weight"] = t[p + "input_layernorm.weight"], t[p + "post_attention_layernorm.weight"]
        for a, b in (("w1", "gate_proj"), ("w3", "up_proj"), ("w2", "down_proj")):
            il[o + f"feed_forward.{a}.weight"] = t[p + f"mlp.{b}.weight"]
    d = tmp_path / "internlm2"
    d.mkdir()
    save_file(il, str(d / "model.safetensors"), metadata={"format": "pt"})
    (d / "config.json").write_text(json.dumps(raw | {"model_type": "internlm2"}))
    ref = load_full_weights(src, ModelConfig.from_path(src), dtype=torch.bfloat16)
    got = load_full_weights(d, ModelConfig.from_path(d), dtype=torch.bfloat16)
    assert torch.equal(got.embed, ref.embed) and torch.equal(got.lm_head, ref.lm_head)
    for a, b in zip(got.layers, ref.layers):
        for f in ("wqkv", "wo", "w_gate_up", "w_down", "ln1", "ln2"):
            assert torch.equal(getattr(a, f), getattr(b, f)), f
    if Hq == Hkv:                                               # Baichuan is multi-head attention only
        bc = dict(t)
        for i in range(L):
            p = f"model.layers.{i}.self_attn."
            bc[p + "W_pack.weight"] = torch.cat([bc.pop(p + "q_proj.weight"), bc.pop(p + "k_proj.weight"), bc.pop(p + "v_proj.weight")])
        d2 = tmp_path / "baichuan"
        d2.mkdir()
        save_file(bc, str(d2 / "model.safetensors"), metadata={"format": "pt"})
        (d2 / "config.json").write_text(json.dumps(raw | {"model_type": "baichuan"}))
        got2 = load_full_weights(d2, ModelConfig.from_path(d2), dtype=torch.bfloat16)
        assert all(torch.equal(a.wqkv, b.wqkv) for a, b in zip(got2.layers, ref.layers))


def test_index_entries_outside_the_checkpoint_directory_are_refused(tmp_path):
    """A weight_map entry may not lead out of the model directory: neither by ``..`` nor into a
    sibling directory whose name merely starts with the model's."""
    import json

    import pytest
    import torch
    from safetensors.torch import save_file

    from mlxcel_b200.loading.checkpoint import TensorSource

    model = tmp_path / "foo"
    evil = tmp_path / "foo-evil"
    model.mkdir()
    evil.mkdir()
    save_file({"a": torch.ones(2)}, str(model / "ok.safetensors"))
    save_file({"b": torch.ones(2)}, str(evil / "x.safetensors"))
    (model / "model.safetensors.index.json").write_text(json.dumps(
        {"weight_map": {"a": "ok.safetensors", "b": "../foo-evil/x.safetensors", "c": "missing.safetensors"}}))
    src = TensorSource(model)
    assert src.get("a").sum().item() == 2
    with pytest.raises(ValueError, match="outside"):
        src.get("b")
    with pytest.raises(ValueError, match="outside"):
        src.footprint()
    with pytest.raises(FileNotFoundError):
        src.get("c")


def test_nvfp4_checkpoint_is_expanded_at_load(tmp_path):
    """MLX ``nvfp4`` (e2m1 codes, one e4m3 scale per 16 inputs): the quantizer's values survive the
    checkpoint round trip, with and without the mode named in the config, as dense matrices."""
    cfg = ModelConfig.from_dict(LLAMA)
    w = random_weights(cfg, seed=5, dtype=torch.float32, std=0.05)
    want = {}
    for li, lw in enumerate(w.layers):
        for name in ("wqkv", "wo", "w_gate_up", "w_down"):
            q = quant.quantize(getattr(lw, name), "nvfp4", 4, 16)
            assert q.scales.dtype == torch.uint8 and q.group_size == 16
            deq = quant.dequantize_ref(q, torch.float32)
            rel = (deq - getattr(lw, name)).abs().max() / getattr(lw, name).abs().max()
            assert rel < 0.3                                         # 4-bit floats: coarse, but the right numbers
            want[(li, name)] = deq
            setattr(lw, name, q)
    for named in (True, False):
        d = tmp_path / f"nvfp4_{int(named)}"
        save_checkpoint(d, LLAMA, w, quantization=dict(mode="nvfp4", bits=4, group_size=16) if named else None)
        cfg2 = ModelConfig.from_path(d)
        w2 = load_full_weights(d, cfg2, dtype=torch.float32)
        for (li, name), t in want.items():
            got = getattr(w2.layers[li], name)
            assert isinstance(got, torch.Tensor) and torch.equal(got, t)


def test_exaone_telechat3_and_deepseek_v1_load_through_their_own_names(tmp_path):
    """EXAONE 3.x names (``transformer.h.N.attn.attention.*``, ``c_fc_0 / c_fc_1 / c_proj``) load into the
    executor layout of the Llama checkpoint they were written from; a TeleChat3 config (``telechat3-yarn``)
    gives the frequencies of the same config spelled ``yarn``; a DeepSeek-MoE (v1) config parses to
    softmax routing with shared experts and runs."""
    import json

    import torch
    from safetensors.torch import load_file, save_file

    from mlxcel_b200.config import ModelConfig, preset
    from mlxcel_b200.loading.checkpoint import load_full_weights, save_checkpoint
    from mlxcel_b200.models.weights import random_weights
    from mlxcel_b200.ops.reference import rope_inv_freq

    cfg = preset("tiny-llama")
    src = tmp_path / "llama"
    base = ModelConfig.from_dict(cfg.to_dict() | {"tie_word_embeddings": False})
    save_checkpoint(src, cfg.to_dict() | {"model_type": "llama", "tie_word_embeddings": False},
                    random_weights(base, seed=0, dtype=torch.bfloat16, std=0.05))
    t = load_file(str(src / "model.safetensors"))
    raw = json.loads((src / "config.json").read_text())
    ex = {"transformer.wte.weight": t["model.embed_tokens.weight"], "transformer.ln_f.weight": t["model.norm.weight"],
          "lm_head.weight": t["lm_head.weight"]}
    for i in range(cfg.num_hidden_layers):
        p, o = f"model.layers.{i}.", f"transformer.h.{i}."
        for n in ("q_proj", "k_proj", "v_proj"):
            ex[o + f"attn.attention.{n}.weight"] = t[p + f"self_attn.{n}.weight"]
        ex[o + "attn.attention.out_proj.weight"] = t[p + "self_attn.o_proj.weight"]
        ex[o + "ln_1.weight"], ex[o + "ln_2.weight"] = t[p + "input_layernorm.weight"], t[p + "post_attention_layernorm.weight"]
        for a, b in (("c_fc_0", "gate_proj"), ("c_fc_1", "up_proj"), ("c_proj", "down_proj")):
            ex[o + f"mlp.{a}.weight"] = t[p + f"mlp.{b}.weight"]
    d = tmp_path / "exaone"
    d.mkdir()
    save_file({k: v.contiguous() for k, v in ex.items()}, str(d / "model.safetensors"), metadata={"format": "pt"})
    r2 = {k: v for k, v in raw.items() if k != "num_hidden_layers"} | {"model_type": "exaone", "num_layers": cfg.num_hidden_layers,
                                                                        "layer_norm_epsilon": raw.get("rms_norm_eps", 1e-5)}
    (d / "config.json").write_text(json.dumps(r2))
    ref = load_full_weights(src, ModelConfig.from_path(src), dtype=torch.bfloat16)
    c2 = ModelConfig.from_path(d)
    got = load_full_weights(d, c2, dtype=torch.bfloat16)
    assert c2.num_hidden_layers == cfg.num_hidden_layers and torch.equal(got.embed, ref.embed) and torch.equal(got.final_norm, ref.final_norm)
    for a, b in zip(got.layers, ref.layers):
        for f in ("wqkv", "wo", "w_gate_up", "w_down", "ln1", "ln2"):
            assert torch.equal(getattr(a, f), getattr(b, f)), f
    ys = dict(factor=4.0, original_max_position_embeddings=64, beta_fast=32, beta_slow=1)
    ct = ModelConfig.from_dict(raw | {"model_type": "telechat3", "rope_scaling": ys | {"rope_type": "telechat3-yarn"}, "attention_bias": True})
    cy = ModelConfig.from_dict(raw | {"model_type": "llama", "rope_scaling": ys | {"rope_type": "yarn"}})
    fa, ma = rope_inv_freq(ct.rot_dim, ct.rope_theta, ct.rope_scaling)
    fb, mb = rope_inv_freq(cy.rot_dim, cy.rope_theta, cy.rope_scaling)
    assert torch.equal(fa, fb) and ma == mb and ct.attention_bias and not torch.equal(fa, rope_inv_freq(cy.rot_dim, cy.rope_theta, None)[0])
    cd = ModelConfig.from_dict(dict(model_type="deepseek", hidden_size=64, intermediate_size=128, moe_intermediate_size=32,
                                    num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=4, vocab_size=200,
                                    n_routed_experts=4, num_experts_per_tok=2, n_shared_experts=2, first_k_dense_replace=1,
                                    routed_scaling_factor=1.0, norm_topk_prob=False))
    assert cd.is_moe and cd.extra["moe_routing"]["score"] == "softmax" and cd.shared_expert_intermediate_size == 64
    assert cd.extra["first_k_dense"] == 1 and not cd.norm_topk_prob
    w = random_weights(cd, seed=1, dtype=torch.float32, std=0.05)
    assert w.layers[0].router_w is None and w.layers[1].router_w is not None and w.layers[1].shared_gate_up is not None
    assert len(_gen(cd, w)) == 6
