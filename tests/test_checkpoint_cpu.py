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
