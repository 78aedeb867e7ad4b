"""Hybrid Mamba2 / attention / MLP stack (Nemotron-H layout): greedy tokens through the engine
(chunked prefill, batching) against a whole-sequence forward written from the block equations;
checkpoint round trip through the CLI. CPU, fp32."""
import argparse

import torch
import torch.nn.functional as F

from mlxcel_b200.config import ModelConfig, preset
from mlxcel_b200.engine.engine import Engine, EngineConfig
from mlxcel_b200.engine.params import SamplingParams
from mlxcel_b200.models.hybrid import HybridModel, block_kinds, load_hybrid_weights, random_hybrid_weights
from mlxcel_b200.models.mamba2 import mamba_dims


def _naive_logits(cfg, w, tokens):
    d = mamba_dims(cfg)
    di, G, N, Hh, P, K = d["d_inner"], d["G"], d["N"], d["heads"], d["P"], d["K"]
    Hq, Hkv, D = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
    h = w.embed.float()[tokens]
    L = h.shape[0]
    rms = lambda x, g: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * g.float()  # noqa: E731
    for blk in w.blocks:
        x = rms(h, blk.norm)
        if blk.kind == "mamba2":
            lw = blk.mamba
            proj = x @ lw.in_proj.float().t()
            z, xBC, dt = proj[:, :di], proj[:, di:di + d["conv_dim"]], proj[:, di + d["conv_dim"]:]
            pad = torch.cat([torch.zeros(K - 1, d["conv_dim"]), xBC])
            conv = F.silu(torch.stack([(pad[t:t + K] * lw.conv_w.float().t()).sum(0) for t in range(L)]) + lw.conv_b.float())
            xs, Bm, Cm = conv[:, :di].reshape(L, Hh, P), conv[:, di:di + G * N].reshape(L, G, N), conv[:, di + G * N:].reshape(L, G, N)
            dtv = F.softplus(dt + lw.dt_bias.float())
            A = -torch.exp(lw.A_log.float())
            S = torch.zeros(Hh, P, N)
            ys = []
            for t in range(L):
                Bh, Ch = Bm[t].repeat_interleave(Hh // G, 0), Cm[t].repeat_interleave(Hh // G, 0)
                S = S * torch.exp(dtv[t] * A)[:, None, None] + (dtv[t][:, None] * xs[t])[..., None] * Bh[:, None, :]
                ys.append(((S * Ch[:, None, :]).sum(-1) + lw.D.float()[:, None] * xs[t]).reshape(-1))
            y = (torch.stack(ys) * F.silu(z)).reshape(L, G, -1)           # gated norm per B/C group
            y = (y * torch.rsqrt(y.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps)).reshape(L, di) * lw.gnorm.float()
            h = h + y @ lw.out_proj.float().t()
        elif blk.kind == "attention":
            qkv = x @ blk.attn.wqkv.float().t()
            q, k, v = qkv.split([Hq * D, Hkv * D, Hkv * D], -1)
            q, k, v = q.reshape(L, Hq, D), k.reshape(L, Hkv, D), v.reshape(L, Hkv, D)
            k, v = k.repeat_interleave(Hq // Hkv, 1), v.repeat_interleave(Hq // Hkv, 1)
            sc = torch.einsum("qhd,khd->hqk", q, k) / D ** 0.5               # no positional encoding
            sc = sc.masked_fill(torch.ones(L, L).triu(1).bool(), float("-inf"))
            a = torch.einsum("hqk,khd->qhd", sc.softmax(-1), v).reshape(L, Hq * D)
            h = h + a @ blk.attn.wo.float().t()
        else:
            h = h + torch.relu(x @ blk.up.float().t()).square() @ blk.down.float().t()
    return rms(h, w.final_norm) @ w.lm_head.float().t()


def test_hybrid_greedy_matches_naive_forward():
    cfg = preset("tiny-nemotron-h")
    assert block_kinds(cfg) == ["mamba2", "mlp", "mamba2", "attention", "mlp", "mamba2", "mlp"]
    w = random_hybrid_weights(cfg, seed=1, dtype=torch.float32, std=0.08)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (41, 6)]
    want = []
    for p in prompts:
        toks = list(p)
        for _ in range(5):
            toks.append(int(_naive_logits(cfg, w, torch.tensor(toks))[-1].argmax()))
        want.append(toks[len(p):])
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    for chunk in (256, 16):
        model = HybridModel(cfg, w, max_seqs=8)
        eng = Engine(model, cfg, EngineConfig(num_blocks=64, block_size=16, max_batch=8, max_model_len=256,
                                              max_num_batched_tokens=chunk))
        assert len(eng.pool.layers) == 1                     # only the attention block owns KV
        outs = eng.generate(prompts, sp)
        assert [s.output for s in outs] == want, chunk
        assert not model.ssm.slot_of


def test_hybrid_checkpoint_round_trip(tmp_path):
    from mlxcel_b200 import cli
    from mlxcel_b200.llm import LLM

    cli.cmd_random_init(argparse.Namespace(preset="tiny-nemotron-h", out=str(tmp_path), seed=3, quantize=None))
    cfg = ModelConfig.from_path(tmp_path)
    assert cfg.extra["hybrid_pattern"] == "M-M*-M-" and cfg.extra["mamba"]["norm_groups"] == 2
    w = load_hybrid_weights(tmp_path, cfg, dtype=torch.float32)
    assert [b.kind for b in w.blocks] == block_kinds(cfg) and len(w.layers) == 1
    llm = LLM.from_pretrained(tmp_path, device="cpu",
                              engine_config=EngineConfig(num_blocks=32, block_size=16, max_batch=4, max_model_len=128))
    assert type(llm.model).__name__ == "HybridModel"
    outs = llm.generate(prompt_token_ids=[[5, 6, 7, 8]], sampling_params=SamplingParams(max_tokens=3, ignore_eos=True))
    assert len(outs[0].output) == 3
