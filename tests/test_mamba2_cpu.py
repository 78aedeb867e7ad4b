"""Mamba2 (state-space) model family: the ragged conv / scan operators against a plain per-sequence
statement of the recurrence, chunked prefill and continuous batching through the engine, and a
checkpoint round trip. CPU, fp32."""
import torch
import torch.nn.functional as F

from mlxcel_b200.config import ModelConfig, preset
from mlxcel_b200.engine.engine import Engine, EngineConfig
from mlxcel_b200.engine.params import SamplingParams
from mlxcel_b200.models.mamba2 import (Mamba2Model, load_mamba2_weights, mamba_dims, random_mamba2_weights,
                                       save_mamba2_checkpoint)


def _naive_logits(cfg, w, tokens):
    """Whole-sequence Mamba2 forward written directly from the block's equations."""
    d = mamba_dims(cfg)
    di, G, N, Hh, P, K = d["d_inner"], d["G"], d["N"], d["heads"], d["P"], d["K"]
    h = w.embed.float()[tokens]
    L = h.shape[0]
    rms = lambda x, g: x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + cfg.rms_norm_eps) * g.float()  # noqa: E731
    for lw in w.layers:
        proj = rms(h, lw.norm) @ lw.in_proj.float().t()
        z, xBC, dt = proj[:, :di], proj[:, di:di + d["conv_dim"]], proj[:, di + d["conv_dim"]:]
        pad = torch.cat([torch.zeros(K - 1, d["conv_dim"]), xBC])
        conv = torch.stack([(pad[t:t + K] * lw.conv_w.float().t()).sum(0) for t in range(L)]) + lw.conv_b.float()
        conv = F.silu(conv)
        xs, Bm, Cm = conv[:, :di].reshape(L, Hh, P), conv[:, di:di + G * N].reshape(L, G, N), conv[:, di + G * N:].reshape(L, G, N)
        dtv = F.softplus(dt + lw.dt_bias.float())
        A = -torch.exp(lw.A_log.float())
        S = torch.zeros(Hh, P, N)
        ys = []
        for t in range(L):
            Bh, Ch = Bm[t].repeat_interleave(Hh // G, 0), Cm[t].repeat_interleave(Hh // G, 0)
            S = S * torch.exp(dtv[t] * A)[:, None, None] + (dtv[t][:, None] * xs[t])[..., None] * Bh[:, None, :]
            ys.append(((S * Ch[:, None, :]).sum(-1) + lw.D.float()[:, None] * xs[t]).reshape(-1))
        y = torch.stack(ys) * F.silu(z)
        h = h + rms(y, lw.gnorm) @ lw.out_proj.float().t()
    return rms(h, w.final_norm) @ w.lm_head.float().t()


def _engine(cfg, w, **kw):
    model = Mamba2Model(cfg, w, max_seqs=16)
    return Engine(model, cfg, EngineConfig(num_blocks=64, block_size=16, max_batch=8, max_model_len=256, **kw))


def test_mamba2_greedy_matches_naive_forward_with_chunked_prefill_and_batching():
    cfg = preset("tiny-mamba2")
    w = random_mamba2_weights(cfg, seed=1, dtype=torch.float32, std=0.08)
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (37, 5, 64)]
    want = []
    for p in prompts:
        toks = list(p)
        for _ in range(6):
            toks.append(int(_naive_logits(cfg, w, torch.tensor(toks))[-1].argmax()))
        want.append(toks[len(p):])
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    # whole-prompt prefill, then small chunks (state carried from chunk to chunk)
    for chunk in (256, 16):
        eng = _engine(cfg, w, max_num_batched_tokens=chunk)
        outs = eng.generate(prompts, sp)
        assert [s.output for s in outs] == want, chunk
        assert not eng.model.slot_of           # every state slot went back
    assert eng.ecfg.prefix_cache is False and eng.ecfg.cuda_graphs is False


def test_mamba2_two_groups_and_checkpoint_round_trip(tmp_path):
    raw = dict(model_type="mamba2", num_hidden_layers=2, hidden_size=64, num_heads=4, head_dim=32,
               state_size=16, conv_kernel=3, n_groups=2, vocab_size=300, tie_word_embeddings=False,
               time_step_limit=[0.001, 0.5])
    cfg = ModelConfig.from_dict(raw)
    w = random_mamba2_weights(cfg, seed=2, dtype=torch.float32, std=0.08)
    save_mamba2_checkpoint(tmp_path, raw, w)
    cfg2 = ModelConfig.from_path(tmp_path)
    w2 = load_mamba2_weights(tmp_path, cfg2, dtype=torch.float32)
    assert cfg2.extra["mamba"]["n_groups"] == 2 and cfg2.extra["mamba"]["time_step_limit"] == (0.001, 0.5)
    sp = SamplingParams(max_tokens=5, temperature=0.0, ignore_eos=True)
    prompt = list(range(3, 40))
    a = _engine(cfg, w).generate([prompt], sp)[0].output
    b = _engine(cfg2, w2).generate([prompt], sp)[0].output
    assert a == b and len(a) == 5


def test_mamba2_cli_random_init_and_llm_front_end(tmp_path):
    """`random-init tiny-mamba2` writes a checkpoint that the LLM front end loads and generates from."""
    import argparse

    from mlxcel_b200 import cli
    from mlxcel_b200.llm import LLM

    cli.cmd_random_init(argparse.Namespace(preset="tiny-mamba2", out=str(tmp_path), seed=0, quantize=None))
    llm = LLM.from_pretrained(tmp_path, device="cpu",
                              engine_config=EngineConfig(num_blocks=32, block_size=16, max_batch=4, max_model_len=128))
    assert type(llm.model).__name__ == "Mamba2Model" and llm.engine.recurrent
    outs = llm.generate(prompt_token_ids=[[1, 2, 3, 4, 5]], sampling_params=SamplingParams(max_tokens=4, ignore_eos=True))
    assert len(outs[0].output) == 4
