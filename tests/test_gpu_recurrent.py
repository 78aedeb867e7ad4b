"""State-space / linear-attention / BitLinear / activation kernels vs their PyTorch references."""
import pytest
import torch

from mlxcel_b200.ops import recurrent as R

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(got, want, rtol=2e-2, atol=2e-2):
    err = (got.float() - want.float()).abs()
    bad = (err > atol + rtol * want.float().abs()).sum().item()
    assert bad == 0, f"{bad}/{err.numel()} mismatches, max err {err.max().item():.4g}"


def _bf(*s, sc=1.0):
    return (torch.randn(*s, device=DEV) * sc).to(torch.bfloat16)


def test_ssm_update():
    B, H, Dh, N, G = 3, 8, 64, 128, 2
    st = torch.randn(B, H, Dh, N, device=DEV)
    x, dt = _bf(B, H, Dh), _bf(B, H)
    A = -torch.rand(H, device=DEV) - 0.1
    Bm, C = _bf(B, G, N), _bf(B, G, N)
    D, db = torch.randn(H, device=DEV), torch.randn(H, device=DEV) * 0.1
    st2 = st.clone()
    y = R.ssm_update(st, x, dt, A, Bm, C, D, db)
    yr = R.ssm_update_ref(st2, x, dt, A, Bm, C, D, db)
    _close(y, yr, atol=0.1)
    _close(st, st2, rtol=1e-3, atol=1e-3)


def test_selective_scan():
    B, L, Di, N = 2, 37, 96, 16
    x, dt = _bf(B, L, Di), _bf(B, L, Di, sc=0.5)
    A = -torch.rand(Di, N, device=DEV) - 0.1
    Bm, C = _bf(B, L, N), _bf(B, L, N)
    D = torch.randn(Di, device=DEV)
    st = torch.randn(B, Di, N, device=DEV) * 0.1
    st2 = st.clone()
    y = R.selective_scan(x, dt, A, Bm, C, D, st)
    yr = R.selective_scan_ref(x, dt, A, Bm, C, D, st2)
    _close(y, yr, atol=0.1)
    _close(st, st2, rtol=2e-3, atol=2e-3)


def test_gated_delta_update():
    B, Hv, Dk, Dv = 2, 4, 128, 128
    S = torch.randn(B, Hv, Dk, Dv, device=DEV) * 0.1
    q = torch.nn.functional.normalize(torch.randn(B, Hv, Dk, device=DEV), dim=-1).to(torch.bfloat16)
    k = torch.nn.functional.normalize(torch.randn(B, Hv, Dk, device=DEV), dim=-1).to(torch.bfloat16)
    v = _bf(B, Hv, Dv)
    g = -torch.rand(B, Hv, device=DEV)
    beta = torch.rand(B, Hv, device=DEV)
    S2 = S.clone()
    o = R.gated_delta_update(S, q, k, v, g, beta, Dk ** -0.5)
    o_r = R.gated_delta_update_ref(S2, q, k, v, g, beta, Dk ** -0.5)
    _close(o, o_r, atol=3e-2)
    _close(S, S2, rtol=1e-3, atol=1e-3)


def test_bitlinear_and_activations():
    M, N, K = 5, 96, 256
    w = torch.randint(-1, 2, (N, K))
    x = _bf(M, K)
    got = R.bitlinear(x, R.pack_ternary(w).to(DEV), 0.37)
    want = (x.float() @ w.float().to(DEV).t()) * 0.37
    _close(got, want, atol=0.1)
    z = _bf(1000, sc=3.0)
    _close(R.gelu_tanh(z), torch.nn.functional.gelu(z.float(), approximate="tanh"))
    _close(R.xielu(z, 0.8, 0.8, 0.5, -1e-6), R.xielu_ref(z, 0.8, 0.8, 0.5, -1e-6), atol=5e-2)
    a, b, c, wt, bs = _bf(7, 640), _bf(7, 640), _bf(7, 640), _bf(640), _bf(640)
    y, s = R.add3_layernorm(a, b, c, wt, bs)
    yr, sr = R.add3_layernorm(a.cpu(), b.cpu(), c.cpu(), wt.cpu(), bs.cpu())
    assert torch.equal(s.cpu(), sr)
    _close(y.cpu(), yr, atol=5e-2)


def _ragged(lens, n_slots):
    cu = [0]
    for n in lens:
        cu.append(cu[-1] + n)
    g = torch.Generator().manual_seed(len(lens))
    slots = torch.randperm(n_slots, generator=g)[: len(lens)].to(torch.int32)
    reset = torch.tensor([1 if i % 3 == 1 else 0 for i in range(len(lens))], dtype=torch.int32)
    return torch.tensor(cu, dtype=torch.int32), slots, reset


@pytest.mark.parametrize("C,K,stride_extra", [(320, 4, 72), (96, 3, 0), (1024 + 8, 2, 8), (77, 4, 11), (75, 7, 0), (64, 8, 0)])
def test_causal_conv_varlen(C, K, stride_extra):
    lens = [1, 1, 1, 37, 5, 130, 2, 64]
    cu, slots, reset = _ragged(lens, 9)
    T = int(cu[-1])
    full = _bf(T, C + stride_extra)
    xin = full[:, :C] if stride_extra == 0 else full[:, 8:8 + C]      # column slice with a row stride
    st = torch.randn(9, K - 1, C, device=DEV)
    st2 = st.clone().cpu()
    w, b = torch.randn(C, K, device=DEV) * 0.3, torch.randn(C, device=DEV) * 0.1
    y = R.causal_conv_varlen(xin, st, slots.to(DEV), cu.to(DEV), reset.to(DEV), w, b)
    yr = R.causal_conv_varlen_ref(xin.cpu(), st2, slots, cu, reset, w.cpu(), b.cpu())
    _close(y.cpu(), yr, atol=3e-2)
    _close(st.cpu(), st2, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("n_short", [0, 3])
@pytest.mark.parametrize("H,P,N,G", [(8, 32, 32, 1), (4, 64, 128, 2), (6, 16, 80, 3), (2, 64, 256, 1), (3, 40, 64, 1),
                                     (2, 8, 16, 2), (4, 32, 30, 1)])
def test_ssm_scan_varlen(H, P, N, G, n_short):
    """Every kernel behind the entry point: float4 step kernel (short pieces), row-per-thread kernel
    (N in 16/32/64/128, also with P not a multiple of the warp), generic warp-per-row kernel."""
    lens = [1, 1, 1, 44, 131, 1, 9]
    cu, slots, reset = _ragged(lens, 7)
    T = int(cu[-1])
    conv = _bf(T, H * P + 2 * G * N, sc=0.5)
    x, Bm, Cm = conv[:, :H * P], conv[:, H * P:H * P + G * N], conv[:, H * P + G * N:]
    dt = _bf(T, H + 8)[:, 8:]
    A = -torch.rand(H, device=DEV) - 0.1
    D, db = torch.randn(H, device=DEV), torch.randn(H, device=DEV) * 0.1
    st = torch.randn(7, H, P, N, device=DEV) * 0.2
    st2 = st.clone().cpu()
    lim = (0.01, 0.8)
    y = R.ssm_scan_varlen(st, slots.to(DEV), cu.to(DEV), reset.to(DEV), x, dt, A, Bm, Cm, D, db, True, lim, n_short)
    yr = R.ssm_scan_varlen_ref(st2, slots, cu, reset, x.cpu(), dt.cpu(), A.cpu(), Bm.cpu(), Cm.cpu(), D.cpu(), db.cpu(),
                               True, lim)
    _close(y.cpu(), yr, atol=0.1)
    _close(st.cpu(), st2, rtol=2e-3, atol=2e-3)


@pytest.mark.parametrize("dim,groups,off", [(640, 1, 40), (640, 5, 40), (644, 2, 3), (8192, 1, 0)])
def test_gated_rmsnorm(dim, groups, off):
    y, full = _bf(77, dim), _bf(77, dim + 360)
    z = full[:, off:off + dim]
    w = _bf(dim, sc=0.2) + 1
    got = R.gated_rmsnorm(y, z, w, 1e-5, groups)
    want = R.gated_rmsnorm(y.cpu().float(), z.cpu().float(), w.cpu().float(), 1e-5, groups)
    _close(got.cpu(), want, atol=3e-2)


def test_relu2():
    x = _bf(33, 257)
    _close(R.relu2(x).cpu(), torch.relu(x.float()).square().cpu(), atol=2e-2)


def test_tiny_nemotron_h_engine_gpu_matches_cpu():
    """Hybrid Mamba2 / attention / MLP stack: bf16 GPU kernels against the fp32 CPU path."""
    import copy
    from mlxcel_b200.config import preset
    from mlxcel_b200.engine.engine import Engine, EngineConfig
    from mlxcel_b200.engine.params import SamplingParams
    from mlxcel_b200.models.hybrid import HybridModel, random_hybrid_weights

    cfg = preset("tiny-nemotron-h")
    w32 = random_hybrid_weights(cfg, seed=4, dtype=torch.float32, std=0.08)
    w16 = copy.deepcopy(w32)

    def conv(obj):
        for k, v in vars(obj).items():
            if isinstance(v, torch.Tensor):
                keep32 = k in ("conv_w", "conv_b", "dt_bias", "A_log", "D")
                setattr(obj, k, (v if keep32 else v.to(torch.bfloat16)).to(DEV))

    conv(w16)
    for blk in w16.blocks:
        conv(blk)
        for sub in (blk.mamba, blk.attn):
            if sub is not None:
                conv(sub)
    w16.layers = [b.attn for b in w16.blocks if b.kind == "attention"]
    from mlxcel_b200.cache.kv_pool import KVPool
    from mlxcel_b200.models.decoder import StepBatch

    T = 50
    ids = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(0), dtype=torch.int32)

    def logits(w, dev, dtype):
        pool = KVPool(cfg, 8, 16, device=dev, dtype=dtype, num_layers=1)
        b = StepBatch(token_ids=ids.to(dev), positions=torch.arange(T, dtype=torch.int32, device=dev),
                      slot_mapping=torch.arange(T, dtype=torch.int32, device=dev), num_prefill_seqs=1,
                      pf_block_tables=torch.arange(8, dtype=torch.int32, device=dev)[None],
                      pf_cu_q=torch.tensor([0, T], dtype=torch.int32, device=dev),
                      pf_context_lens=torch.tensor([T], dtype=torch.int32, device=dev), pf_max_q_len=T,
                      pf_cu_q_host=[0, T], logits_rows=torch.tensor([T - 1, T // 2], device=dev))
        b.seq_ids, b.pf_starts = [0], [0]
        return HybridModel(cfg, w, max_seqs=4).forward(b, pool.layers).float().cpu()

    lc, lg = logits(w32, "cpu", torch.float32), logits(w16, DEV, torch.bfloat16)
    assert (lc - lg).abs().max().item() < 0.05 * lc.abs().max().item() + 0.03
    sp = SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)
    eng = Engine(HybridModel(cfg, w16, max_seqs=8), cfg,
                 EngineConfig(num_blocks=64, block_size=16, max_batch=8, max_model_len=256, max_num_batched_tokens=32))
    outs = eng.generate([ids[:45].tolist(), ids[3:12].tolist()], sp)
    assert all(len(o.output) == 6 for o in outs) and not eng.model.ssm.slot_of
    from mlxcel_b200.ops import _lib
    torch.cuda.synchronize()
    assert _lib.read_status(torch.device(DEV)) == 0


def test_tiny_mamba2_engine_gpu_matches_cpu():
    """bf16 kernels on the GPU against the fp32 CPU path, through the engine (chunked prefill + batching)."""
    import copy
    from mlxcel_b200.config import preset
    from mlxcel_b200.engine.engine import Engine, EngineConfig
    from mlxcel_b200.engine.params import SamplingParams
    from mlxcel_b200.models.decoder import StepBatch
    from mlxcel_b200.models.mamba2 import Mamba2Model, random_mamba2_weights

    cfg = preset("tiny-mamba2")
    w32 = random_mamba2_weights(cfg, seed=4, dtype=torch.float32, std=0.08)
    w16 = copy.deepcopy(w32)
    for obj in [w16, *w16.layers]:
        for k, v in vars(obj).items():
            if isinstance(v, torch.Tensor):
                keep32 = k in ("conv_w", "conv_b", "dt_bias", "A_log", "D")
                setattr(obj, k, (v if keep32 else v.to(torch.bfloat16)).to(DEV))
    w16.lm_head = w16.embed
    T = 50
    ids = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(0), dtype=torch.int32)

    def logits(w, dev):
        m = Mamba2Model(cfg, w, max_seqs=4)
        b = StepBatch(token_ids=ids.to(dev), positions=torch.arange(T, dtype=torch.int32, device=dev),
                      slot_mapping=torch.arange(T, dtype=torch.int32, device=dev), num_prefill_seqs=1,
                      pf_cu_q_host=[0, T], pf_max_q_len=T, logits_rows=torch.tensor([T - 1, T // 2], device=dev))
        b.seq_ids, b.pf_starts = [0], [0]
        return m.forward(b).float().cpu()

    lc, lg = logits(w32, "cpu"), logits(w16, DEV)
    assert (lc - lg).abs().max().item() < 0.05 * lc.abs().max().item() + 0.03
    sp = SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True)
    eng = Engine(Mamba2Model(cfg, w16, max_seqs=16), cfg,
                 EngineConfig(num_blocks=64, block_size=16, max_batch=8, max_model_len=256, max_num_batched_tokens=32))
    outs = eng.generate([ids[:40].tolist(), ids[5:12].tolist()], sp)
    assert all(len(s.output) == 8 for s in outs) and not eng.model.slot_of
    from mlxcel_b200.ops import _lib
    torch.cuda.synchronize()
    assert _lib.read_status(torch.device(DEV)) == 0


def test_tiny_mamba1_engine_gpu_matches_cpu():
    """First-generation Mamba: bf16 GPU kernels (ragged conv, selective scan) against the fp32 CPU path."""
    import copy
    from mlxcel_b200.config import preset
    from mlxcel_b200.engine.engine import Engine, EngineConfig
    from mlxcel_b200.engine.params import SamplingParams
    from mlxcel_b200.models.decoder import StepBatch
    from mlxcel_b200.models.mamba1 import Mamba1Model, random_mamba1_weights

    cfg = preset("tiny-mamba")
    w32 = random_mamba1_weights(cfg, seed=4, dtype=torch.float32, std=0.08)
    w16 = copy.deepcopy(w32)
    for obj in [w16, *w16.layers]:
        for k, v in vars(obj).items():
            if isinstance(v, torch.Tensor):
                keep32 = k in ("conv_w", "conv_b", "A_log", "D")
                setattr(obj, k, (v if keep32 else v.to(torch.bfloat16)).to(DEV))
    w16.lm_head = w16.embed
    T = 50
    ids = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(0), dtype=torch.int32)

    def logits(w, dev):
        m = Mamba1Model(cfg, w, max_seqs=4)
        b = StepBatch(token_ids=ids.to(dev), positions=torch.arange(T, dtype=torch.int32, device=dev),
                      slot_mapping=torch.arange(T, dtype=torch.int32, device=dev), num_prefill_seqs=1,
                      pf_cu_q_host=[0, T], pf_max_q_len=T, logits_rows=torch.tensor([T - 1, T // 2], device=dev))
        b.seq_ids, b.pf_starts = [0], [0]
        return m.forward(b).float().cpu()

    lc, lg = logits(w32, "cpu"), logits(w16, DEV)
    assert (lc - lg).abs().max().item() < 0.05 * lc.abs().max().item() + 0.03
    eng = Engine(Mamba1Model(cfg, w16, max_seqs=16), cfg,
                 EngineConfig(num_blocks=64, block_size=16, max_batch=8, max_model_len=256, max_num_batched_tokens=32))
    outs = eng.generate([ids[:40].tolist(), ids[5:12].tolist()], SamplingParams(max_tokens=8, temperature=0.0, ignore_eos=True))
    assert all(len(s.output) == 8 for s in outs) and not eng.model.slot_of
    from mlxcel_b200.ops import _lib
    torch.cuda.synchronize()
    assert _lib.read_status(torch.device(DEV)) == 0


def _tiny_hf_hybrid(name):
    """A tiny random checkpoint of a hybrid family written by transformers (skipped where it is missing)."""
    import tempfile
    transformers = pytest.importorskip("transformers")
    from transformers import AutoConfig, AutoModelForCausalLM
    common = dict(hidden_size=128, intermediate_size=256, num_hidden_layers=4, num_attention_heads=2,
                  num_key_value_heads=1, vocab_size=512, max_position_embeddings=256, pad_token_id=0)   # head size 64
    kw = {
        "jamba": dict(attn_layer_period=4, attn_layer_offset=2, expert_layer_period=2, expert_layer_offset=1,
                      num_experts=8, num_experts_per_tok=2, mamba_d_state=16, mamba_d_conv=4, mamba_expand=2,
                      mamba_dt_rank=8, use_mamba_kernels=False),
        "qwen3_next": dict(head_dim=64, layer_types=["linear_attention", "linear_attention", "full_attention",
                                                     "linear_attention"],
                           linear_conv_kernel_dim=4, linear_key_head_dim=32, linear_value_head_dim=32,
                           linear_num_key_heads=2, linear_num_value_heads=4, num_experts=8, num_experts_per_tok=2,
                           moe_intermediate_size=128, shared_expert_intermediate_size=128, decoder_sparse_step=1,
                           mlp_only_layers=[0, 1, 2, 3]),     # dense MLPs: no expert choice that bf16 could flip
        "granitemoehybrid": dict(shared_intermediate_size=256, layer_types=["mamba", "attention", "mamba", "mamba"],
                                 num_local_experts=0, mamba_n_heads=8, mamba_d_head=32, mamba_d_state=32,
                                 mamba_n_groups=2, mamba_d_conv=4, mamba_expand=2, mamba_chunk_size=8,
                                 embedding_multiplier=2.0, residual_multiplier=0.5, attention_multiplier=0.125,
                                 logits_scaling=2.0),
        "lfm2": dict(layer_types=["conv", "full_attention", "conv", "conv"], conv_L_cache=3, conv_bias=False,
                     block_auto_adjust_ff_dim=False),
        "recurrent_gemma": dict(head_dim=64, lru_width=128, attention_window_size=32, conv1d_width=4, intermediate_size=512),
        "qwen3_5_text": dict(head_dim=64, layer_types=["linear_attention", "linear_attention", "full_attention",
                                                       "linear_attention"],
                             linear_conv_kernel_dim=4, linear_key_head_dim=32, linear_value_head_dim=32,
                             linear_num_key_heads=2, linear_num_value_heads=4),
    }[name]
    if name == "recurrent_gemma":
        common = {k: v for k, v in common.items() if k != "intermediate_size"}
    torch.manual_seed(0)
    try:
        model = AutoModelForCausalLM.from_config(AutoConfig.for_model(name, **common, **kw)).float()
    except (KeyError, ValueError, ImportError) as e:
        pytest.skip(f"transformers cannot build {name}: {e}")
    with torch.no_grad():
        for n, p in model.named_parameters():
            if p.dim() >= 2 and "A_log" not in n and "recurrent_param" not in n:
                p.normal_(0, 0.05)
    d = tempfile.mkdtemp(prefix=f"hyb_{name}_")
    model.save_pretrained(d, safe_serialization=True)
    return d


@pytest.mark.parametrize("name", ["jamba", "qwen3_next", "granitemoehybrid", "lfm2", "recurrent_gemma", "qwen3_5_text"])
def test_hybrid_checkpoints_gpu_matches_cpu(name):
    """Hybrid layouts end to end on the GPU (bf16 kernels) against this package's fp32 CPU path, from a
    checkpoint written by transformers: prompt logits, then a short greedy run through the engine."""
    from mlxcel_b200.cache.kv_pool import KVPool
    from mlxcel_b200.config import ModelConfig
    from mlxcel_b200.engine.engine import Engine, EngineConfig
    from mlxcel_b200.engine.params import SamplingParams
    from mlxcel_b200.models import hybrid
    from mlxcel_b200.models.decoder import StepBatch

    d = _tiny_hf_hybrid(name)
    cfg = ModelConfig.from_path(d)
    load = {"jamba": hybrid.load_jamba_weights, "qwen3_next": hybrid.load_qwen3_next_weights,
            "granitemoehybrid": hybrid.load_granite_hybrid_weights, "lfm2": hybrid.load_lfm2_weights,
            "recurrent_gemma": hybrid.load_recurrent_gemma_weights, "qwen3_5_text": hybrid.load_qwen3_next_weights}[name]
    T = 40
    ids = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(0), dtype=torch.int32)

    def logits(dev, dtype):
        m = hybrid.HybridModel(cfg, load(d, cfg, dtype=dtype, device=dev), max_seqs=4)
        pool = KVPool(cfg, 8, 16, device=dev, dtype=dtype, num_layers=m.num_kv_layers)
        b = StepBatch(token_ids=ids.to(dev), positions=torch.arange(T, dtype=torch.int32, device=dev),
                      slot_mapping=torch.arange(T, dtype=torch.int32, device=dev), num_prefill_seqs=1,
                      pf_block_tables=torch.arange(8, dtype=torch.int32, device=dev)[None],
                      pf_cu_q=torch.tensor([0, T], dtype=torch.int32, device=dev),
                      pf_context_lens=torch.tensor([T], dtype=torch.int32, device=dev), pf_max_q_len=T,
                      pf_cu_q_host=[0, T], logits_rows=torch.arange(T, device=dev))
        b.seq_ids, b.pf_starts = [0], [0]
        return m.forward(b, pool.layers).float().cpu(), m

    lc, _ = logits("cpu", torch.float32)
    lg, m16 = logits(DEV, torch.bfloat16)
    # row by row: bf16 rounding may flip a top-k expert choice of a token, which moves that row (and
    # through the recurrent state a few later ones) by more than rounding; a wrong kernel moves all rows
    row_err = (lc - lg).abs().amax(-1)
    good = row_err < 0.06 * lc.abs().max().item() + 0.04
    assert good.float().mean().item() >= 0.75 and bool(good[:4].all()), (name, row_err.tolist())
    m16.release_seq(0)
    eng = Engine(m16, cfg, EngineConfig(num_blocks=64, block_size=16, max_batch=8, max_model_len=256,
                                        max_num_batched_tokens=32))
    outs = eng.generate([ids[:37].tolist(), ids[5:12].tolist()], SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True))
    assert all(len(s.output) == 6 for s in outs) and not m16.ssm.slot_of
    from mlxcel_b200.ops import _lib
    torch.cuda.synchronize()
    assert _lib.read_status(torch.device(DEV)) == 0


def test_plain_expert_moe_matches_reference():
    """Non-gated experts (``down(relu(up x)^2)``, the Nemotron-H MoE block): grouped GEMM, activation
    kernel, grouped GEMM against the dense fp32 statement of the same routing."""
    from mlxcel_b200.ops import moe as moe_ops

    g = torch.Generator().manual_seed(0)
    T, H, I, E, k = 96, 128, 192, 8, 3
    x = (torch.randn(T, H, generator=g) * 0.5).to(torch.bfloat16)
    up = (torch.randn(E, I, H, generator=g) * 0.08).to(torch.bfloat16)
    down = (torch.randn(E, H, I, generator=g) * 0.08).to(torch.bfloat16)
    ids, wts = moe_ops.route_sigmoid_grouped(torch.randn(T, E, generator=g), k, None, 4, 2, True, 1.7)
    want = moe_ops.moe_ref(x, ids, wts, up, down, I, "relu2", gated=False)
    got = moe_ops.moe_experts(x.to(DEV), ids.to(DEV).int().contiguous(), wts.to(DEV).float().contiguous(), up.to(DEV),
                              down.to(DEV), I, "relu2", gated=False).float().cpu()
    err = (got - want).abs().max().item()
    assert err < 2e-2 * max(want.abs().max().item(), 1.0), err
