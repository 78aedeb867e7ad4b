"""Quantized-weight kernels, MoE routing / permutation / grouped GEMM vs PyTorch fp32 references."""
import pytest
import torch

from mlxcel_b200 import ops
from mlxcel_b200.ops import moe as moe_ops, quant

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _close(got, want, rtol=2e-2, atol=2e-2):
    err = (got.float() - want.float()).abs()
    bad = (err > atol + rtol * want.float().abs()).sum().item()
    assert bad == 0, f"{bad}/{err.numel()} mismatches, max err {err.max().item():.4g}"


def _qt_to(qt, dev):
    return qt.to(dev)


@pytest.mark.parametrize("mode,bits,group", [("affine", 2, 64), ("affine", 3, 32), ("affine", 4, 64),
                                             ("affine", 5, 64), ("affine", 6, 128), ("affine", 8, 64),
                                             ("mxfp4", 4, 32), ("mxfp8", 8, 32)])
def test_dequantize(mode, bits, group):
    w = torch.randn(96, 512) * 0.1
    qt = quant.quantize(w, mode, bits, group)
    want = quant.dequantize_ref(qt)
    got = quant.dequantize(_qt_to(qt, DEV))
    _close(got.cpu(), want, rtol=1e-2, atol=1e-3)


@pytest.mark.parametrize("mode,bits,group", [("affine", 4, 64), ("affine", 8, 64), ("affine", 4, 32),
                                             ("mxfp4", 4, 32), ("mxfp8", 8, 32), ("affine", 3, 64)])
@pytest.mark.parametrize("M", [1, 3, 8, 40, 300])
def test_qlinear(mode, bits, group, M):
    N, K = 384, 1024
    w = torch.randn(N, K) * 0.05
    qt = quant.quantize(w, mode, bits, group)
    wd = quant.dequantize_ref(qt)
    x = torch.randn(M, K).to(torch.bfloat16)
    res = torch.randn(M, N).to(torch.bfloat16)
    want = x.float() @ wd.t() + res.float()
    got = quant.qlinear(x.to(DEV), _qt_to(qt, DEV), residual=res.to(DEV))
    _close(got.cpu(), want, rtol=2e-2, atol=6e-2)


@pytest.mark.parametrize("mode,bits,group", [("affine", 4, 64), ("affine", 4, 128), ("affine", 8, 32), ("mxfp4", 4, 32)])
@pytest.mark.parametrize("M", [1, 16, 64, 200])
def test_fused_dequant_gemm(monkeypatch, mode, bits, group, M):
    """Packed weights dequantised inside the tcgen05 GEMM (transform warps): plain with bias and
    residual, and the gated projection, for every batch size the path serves (M <= 256)."""
    monkeypatch.setattr(quant, "_QMV_MAX_M", 0)      # also M <= 8 through the GEMM path
    N, K, I = 640, 1536, 384                        # N not a multiple of the 128-row tile
    g = torch.Generator().manual_seed(M)
    w = torch.randn(N, K, generator=g) * 0.05
    qt = quant.quantize(w, mode, bits, group)
    wd = quant.dequantize_ref(qt)
    x = (torch.randn(M, K, generator=g)).to(torch.bfloat16)
    res = torch.randn(M, N, generator=g).to(torch.bfloat16)
    bias = torch.randn(N, generator=g).to(torch.bfloat16)
    assert quant.fused_wq(_qt_to(qt, DEV), M, K) != 0
    got = quant.qlinear(x.to(DEV), _qt_to(qt, DEV), residual=res.to(DEV))
    _close(got.cpu(), x.float() @ wd.t() + res.float(), rtol=2e-2, atol=6e-2)
    got = quant.qlinear(x.to(DEV), _qt_to(qt, DEV), bias=bias.to(DEV))
    _close(got.cpu(), x.float() @ wd.t() + bias.float(), rtol=2e-2, atol=6e-2)
    wg = torch.randn(2 * I, K, generator=g) * 0.05
    qg = quant.quantize(wg, mode, bits, group)
    y = x.float() @ quant.dequantize_ref(qg).t()
    want = torch.nn.functional.silu(y[:, :I]) * y[:, I:]
    got = quant.qglu_linear(x.to(DEV), _qt_to(qg, DEV), I, "silu")
    _close(got.cpu(), want, rtol=3e-2, atol=6e-2)


@pytest.mark.parametrize("mode,norm", [("topk_softmax", True), ("softmax_topk", True), ("softmax_topk", False)])
@pytest.mark.parametrize("E,k", [(8, 2), (128, 4), (60, 8)])
def test_route(mode, norm, E, k):
    lg = torch.randn(77, E, device=DEV).to(torch.bfloat16)
    ids, w = moe_ops.route(lg, k, mode, norm)
    ids_r, w_r = moe_ops.route_ref(lg, k, mode, norm)
    # compare as sets per row: order of equal logits may differ
    assert torch.equal(ids.sort(-1).values, ids_r.sort(-1).values)
    order, order_r = ids.argsort(-1), ids_r.argsort(-1)
    _close(w.gather(1, order), w_r.gather(1, order_r), rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("T,E,k,H,I,act", [(5, 8, 2, 256, 512, "silu"), (64, 16, 4, 256, 256, "clipped_swiglu"),
                                           (700, 8, 2, 512, 384, "silu"), (128, 32, 4, 2880 // 8 * 8, 256, "clipped_swiglu")])
@pytest.mark.parametrize("local", [False, True])
def test_moe_experts(T, E, k, H, I, act, local):
    g = torch.Generator(device=DEV).manual_seed(T + E)
    r = lambda *s, sc=1.0: (torch.randn(*s, generator=g, device=DEV) * sc).to(torch.bfloat16)  # noqa: E731
    x = r(T, H)
    lg = r(T, E)
    ids, wts = moe_ops.route(lg, k, "topk_softmax", True)
    e0, e1 = (E // 4, E // 2) if local else (0, E)
    wgu, wd = r(e1 - e0, 2 * I, H, sc=0.05), r(e1 - e0, H, I, sc=0.05)
    bias = act == "clipped_swiglu"
    bgu = r(e1 - e0, 2 * I, sc=0.1) if bias else None
    bd = r(e1 - e0, H, sc=0.1) if bias else None
    res = r(T, H)
    want = moe_ops.moe_ref(x, ids, wts, wgu, wd, I, act, bgu, bd, e_begin=e0) + res.float()
    got = moe_ops.moe_experts(x, ids, wts, wgu, wd, I, act, bgu, bd, e_begin=e0, residual=res)
    _close(got, want, rtol=3e-2, atol=5e-2)
    from mlxcel_b200.ops import _lib
    torch.cuda.synchronize()
    assert _lib.read_status(torch.device(DEV)) == 0


@pytest.mark.parametrize("mode,bits,group", [("mxfp4", 4, 32), ("affine", 4, 64)])
@pytest.mark.parametrize("T,E,k,H,I,act", [(5, 8, 2, 256, 512, "silu"), (64, 16, 4, 320, 192, "clipped_swiglu"),
                                           (128, 32, 4, 2880, 384, "clipped_swiglu")])
def test_moe_experts_packed(mode, bits, group, T, E, k, H, I, act):
    """Packed (mxfp4 / affine 4-bit) expert weights through the grouped fused dequant GEMM; hidden
    and expert sizes that are not multiples of the 128-row tile (gpt-oss: 2880)."""
    g = torch.Generator().manual_seed(T + E)
    r = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc)  # noqa: E731
    x = r(T, H).to(torch.bfloat16).to(DEV)
    ids, wts = moe_ops.route(r(T, E).to(torch.bfloat16).to(DEV), k, "topk_softmax", True)
    qgu = quant.quantize(r(E, 2 * I, H, sc=0.05), mode, bits, group)
    qd = quant.quantize(r(E, H, I, sc=0.05), mode, bits, group)
    bias = act == "clipped_swiglu"
    bgu = r(E, 2 * I, sc=0.1).to(torch.bfloat16).to(DEV) if bias else None
    bd = r(E, H, sc=0.1).to(torch.bfloat16).to(DEV) if bias else None
    res = r(T, H).to(torch.bfloat16).to(DEV)
    wgu_d = quant.dequantize_ref(qgu).to(torch.bfloat16).to(DEV)
    wd_d = quant.dequantize_ref(qd).to(torch.bfloat16).to(DEV)
    want = moe_ops.moe_ref(x, ids, wts, wgu_d, wd_d, I, act, bgu, bd) + res.float()
    got = moe_ops.moe_experts(x, ids, wts, _qt_to(qgu, DEV), _qt_to(qd, DEV), I, act, bgu, bd, residual=res)
    _close(got, want, rtol=3e-2, atol=6e-2)
    from mlxcel_b200.ops import _lib
    torch.cuda.synchronize()
    assert _lib.read_status(torch.device(DEV)) == 0


@pytest.mark.parametrize("mode,bits,group", [("mxfp4", 4, 32), ("affine", 4, 64), ("affine", 4, 32)])
@pytest.mark.parametrize("T,E,k,H,I,act,skew", [(3, 8, 2, 256, 512, "silu", False), (24, 16, 4, 2880, 352, "clipped_swiglu", False),
                                                (40, 8, 2, 320, 200, "gelu_tanh", True), (128, 128, 4, 2880, 96, "clipped_swiglu", False)])
def test_moe_experts_weight_streaming_gemv(monkeypatch, mode, bits, group, T, E, k, H, I, act, skew):
    """Decode-sized groups take the grouped 4-bit GEMV (packed rows streamed once, activations in
    registers): experts without rows, one row, odd counts and one overloaded expert (several token
    passes), feature counts that do not fill the last block, against the dequantised fp32 reference."""
    monkeypatch.setattr(moe_ops, "_QGEMV_MAX_ROWS", 1 << 20)          # every case through the GEMV
    g = torch.Generator().manual_seed(T * 7 + E)
    r = lambda *s, sc=1.0: (torch.randn(*s, generator=g) * sc)  # noqa: E731
    x = r(T, H).to(torch.bfloat16).to(DEV)
    logits = r(T, E)
    if skew:
        logits[:, 3] += 6.0                                            # most tokens pick expert 3
    ids, wts = moe_ops.route(logits.to(torch.bfloat16).to(DEV), k, "topk_softmax", True)
    qgu = quant.quantize(r(E, 2 * I, H, sc=0.05), mode, bits, group)
    qd = quant.quantize(r(E, H, I, sc=0.05), mode, bits, group) if I % group == 0 and I % 32 == 0 else None
    bias = act == "clipped_swiglu"
    bgu = r(E, 2 * I, sc=0.1).to(torch.bfloat16).to(DEV) if bias else None
    bd = r(E, H, sc=0.1).to(torch.bfloat16).to(DEV) if bias else None
    wgu_d = quant.dequantize_ref(qgu).to(torch.bfloat16).to(DEV)
    wd = r(E, H, I, sc=0.05)
    wd_d = (quant.dequantize_ref(qd) if qd is not None else wd).to(torch.bfloat16).to(DEV)
    res = r(T, H).to(torch.bfloat16).to(DEV)
    want = moe_ops.moe_ref(x, ids, wts, wgu_d, wd_d, I, act, bgu, bd) + res.float()
    from mlxcel_b200.ops import _lib
    n0 = _lib.launches()
    got = moe_ops.moe_experts(x, ids, wts, _qt_to(qgu, DEV), _qt_to(qd, DEV) if qd is not None else wd_d, I, act, bgu, bd,
                              residual=res)
    _close(got, want, rtol=3e-2, atol=6e-2)
    torch.cuda.synchronize()
    assert _lib.read_status(torch.device(DEV)) == 0
    # the same call through the tensor-core path agrees too (both are checked against the reference above)
    monkeypatch.setattr(moe_ops, "_QGEMV_MAX_ROWS", 0)
    other = moe_ops.moe_experts(x, ids, wts, _qt_to(qgu, DEV), _qt_to(qd, DEV) if qd is not None else wd_d, I, act, bgu, bd,
                                residual=res)
    _close(other, want, rtol=3e-2, atol=6e-2)


def test_tiny_moe_models_gpu_vs_cpu_logits():
    from mlxcel_b200.config import preset
    from mlxcel_b200.models.decoder import DecoderModel, StepBatch
    from mlxcel_b200.models.weights import random_weights
    from mlxcel_b200.cache.kv_pool import KVPool
    import copy

    for name in ("tiny-moe", "tiny-gpt-oss", "tiny-qwen3"):
        cfg = preset(name)
        w32 = random_weights(cfg, seed=3, dtype=torch.float32, std=0.05)
        w16 = copy.deepcopy(w32)
        for obj in [w16, *w16.layers]:
            for kname, v in vars(obj).items():
                if isinstance(v, torch.Tensor):
                    setattr(obj, kname, (v.to(torch.bfloat16) if (v.dtype == torch.float32 and kname != "sinks") else v).to(DEV))
        T = 40
        ids = torch.randint(0, cfg.vocab_size, (T,), generator=torch.Generator().manual_seed(0), dtype=torch.int32)

        def one_pass(w, dev, dtype):
            pool = KVPool(cfg, 8, 16, device=dev, dtype=dtype)
            b = StepBatch(token_ids=ids.to(dev), positions=torch.arange(T, dtype=torch.int32, device=dev),
                          slot_mapping=torch.arange(T, dtype=torch.int32, device=dev), num_prefill_seqs=1,
                          pf_block_tables=torch.arange(8, dtype=torch.int32, device=dev)[None],
                          pf_cu_q=torch.tensor([0, T], dtype=torch.int32, device=dev),
                          pf_context_lens=torch.tensor([T], dtype=torch.int32, device=dev), pf_max_q_len=T,
                          logits_rows=torch.tensor([T - 1, T // 2], device=dev))
            return DecoderModel(cfg, w).forward(b, pool.layers).float().cpu()

        lc, lg = one_pass(w32, "cpu", torch.float32), one_pass(w16, DEV, torch.bfloat16)
        assert (lc - lg).abs().max().item() < 0.06 * lc.abs().max().item() + 0.03, name
