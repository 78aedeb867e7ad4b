"""Small, self-terminating workloads for profiler captures and kernel timing.

    python -m benchmarks.profile_cases gemm_decode      # M=64 projections, 6 distinct weights
    python -m benchmarks.profile_cases gemm_prefill     # 8192 x 6144 x 4096
    python -m benchmarks.profile_cases attn_decode      # B=64, ctx 1152, GQA 32/8, D=128
    python -m benchmarks.profile_cases attn_prefill     # 8 x 1024-token prompts
    python -m benchmarks.profile_cases decode_steps N   # N eager decode steps of the bench workload
    python -m benchmarks.profile_cases kbench           # CUDA-event timings of the hot kernels (JSON lines)
    python -m benchmarks.profile_cases gemm_graph       # decode GEMMs back to back inside a CUDA graph, us per kernel
    python -m benchmarks.profile_cases gemm_phases      # per-CTA phase timestamps of the decode GEMMs
    python -m benchmarks.profile_cases qgemm_graph      # 4-bit weights: fused dequant GEMM vs GEMV vs dequantise + GEMM
    python -m benchmarks.profile_cases mamba2           # Mamba2-2.7B mixer kernels (decode B=64, prefill 8 x 1024) + engine run

Every case holds at most a few GB on the device and launches a handful of kernels, so that a
capture with ``ncu --set full -k regex:<kernel> -c <n>`` ends by itself. ``decode_steps`` brackets
the measured steps with cudaProfilerStart/Stop (use ``--profile-from-start off``).
"""
from __future__ import annotations

import json
import math
import sys

import torch

from mlxcel_b200 import ops
from mlxcel_b200.ops import KVLayer

DEV = "cuda"


def _bf(*shape, scale=1.0):
    return (torch.randn(*shape, device=DEV) * scale).to(torch.bfloat16)


def gemm_decode():
    x = _bf(64, 4096)
    ws = [_bf(4096, 4096, scale=0.02) for _ in range(6)]     # 192 MB of weights > L2
    res = _bf(64, 4096)
    for w in ws:
        ops.linear(x, w, residual=res)
    wg = _bf(2 * 14336, 4096, scale=0.02)
    ops.glu_linear(x, wg, 14336, "silu")


def gemm_prefill():
    x, w = _bf(8192, 4096), _bf(6144, 4096, scale=0.02)
    for _ in range(3):
        ops.linear(x, w)
    wg = _bf(2 * 14336, 4096, scale=0.02)
    ops.glu_linear(x, wg, 14336, "silu")


def _pool(B, ctx, Hkv, D, bs=16):
    nbs = (ctx + bs - 1) // bs
    nb = B * nbs + 8
    kv = KVLayer(_bf(nb, Hkv, bs, D), _bf(nb, Hkv, bs, D), None, None, bs, 16)
    tab = torch.randperm(nb - 8, device=DEV)[: B * nbs].reshape(B, nbs).to(torch.int32)
    return kv, tab


def _qpool(B, ctx, Hkv, D, bits, bs=16):
    """Quantized pool (8- or 4-bit affine per 64 values): random codes, scales / offsets of plausible size."""
    nbs = (ctx + bs - 1) // bs
    nb = B * nbs + 8
    shape = (nb, Hkv, bs, D if bits == 8 else D // 2)
    k = torch.randint(0, 256, shape, dtype=torch.uint8, device=DEV)
    v = torch.randint(0, 256, shape, dtype=torch.uint8, device=DEV)
    meta = lambda: torch.stack([_bf(nb, Hkv, bs, D // 64, scale=0.01).abs() + 0.005,          # noqa: E731
                                _bf(nb, Hkv, bs, D // 64, scale=0.5)], dim=-1).contiguous()
    kv = KVLayer(k, v, meta(), meta(), bs, bits)
    tab = torch.randperm(nb - 8, device=DEV)[: B * nbs].reshape(B, nbs).to(torch.int32)
    return kv, tab


def attn_decode(B=64, ctx=1152, Hq=32, Hkv=8, D=128, reps=3, bits=16):
    """``bits`` 8 / 4: the quantized-KV variants of the decode kernel (positional argument 7)."""
    kv, tab = _pool(B, ctx, Hkv, D) if bits == 16 else _qpool(B, ctx, Hkv, D, bits)
    cl = torch.full((B,), ctx, dtype=torch.int32, device=DEV)
    q = _bf(B, Hq * D)
    for _ in range(reps):
        ops.paged_decode(q, kv, tab, cl, Hq=Hq, Hkv=Hkv, D=D, scale=1 / math.sqrt(D), max_len=ctx)


def attn_decode_kv(B=64, ctx=1152, Hq=32, Hkv=8, D=128):
    """CUDA-event time of the decode kernel at 16 / 8 / 4-bit KV (L2 flushed between launches) with the
    bytes each variant has to read: codes plus one bf16 scale and offset per 64 values."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)

    def timeit(fn, n=10):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(n):
            flush.zero_()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2]
    cl = torch.full((B,), ctx, dtype=torch.int32, device=DEV)
    q = _bf(B, Hq * D)
    for bits in (16, 8, 4):
        kv, tab = _pool(B, ctx, Hkv, D) if bits == 16 else _qpool(B, ctx, Hkv, D, bits)
        t = timeit(lambda: ops.paged_decode(q, kv, tab, cl, Hq=Hq, Hkv=Hkv, D=D, scale=1 / math.sqrt(D), max_len=ctx))
        per_tok = Hkv * 2 * (D * bits // 8 + (0 if bits == 16 else D // 64 * 4))
        by = B * ctx * per_tok
        print(json.dumps(dict(op="attn_decode_kv", kv_bits=bits, B=B, ctx=ctx, Hq=Hq, Hkv=Hkv, D=D, us=round(t * 1e3, 1),
                              mbytes=round(by / 1e6, 1), gbs=round(by / t / 1e6, 1))), flush=True)


def attn_prefill(S=8, qlen=1024, Hq=32, Hkv=8, D=128, reps=2):
    kv, tab = _pool(S, qlen, Hkv, D)
    cl = torch.full((S,), qlen, dtype=torch.int32, device=DEV)
    cu = (torch.arange(S + 1, device=DEV) * qlen).to(torch.int32)
    q = _bf(S * qlen, Hq * D)
    for _ in range(reps):
        ops.paged_prefill(q, kv, tab, cu, cl, Hq=Hq, Hkv=Hkv, D=D, scale=1 / math.sqrt(D), max_q_len=qlen)


def decode_steps(n_steps=2, requests=64, prompt_len=1024, model="llama-3.1-8b"):
    from mlxcel_b200.engine import EngineConfig, SamplingParams
    from mlxcel_b200.llm import LLM
    ecfg = EngineConfig(max_batch=requests, max_num_batched_tokens=8192, prefill_chunk_alone=2048,
                        prefill_chunk_contended=prompt_len, max_prefill_seqs=8, prefix_cache=False,
                        max_model_len=prompt_len + 300, cuda_graphs=False, lookahead=False,
                        num_blocks=(prompt_len + 300) // 16 * requests + 128)
    llm = LLM.from_preset(model, device=DEV, engine_config=ecfg)
    g = torch.Generator().manual_seed(0)
    eng = llm.engine
    for p in torch.randint(0, llm.cfg.vocab_size, (requests, prompt_len), generator=g).tolist():
        eng.add_request(p, SamplingParams(max_tokens=200, ignore_eos=True))
    while eng.waiting or any(s.status.value == "prefilling" for s in eng.running):
        eng.step()
    for _ in range(3):
        eng.step()
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    for _ in range(n_steps):
        eng.step()
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()


def kbench():
    """CUDA-event medians with an L2 flush between iterations; cuBLAS (torch.matmul) beside each GEMM."""
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)

    def timeit(fn, iters=10, warm=3):
        for _ in range(warm):
            fn()
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2]

    def gemm(M, N, K, glu=False):
        x, w = _bf(M, K), _bf(N * (2 if glu else 1), K, scale=0.02)
        t = timeit((lambda: ops.glu_linear(x, w, N, "silu")) if glu else (lambda: ops.linear(x, w)))
        tc = timeit(lambda: x @ w.t())
        fl, by = 2 * M * N * K * (2 if glu else 1), (N * K * (2 if glu else 1) + M * K + M * N) * 2
        print(json.dumps(dict(op="glu" if glu else "gemm", M=M, N=N, K=K, ms=round(t, 4), cublas_ms=round(tc, 4),
                              tflops=round(fl / t / 1e9, 1), gbs=round(by / t / 1e6, 1))), flush=True)

    for N, K, glu in [(6144, 4096, False), (4096, 4096, False), (14336, 4096, True), (4096, 14336, False)]:
        gemm(8192, N, K, glu)
    for N, K, glu in [(6144, 4096, False), (4096, 4096, False), (14336, 4096, True), (4096, 14336, False),
                      (128256, 4096, False)]:
        gemm(64, N, K, glu)
    for B, ctx, Hq, Hkv, D in [(64, 1152, 32, 8, 128), (64, 1152, 4, 1, 128), (128, 2304, 64, 8, 64)]:
        kv, tab = _pool(B, ctx, Hkv, D)
        cl = torch.full((B,), ctx, dtype=torch.int32, device=DEV)
        q = _bf(B, Hq * D)
        t = timeit(lambda: ops.paged_decode(q, kv, tab, cl, Hq=Hq, Hkv=Hkv, D=D, scale=1 / math.sqrt(D), max_len=ctx))
        print(json.dumps(dict(op="attn_decode", B=B, ctx=ctx, Hq=Hq, Hkv=Hkv, D=D, ms=round(t, 4),
                              gbs=round(B * ctx * Hkv * D * 4 / t / 1e6, 1))), flush=True)
    for S, ql, Hq, Hkv, D in [(8, 1024, 32, 8, 128), (8, 1024, 64, 8, 64)]:
        kv, tab = _pool(S, ql, Hkv, D)
        cl = torch.full((S,), ql, dtype=torch.int32, device=DEV)
        cu = (torch.arange(S + 1, device=DEV) * ql).to(torch.int32)
        q = _bf(S * ql, Hq * D)
        t = timeit(lambda: ops.paged_prefill(q, kv, tab, cu, cl, Hq=Hq, Hkv=Hkv, D=D, scale=1 / math.sqrt(D),
                                             max_q_len=ql))
        print(json.dumps(dict(op="attn_prefill", S=S, qlen=ql, Hq=Hq, D=D, ms=round(t, 4),
                              tflops=round(4 * S * Hq * D * ql * ql / 2 / t / 1e9, 1))), flush=True)


def gemm_graph(M=64, full=1):
    """Decode-shape GEMMs as they run inside a decode step: 24 dependent launches over 6 rotating
    weight copies (no L2 reuse) captured in one CUDA graph; prints us per kernel for this library
    (split-K forced to several values when ``full``) and for cuBLAS (torch.matmul) under the same
    conditions, plus the time the weight stream alone would take at the measured copy bandwidth."""
    nrep, ncopy = 24, 6

    def graph_time(fn):
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                fn()
        torch.cuda.synchronize()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(7):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2] * 1e3 / nrep

    def case(N, K, glu=False, splits=(0,)):
        x = _bf(M, K)
        ws = [_bf(N * (2 if glu else 1), K, scale=0.02) for _ in range(ncopy)]
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        outc = torch.empty(M, N * (2 if glu else 1), dtype=torch.bfloat16, device=DEV)
        r = dict(M=M, N=N, K=K, glu=glu, stream_us_at_measured_copy_bw=round(ws[0].numel() * 2 / 6.5514e6, 1))
        for sp in splits:
            if glu:
                f = lambda: [ops.glu_linear(x, ws[i % ncopy], N, "silu", out=out, force_splits=sp) for i in range(nrep)]
            else:
                f = lambda: [ops.linear(x, ws[i % ncopy], out=out, force_splits=sp) for i in range(nrep)]
            r[f"us_splits_{sp or 'auto'}"] = round(graph_time(f), 1)
        r["us_cublas"] = round(graph_time(lambda: [torch.matmul(x, ws[i % ncopy].t(), out=outc) for i in range(nrep)]), 1)
        print(json.dumps(r), flush=True)

    sp = (0, 1, 2, 4, 8) if full else (0,)
    case(6144, 4096, splits=sp)
    case(4096, 4096, splits=sp)
    case(4096, 14336, splits=sp)
    case(14336, 4096, glu=True, splits=(0, 2) if full else (0,))
    # tensor-parallel 8 shards of the same model
    case(768, 4096, splits=(0,))
    case(4096, 512, splits=(0,))
    case(1792, 4096, glu=True, splits=(0,))
    case(4096, 1792, splits=(0,))


def gemm_phases(M=64):
    """Where a decode GEMM spends its time: device timestamps (globaltimer) that every CTA records
    at entry, after set-up, at the first load, when the first tile lands, at the last MMA, when
    the accumulator is ready, before/after the vector epilogue and at exit
    (MLXCEL_B200_GEMM_TRACE=1 must be set before the library is loaded)."""
    import os

    import numpy as np

    from mlxcel_b200.ops import _lib
    if os.environ.get("MLXCEL_B200_GEMM_TRACE") != "1":
        raise SystemExit("set MLXCEL_B200_GEMM_TRACE=1")
    names = ["entry", "setup", "loads0", "tile0", "mma_end", "acc_ready", "stored", "exit", "phaseB_begin", "phaseB_end"]
    off, nb = 98304, 256 * 128

    def case(N, K, glu=False):
        x = _bf(M, K)
        ws = [_bf(N * (2 if glu else 1), K, scale=0.02) for _ in range(4)]
        out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
        wsp = _lib.workspace(x.device)
        f = (lambda w: ops.glu_linear(x, w, N, "silu", out=out)) if glu else (lambda w: ops.linear(x, w, out=out))
        for w in ws:
            f(w)
        torch.cuda.synchronize()
        wsp[off:off + nb].zero_()
        for w in ws:
            f(w)
        torch.cuda.synchronize()
        t = wsp[off:off + nb].view(torch.int64).view(256, 16).cpu().numpy()
        t = t[t[:, 0] > 0]
        r = (t - t[:, 0].min()) / 1e3
        print(f"M={M} N={N} K={K} glu={glu} ctas={len(t)} span_us={r[:, 7].max():.2f}")
        for i, n in enumerate(names):
            c = r[:, i]
            c = c[c > -1e6]
            if len(c):
                print(f"   {n:13s} min {c.min():7.2f} med {np.median(c):7.2f} max {c.max():7.2f}")

    case(4096, 4096)
    case(6144, 4096)
    case(4096, 14336)
    case(14336, 4096, glu=True)


def qgemm_graph():
    """Affine 4-bit (group 64) Llama-3.1-8B projections inside a CUDA graph (16 dependent launches over
    4 rotating weight copies): the fused dequant GEMM (packed weights unpacked by the GEMM's transform
    warps), the GEMV kernel (M <= 8) and dequantise-then-GEMM, with the time the packed weight stream
    alone would take at the measured copy bandwidth."""
    from mlxcel_b200.ops import quant
    nrep, ncopy = 16, 4

    def graph_time(fn):
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                fn()
        torch.cuda.synchronize()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(7):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2] * 1e3 / nrep

    for N, K in [(6144, 4096), (4096, 4096), (4096, 14336), (28672, 4096)]:
        qts = []
        for i in range(ncopy):
            w = torch.randn(N, K, device=DEV) * 0.02
            qts.append(quant.quantize(w, "affine", 4, 64))
            del w
        packed_bytes = qts[0].nbytes()
        for M in (1, 4, 8, 32, 64):
            x = _bf(M, K)
            out = torch.empty(M, N, dtype=torch.bfloat16, device=DEV)
            r = dict(M=M, N=N, K=K, packed_MB=round(packed_bytes / 1e6, 1),
                     stream_us_at_measured_copy_bw=round(packed_bytes / 6.5514e6, 1))
            old = quant._QMV_MAX_M
            keep = quant._QGEMV4
            if M <= 8:      # the grouped mma.sync weight-streaming kernel used as a dense GEMV (one group)
                quant._QGEMV4 = True
                r["gemv4_us"] = round(graph_time(lambda: [quant.qlinear(x, qts[i % ncopy], out=out) for i in range(nrep)]), 1)
            quant._QGEMV4 = False
            quant._QMV_MAX_M = 0
            r["fused_qgemm_us"] = round(graph_time(lambda: [quant.qlinear(x, qts[i % ncopy], out=out) for i in range(nrep)]), 1)
            quant._QMV_MAX_M = old
            if M <= 8:      # the older one-warp-per-row fp32 GEMV
                r["qmv_us"] = round(graph_time(lambda: [quant.qlinear(x, qts[i % ncopy], out=out) for i in range(nrep)]), 1)
            quant._QGEMV4 = keep
            quant._FUSED_QGEMM = False
            if M > 8:
                r["dequant_then_gemm_us"] = round(
                    graph_time(lambda: [quant.qlinear(x, qts[i % ncopy], out=out) for i in range(nrep)]), 1)
            quant._FUSED_QGEMM = True
            print(json.dumps(r), flush=True)


def qgemm_decode(M=32):
    """Three launches of the fused dequant GEMM (affine 4-bit, group 64) at M tokens, 4096 x 14336."""
    from mlxcel_b200.ops import quant
    quant._QMV_MAX_M = 0
    x = _bf(M, 14336)
    out = torch.empty(M, 4096, dtype=torch.bfloat16, device=DEV)
    for _ in range(3):
        qt = quant.quantize(torch.randn(4096, 14336, device=DEV) * 0.02, "affine", 4, 64)
        quant.qlinear(x, qt, out=out)


def mamba2(engine_run=1):
    """Mamba2-2.7B geometry (80 heads x 64, state 128, conv 4): the ragged conv / scan / gated-norm
    kernels as decode rows (64 pieces of one token) and as prefill chunks (8 pieces of 1024), then
    64 requests of 1024 prompt + 64 generated tokens through the engine."""
    import time

    from mlxcel_b200.ops import recurrent as R

    H, P, N, G, K, hid = 80, 64, 128, 1, 4, 2560
    di, cd = H * P, H * P + 2 * G * N
    slots_n = 128
    conv_state = torch.zeros(slots_n, K - 1, cd, device=DEV)
    state = torch.randn(slots_n, H, P, N, device=DEV) * 0.1
    A = -torch.rand(H, device=DEV) - 0.1
    D, db = torch.randn(H, device=DEV), torch.randn(H, device=DEV) * 0.1
    cw, cb = torch.randn(cd, K, device=DEV) * 0.3, torch.randn(cd, device=DEV) * 0.1
    gw = _bf(di) + 1
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)

    def timeit(fn, iters=7, warm=3):
        for _ in range(warm):
            fn()
        ts = []
        for _ in range(iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[len(ts) // 2]

    for label, lens in (("decode_b64", [1] * 64), ("prefill_8x1024", [1024] * 8)):
        T = sum(lens)
        cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=DEV)
        sl = torch.arange(len(lens), dtype=torch.int32, device=DEV)
        rs = torch.zeros(len(lens), dtype=torch.int32, device=DEV)
        proj = _bf(T, 2 * di + 2 * G * N + H, scale=0.5)
        z, xBC, dt = proj[:, :di], proj[:, di:di + cd], proj[:, di + cd:]
        ml, ns = max(lens), (len(lens) if max(lens) == 1 else 0)
        conv = R.causal_conv_varlen(xBC, conv_state, sl, cu, rs, cw, cb, True, ml)
        y = R.ssm_scan_varlen(state, sl, cu, rs, conv[:, :di], dt, A, conv[:, di:di + G * N], conv[:, di + G * N:], D, db,
                              n_short=ns)
        t_conv = timeit(lambda: R.causal_conv_varlen(xBC, conv_state, sl, cu, rs, cw, cb, True, ml))
        t_scan = timeit(lambda: R.ssm_scan_varlen(state, sl, cu, rs, conv[:, :di], dt, A, conv[:, di:di + G * N],
                                                  conv[:, di + G * N:], D, db, n_short=ns))
        t_norm = timeit(lambda: R.gated_rmsnorm(y, z, gw, 1e-5))
        st_bytes = len(lens) * H * P * N * 4 * 2
        print(json.dumps(dict(op="mamba2_" + label, conv_us=round(t_conv * 1e3, 1), scan_us=round(t_scan * 1e3, 1),
                              gated_norm_us=round(t_norm * 1e3, 1),
                              scan_state_gbs=round(st_bytes / t_scan / 1e6, 1),
                              scan_us_per_token_step=round(t_scan * 1e3 / max(lens), 3))), flush=True)
    if not engine_run:
        return
    from mlxcel_b200.engine.engine import EngineConfig
    from mlxcel_b200.engine.params import SamplingParams
    from mlxcel_b200.llm import LLM

    del state, conv_state
    llm = LLM.from_preset("mamba2-2.7b", engine_config=EngineConfig(max_batch=64, max_model_len=2048, block_size=16,
                                                                      max_num_batched_tokens=8192, num_blocks=64 * 132))
    g = torch.Generator().manual_seed(0)
    prompts = [torch.randint(0, 50000, (1024,), generator=g).tolist() for _ in range(64)]
    sp = SamplingParams(max_tokens=64, temperature=0.0, ignore_eos=True)
    llm.generate(prompt_token_ids=prompts[:8], sampling_params=SamplingParams(max_tokens=4, temperature=0.0, ignore_eos=True))
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = llm.generate(prompt_token_ids=prompts, sampling_params=sp)
    torch.cuda.synchronize()
    dt_s = time.perf_counter() - t0
    n = sum(len(o.output) for o in outs)
    print(json.dumps(dict(op="mamba2_2.7b_engine", requests=64, prompt=1024, new_tokens=n, seconds=round(dt_s, 3),
                          output_tok_s=round(n / dt_s, 1), total_tok_s=round((n + 64 * 1024) / dt_s, 1),
                          steps=llm.engine.stats["steps"])), flush=True)


def moe_decode(T=128, E=128, k=4, H=2880, inter=2880, reps=0):
    """One gpt-oss-120b shaped MoE block at decode (T rows, top-k of E mxfp4 experts): the grouped
    weight-streaming GEMV against the tensor-core grouped GEMM with unpack warps, both in a CUDA graph
    of 8 launches over 4 rotating weight copies (CUDA events around the replay, median of 7).
    ``reps`` > 0: just run the GEMV path that many times (for a profiler capture)."""
    import os

    from mlxcel_b200.models.weights import QuantizedTensor
    from mlxcel_b200.ops import moe as moe_ops

    def rand_q(n_rows, kdim):
        packed = torch.randint(0, 2 ** 31 - 1, (E, n_rows, kdim // 8), dtype=torch.int32, device=DEV).view(torch.uint32)
        scales = torch.randint(118, 124, (E, n_rows, kdim // 32), dtype=torch.uint8, device=DEV)
        return QuantizedTensor(packed, scales, None, 4, 32, "mxfp4")
    ncopy = 1 if reps else 4
    wgu = [rand_q(2 * inter, H) for _ in range(ncopy)]
    wd = [rand_q(H, inter) for _ in range(ncopy)]
    x = _bf(T, H)
    ids, wts = moe_ops.route(_bf(T, E), k, "topk_softmax", True)
    bgu, bd = _bf(E, 2 * inter, scale=0.1), _bf(E, H, scale=0.1)
    run = lambda i: moe_ops.moe_experts(x, ids, wts, wgu[i % ncopy], wd[i % ncopy], inter, "clipped_swiglu", bgu, bd)  # noqa: E731
    if reps:
        for i in range(reps):
            run(i)
        return
    packed_bytes = E * (2 * inter * H + H * inter) // 2 * 33 // 32

    def graph_us(n=8):
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            for i in range(2):
                run(i)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                for i in range(n):
                    run(i)
        ts = []
        for _ in range(7):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        return sorted(ts)[3] * 1e3 / n
    for label, limit, expand in (("gemv", 1 << 20, 0), ("tensor_core_gemm", 0, 0), ("expand_then_dense_gemm", 0, 1)):
        if label == "gemv" and T * k > 64 * E:
            continue                      # prefill-sized: the streaming kernel is not a candidate
        moe_ops._QGEMV_MAX_ROWS, moe_ops._DEQUANT_MIN_ROWS = limit, expand
        us = graph_us(2 if T * k > 64 * E else 8)
        print(json.dumps(dict(op="moe_decode", path=label, T=T, E=E, k=k, H=H, inter=inter, us=round(us, 1),
                              packed_mbytes=round(packed_bytes / 1e6, 1), gbs=round(packed_bytes / us / 1e3, 1))), flush=True)


def prefill_helpers(T=8192, Hq=64, Hkv=8, D=64, E=128, k=4):
    """CUDA-event times (L2 flushed between launches, median of 9) of two helper kernels of a prefill step
    at gpt-oss-120b sizes, each in both of its forms: the register-resident RoPE + KV-append kernel
    (8-byte against 2/4-byte accesses) and the MoE alignment kernel (slice-per-warp against
    scan-per-expert)."""
    from mlxcel_b200.ops import KVLayer, _lib, moe as moe_ops, reference as ref

    lib = _lib.load()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=DEV)

    def timeit(fn, n=9):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(n):
            flush.zero_()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1) * 1e3)
        return round(sorted(ts)[n // 2], 1)
    bs = 16
    nb = T // bs + 1
    qkv = _bf(T, (Hq + 2 * Hkv) * D)
    pos = torch.arange(T, dtype=torch.int32, device=DEV)
    slots = torch.arange(T, dtype=torch.int32, device=DEV)
    inv = ref.rope_inv_freq(D, 150000.0, None)[0].to(DEV)
    kv = KVLayer(torch.zeros(nb, Hkv, bs, D, dtype=torch.bfloat16, device=DEV),
                 torch.zeros(nb, Hkv, bs, D, dtype=torch.bfloat16, device=DEV), None, None, bs, 16)
    rope = lambda: ops.rope_append(qkv, pos, slots, inv, kv, Hq=Hq, Hkv=Hkv, D=D, rot_dim=D)  # noqa: E731
    out = dict(op="prefill_helpers", T=T, heads=[Hq, Hkv, D], rope_mbytes=round((2 * qkv.numel() * 2) / 1e6, 1))
    for name, on in (("rope_vec8_us", 1), ("rope_narrow_us", 0)):
        lib.mx_set_rope_vec(on)
        out[name] = timeit(rope)
    lib.mx_set_rope_vec(1)
    ids, _ = moe_ops.route(_bf(T, E), k, "topk_softmax", True)
    offs = torch.empty(E + 1, dtype=torch.int32, device=DEV)
    sp = torch.empty(T * k, dtype=torch.int32, device=DEV)
    stok = torch.empty(T * k, dtype=torch.int32, device=DEV)
    st = _lib.stream()
    align = lambda: lib.mx_moe_align(ids.data_ptr(), offs.data_ptr(), sp.data_ptr(), stok.data_ptr(), T, k, 0, 0, E, st)  # noqa: E731
    res = {}
    for name, on in (("align_slices_us", 1), ("align_scan_us", 0)):
        lib.mx_set_moe_align_fast(on)
        out[name] = timeit(align)
        torch.cuda.synchronize()
        res[name] = (offs.clone(), sp.clone(), stok.clone())
    lib.mx_set_moe_align_fast(1)
    a, b = res["align_slices_us"], res["align_scan_us"]
    out["align_forms_agree"] = bool(all(torch.equal(x, y) for x, y in zip(a, b)))
    print(json.dumps(out), flush=True)


def ep_stage(T=16, world=8, max_tokens=8192, E=128, k=4, H=2880, inter=2880):
    """The all-to-all MoE layer of one data-parallel rank at serving sizes, with the ``world`` ranks
    emulated on this GPU (their stages run rank after rank, so no kernel waits on another): T rows
    per rank, receive areas sized for ``max_tokens`` rows per rank (what the engine allocates), E mxfp4
    experts in all. CUDA events around rank 0's dispatch, expert stage and combine, median of 7
    layers; the other ranks' stages run in between, untimed."""
    from mlxcel_b200.models.weights import QuantizedTensor
    from mlxcel_b200.ops import moe as moe_ops
    from mlxcel_b200.parallel.ep_a2a import EpAllToAll

    epr = E // world
    eps = EpAllToAll.emulated(world, torch.device(DEV), H, max_tokens * k, epr, max_tokens, k)

    def rand_q(n_rows, kdim):
        packed = torch.randint(0, 2 ** 31 - 1, (epr, n_rows, kdim // 8), dtype=torch.int32, device=DEV).view(torch.uint32)
        scales = torch.randint(118, 124, (epr, n_rows, kdim // 32), dtype=torch.uint8, device=DEV)
        return QuantizedTensor(packed, scales, None, 4, 32, "mxfp4")
    wgu, wd = rand_q(2 * inter, H), rand_q(H, inter)          # one shard, used by every emulated rank
    bgu, bd = _bf(epr, 2 * inter, scale=0.1), _bf(epr, H, scale=0.1)
    x = _bf(T, H)
    ids, wts = moe_ops.route(_bf(T, E), k, "topk_softmax", True)
    ev = lambda: torch.cuda.Event(enable_timing=True)  # noqa: E731
    rec = dict(dispatch=[], experts=[], combine=[])
    for it in range(9):
        marks = [ev() for _ in range(6)]
        torch.cuda.synchronize()
        marks[0].record()
        eps[0].dispatch(x, ids)
        marks[1].record()
        for r in range(1, world):
            eps[r].dispatch(x, ids)
        marks[2].record()
        eps[0].expert_stage(wgu, wd, inter, "clipped_swiglu", bgu, bd)
        marks[3].record()
        for r in range(1, world):
            eps[r].expert_stage(wgu, wd, inter, "clipped_swiglu", bgu, bd)
        marks[4].record()
        out = eps[0].combine(wts, x)
        marks[5].record()
        for r in range(1, world):
            eps[r].combine(wts, x)
        torch.cuda.synchronize()
        if it >= 2:
            rec["dispatch"].append(marks[0].elapsed_time(marks[1]) * 1e3)
            rec["experts"].append(marks[2].elapsed_time(marks[3]) * 1e3)
            rec["combine"].append(marks[4].elapsed_time(marks[5]) * 1e3)
    med = {n: round(sorted(v)[len(v) // 2], 1) for n, v in rec.items()}
    print(json.dumps(dict(op="ep_stage", T=T, world=world, cap=max_tokens * k, E=E, k=k, H=H, inter=inter,
                          eager_us=med, finite=bool(torch.isfinite(out.float()).all()))), flush=True)


CASES = dict(prefill_helpers=prefill_helpers, ep_stage=ep_stage, mamba2=mamba2, moe_decode=moe_decode, attn_decode_kv=attn_decode_kv, qgemm_decode=qgemm_decode, qgemm_graph=qgemm_graph, gemm_graph=gemm_graph, gemm_phases=gemm_phases, gemm_decode=gemm_decode, gemm_prefill=gemm_prefill, attn_decode=attn_decode,
             attn_prefill=attn_prefill, decode_steps=decode_steps, kbench=kbench)

if __name__ == "__main__":
    name = sys.argv[1] if len(sys.argv) > 1 else "kbench"
    args = [int(a) for a in sys.argv[2:]]
    CASES[name](*args)
    torch.cuda.synchronize()
    print("done", name)
