"""Multi-rank timing of the fused GEMM + collective kernels against GEMM + NCCL.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 \\
        -m mlxcel_b200.utils.profile_comm [decode|prefill]

Every case runs 16 dependent launches over 4 rotating weight shards inside one CUDA graph (CUDA
events around the replay, median of 7, MAX over ranks). Printed per shape: the fused kernel, the
plain GEMM followed by an NCCL all-reduce (the baseline), the plain GEMM alone, and the roofline
time = max(weight stream at the measured copy bandwidth, FLOPs at the measured bf16 peak, bytes
that must cross NVLink per GPU at the measured 770 GB/s per direction).
With MLXCEL_B200_GEMM_TRACE=1 the per-CTA phase timestamps of the fused kernel are printed too.
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

from .. import ops
from ..ops import _lib
from ..parallel.tp import TPComm

HBM_GBS, BF16_TFLOPS, NVLINK_GBS = 6551.4, 1658.9, 770.0


def main() -> None:
    mode = sys.argv[1] if len(sys.argv) > 1 else "decode"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    lr = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("nccl", device_id=dev)
    comm = TPComm(dist.group.WORLD, dev, backend="fused", max_tokens=8192, hidden=4096, vocab=131072)
    assert comm.backend == "fused"
    nrep, ncopy = 16, 4

    def graph_time(fn):
        s = torch.cuda.Stream()
        with torch.cuda.stream(s):
            for _ in range(2):
                fn()
            torch.cuda.synchronize()
            dist.barrier()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=s):
                fn()
        torch.cuda.synchronize()
        dist.barrier()
        for _ in range(3):
            g.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(7):
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            g.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0]) * 1e3 / nrep

    def case(name, M, N, K_full):
        K = K_full // world
        g = torch.Generator(device=dev).manual_seed(1 + rank)
        x = (torch.randn(M, K, device=dev, generator=g)).to(torch.bfloat16)
        ws = [(torch.randn(N, K, device=dev, generator=g) * 0.02).to(torch.bfloat16) for _ in range(ncopy)]
        res = torch.zeros(M, N, device=dev, dtype=torch.bfloat16)
        hb = comm.fused.hidden_buffer(M, N)
        hb.zero_()
        tmp = torch.empty(M, N, device=dev, dtype=torch.bfloat16)
        fused = graph_time(lambda: [comm.fused.gemm_allreduce(x, ws[i % ncopy], None, hb) for i in range(nrep)])

        def base():
            for i in range(nrep):
                ops.linear(x, ws[i % ncopy], out=tmp)
                dist.all_reduce(tmp)
        nccl = graph_time(base)
        alone = graph_time(lambda: [ops.linear(x, ws[i % ncopy], residual=res, out=tmp) for i in range(nrep)])
        nv_bytes = M * N * 2 * (world - 1)       # one-shot: every rank receives world-1 partial tiles
        if M > 256:
            nv_bytes = 2 * M * N * 2 * (world - 1) // world   # two-shot: reduce-scatter + all-gather
        roof = max(N * K * 2 / (HBM_GBS * 1e3), 2.0 * M * N * K / (BF16_TFLOPS * 1e6), nv_bytes / (NVLINK_GBS * 1e3))
        if rank == 0:
            print(json.dumps(dict(case=name, world=world, M=M, N=N, K_per_rank=K, fused_us=round(fused, 1),
                                  gemm_plus_nccl_us=round(nccl, 1), gemm_alone_us=round(alone, 1),
                                  roofline_us=round(roof, 1), fused_of_roofline=round(roof / fused, 2))), flush=True)
        if os.environ.get("MLXCEL_B200_GEMM_TRACE") == "1":
            wsp = _lib.workspace(dev)
            off, nb = 98304, 256 * 128
            torch.cuda.synchronize()
            dist.barrier()
            wsp[off:off + nb].zero_()
            for i in range(3):   # every rank takes part; the last launch is the one read back
                comm.fused.gemm_allreduce(x, ws[i], None, hb)
            torch.cuda.synchronize()
            t = wsp[off:off + nb].view(torch.int64).view(256, 16).cpu().numpy()
            t = t[t[:, 0] > 0]
            r = (t - t[:, 0].min()) / 1e3
            names = ["entry", "setup", "loads0", "tile0", "mma_end", "acc_ready", "stored", "exit", "phaseB_begin",
                     "pushed", "peers_arrived", "cta_synced"]
            for i, n in enumerate(names):
                c = r[:, i]
                c = c[c > -1e6]
                if len(c) and rank == 0:
                    print(f"   {n:14s} min {c.min():7.2f} med {np.median(c):7.2f} max {c.max():7.2f}", flush=True)
        dist.barrier()

    if mode == "decode":
        case("o_proj", 64, 4096, 4096)
        case("down_proj", 64, 4096, 14336)
        case("o_proj_m16", 16, 4096, 4096)
    else:
        case("o_proj_prefill", 8192, 4096, 4096)
        case("down_proj_prefill", 8192, 4096, 14336)
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)


if __name__ == "__main__":
    main()
