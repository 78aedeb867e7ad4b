"""Multi-rank timing of the fused GEMM + collective kernels against GEMM + NCCL.

    python -m torch.distributed.run --nproc-per-node N --master-addr 127.0.0.1 \\
        -m benchmarks.profile_comm [decode|prefill|ep]

Every case runs 16 dependent launches over 4 rotating weight shards inside one CUDA graph (CUDA
events around the replay, median of 7, MAX over ranks). Printed per shape: the fused kernel, the
plain GEMM followed by an NCCL all-reduce (the baseline), the plain GEMM alone, and the roofline
time = max(weight stream at the measured copy bandwidth, FLOPs at the measured bf16 peak, bytes
that must cross NVLink per GPU at the measured 770 GB/s per direction).
With MLXCEL_B200_GEMM_TRACE=1 the per-CTA phase timestamps of the fused kernel are printed too.

``ep``: expert-parallel MoE layer with token-sharded ranks (GPT-OSS-120B expert geometry: 128 experts,
top-4, hidden 2880): the dispatch / combine kernels over peer memory against the same exchange done
with NCCL (count all-to-all, host read of the counts, two uneven all_to_all_single, torch index ops
for the permutation and the weighted sum), with and without the expert GEMMs between them.
"""
from __future__ import annotations

import json
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

from mlxcel_b200 import ops
from mlxcel_b200.ops import _lib
from mlxcel_b200.parallel.tp import TPComm

HBM_GBS, BF16_TFLOPS, NVLINK_GBS = 6551.4, 1658.9, 770.0


def ep_main(rank: int, world: int, dev: torch.device) -> None:
    from mlxcel_b200.ops import moe as moe_ops
    from ..parallel.ep_a2a import EpAllToAll
    from mlxcel_b200.parallel.symm import SymmetricHeap

    E, k, H, I = 128, 4, 2880, 2880
    epr = E // world
    Tmax = 1024
    cap = Tmax * k
    heap = SymmetricHeap(dist.group.WORLD, dev, EpAllToAll.required_bytes(world, H, cap) + (4 << 20))
    ep = EpAllToAll.from_heap(heap, H, cap, epr, Tmax, k)
    g = torch.Generator(device=dev).manual_seed(3 + rank)
    wgu = (torch.randn(epr, 2 * I, H, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    wd = (torch.randn(epr, H, I, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    layers = 8          # back-to-back layers per timed region (the launches queue up behind the first)

    def timeit(fn, iters=7, warm=2):
        for _ in range(warm):
            fn()
        ts = []
        for _ in range(iters):
            flush.zero_()
            torch.cuda.synchronize()
            dist.barrier()
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(layers):
                fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        t = torch.tensor([sorted(ts)[len(ts) // 2]], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t[0]) * 1e3 / layers

    for T in (64, 1024):
        x = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
        res = torch.randn(T, H, device=dev, generator=g).to(torch.bfloat16)
        ids, wts = moe_ops.route(torch.randn(T, E, device=dev, generator=g).to(torch.bfloat16), k, "topk_softmax", True)
        ids, wts = ids.contiguous(), wts.contiguous()

        def ours_comm():
            ep.dispatch(x, ids)
            ep._call(1)
            ep._call(2)
            return ep.combine(wts, res)

        def ours_full():
            return ep.moe(x, ids, wts, wgu, wd, I, "clipped_swiglu", residual=res)

        def nccl(with_gemm: bool):
            flat = ids.reshape(-1).long()
            order = torch.argsort(flat // epr, stable=True)
            send_counts = torch.bincount(flat // epr, minlength=world)
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts)
            sc, rc = send_counts.tolist(), recv_counts.tolist()            # host read of the counts
            rows = x.index_select(0, order // k)
            eids = flat.index_select(0, order).to(torch.int32)
            got = torch.empty(sum(rc), H, dtype=x.dtype, device=dev)
            got_e = torch.empty(sum(rc), dtype=torch.int32, device=dev)
            dist.all_to_all_single(got, rows, rc, sc)
            dist.all_to_all_single(got_e, eids, rc, sc)
            if with_gemm:
                y = moe_ops.moe_experts(got, got_e.view(-1, 1), torch.ones(sum(rc), 1, device=dev), wgu, wd, I,
                                        "clipped_swiglu", e_begin=rank * epr)
            else:
                y = got
            back = torch.empty(T * k, H, dtype=x.dtype, device=dev)
            dist.all_to_all_single(back, y, sc, rc)
            unsorted = torch.empty_like(back)
            unsorted.index_copy_(0, order, back)
            return (res.float() + (unsorted.view(T, k, H).float() * wts.unsqueeze(-1)).sum(1)).to(x.dtype)

        a, b = ours_full(), nccl(True)
        torch.cuda.synchronize()
        err = (a.float() - b.float()).abs().max().item()
        def graphed(fn):
            """The same 8 layers inside one CUDA graph (the epoch lives on the device, so a replay
            raises fresh flags)."""
            st = torch.cuda.Stream()
            with torch.cuda.stream(st):
                fn()
                torch.cuda.synchronize()
                dist.barrier()
                gr = torch.cuda.CUDAGraph()
                with torch.cuda.graph(gr, stream=st):
                    for _ in range(layers):
                        fn()
            torch.cuda.synchronize()
            dist.barrier()
            return timeit(gr.replay) / layers

        t_comm, t_full = timeit(ours_comm), timeit(ours_full)
        g_comm, g_full = graphed(ours_comm), graphed(ours_full)
        n_comm, n_full = timeit(lambda: nccl(False)), timeit(lambda: nccl(True))
        nv = T * k * H * 2 * (world - 1) / world            # bytes leaving one GPU per direction, uniform routing
        roof = 2 * nv / (NVLINK_GBS * 1e3)
        if rank == 0:
            print(json.dumps(dict(case="ep_moe_a2a", world=world, tokens_per_rank=T, top_k=k, hidden=H, experts=E,
                                  ours_comm_us=round(t_comm, 1), nccl_comm_us=round(n_comm, 1),
                                  ours_layer_us=round(t_full, 1), nccl_layer_us=round(n_full, 1),
                                  ours_comm_graph_us=round(g_comm, 1), ours_layer_graph_us=round(g_full, 1),
                                  nvlink_roofline_us=round(roof, 1), comm_graph_of_roofline=round(roof / g_comm, 3),
                                  max_abs_diff_vs_nccl_path=round(err, 4))), flush=True)
    st = _lib.read_status(dev)
    assert st == 0, f"kernel status {st}"
    dist.barrier()
    torch.cuda.synchronize()
    sys.stdout.flush()
    os._exit(0)


def main() -> None:
    mode = sys.argv[1] if len(sys.argv) > 1 else "decode"
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    lr = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    dist.init_process_group("nccl", device_id=dev)
    if mode == "ep":
        return ep_main(rank, world, dev)
    os.environ.setdefault("MLXCEL_B200_NVLS_ONESHOT", "1")       # "fused_us" = everything through the switch
    comm = TPComm(dist.group.WORLD, dev, backend="fused", max_tokens=8192, hidden=4096, vocab=131072)
    assert comm.backend == "fused"
    # second channel set on the peer-store protocol, so that one run shows NVLS (multimem) beside it
    comm_peer = None
    if comm.fused.nvls:
        os.environ["MLXCEL_B200_NVLS"] = "0"
        comm_peer = TPComm(dist.group.WORLD, dev, backend="fused", max_tokens=8192, hidden=4096, vocab=131072)
        os.environ["MLXCEL_B200_NVLS"] = "1"
    # third channel set whose one-shot limit is 8 rows: decode-sized cases then take the two-shot
    # (reduce-scatter + broadcast through the switch) kernel, for comparison with the one-shot ones
    fused_two = None
    if comm.fused.nvls:
        from mlxcel_b200.parallel.symm import FusedOps, SymmetricHeap
        heap2 = SymmetricHeap(dist.group.WORLD, dev, FusedOps.required_bytes(world, 8192, 4096, 8 * 1024, small_m=8))
        fused_two = FusedOps(heap2, 8192, 4096, 8 * 1024, small_m=8)
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
        fused_peer = None
        if comm_peer is not None:
            hb2 = comm_peer.fused.hidden_buffer(M, N)
            hb2.zero_()
            fused_peer = graph_time(lambda: [comm_peer.fused.gemm_allreduce(x, ws[i % ncopy], None, hb2)
                                             for i in range(nrep)])

        two_shot = None
        if fused_two is not None and M <= 256:
            hb3 = fused_two.hidden_buffer(M, N)
            hb3.zero_()
            try:
                two_shot = graph_time(lambda: [fused_two.gemm_allreduce(x, ws[i % ncopy], None, hb3) for i in range(nrep)])
            except Exception as e:          # shape not covered by the two-shot kernel: report the rest
                if rank == 0:
                    print(f"two-shot at M={M} not measured: {e}", flush=True)

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
            print(json.dumps(dict(case=name, world=world, M=M, N=N, K_per_rank=K, nvls=bool(comm.fused.nvls),
                                  fused_us=round(fused, 1),
                                  fused_peer_store_us=round(fused_peer, 1) if fused_peer is not None else None,
                                  fused_two_shot_switch_us=round(two_shot, 1) if two_shot is not None else None,
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
