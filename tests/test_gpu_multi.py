"""Multi-GPU checks of the fused GEMM + collective kernels and the tensor-parallel executor.
Each test spawns one process per GPU (NCCL for bootstrap) and is skipped on boxes with one GPU."""
import os
import socket
import subprocess
import sys
import textwrap

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _run(world: int, body: str, timeout: int = 600) -> str:
    script = textwrap.dedent("""
        import os, sys, torch, torch.distributed as dist
        sys.path.insert(0, %r)
        rank = int(os.environ["RANK"]); world = int(os.environ["WORLD_SIZE"])
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", device_id=dev)
        from mlxcel_b200 import ops
        from mlxcel_b200.ops import _lib
        from mlxcel_b200.parallel.tp import TPComm
    """ % ROOT) + textwrap.dedent(body) + textwrap.dedent("""
        torch.cuda.synchronize()
        st = _lib.read_status(dev)
        assert st == 0, f"kernel status {st}"
        dist.barrier()
        if rank == 0:
            print("MULTI_OK")
        dist.destroy_process_group()
    """)
    import tempfile
    path = os.path.join(tempfile.mkdtemp(prefix="mlxcel_multi_"), "ranks.py")
    with open(path, "w") as f:
        f.write(script)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0", MLXCEL_B200_REQUIRE_FUSED="1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), path]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and "MULTI_OK" in out, out[-4000:]
    return out


def _world() -> int:
    n = torch.cuda.device_count()
    return 8 if n >= 8 else 4 if n >= 4 else 2 if n >= 2 else 1


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_fused_gemm_allreduce_and_allgather():
    _run(_world(), """
        comm = TPComm(dist.group.WORLD, dev, backend="fused", max_tokens=2048, hidden=1024, vocab=8192)
        assert comm.backend == "fused"
        torch.manual_seed(0)   # same full tensors on every rank, each takes its shard
        for M in (1, 7, 64, 200, 300, 1500):
            K, N = 512 * world, 1024
            x = torch.randn(M, K, device=dev).to(torch.bfloat16)
            w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
            bias = torch.randn(N, device=dev).to(torch.bfloat16)
            res = torch.randn(M, N, device=dev).to(torch.bfloat16)
            ks = slice(rank * 512, (rank + 1) * 512)
            want = x.float() @ w.float().t() + bias.float() + res.float()
            for rep in range(3):
                got = comm.row_parallel_linear(x[:, ks].contiguous(), w[:, ks].contiguous(), bias, res.clone())
                torch.cuda.synchronize()
                err = (got.float() - want).abs().max().item()
                assert err < 0.25, (M, rep, err)
                # bitwise identical on every rank
                ref0 = got.clone(); dist.broadcast(ref0, 0)
                assert torch.equal(ref0, got), (M, rep)
                if M > 256:   # the fused two-shot kernel (prefill chunks take GEMM + NCCL by default)
                    got2 = comm.fused.gemm_allreduce(x[:, ks].contiguous(), w[:, ks].contiguous(), bias, res.clone())
                    torch.cuda.synchronize()
                    assert (got2.float() - want).abs().max().item() < 0.25, (M, rep)
                    ref0 = got2.clone(); dist.broadcast(ref0, 0)
                    assert torch.equal(ref0, got2), (M, rep)
            # quantized row-parallel projection -> all-reduce in one kernel (packed 4-bit shards)
            if M <= 256:
                from mlxcel_b200.ops import quant
                qts = quant.quantize(w[:, ks].float().cpu(), "affine", 4, 64)
                qts = qts.to(dev)
                wdq = quant.dequantize_ref(qts).float()
                parts = [torch.empty(N, 512, device=dev) for _ in range(world)]
                dist.all_gather(parts, wdq.contiguous())
                want_q = x.float() @ torch.cat(parts, dim=1).t() + bias.float() + res.float()
                got_q = comm.row_parallel_linear(x[:, ks].contiguous(), qts, bias, res.clone())
                torch.cuda.synchronize()
                assert (got_q.float() - want_q).abs().max().item() < 0.3, (M, "q4")
                ref0 = got_q.clone(); dist.broadcast(ref0, 0)
                assert torch.equal(ref0, got_q), (M, "q4")
            # stand-alone all-reduce (one-shot for small, two-shot for large tensors)
            part = torch.randn(M, N, device=dev).to(torch.bfloat16) * (rank + 1)
            parts = [torch.empty_like(part) for _ in range(world)]
            dist.all_gather(parts, part)
            want_ar = sum(p.float() for p in parts)
            got_ar = comm.all_reduce(part.clone())
            torch.cuda.synchronize()
            assert (got_ar.float() - want_ar).abs().max().item() < 0.1 * world, M
            # all-gather of a vocab-parallel projection
            if M <= 256:
                Vl = 1024
                wl = (torch.randn(world * Vl, 256, device=dev) * 0.05).to(torch.bfloat16)
                xs = torch.randn(M, 256, device=dev).to(torch.bfloat16)
                lg = comm.lm_head(xs, wl[rank * Vl:(rank + 1) * Vl].contiguous())
                torch.cuda.synchronize()
                wantl = xs.float() @ wl.float().t()
                assert (lg.float() - wantl).abs().max().item() < 0.1
    """)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_tp_engine_fused_matches_nccl_and_single_gpu():
    _run(_world(), """
        from mlxcel_b200.config import preset
        from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams
        from mlxcel_b200.models.decoder import DecoderModel
        from mlxcel_b200.models.weights import random_weights
        from mlxcel_b200.loading.shard import shard_weights
        cfg = preset("tiny-llama")
        cfg.num_attention_heads, cfg.num_key_value_heads = 8, 8
        cfg.hidden_size, cfg.head_dim, cfg.intermediate_size = 512, 64, 1024
        full = random_weights(cfg, seed=3, dtype=torch.bfloat16, device=dev, std=0.05)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (20, 7, 33, 300)]
        sp = SamplingParams(max_tokens=10, ignore_eos=True)
        ec = lambda: EngineConfig(max_batch=4, max_num_batched_tokens=512, num_blocks=128, max_model_len=512)
        single = [s.output for s in Engine(DecoderModel(cfg, full), cfg, ec()).generate(prompts, sp)]
        outs = {}
        for backend in ("nccl", "fused"):
            comm = TPComm(dist.group.WORLD, dev, backend=backend, max_tokens=512, hidden=512, vocab=2048)
            w = shard_weights(cfg, full, comm.tp_rank, comm.tp_size)
            eng = Engine(DecoderModel(cfg, w, comm=comm), cfg, ec())
            outs[backend] = [s.output for s in eng.generate(prompts, sp)]
        agree = lambda a, b: sum(x == y for sa, sb in zip(a, b) for x, y in zip(sa, sb)) / sum(map(len, a))
        assert all(a[0] == b[0] for a, b in zip(single, outs["fused"])), (single, outs)
        assert agree(single, outs["fused"]) >= 0.6 and agree(single, outs["nccl"]) >= 0.6, (single, outs)
    """)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_ep_all_to_all_moe_matches_local_reference():
    """Token-sharded expert parallelism: dispatch / combine kernels over peer memory, three layers
    back to back on the same buffers, every rank with its own token count."""
    _run(_world(), """
        from mlxcel_b200.ops import moe as moe_ops
        from mlxcel_b200.parallel.symm import SymmetricHeap
        from mlxcel_b200.parallel.ep_a2a import EpAllToAll
        E, k, H, I, Tmax = 16, 2, 512, 256, 96
        epr = E // world
        cap = Tmax * k
        heap = SymmetricHeap(dist.group.WORLD, dev, EpAllToAll.required_bytes(world, H, cap) + (4 << 20))
        ep = EpAllToAll.from_heap(heap, H, cap, epr, Tmax, k)
        g = torch.Generator().manual_seed(7)                      # same expert weights on every rank
        wgu = (torch.randn(E, 2 * I, H, generator=g) * 0.05).to(torch.bfloat16).to(dev)
        wd = (torch.randn(E, H, I, generator=g) * 0.05).to(torch.bfloat16).to(dev)
        lo, hi = rank * epr, (rank + 1) * epr
        gl = torch.Generator().manual_seed(100 + rank)            # own tokens
        T = [96, 5, 33, 64, 1, 77, 18, 50][rank]
        for layer in range(3):
            x = torch.randn(T, H, generator=gl).to(torch.bfloat16).to(dev)
            res = torch.randn(T, H, generator=gl).to(torch.bfloat16).to(dev)
            ids, wts = moe_ops.route(torch.randn(T, E, generator=gl).to(torch.bfloat16).to(dev), k, "topk_softmax", True)
            got = ep.moe(x, ids, wts, wgu[lo:hi].contiguous(), wd[lo:hi].contiguous(), I, "silu", residual=res)
            want = moe_ops.moe_ref(x, ids, wts, wgu, wd, I, "silu") + res.float()
            err = (got.float() - want).abs().max().item()
            assert err < 0.06, (rank, layer, err)
    """)
