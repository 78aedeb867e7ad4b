"""Multi-GPU checks of the fused GEMM + collective kernels and the tensor-parallel executor.
Each test spawns one process per GPU (NCCL for bootstrap), prints which test ran at which world
size, and is skipped on boxes with one GPU.

Error bounds come from an fp32 reduction of the same shards. bf16 keeps 8 significant bits, so one
round-to-nearest changes a value v by at most ``u |v|`` with ``u = 2^-8``. A fused result differs
from the fp32 sum of the per-rank products by the rounding of each partial tile (the peer-store
kernels round partials to bf16 before they cross NVLink) and by the rounding of the result itself:
at most ``u (sum_r |partial_r| + |result|)`` per element. The one-shot NVLS kernels keep fp32
partials and let the switch add them in fp32, so only ``u |result|`` remains there. The two-shot
NVLS kernel moves bf16 partials and the switch hands its fp32 sum back TRUNCATED to bf16
(measured), which adds ``2u |sum_r partial_r|``.
"""
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


def _run(name: str, world: int, body: str, timeout: int = 600, nvls: bool = False, extra_env=None) -> str:
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
        EPS = 2.0 ** -8
        def bound(parts_abs_sum, want, switch_sum=None):
            b = want.abs()
            if parts_abs_sum is not None:
                b = b + parts_abs_sum
            if switch_sum is not None:
                b = b + 2 * switch_sum.abs()
            return 1.01 * EPS * b + 1e-3
    """ % ROOT) + textwrap.dedent(body) + textwrap.dedent("""
        torch.cuda.synchronize()
        st = _lib.read_status(dev)
        assert st == 0, f"kernel status {st}"
        dist.barrier()
        torch.cuda.synchronize()
        if rank == 0:
            print("MULTI_OK %s world=%%d nvls=%%s" %% (world, os.environ.get("MLXCEL_B200_NVLS")), flush=True)
        sys.stdout.flush()
        # every rank is past its last collective and kernel: leave without tearing the communicator
        # down under live symmetric-memory mappings
        os._exit(0)
    """ % name)
    import tempfile
    path = os.path.join(tempfile.mkdtemp(prefix="mlxcel_multi_"), "ranks.py")
    with open(path, "w") as f:
        f.write(script)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0", MLXCEL_B200_REQUIRE_FUSED="1",
               MLXCEL_B200_NVLS="1" if nvls else "0",
               MLXCEL_B200_NVLS_ONESHOT="1" if nvls else "0")     # the nvls variants cover the in-switch one-shot path too
    env.update(extra_env or {})
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), path]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env)
    out = r.stdout + r.stderr
    assert r.returncode == 0 and "MULTI_OK" in out, out[-4000:]
    for line in out.splitlines():
        if line.startswith(("MULTI_OK", "INFO ")):
            print(line)
    return out


def _world() -> int:
    n = torch.cuda.device_count()
    return 8 if n >= 8 else 4 if n >= 4 else 2 if n >= 2 else 1


_FUSED_BODY = """
    comm = TPComm(dist.group.WORLD, dev, backend="fused", max_tokens=2048, hidden=1024, vocab=8192)
    assert comm.backend == "fused"
    nvls = comm.fused.nvls
    if os.environ["MLXCEL_B200_NVLS"] == "1" and not nvls and rank == 0:
        print("INFO no multicast mapping on this box: the peer-store protocol ran instead", flush=True)
    torch.manual_seed(0)   # same full tensors on every rank, each takes its shard
    worst = 0.0
    for M in (1, 7, 64, 200, 300, 1500):
        K, N = 512 * world, 1024
        x = torch.randn(M, K, device=dev).to(torch.bfloat16)
        w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
        bias = torch.randn(N, device=dev).to(torch.bfloat16)
        res = torch.randn(M, N, device=dev).to(torch.bfloat16)
        ks = slice(rank * 512, (rank + 1) * 512)
        parts = [x[:, r * 512:(r + 1) * 512].float() @ w[:, r * 512:(r + 1) * 512].float().t() for r in range(world)]
        want = sum(parts) + bias.float() + res.float()           # the fp32 reduction
        pabs = sum(p.abs() for p in parts)
        sw = sum(parts) if nvls else None                        # what the switch narrows on the two-shot NVLS path
        for rep in range(3):
            got = comm.row_parallel_linear(x[:, ks].contiguous(), w[:, ks].contiguous(), bias, res.clone())
            torch.cuda.synchronize()
            diff = (got.float() - want).abs()
            # row_parallel_linear: one-shot for M <= 256 (NVLS: fp32 partials), two-shot above
            bnd = bound(None, want) if (nvls and M <= 256) else bound(pabs, want, sw)
            if not bool((diff <= bnd).all()):
                i = int((diff - bnd).argmax())
                r_, c_ = divmod(i, N)
                detail = dict(M=M, rep=rep, diff=diff[r_, c_].item(), bound=bnd[r_, c_].item(), got=got[r_, c_].item(),
                              want=want[r_, c_].item(), parts=[p[r_, c_].item() for p in parts],
                              bias=bias[c_].item(), res=res[r_, c_].item(), bad=int((diff > bnd).sum()))
                raise AssertionError(f"DETAIL {detail}")
            worst = max(worst, diff.max().item())
            ref0 = got.clone(); dist.broadcast(ref0, 0)
            if nvls:
                # every rank asks the switch for its own sum: equal up to the result's rounding
                assert bool(((ref0.float() - got.float()).abs() <= 2 * EPS * want.abs() + 1e-3).all()), (M, rep)
            else:
                assert torch.equal(ref0, got), (M, rep)          # rank-ordered sums: bitwise identical
            if M > 256:   # the fused two-shot kernel: one owner reduces, everyone receives the same bits
                got2 = comm.fused.gemm_allreduce(x[:, ks].contiguous(), w[:, ks].contiguous(), bias, res.clone())
                torch.cuda.synchronize()
                d2 = (got2.float() - want).abs()
                assert bool((d2 <= bound(pabs, want, sw)).all()), (M, rep, d2.max().item())
                ref0 = got2.clone(); dist.broadcast(ref0, 0)
                assert torch.equal(ref0, got2), (M, rep)
        # quantized row-parallel projection -> all-reduce in one kernel (packed 4-bit shards)
        if M <= 256:
            from mlxcel_b200.ops import quant
            qts = quant.quantize(w[:, ks].float().cpu(), "affine", 4, 64)
            qts = qts.to(dev)
            wdq = quant.dequantize_ref(qts).float()
            wparts = [torch.empty(N, 512, device=dev) for _ in range(world)]
            dist.all_gather(wparts, wdq.contiguous())
            qparts = [x[:, r * 512:(r + 1) * 512].float() @ wparts[r].t() for r in range(world)]
            want_q = sum(qparts) + bias.float() + res.float()
            # the GEMM form rounds every dequantised weight to bf16 before the MMA: an error of up to
            # u on each product, i.e. on sum_k |x_k| |w_k| (no cancellation), on top of the partial rounding
            prod_abs = sum(x[:, r * 512:(r + 1) * 512].float().abs() @ wparts[r].abs().t() for r in range(world))
            qbound = bound(None if nvls else sum(p.abs() for p in qparts), want_q) + EPS * prod_abs
            got_q = comm.row_parallel_linear(x[:, ks].contiguous(), qts, bias, res.clone())
            torch.cuda.synchronize()
            dq = (got_q.float() - want_q).abs()
            assert bool((dq <= qbound).all()), (M, "q4", dq.max().item())
            if M <= 8:
                # M <= 8 took the GEMV -> all-reduce kernel above; the GEMM form of the same projection must agree
                import mlxcel_b200.parallel.tp as tpm
                old, tpm._QMV_AR_MAX_M = tpm._QMV_AR_MAX_M, 0
                got_g = comm.row_parallel_linear(x[:, ks].contiguous(), qts, bias, res.clone())
                tpm._QMV_AR_MAX_M = old
                torch.cuda.synchronize()
                dg = (got_g.float() - want_q).abs()
                assert bool((dg <= qbound).all()), (M, "q4 gemm", dg.max().item())
                for rep in range(2):      # repeated calls reuse the channel (parity, flags)
                    again = comm.row_parallel_linear(x[:, ks].contiguous(), qts, bias, res.clone())
                    torch.cuda.synchronize()
                    assert bool(((again.float() - got_q.float()).abs() <= 2 * EPS * want_q.abs() + 1e-3).all()), (M, rep)
        # stand-alone all-reduce (one-shot for small, two-shot for large tensors)
        part = torch.randn(M, N, device=dev).to(torch.bfloat16) * (rank + 1)
        aparts = [torch.empty_like(part) for _ in range(world)]
        dist.all_gather(aparts, part)
        want_ar = sum(p.float() for p in aparts)
        got_ar = comm.all_reduce(part.clone())
        torch.cuda.synchronize()
        assert bool(((got_ar.float() - want_ar).abs() <= 3.03 * EPS * want_ar.abs() + 1e-3).all()), M
        # all-gather of a vocab-parallel projection
        if M <= 256:
            Vl = 1024
            wl = (torch.randn(world * Vl, 256, device=dev) * 0.05).to(torch.bfloat16)
            xs = torch.randn(M, 256, device=dev).to(torch.bfloat16)
            lg = comm.lm_head(xs, wl[rank * Vl:(rank + 1) * Vl].contiguous())
            torch.cuda.synchronize()
            wantl = xs.float() @ wl.float().t()
            assert bool(((lg.float() - wantl).abs() <= 1.01 * EPS * wantl.abs() + 1e-3).all())
    if rank == 0:
        print("INFO fused GEMM->all-reduce max |err| vs the fp32 reduction: %.4f (world %d, nvls %s)" % (worst, world, nvls),
              flush=True)
"""


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
@pytest.mark.parametrize("nvls", [False, True], ids=["peer_stores", "nvls_multimem"])
def test_fused_gemm_allreduce_and_allgather(nvls):
    _run(f"test_fused_gemm_allreduce_and_allgather[{'nvls' if nvls else 'peer'}]", _world(), _FUSED_BODY, nvls=nvls)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
@pytest.mark.parametrize("nvls", [False, True], ids=["peer_stores", "nvls_multimem"])
def test_tp_engine_fused_matches_nccl_and_single_gpu(nvls):
    """Teacher-forced log-probabilities of the tensor-parallel executors against the single-GPU
    executor (one prefill each), then greedy generation through the engine."""
    _run(f"test_tp_engine_fused_matches_nccl_and_single_gpu[{'nvls' if nvls else 'peer'}]", _world(), """
        from mlxcel_b200.config import preset
        from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams
        from mlxcel_b200.engine.scoring import sequence_logprobs
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
        single_model = DecoderModel(cfg, full)
        lp_single = sequence_logprobs(single_model, cfg, prompts[3])
        single = [s.output for s in Engine(single_model, cfg, ec()).generate(prompts, sp)]
        outs = {}
        for backend in ("nccl", "fused"):
            comm = TPComm(dist.group.WORLD, dev, backend=backend, max_tokens=512, hidden=512, vocab=4096)
            w = shard_weights(cfg, full, comm.tp_rank, comm.tp_size)
            model = DecoderModel(cfg, w, comm=comm)
            lp = sequence_logprobs(model, cfg, prompts[3])
            d = (lp - lp_single).abs().max().item()
            # 299 teacher-forced positions through 2 layers in bf16: the two executors differ only by
            # where partial sums are rounded
            assert d < 0.08, (backend, d)
            if rank == 0:
                print("INFO %s: max |logprob - single GPU| = %.4f over %d positions" % (backend, d, lp.numel()), flush=True)
            eng = Engine(model, cfg, ec())
            outs[backend] = [s.output for s in eng.generate(prompts, sp)]
        assert all(a[0] == b[0] for a, b in zip(single, outs["fused"])), (single, outs)
        assert all(len(o) == 10 for o in outs["fused"] + outs["nccl"])
    """, nvls=nvls)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_ep_all_to_all_moe_matches_local_reference():
    """Token-sharded expert parallelism: dispatch / combine kernels over peer memory, three layers
    back to back on the same buffers, every rank with its own token count."""
    _run("test_ep_all_to_all_moe_matches_local_reference", _world(), """
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


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_dp_attention_ep_engine_matches_the_single_gpu_engine():
    """Data-parallel attention + expert-parallel MoE in the engine: every rank serves its own requests
    (one rank none at all), MoE rows cross NVLink through the dispatch / combine kernels, ticks are in
    lockstep. Tokens are compared with the same requests on one GPU holding every expert."""
    _run("test_dp_attention_ep_engine_matches_the_single_gpu_engine", _world(), """
        from mlxcel_b200.config import preset
        from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams
        from mlxcel_b200.loading.shard import shard_weights
        from mlxcel_b200.models.decoder import DecoderModel
        from mlxcel_b200.models.weights import random_weights
        from mlxcel_b200.parallel.dp_ep import DpEpComm
        cfg = preset("tiny-gpt-oss")
        if cfg.num_experts % world:
            sys.exit(0)
        full = random_weights(cfg, seed=5, dtype=torch.bfloat16, std=0.05)
        ecfg = lambda: EngineConfig(max_batch=8, max_num_batched_tokens=128, num_blocks=128, max_model_len=256,
                                    prefill_chunk_alone=32, prefill_chunk_contended=32)
        g = torch.Generator().manual_seed(100 + rank)
        lens = [(9, 21, 14), (), (33, 40), (12,), (5, 6, 7, 8), (64,), (3,), (17, 19)][rank]
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
        sp = SamplingParams(max_tokens=12, ignore_eos=True)
        import copy
        to_dev = lambda w: __import__("mlxcel_b200.loading.checkpoint", fromlist=["_to_device"])._to_device(w, dev)
        ref = Engine(DecoderModel(cfg, to_dev(copy.deepcopy(full))), cfg, ecfg())
        want = [s.output for s in ref.generate(prompts, sp)] if prompts else []
        del ref
        w = to_dev(shard_weights(cfg, full, 0, 1, ep=world, ep_rank=rank, vocab_parallel=False))
        comm = DpEpComm(dist.group.WORLD, dev, hidden=cfg.hidden_size, top_k=cfg.num_experts_per_tok,
                        num_experts=cfg.num_experts, max_tokens=128)
        eng = Engine(DecoderModel(cfg, w, comm=comm), cfg, ecfg())
        assert eng.dp_lockstep and not eng.ecfg.lookahead
        ids = [eng.add_request(p, sp) for p in prompts]
        ticks = 0
        while True:
            eng.step()
            ticks += 1
            if not eng.dp_active:
                break
            assert ticks < 1000
        got = [eng.seqs[i].output for i in ids]
        # bf16 partial sums are ordered differently (per-expert rows return one by one): allow late divergence
        for a, b in zip(got, want):
            assert a[0] == b[0], (rank, a, b)
        agree = sum(x == y for a, b in zip(got, want) for x, y in zip(a, b)) / max(1, sum(len(b) for b in want))
        assert not want or agree >= 0.75, (rank, agree, got, want)
        if rank == 1:
            assert eng.stats.get("null_forwards", 0) == ticks - 1
        elif prompts:
            assert eng.stats["graph_replays"] > 0            # decode ticks replay CUDA graphs (captured after a dry warm-up)
    """)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs >= 2 GPUs")
def test_rank_leaving_between_steps_is_seen_by_the_survivors():
    """A rank leaves a GPU job between steps, with none of its kernels or collectives in flight; the
    others learn of it on the host from the heartbeat before their next launch. NCCL only (NVLS off),
    no symmetric heap and no multicast mapping, so the leaving rank has no memory bound to one."""
    world = min(_world(), 4)
    script = textwrap.dedent("""
        import os, sys, time, torch, torch.distributed as dist
        sys.path.insert(0, %r)
        from mlxcel_b200 import ops
        from mlxcel_b200.parallel.health import Heartbeat, FailureDetector, PeerFailure
        rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
        torch.cuda.set_device(rank)
        dev = torch.device("cuda", rank)
        dist.init_process_group("nccl", device_id=dev)
        store = dist.TCPStore("127.0.0.1", int(os.environ["HB_PORT"]), world, rank == 0)
        hb = Heartbeat(store, rank, interval=0.1).start()
        det = FailureDetector(store, rank, world, interval=0.1, threshold=5)
        x = torch.randn(64, 256, device=dev).to(torch.bfloat16)
        for step in range(3):                      # three healthy steps: kernel + collective
            det.raise_if_failed()
            y = ops.linear(x, x[:32].contiguous())
            dist.all_reduce(y)
            torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        if rank == world - 1:
            hb.stop()
            sys.stdout.flush()
            os._exit(0)                            # leaves between steps, nothing in flight
        deadline = time.time() + 20
        seen = None
        while time.time() < deadline and seen is None:
            try:
                det.raise_if_failed()              # what the step loop does before every launch
                time.sleep(0.05)
            except PeerFailure as e:
                seen = e.ranks
        print("SURVIVOR", rank, "DETECTED" if seen == [world - 1] else "MISSED", seen, flush=True)
        sys.stdout.flush()
        os._exit(0 if seen == [world - 1] else 3)   # no further collective is started with the lost rank
    """ % ROOT)
    import tempfile
    path = os.path.join(tempfile.mkdtemp(prefix="mlxcel_leave_"), "ranks.py")
    with open(path, "w") as f:
        f.write(script)
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), NCCL_NVLS_ENABLE="0",
               WORLD_SIZE=str(world), HB_PORT=str(_free_port()))
    procs = [subprocess.Popen([sys.executable, path], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(world)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    for r in range(world - 1):
        assert f"SURVIVOR {r} DETECTED" in outs[r], outs
    print(f"MULTI_OK test_rank_leaving_between_steps_is_seen_by_the_survivors world={world}")
