"""Tensor-parallel sharding and lockstep execution on CPU (gloo, world_size 2): the sharded
executor must reproduce the single-rank greedy tokens exactly in fp32."""
import os
import socket
import subprocess
import sys
import textwrap

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_tp2_gloo_matches_single_rank(tmp_path):
    script = tmp_path / "tp_cpu.py"
    script.write_text(textwrap.dedent("""
        import os, sys, torch, torch.distributed as dist
        sys.path.insert(0, %r)
        dist.init_process_group("gloo")
        rank, world = dist.get_rank(), dist.get_world_size()
        from mlxcel_b200.config import preset
        from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams
        from mlxcel_b200.models.decoder import DecoderModel
        from mlxcel_b200.models.weights import random_weights
        from mlxcel_b200.loading.shard import shard_weights
        from mlxcel_b200.parallel.tp import TPComm
        for name in ("tiny-llama", "tiny-qwen3"):
            cfg = preset(name)
            full = random_weights(cfg, seed=9, dtype=torch.float32, std=0.05)
            g = torch.Generator().manual_seed(2)
            prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (12, 40, 5)]
            sp = SamplingParams(max_tokens=8, ignore_eos=True)
            ec = lambda: EngineConfig(max_batch=4, max_num_batched_tokens=64, num_blocks=64,
                                      max_model_len=128, cuda_graphs=False, prefill_chunk_alone=32)
            want = [s.output for s in Engine(DecoderModel(cfg, full), cfg, ec()).generate(prompts, sp)]
            comm = TPComm(dist.group.WORLD, torch.device("cpu"), backend="nccl")
            w = shard_weights(cfg, full, rank, world)
            got = [s.output for s in Engine(DecoderModel(cfg, w, comm=comm), cfg, ec()).generate(prompts, sp)]
            assert got == want, (name, got, want)
        dist.barrier()
        if rank == 0:
            print("TP_CPU_OK")
    """ % ROOT))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600, env=env)
    assert r.returncode == 0 and "TP_CPU_OK" in r.stdout, (r.stdout + r.stderr)[-3000:]
