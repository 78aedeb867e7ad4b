"""Pipeline parallelism on CPU (gloo): 2 stages with micro-batching, and TP2 x PP2 on 4 ranks, must
reproduce the single-rank greedy tokens exactly in fp32."""
import os
import socket
import subprocess
import sys
import textwrap

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


BODY = """
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, %r)
dist.init_process_group("gloo")
rank, world = dist.get_rank(), dist.get_world_size()
TP = int(os.environ["TEST_TP"]); PP = world // TP
from mlxcel_b200.config import preset
from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams
from mlxcel_b200.models.decoder import DecoderModel
from mlxcel_b200.models.weights import random_weights
from mlxcel_b200.loading.shard import shard_weights, partition_layers
from mlxcel_b200.parallel.tp import TPComm
from mlxcel_b200.parallel.pp import PipelineContext, PipelineModel
cfg = preset("tiny-qwen3"); cfg.num_hidden_layers = 4
full = random_weights(cfg, seed=9, dtype=torch.float32, std=0.05)
g = torch.Generator().manual_seed(2)
prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (12, 40, 5, 19)]
sp = SamplingParams(max_tokens=8, ignore_eos=True)
ec = lambda: EngineConfig(max_batch=4, max_num_batched_tokens=64, num_blocks=64, max_model_len=128,
                          cuda_graphs=False, prefill_chunk_alone=32)
want = [s.output for s in Engine(DecoderModel(cfg, full), cfg, ec()).generate(prompts, sp)]
stage, tp_rank = rank // TP, rank %% TP
tp_group = None
for st in range(PP):
    grp = dist.new_group(list(range(st * TP, (st + 1) * TP)))
    if st == stage:
        tp_group = grp
comm = TPComm(tp_group, torch.device("cpu"), backend="nccl") if TP > 1 else None
ranges = partition_layers(cfg.num_hidden_layers, PP)
w = shard_weights(cfg, full, tp_rank, TP, layers=ranges[stage], vocab_parallel=TP > 1)
ctx = PipelineContext(dist.group.WORLD, stage, PP, tp_size=TP, tp_rank=tp_rank)
model = PipelineModel(cfg, w, ctx, comm=comm, num_micro=2, layer_range=ranges[stage])
eng = Engine(model, cfg, ec())
if os.environ.get("TEST_MTP") == "1":
    # the MTP head lives on the last stage; the other stages take part in the draft broadcast only
    from mlxcel_b200.speculative import MTPDrafter, random_mtp_weights
    from mlxcel_b200.parallel.pp import RemoteDrafter
    if ctx.is_last:
        mw = random_mtp_weights(cfg, dtype=torch.float32, std=0.05, tp_rank=tp_rank, tp_size=TP)
        eng.drafter = MTPDrafter(model, cfg, mw, num_blocks=64)
    else:
        eng.drafter = RemoteDrafter()
    eng.spec_k = 4
got = [s.output for s in eng.generate(prompts, sp)]
assert got == want, (rank, got, want)
assert ctx.stats["microbatches"] > 0
if os.environ.get("TEST_MTP") == "1":
    assert eng.stats["spec_rounds"] > 0 and eng.stats["spec_drafted"] > 0, eng.stats
assert ctx.stats.get("token_bytes", 0) > 0 or os.environ.get("TEST_MTP") == "1"
dist.barrier()
if rank == 0:
    print("PP_CPU_OK")
"""


@pytest.mark.parametrize("world,tp,mtp", [(2, 1, 0), (4, 2, 0), (2, 1, 1), (4, 2, 1)])
def test_pipeline_gloo(tmp_path, world, tp, mtp):
    script = tmp_path / "pp_cpu.py"
    script.write_text(textwrap.dedent(BODY % ROOT))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", TEST_TP=str(tp), OMP_NUM_THREADS="2", TEST_MTP=str(mtp))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0 and "PP_CPU_OK" in r.stdout, (r.stdout + r.stderr)[-3000:]
