"""Data-parallel attention + expert-parallel MoE over gloo ranks: every rank serves its own requests,
MoE rows travel to the experts' owners, ticks are taken in lockstep (null forwards on idle ranks).
Each rank's greedy tokens must equal what one process with all experts produces for those requests."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from mlxcel_b200.config import preset
from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams
from mlxcel_b200.loading.shard import shard_weights
from mlxcel_b200.models.decoder import DecoderModel
from mlxcel_b200.models.weights import random_weights

PRESET = "tiny-gpt-oss"


def _prompts(cfg, rank):
    g = torch.Generator().manual_seed(100 + rank)
    lens = [(9, 21, 14), (33,), (), (12,)][rank]       # rank 2 (when present) never has a request
    return [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]


def _ecfg():
    return EngineConfig(max_batch=4, max_num_batched_tokens=64, num_blocks=64, max_model_len=256, cuda_graphs=False,
                        prefill_chunk_alone=16, prefill_chunk_contended=16)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from mlxcel_b200.parallel.dp_ep import DpEpComm
        cfg = preset(PRESET)
        full = random_weights(cfg, seed=5, dtype=torch.float32, std=0.05)
        w = shard_weights(cfg, full, 0, 1, ep=world, ep_rank=rank, vocab_parallel=False)
        comm = DpEpComm(dist.group.WORLD, "cpu", hidden=cfg.hidden_size, top_k=cfg.num_experts_per_tok,
                        num_experts=cfg.num_experts, max_tokens=64)
        eng = Engine(DecoderModel(cfg, w, comm=comm), cfg, _ecfg())
        assert eng.dp_lockstep and w.layers[0].experts_gate_up.shape[0] == cfg.num_experts // world
        sp = SamplingParams(max_tokens=10, ignore_eos=True)
        ids = [eng.add_request(p, sp) for p in _prompts(cfg, rank)]
        ticks = 0
        while True:
            eng.step()
            ticks += 1
            if not eng.dp_active:
                break
            assert ticks < 500
        q.put((rank, [eng.seqs[i].output for i in ids], ticks, eng.stats.get("null_forwards", 0),
               comm.a2a.stats["rows_served"]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 4])
def test_dp_ep_ranks_match_the_single_process_engine(world):
    cfg = preset(PRESET)
    if cfg.num_experts % world:
        pytest.skip("expert count not divisible")
    full = random_weights(cfg, seed=5, dtype=torch.float32, std=0.05)
    sp = SamplingParams(max_tokens=10, ignore_eos=True)
    want = {}
    for r in range(world):
        eng = Engine(DecoderModel(cfg, full), cfg, _ecfg())
        want[r] = [s.output for s in eng.generate(_prompts(cfg, r), sp)] if _prompts(cfg, r) else []
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + os.getpid() % 300 + world
    procs = [ctx.Process(target=_worker, args=(r, world, port, q)) for r in range(world)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(world):
        r, outs, ticks, nulls, served = q.get(timeout=300)
        got[r] = (outs, ticks, nulls, served)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    for r in range(world):
        assert got[r][0] == want[r], r
    # every rank took the same number of ticks; the rank with the short job (or none) idled through null forwards
    assert len({got[r][1] for r in range(world)}) == 1
    assert all(got[r][3] > 0 for r in range(world))
    if world == 4:
        assert got[2][2] == got[2][1] - 1           # the rank without requests ran a null forward in every working tick
