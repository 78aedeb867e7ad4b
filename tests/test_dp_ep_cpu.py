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


def test_serve_ep_mode_a2a_gives_every_rank_its_own_listener():
    """`torch.distributed.run ... serve --ep-mode a2a`: rank r listens on port + r, serves its own requests,
    and the text equals what a single-process server of the same preset answers."""
    import json
    import signal
    import socket
    import subprocess
    import time
    import urllib.request

    def free_port():
        with socket.socket() as s:
            s.bind(("127.0.0.1", 0))
            return s.getsockname()[1]

    def ask(port, prompt):
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions",
                                     data=json.dumps({"prompt": prompt, "max_tokens": 8, "temperature": 0, "ignore_eos": True}).encode(),
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=120) as r:
            return json.loads(r.read())["choices"][0]["text"]

    def wait_up(port, proc):
        for _ in range(600):
            if proc.poll() is not None:
                raise AssertionError(f"server exited with {proc.returncode}")
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=2) as r:
                    if r.status == 200:
                        return
            except OSError:
                time.sleep(0.5)
        raise AssertionError("server did not come up")
    env = dict(os.environ, CUDA_VISIBLE_DEVICES="")
    common = ["-m", "preset:tiny-gpt-oss", "--device", "cpu", "--no-warmup", "-c", "256", "--no-preflight"]
    p1 = free_port()
    single = subprocess.Popen([sys.executable, "-m", "mlxcel_b200.cli", "serve", *common, "--port", str(p1)], env=env)
    base = free_port()
    duo = subprocess.Popen([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                            "--master-addr", "127.0.0.1", "--master-port", str(free_port()), "-m", "mlxcel_b200.cli",
                            "serve", *common, "--ep-mode", "a2a", "--port", str(base)], env=env, start_new_session=True)
    try:
        wait_up(p1, single)
        wait_up(base, duo)
        wait_up(base + 1, duo)
        want = [ask(p1, "hello there"), ask(p1, "another prompt, longer than the first one")]
        assert ask(base, "hello there") == want[0]
        assert ask(base + 1, "another prompt, longer than the first one") == want[1]
        assert ask(base + 1, "hello there") == want[0]
    finally:
        single.terminate()
        os.killpg(duo.pid, signal.SIGTERM)
        for p in (single, duo):
            try:
                p.wait(timeout=30)
            except subprocess.TimeoutExpired:
                p.kill()
