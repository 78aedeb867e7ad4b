"""Serving control plane on CPU (gloo, 2 ranks): rank 0 takes requests and broadcasts step
descriptors, rank 1 runs the executor loop. Under concurrent requests, a cancellation and KV
pressure (preemption) the tokens must equal a single-process run, and both ranks must end in
the same scheduler state."""
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


BODY = """
import os, sys, queue, time, torch, torch.distributed as dist
sys.path.insert(0, %r)
from mlxcel_b200.parallel.control import ControlPlane, init_distributed, engine_digest
dev, ctl_group = init_distributed("cpu")
rank, world = dist.get_rank(), dist.get_world_size()
from mlxcel_b200.config import preset
from mlxcel_b200.engine import Engine, EngineConfig, SamplingParams
from mlxcel_b200.models.decoder import DecoderModel
from mlxcel_b200.models.weights import random_weights
from mlxcel_b200.loading.shard import shard_weights
from mlxcel_b200.parallel.tp import TPComm
from mlxcel_b200.server.worker import GenRequest, ModelWorker
from mlxcel_b200.tokenizer import ByteTokenizer
cfg = preset("tiny-llama")
full = random_weights(cfg, seed=9, dtype=torch.float32, std=0.05)
g = torch.Generator().manual_seed(2)
prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (30, 44, 21, 37, 26)]
# 10 blocks of 16 tokens for up to 3 rows of ~70 tokens: rows get preempted and recomputed
ec = lambda: EngineConfig(max_batch=3, max_num_batched_tokens=64, num_blocks=10, max_model_len=128,
                          cuda_graphs=False, prefill_chunk_alone=32, prefix_cache=False)
sp = lambda: SamplingParams(max_tokens=24, ignore_eos=True)
tok = ByteTokenizer(cfg.vocab_size)
comm = TPComm(dist.group.WORLD, torch.device("cpu"), backend="nccl")
eng = Engine(DecoderModel(cfg, shard_weights(cfg, full, rank, world), comm=comm), cfg, ec())
worker = ModelWorker(eng, tok, control=ControlPlane(ctl_group))
if rank != 0:
    worker.follow()
    st = torch.tensor([eng.stats["steps"], eng.stats["preemptions"], engine_digest(eng) & 0x7FFFFFFF])
    dist.send(st, 0)
    sys.exit(0)
outs = [queue.Queue() for _ in prompts]
reqs = [GenRequest(prompt_ids=p, params=sp(), out=o, request_id=f"r{i}") for i, (p, o) in enumerate(zip(prompts, outs))]
for r in reqs[:4]:
    worker.submit(r)
got, texts, done = [[] for _ in prompts], [""] * len(prompts), [None] * len(prompts)
cancelled = late = False
deadline = time.time() + 300
while time.time() < deadline and not all(done[i] for i in (0, 1, 3, 4)):
    for i, o in enumerate(outs):
        try:
            ev = o.get(timeout=0.01)
        except queue.Empty:
            continue
        if ev.kind == "token":
            got[i].append(ev.token_id)
        elif ev.kind in ("done", "error"):
            done[i] = ev
    if not cancelled and len(got[2]) >= 3:
        worker.cancel(reqs[2]); cancelled = True           # a client goes away mid-generation
    if not late and len(got[0]) >= 5:
        worker.submit(reqs[4]); late = True                # a request arrives while others decode
assert all(done[i] is not None and done[i].kind == "done" for i in (0, 1, 3, 4)), done
worker.shutdown()
other = torch.zeros(3, dtype=torch.long)
dist.recv(other, 1)
single = Engine(DecoderModel(cfg, full), cfg, EngineConfig(max_batch=8, max_num_batched_tokens=256, num_blocks=64,
                max_model_len=128, cuda_graphs=False, prefix_cache=False))
want = [s.output for s in single.generate(prompts, sp())]
for i in (0, 1, 3, 4):
    assert got[i] == want[i], (i, got[i], want[i])
assert 3 <= len(got[2]) < 24 and got[2] == want[2][:len(got[2])]
assert eng.stats["preemptions"] > 0, eng.stats
mine = [eng.stats["steps"], eng.stats["preemptions"], engine_digest(eng) & 0x7FFFFFFF]
assert other.tolist() == mine, (other.tolist(), mine)
print("CONTROL_OK", eng.stats["steps"], eng.stats["preemptions"], worker.control.stats)
"""


def test_two_rank_control_plane_matches_single_process(tmp_path):
    script = tmp_path / "ctl.py"
    script.write_text(textwrap.dedent(BODY % ROOT))
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), str(script)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
    assert r.returncode == 0 and "CONTROL_OK" in r.stdout, (r.stdout + r.stderr)[-4000:]


def _torchrun(args, n=2, timeout=600):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={n}",
           "--master-addr", "127.0.0.1", "--master-port", str(_free_port()), "-m", "mlxcel_b200.cli", *args]
    return subprocess.run(cmd, capture_output=True, text=True, timeout=timeout, env=env, cwd=ROOT)


def test_cli_generate_under_tp_and_pp():
    """`generate --tp 2` and `generate --pp 2` from the command line: the package joins the job by
    itself (device, process group), one rank prints."""
    single = subprocess.run([sys.executable, "-m", "mlxcel_b200.cli", "generate", "-m", "preset:tiny-llama", "--device", "cpu",
                             "-p", "hello", "-n", "6", "--ignore-eos"], capture_output=True, text=True, timeout=600,
                            env=dict(os.environ, PYTHONPATH=ROOT), cwd=ROOT)
    assert single.returncode == 0, single.stderr[-2000:]
    for flags in (["--tp", "2"], ["--pp", "2"]):
        r = _torchrun(["generate", "-m", "preset:tiny-llama", "--device", "cpu", "-p", "hello", "-n", "6", "--ignore-eos", *flags])
        assert r.returncode == 0, (flags, (r.stdout + r.stderr)[-3000:])
        assert "generated 6 tok" in r.stderr, (flags, r.stderr[-2000:])
        assert r.stderr.count("generated 6 tok") == 1          # one rank reports
    # pipeline stages hold the same replicated weights as the single process: same text
    assert r.stdout.strip() == single.stdout.strip(), (r.stdout, single.stdout)
    bad = _torchrun(["generate", "-m", "preset:tiny-llama", "--device", "cpu", "-p", "x", "-n", "2"])
    assert bad.returncode != 0 and "neither --tp nor --pp" in (bad.stdout + bad.stderr)


def test_serve_tp2_streams_chat_completions():
    """`serve --tp 2`: rank 0 listens, rank 1 follows the step descriptors; a streamed chat completion
    and a plain completion come back, then the job is stopped."""
    import json
    import signal
    import time
    import urllib.request

    port = _free_port()
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", str(_free_port()), "-m", "mlxcel_b200.cli", "serve", "-m", "preset:tiny-llama", "--device", "cpu",
           "--tp", "2", "--port", str(port), "--parallel", "2", "--no-preflight"]
    proc = subprocess.Popen(cmd, env=env, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True,
                            start_new_session=True)
    try:
        ok = False
        for _ in range(240):
            try:
                with urllib.request.urlopen(f"http://127.0.0.1:{port}/health", timeout=1) as r:
                    ok = r.status == 200
                    break
            except Exception:
                if proc.poll() is not None:
                    break
                time.sleep(0.5)
        assert ok, proc.stdout.read()[-3000:] if proc.poll() is not None else "server did not come up"
        body = json.dumps({"messages": [{"role": "user", "content": "hi"}], "max_tokens": 5, "stream": True,
                           "temperature": 0, "ignore_eos": True}).encode()
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/chat/completions", data=body,
                                     headers={"Content-Type": "application/json"})
        chunks = []
        with urllib.request.urlopen(req, timeout=120) as r:
            for line in r:
                line = line.decode().strip()
                if line.startswith("data: ") and line != "data: [DONE]":
                    chunks.append(json.loads(line[6:]))
        assert len(chunks) >= 2 and chunks[-1]["choices"][0]["finish_reason"] in ("length", "stop")
        body = json.dumps({"prompt": "abc", "max_tokens": 4, "temperature": 0, "ignore_eos": True}).encode()
        req = urllib.request.Request(f"http://127.0.0.1:{port}/v1/completions", data=body,
                                     headers={"Content-Type": "application/json"})
        with urllib.request.urlopen(req, timeout=120) as r:
            out = json.loads(r.read())
        assert out["usage"]["completion_tokens"] == 4
    finally:
        os.killpg(proc.pid, signal.SIGTERM)
        try:
            proc.wait(timeout=30)
        except subprocess.TimeoutExpired:
            os.killpg(proc.pid, signal.SIGKILL)
