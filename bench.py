#!/usr/bin/env python
"""Headline benchmark: continuous-batching serving throughput of the Llama-3.1-8B architecture
(bf16, random-init weights, synthetic token-id prompts), tensor-parallel over N GPUs of one node.

One "step" is one complete serving round of the configured workload. The default (--config 2) is
the headline: 64 concurrent requests, each a 1024-token prompt and 256 greedy output tokens, paged
KV with 16-token blocks. The metric is output tokens per second over the whole round (prefill
included).

    python bench.py --gpus N --steps K --warmup W            # this framework, headline configuration
    python bench.py --config 3|4|5 --gpus N ...              # the other benchmark configurations
    python bench.py --impl torch --gpus N ...                # plain PyTorch (cuBLAS / SDPA / NCCL) executor
                                                             # under the same engine and workload
    python bench.py --impl reference ...                      # the reference (not installable here)

Configurations (synthetic token ids, random-init weights of the named architecture):
  2  Llama-3.1-8B bf16, TP = N, 64 x (1024 -> 256)
  3  Llama-3.1-8B MLX affine 4-bit (group 64) + 8-bit KV, TP = N, 512 -> 1024 at batch 32 (the
     reported value) and batch 1 (reported under "batch1")
  4  gpt-oss-120b shape, mxfp4 experts, attention tensor-parallel and experts expert-parallel over
     the N ranks, 128 x (2048 -> 512)
  5  Qwen3-32B bf16, TP x PP = N (TP4 x PP2 at N = 8), one-layer MTP drafter proposing 3 tokens per
     round, 16 x (4096 -> 256) with 512-token prefill chunks

For N > 1 launch with ``python -m torch.distributed.run --nproc-per-node N ... bench.py --gpus N``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

CONFIGS = {
    2: dict(model="llama-3.1-8b", requests=64, prompt_len=1024, output_len=256, kv_bits=16, quantize=None,
            chunk=None),
    3: dict(model="llama-3.1-8b", requests=32, prompt_len=512, output_len=1024, kv_bits=8,
            quantize=dict(dense=("affine", 4, 64), lm_head=True), chunk=None),
    4: dict(model="gpt-oss-120b", requests=128, prompt_len=2048, output_len=512, kv_bits=16,
            quantize=dict(experts=("mxfp4", 4, 32)), chunk=None),
    5: dict(model="qwen3-32b", requests=16, prompt_len=4096, output_len=256, kv_bits=16, quantize=None, chunk=512),
}

BASELINE_TOK_S = 105.1  # reference's best published serving aggregate (8 clients, llama-3.1-8b-4bit,
#                         M1 Ultra, docs/CONTINUOUS_BATCHING.md:240-245); it publishes no B200 number.


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.gpu_index, self.rows, self.proc = gpu_index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits", "-lms", "200",
                 "-i", str(self.gpu_index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, power = [], [], set(), []
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 9:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                power.append(float(r[3]))
            except ValueError:
                continue
            for n, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        # under load = the upper half of the power samples
        if sm:
            order = sorted(range(len(sm)), key=lambda i: power[i])
            load = [sm[i] for i in order[len(order) // 2:]]
        else:
            load = []
        return {"sm_mhz": statistics.median(load) if load else None,
                "sm_max_mhz": max(mx) if mx else None, "reasons": sorted(reasons),
                "samples": len(sm), "power_w_max": max(power) if power else None}


def reference_arm(args) -> None:
    # The reference is a Rust workspace over a C++ MLX runtime that it downloads at build time;
    # pip cannot install it and this image has no cargo/rustc, so there is nothing to run.
    print(json.dumps({"impl": "reference", "unavailable":
                      "reference is a Rust/C++ project (no setup.py/pyproject.toml at its root; "
                      "MLX/CUTLASS fetched at build time; no cargo in the image): pip install failed"}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "torch", "reference"])
    ap.add_argument("--config", type=int, default=2, choices=[2, 3, 4, 5])
    ap.add_argument("--model", default=None)
    ap.add_argument("--requests", type=int, default=None)
    ap.add_argument("--prompt-len", type=int, default=None)
    ap.add_argument("--output-len", type=int, default=None)
    ap.add_argument("--kv-bits", type=int, default=None)
    ap.add_argument("--layers", type=int, default=0, help="debugging only: fewer layers (the line is then marked invalid)")
    ap.add_argument("--no-mtp", action="store_true", help="config 5 without the drafter (classic decoding)")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--tp-backend", default="fused", choices=["fused", "nccl"])
    ap.add_argument("--ep-mode", default="replicated", choices=["replicated", "a2a"],
                    help="config 4 on several GPUs: 'replicated' = tensor-parallel attention, tokens on every rank, "
                         "experts sharded, all-reduce combine; 'a2a' = data-parallel attention (every rank serves "
                         "requests / N of the batch), MoE rows exchanged by the dispatch / combine kernels")
    ap.add_argument("--watchdog", type=int, default=1500,
                    help="seconds without finishing a round before every thread's stack is dumped and the "
                         "process exits (a stuck multi-rank run then ends by itself)")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm(args)
    if args.warmup < 3:
        args.warmup = 3
    preset = CONFIGS[args.config]
    for k in ("model", "requests", "prompt_len", "output_len", "kv_bits"):
        if getattr(args, k) is None:
            setattr(args, k, preset[k])
    if args.impl == "torch":
        if args.config != 2:
            raise SystemExit("--impl torch covers the headline configuration (--config 2)")
        sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
        from benchmarks import torch_executor
        torch_executor.install()
        args.tp_backend = "nccl"

    import faulthandler

    faulthandler.dump_traceback_later(args.watchdog, exit=True)   # re-armed at every round
    import torch

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("launch with torch.distributed.run --nproc-per-node N for --gpus N > 1")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)

    from mlxcel_b200.engine import EngineConfig, SamplingParams
    from mlxcel_b200.llm import LLM
    from mlxcel_b200.ops import _lib

    comm = None
    pp = 1
    dp = 1                      # data-parallel ranks (each serves requests / dp of the batch)
    if args.config == 5 and world > 1:
        pp = 2
    tp = world // pp
    ctx = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=dev)
        from mlxcel_b200.parallel.tp import TPComm
        group = dist.group.WORLD
        if pp > 1:
            stage, tp_rank = rank // tp, rank % tp
            for st in range(pp):
                grp = dist.new_group(list(range(st * tp, (st + 1) * tp)))
                if st == stage:
                    group = grp
        if args.config == 4 and args.ep_mode == "a2a":
            from mlxcel_b200.config import preset as _cp
            from mlxcel_b200.parallel.dp_ep import DpEpComm
            c4 = _cp(args.model)
            comm = DpEpComm(group, dev, hidden=c4.hidden_size, top_k=c4.num_experts_per_tok, num_experts=c4.num_experts,
                            max_tokens=8192)
            dp = world
            tp = 1
        elif tp > 1:
            hidden = {"llama-3.1-8b": 4096, "qwen3-32b": 5120, "gpt-oss-120b": 2880}.get(args.model, 8192)
            comm = TPComm(group, dev, backend=args.tp_backend, hidden=max(4096, hidden), max_tokens=8192)

    max_len = args.prompt_len + args.output_len + 16
    chunk = preset["chunk"]
    ecfg = EngineConfig(max_batch=max(1, args.requests // dp), max_num_batched_tokens=8192,
                        prefill_chunk_alone=chunk or max(2048, args.prompt_len),
                        prefill_chunk_contended=chunk or max(512, args.prompt_len),
                        max_prefill_seqs=16 if chunk else 8,
                        block_size=16, kv_bits=args.kv_bits, prefix_cache=False,
                        max_model_len=max_len, cuda_graphs=not args.no_graphs,
                        num_blocks=(max_len // 16 + 2) * max(1, args.requests // dp) + 64)
    drafter_note = None
    if pp > 1:
        import torch.distributed as dist

        from mlxcel_b200.config import preset as cfg_preset
        from mlxcel_b200.loading.shard import partition_layers
        from mlxcel_b200.models.weights import random_weights
        from mlxcel_b200.parallel.pp import PipelineContext, PipelineModel
        cfg = cfg_preset(args.model)
        if args.layers:
            cfg.num_hidden_layers = args.layers
        stage, tp_rank = rank // tp, rank % tp
        ranges = partition_layers(cfg.num_hidden_layers, pp)
        w = random_weights(cfg, seed=0, dtype=torch.bfloat16, device=dev, tp_rank=tp_rank, tp_size=tp, ep_rank=tp_rank,
                           ep_size=tp, layers=ranges[stage], vocab_parallel=tp > 1 and cfg.vocab_size % tp == 0)
        ctx = PipelineContext(dist.group.WORLD, stage, pp, tp_size=tp, tp_rank=tp_rank)
        model = PipelineModel(cfg, w, ctx, comm=comm, num_micro=2, layer_range=ranges[stage], kv_bits=args.kv_bits)
        llm = LLM(cfg, w, ecfg, comm=comm, model=model)
    else:
        if args.layers:
            import mlxcel_b200.config as _c
            _orig = _c.preset

            def _fewer(name):
                c = _orig(name)
                c.num_hidden_layers = args.layers
                return c
            import mlxcel_b200.llm as _l
            _l.preset = _fewer
        llm = LLM.from_preset(args.model, device=dev, seed=0, engine_config=ecfg, comm=comm, quantize=preset["quantize"])
    if args.config == 5 and not args.no_mtp:
        # one-layer MTP drafter of the same layer shape: K = 4 (3 drafts + the bonus token per round)
        from mlxcel_b200.speculative import MTPDrafter, random_mtp_weights
        eng0 = llm.engine
        on_last = ctx is None or ctx.is_last
        if on_last:
            mw = random_mtp_weights(llm.cfg, dtype=torch.bfloat16, device=dev,
                                    tp_rank=comm.tp_rank if comm is not None else 0, tp_size=tp)
            eng0.drafter = MTPDrafter(eng0.model, llm.cfg, mw, num_blocks=ecfg.num_blocks, block_size=16)
        else:
            from mlxcel_b200.parallel.pp import RemoteDrafter
            eng0.drafter = RemoteDrafter()
        eng0.spec_k = 4
        drafter_note = "1-layer MTP head, K=4, random-init (acceptance is that of an untrained head)"
    eng = llm.engine
    sp = SamplingParams(max_tokens=args.output_len, temperature=0.0, ignore_eos=True)

    # Synthetic prompts live in pinned host memory; every engine step copies that step's token
    # ids / positions / slots / page tables host→device and reads the sampled tokens back.
    g = torch.Generator().manual_seed(1234 + (rank if dp > 1 else 0))
    vocab = llm.cfg.vocab_size

    def make_prompts(n_req: int) -> list[list[int]]:
        if dp > 1:              # this rank's share of the batch
            n_req = n_req // dp + (1 if rank < n_req % dp else 0)
        return torch.randint(0, vocab, (n_req, args.prompt_len), generator=g).tolist()

    def barrier():
        if world > 1:
            import torch.distributed as dist
            dist.barrier()
        torch.cuda.synchronize()

    verbose = os.environ.get("MLXCEL_B200_BENCH_VERBOSE") == "1"
    n_round = [0]

    def run_round(prompts):
        faulthandler.dump_traceback_later(args.watchdog, exit=True)
        outs = llm.generate(prompt_token_ids=prompts, sampling_params=sp)
        n_round[0] += 1
        if verbose:
            print(f"[bench rank {rank}] round {n_round[0]} done, status {_lib.read_status(dev)}",
                  file=sys.stderr, flush=True)
        return outs

    def launches_now() -> int:
        if args.impl == "torch":
            from benchmarks import torch_executor
            return torch_executor.CALLS
        return _lib.launches() + eng.stats.get("graph_kernel_launches", 0)

    def measure(n_req: int, warmup: int, steps: int, sample_clocks: bool) -> dict:
        """``warmup`` untimed rounds, then exactly ``steps`` rounds timed on the device (CUDA events,
        barrier + synchronize on both sides, max over ranks), then the same number of rounds timed end
        to end on the wall clock through ``LLM.generate``."""
        for _ in range(warmup):
            run_round(make_prompts(n_req))
        barrier()
        rounds = [make_prompts(n_req) for _ in range(steps)]
        sampler = ClockSampler(local_rank) if sample_clocks else None
        if sampler is not None and rank == 0:
            sampler.start()
        l0, h2d0, d2h0 = launches_now(), eng.stats.get("h2d_bytes", 0), eng.stats.get("d2h_bytes", 0)
        sp0 = {k: eng.stats.get(k, 0) for k in ("spec_rounds", "spec_drafted", "spec_accepted")}
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        ev0.record()
        ttft, tpot, n_out = [], [], 0
        for pr in rounds:
            for s in run_round(pr):
                n_out += len(s.output)
                ttft.append((s.first_token_time - s.arrival) * 1e3)
                if len(s.output) > 1:
                    tpot.append((s.finish_time - s.first_token_time) * 1e3 / (len(s.output) - 1))
        ev1.record()
        barrier()
        dev_ms = ev0.elapsed_time(ev1)
        clocks = sampler.stop() if (sampler is not None and rank == 0) else None
        launches = launches_now() - l0
        h2d = (eng.stats.get("h2d_bytes", 0) - h2d0) / max(1, steps)
        d2h = (eng.stats.get("d2h_bytes", 0) - d2h0) / max(1, steps)
        spec = {k: eng.stats.get(k, 0) - v for k, v in sp0.items()}
        rounds2 = [make_prompts(n_req) for _ in range(steps)]
        barrier()
        t0 = time.perf_counter()
        n_out2 = 0
        for pr in rounds2:
            n_out2 += sum(len(s.output) for s in run_round(pr))
        barrier()
        wall_s = time.perf_counter() - t0
        if world > 1:
            import torch.distributed as dist
            t = torch.tensor([dev_ms, wall_s], device=dev, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            dev_ms, wall_s = float(t[0]), float(t[1])
            if dp > 1:          # every rank produced its own tokens: the job's output is their sum
                c = torch.tensor([n_out, n_out2, launches, h2d, d2h], device=dev, dtype=torch.float64)
                dist.all_reduce(c)
                n_out, n_out2, launches, h2d, d2h = (float(v) for v in c)
                gathered = [None] * world
                dist.all_gather_object(gathered, (ttft, tpot))
                ttft = [v for a, _ in gathered for v in a]
                tpot = [v for _, b in gathered for v in b]
        return dict(value=n_out / (dev_ms / 1e3), ms_per_step=dev_ms / steps, e2e=n_out2 / wall_s, h2d=h2d, d2h=d2h,
                    launches=launches, clocks=clocks, spec=spec,
                    ttft=statistics.median(ttft) if ttft else None, tpot=statistics.median(tpot) if tpot else None)

    m = measure(args.requests, args.warmup, args.steps, True)
    extra = {}
    if args.config == 3:
        # the same engine at batch 1 (the GEMV -> all-reduce regime)
        b1 = measure(1, 3, args.steps, False)
        extra["batch1"] = {"value": round(b1["value"], 2), "unit": "tok/s", "ms_per_step": round(b1["ms_per_step"], 3),
                           "p50_tpot_ms": round(b1["tpot"], 3) if b1["tpot"] else None,
                           "e2e": round(b1["e2e"], 2), "gpu_launches": int(b1["launches"]),
                           "vs_baseline": round(b1["value"] / 49.75, 2),
                           "baseline": "reference llama-3.1-8b-4bit decode, batch 1, GB10 (docs/benchmark_results/model_tests_gb10.md:47)"}
    if args.config == 5:
        sd = m["spec"]
        extra["speculative"] = {"kind": drafter_note, "rounds": sd["spec_rounds"], "drafted": sd["spec_drafted"],
                                "accepted": sd["spec_accepted"],
                                "acceptance": round(sd["spec_accepted"] / sd["spec_drafted"], 4) if sd["spec_drafted"] else None}
    if os.environ.get("MLXCEL_B200_STEP_TIMING", "0") == "1":
        # whole-run sums of the engine's per-step event timings (warm-up rounds included): the gap between
        # wall and device time is host work, which the lookahead pipeline hides where it is on
        extra["step_timing"] = {k: round(v, 1) if isinstance(v, float) else v for k, v in eng.stats.items()
                                if k.endswith(("_gpu_ms", "_wall_ms", "_timed_steps", "tick_sync_ms", "null_forwards"))}
    status = _lib.read_status(dev)
    if rank == 0:
        value = m["value"]
        if args.config == 5:
            par = f"tp{tp}xpp{pp}"
        elif args.config == 4 and dp > 1:
            par = f"dp{dp} attention + ep{dp} experts (all-to-all dispatch / combine)"
        elif args.config == 4:
            par = f"ep{args.gpus} (attention tp{args.gpus})"
        else:
            par = f"tp{args.gpus}"
        out = {
            "metric": f"output tok/s (continuous batching, {args.requests} concurrent requests, prefill included)",
            "value": round(value, 2), "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(m["ms_per_step"], 3),
            "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(value / BASELINE_TOK_S, 2) if args.config == 2 else None, "dtype": "bf16",
            "data": "synthetic token-id prompts (uniform over vocab), random-init N(0,0.02) weights",
            "config": {"benchmark_config": args.config, "model": f"{args.model} architecture",
                       "global_batch": args.requests, "seq_len": args.prompt_len, "output_len": args.output_len,
                       "parallelism": par, "kv_block": 16, "kv_bits": args.kv_bits,
                       "weights": ("MLX affine 4-bit, group 64 (bf16 scales and biases), LM head included" if args.config == 3
                                   else "mxfp4 experts (e2m1 + e8m0 per 32), bf16 attention and embeddings" if args.config == 4
                                   else "bf16"),
                       "prefill_chunk": chunk or args.prompt_len,
                       "l2": "working set (weights + KV pool, > 16 GB) exceeds the 126 MB L2; no flush needed",
                       "step": "one serving round of global_batch requests",
                       "cuda_graphs": eng.ecfg.cuda_graphs,
                       "tp_backend": (comm.backend + ("+nvls" if getattr(getattr(comm, "fused", None), "nvls", False) else ""))
                       if comm is not None else "none"},
            "p50_ttft_ms": round(m["ttft"], 2) if m["ttft"] else None,
            "p50_tpot_ms": round(m["tpot"], 3) if m["tpot"] else None,
            "clocks": m["clocks"],
            "e2e": {"value": round(m["e2e"], 2), "unit": "tok/s",
                    "h2d_bytes_per_step": int(m["h2d"]), "d2h_bytes_per_step": int(m["d2h"])},
            "gpu_launches": int(m["launches"]),
            "kernel_status": status,
            "impl": args.impl,
        }
        out.update(extra)
        if args.layers:
            out["invalid"] = f"debug run with {args.layers} layers"
        if args.impl == "torch":
            out["note"] = ("plain PyTorch executor (cuBLAS linear, SDPA over K/V gathered from the paged pool, NCCL "
                           "collectives) under the same engine; gpu_launches counts library calls issued")
        if status != 0:
            out["error"] = f"a kernel recorded failure code {status} (bounded wait ran out): the numbers are not valid"
        print(json.dumps(out))
    code = 0 if status == 0 else 4
    if world > 1:
        # Tearing the NCCL communicator down while the symmetric-memory mappings are alive was
        # seen to block for minutes; every rank is past its last collective here, so leave directly.
        barrier()
        sys.stdout.flush()
        sys.stderr.flush()
        os._exit(code)
    if code:
        sys.exit(code)


if __name__ == "__main__":
    main()
