"""Serving control plane for multi-process (tensor / expert / pipeline parallel) engines.

One process per GPU runs the same deterministic engine. Rank 0 (the leader) owns everything that
talks to the outside: the HTTP listener, the tokenizer front end, request validation. Before every
engine step it broadcasts a compact *step descriptor* — the requests admitted since the last step
(token ids, sampling parameters, constraint specification), the cancellations, named maintenance
calls — together with a digest of its own scheduler state; the other ranks (followers) apply the
same descriptor to their own engine, block manager and stop matchers, check the digest and run the
step. Token decisions never differ between ranks (every rank samples from the same gathered
logits), so the engines stay in lockstep without shipping schedules or tokens; the digest turns a
divergence (a bug, a rank that lost a message) into an error instead of a hang.

The descriptor travels over a CPU (gloo) process group: a few hundred bytes per step, no GPU
synchronisation, and the leader's loop doubles as a heartbeat (an empty descriptor at least every
``idle_interval`` seconds), which the failure detector of ``parallel/health.py`` rides on.

Reference design: the lockstep types of src/distributed/tensor_parallel/synchronized.rs:117
(``StepDecision``), tp_scheduler.rs (rank-0 scheduler) and tp_executor.rs (executor loop); the
reference exercises them in tests only, its live TP runtime is one process.
"""
from __future__ import annotations

import dataclasses
import os
import time
from dataclasses import dataclass, field

import torch
import torch.distributed as dist


@dataclass
class StepDescriptor:
    """What the leader decided to feed the engines before one step."""

    step: int = 0
    requests: list = field(default_factory=list)     # [dict(request_id, prompt_ids, params, constraint)]
    cancels: list = field(default_factory=list)      # [request_id]
    calls: list = field(default_factory=list)        # [(name, args)] maintenance calls replicated by name
    stop: bool = False
    digest: int = 0                                   # leader's engine digest BEFORE applying this descriptor
    sent_at: float = 0.0


def params_to_wire(p) -> dict:
    return dataclasses.asdict(p)


def params_from_wire(d: dict):
    from ..engine import SamplingParams
    d = dict(d)
    if d.get("logit_bias"):
        d["logit_bias"] = {int(k): float(v) for k, v in d["logit_bias"].items()}
    return SamplingParams(**d)


def engine_digest(engine) -> int:
    """A cheap fingerprint of the scheduler-visible state: which sequences exist, how far each has
    got, how many blocks are free. Equal on all ranks that are in lockstep."""
    h = 1469598103934665603
    for s in list(engine.running) + list(engine.waiting):
        for v in (s.seq_id, len(s.prompt), len(s.output), s.num_computed, s.output[-1] if s.output else -1):
            h = ((h ^ (v & 0xFFFFFFFF)) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    h = ((h ^ (engine.stats.get("steps", 0) & 0xFFFFFFFF)) * 1099511628211) & 0xFFFFFFFFFFFFFFFF
    return h


class LockstepError(RuntimeError):
    pass


class ControlPlane:
    def __init__(self, group, rank: int | None = None, world: int | None = None, leader: int = 0,
                 idle_interval: float = 0.2, detector=None):
        """``group``: a gloo (CPU) process group over all ranks that run the engine together."""
        self.group = group
        self.rank = dist.get_rank(group) if rank is None else rank
        self.world = dist.get_world_size(group) if world is None else world
        self.leader = leader
        self.idle_interval = idle_interval
        self.detector = detector            # optional FailureDetector polled between steps
        self.step = 0
        self.stats = dict(descriptors=0, bytes=0, empty=0)

    @property
    def is_leader(self) -> bool:
        return self.rank == self.leader

    def exchange(self, desc: StepDescriptor | None) -> StepDescriptor:
        """Leader: send ``desc``. Follower: receive the leader's descriptor (``desc`` is ignored)."""
        if self.detector is not None:
            self.detector.raise_if_failed()       # before anything that waits on a peer
        box = [None]
        if self.is_leader:
            desc.step = self.step
            desc.sent_at = time.time()
            box[0] = desc
        dist.broadcast_object_list(box, src=dist.get_global_rank(self.group, self.leader), group=self.group)
        d: StepDescriptor = box[0]
        if d.step != self.step:
            raise LockstepError(f"rank {self.rank}: descriptor {d.step} arrived at local step {self.step}")
        self.step += 1
        self.stats["descriptors"] += 1
        if not (d.requests or d.cancels or d.calls or d.stop):
            self.stats["empty"] += 1
        return d

    def check_digest(self, d: StepDescriptor, engine) -> None:
        mine = engine_digest(engine)
        if d.digest and mine != d.digest:
            raise LockstepError(f"rank {self.rank} diverged from the leader before step {d.step} "
                                f"(digest {mine:#x} != {d.digest:#x})")


def agree_min(value: int, group=None) -> int:
    """The smallest ``value`` over the ranks of the default (or given) group: sizes that every rank
    derives from its own free memory (KV blocks) must agree or the schedulers diverge under pressure."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return int(value)
    backend = dist.get_backend(group)
    dev = torch.device("cuda", torch.cuda.current_device()) if "nccl" in str(backend) else torch.device("cpu")
    t = torch.tensor([int(value)], dtype=torch.int64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MIN, group=group)
    return int(t.item())


def init_distributed(device: str | None = None):
    """Join the job a ``torch.distributed.run`` launch describes (environment variables only):
    selects this rank's GPU, initialises the default process group (NCCL on GPUs, gloo on CPU) and
    returns ``(device, control_group)`` where ``control_group`` is a gloo group over all ranks for
    the step descriptors. With WORLD_SIZE unset or 1 nothing is initialised."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world <= 1:
        return device, None
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    local = int(os.environ.get("LOCAL_RANK", os.environ.get("RANK", "0")))
    use_cuda = torch.cuda.is_available() and (device is None or str(device).startswith("cuda"))
    if use_cuda:
        torch.cuda.set_device(local)
        device = f"cuda:{local}"
    else:
        device = "cpu"
    if not dist.is_initialized():
        if use_cuda:
            dist.init_process_group("nccl", device_id=torch.device(device))
        else:
            dist.init_process_group("gloo")
    if "gloo" in str(dist.get_backend()):
        ctl = dist.group.WORLD
    else:
        ctl = dist.new_group(backend="gloo")
    return device, ctl
