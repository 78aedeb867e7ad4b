"""Data-parallel attention with expert-parallel MoE layers (token-sharded ranks).

Every rank is a complete engine for its OWN requests: attention, dense projections, router, KV
pool and scheduler are local and need no communication. Only the routed experts are shared: rank r
holds experts ``[r * E / world, (r + 1) * E / world)``, and a MoE layer sends every (token, k) row
to the rank that owns its expert and brings the expert's output back (`EpAllToAll`, one fused
permutation + NVLink transfer each way). Against the replicated-token mode of the tensor-parallel
engine this removes the two all-reduces per layer and the replicated attention work, and lets the
batch grow with the number of GPUs; it needs every rank to enter every MoE layer together.

Lockstep. The all-to-all kernels wait for their peers (bounded waits), so all ranks must run the same
number of forward passes, close in time. `Engine` does that when it is given a ``dp_group``: a
scheduler tick starts with a one-integer all-reduce ("does anyone have work?"), a rank with nothing
to run this tick runs a *null forward* (its MoE layers exchange zero rows and serve the others'
tokens), and the tick is skipped everywhere when nobody has work (reference: the expert-parallel
runtime around SwitchGLU, src/distributed/, src/models/switch_layers.rs:98-220; the engine-side
lockstep is the counterpart of src/distributed/tensor_parallel/synchronized.rs for token-sharded
ranks).

On CPU (tests, gloo) `GlooAllToAll` stands in for the kernels with object collectives.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..models.decoder import LocalComm
from ..ops import moe as moe_ops


class GlooAllToAll:
    """Reference exchange for CPU ranks: same interface as `EpAllToAll.moe`."""

    def __init__(self, group, experts_per_rank: int):
        self.group, self.epr = group, experts_per_rank
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.stats = dict(layers=0, rows_sent=0, rows_served=0)

    def moe(self, x, ids, wts, w_gate_up, w_down, inter: int, act: str, b_gate_up=None, b_down=None,
            residual=None, alpha: float = 1.702, limit: float = 7.0) -> torch.Tensor:
        T, k = ids.shape
        owner = torch.div(ids, self.epr, rounding_mode="floor")
        send = []
        for r in range(self.world):
            sel = (owner == r).nonzero()                   # [n, 2] (token, slot)
            send.append((x[sel[:, 0]].float(), ids[sel[:, 0], sel[:, 1]].clone(), sel))
        box = [None] * self.world
        dist.all_gather_object(box, [(s[0], s[1]) for s in send], group=self.group)
        outs = []
        for src in range(self.world):                      # rows every source addressed to this rank
            rows, eids = box[src][self.rank]
            if rows.shape[0]:
                o = moe_ops.moe_experts(rows.to(x.dtype), eids.view(-1, 1).int(), torch.ones(rows.shape[0], 1),
                                        w_gate_up, w_down, inter, act, b_gate_up, b_down, e_begin=self.rank * self.epr,
                                        alpha=alpha, limit=limit).float()
            else:
                o = rows
            outs.append(o)
            self.stats["rows_served"] += int(rows.shape[0])
        back = [None] * self.world
        dist.all_gather_object(back, outs, group=self.group)
        out = residual.float().clone() if residual is not None else torch.zeros(T, x.shape[1])
        for r in range(self.world):
            sel = send[r][2]
            if sel.shape[0]:
                got = back[r][self.rank]                   # what rank r computed for this rank's rows
                out.index_add_(0, sel[:, 0], got * wts[sel[:, 0], sel[:, 1]].float()[:, None])
        self.stats["layers"] += 1
        self.stats["rows_sent"] += T * k
        return out.to(x.dtype)


class DpEpComm(LocalComm):
    """Communication context of one data-parallel rank: everything local except the routed experts."""

    backend = "a2a"

    def __init__(self, group, device, *, hidden: int, top_k: int, num_experts: int, max_tokens: int, host_group=None):
        self.group = group
        self.ep_size, self.ep_rank = dist.get_world_size(group), dist.get_rank(group)
        if num_experts % self.ep_size:
            raise ValueError("the expert count must be a multiple of the number of ranks")
        epr = num_experts // self.ep_size
        device = torch.device(device)
        if device.type == "cuda":
            from .ep_a2a import EpAllToAll
            from .symm import SymmetricHeap
            cap = max_tokens * top_k                       # worst case: one source sends all its rows to one rank
            need = EpAllToAll.required_bytes(self.ep_size, hidden, cap) + (1 << 20)
            self.heap = SymmetricHeap(group, device, need)
            self.a2a = EpAllToAll.from_heap(self.heap, hidden, cap, epr, max_tokens, top_k)
            # the per-tick "does anyone have work" count travels over a host (gloo) group
            self.host_group = host_group or dist.new_group(list(range(self.ep_size)), backend="gloo")
        else:
            self.a2a = GlooAllToAll(group, epr)
            self.a2a.dry = False
            self.host_group = host_group or group
        self.tick_tokens, self.heavy = 0, False

    def any_work(self, mine: bool, tokens: int = 0) -> int:
        """How many ranks have work this tick (one small host all-reduce). The same message sums the
        ranks' token counts of the tick: every rank's experts see rows of all ranks, so the expected
        rows per rank (what picks the weight-streaming or the dense expert kernels) is a global
        figure, not this rank's. ``heavy`` afterwards says whether that figure is beyond the
        weight-streaming kernel's range (a rank that decodes while another one prefills)."""
        t = torch.tensor([1 if mine else 0, int(tokens)], dtype=torch.int64)
        dist.all_reduce(t, group=self.host_group)
        self.tick_tokens = int(t[1])
        k = getattr(self.a2a, "k", 1)
        hint = max(1, -(-self.tick_tokens * k // self.ep_size))
        if hasattr(self.a2a, "rows_hint"):
            self.a2a.rows_hint = hint
        from ..ops import moe as moe_ops
        self.heavy = hint > moe_ops._QGEMV_MAX_ROWS * getattr(self.a2a, "epr", 1)
        return int(t[0])
