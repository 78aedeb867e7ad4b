"""Tensor-parallel runtime: one process per GPU, SPMD lockstep.

Every rank runs the same scheduler on the same request stream (the step descriptor is
deterministic), holds a column/row shard of every projection and 1/tp of the KV heads, and keeps
the residual stream replicated. Two interchangeable communication back ends:

* ``fused`` (default on NVLink/NVSwitch): the row-parallel projections (o_proj, down_proj) run
  ONE kernel that computes the GEMM tile on tensor cores and reduces it across ranks by peer
  stores/loads into a symmetric heap (push partial tile → per-tile arrival flags → ordered sum +
  residual), and the vocab-parallel LM head pushes its logits tile straight into every peer's
  logits buffer (GEMM → all-gather). See ``csrc/gemm.cu`` (COMM modes).
* ``nccl``: cuBLAS-free GEMM kernel + ``torch.distributed`` all-reduce / all-gather. This is the
  measured baseline the fused path is compared against.

The reference simulates TP inside one process (``reduce_sum`` = a chain of adds,
src/distributed/tensor_parallel/llama_runtime.rs:3133-3153); its shard plan (column-parallel
q/k/v/gate/up, row-parallel o/down, src/distributed/tensor_parallel/plan_generator.rs) is what the
weight sharding here follows.
"""
from __future__ import annotations

import os

import torch
import torch.distributed as dist

from .. import ops
from ..ops import _lib


# Prefill-sized M (> 256 tokens) uses the fused two-shot GEMM -> all-reduce as well. In isolation
# GEMM + NCCL all-reduce is faster at 8192 x 4096 (the two-shot kernel's peer stores are 16-byte
# pieces of 32 different rows per instruction), but inside a serving step the fused path wins
# (TP2 p50 TTFT 387 ms vs 444 ms): no separate residual pass, no extra launches. Set to 0 to compare.
_FUSED_PREFILL = os.environ.get("MLXCEL_B200_FUSED_PREFILL", "1") == "1"
# Largest token count served by the fused quantized GEMV -> all-reduce kernel (0 = always the GEMM form).
_QMV_AR_MAX_M = int(os.environ.get("MLXCEL_B200_QMV_AR_MAX_M", "8"))


class TPComm:
    def __init__(self, group, device: torch.device, backend: str = "fused", max_tokens: int = 8192,
                 hidden: int = 8192, vocab: int = 262144, ep: bool = True):
        self.group = group
        self.device = device
        self.tp_size = dist.get_world_size(group)
        self.tp_rank = dist.get_rank(group)
        self.ep_size = self.tp_size if ep else 1
        self.ep_rank = self.tp_rank if ep else 0
        self.backend = backend
        self.heap = None
        self.calls = 0
        if backend == "fused" and self.tp_size > 1:
            from .symm import SymmetricHeap, FusedOps

            try:
                self.heap = SymmetricHeap(group, device, FusedOps.required_bytes(
                    self.tp_size, max_tokens=max_tokens, hidden=hidden, vocab=vocab))
                self.fused = FusedOps(self.heap, max_tokens=max_tokens, hidden=hidden, vocab=vocab)
            except Exception as e:  # symmetric memory unavailable: say so loudly, use NCCL
                if os.environ.get("MLXCEL_B200_REQUIRE_FUSED") == "1":
                    raise
                print(f"[mlxcel_b200] fused TP backend unavailable ({type(e).__name__}: {e}); using NCCL",
                      flush=True)
                self.backend = "nccl"

    # ------------------------------------------------------------------ collectives
    def all_reduce(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp_size > 1:
            if self.backend == "fused" and x.is_cuda and x.dtype == torch.bfloat16 and x.numel() % 8 == 0:
                return self.fused.all_reduce(x)
            dist.all_reduce(x, group=self.group)
        return x

    def row_parallel_linear(self, x, w, bias, residual, ssq_out=None):
        """``residual + all_reduce(x_shard @ w_shard^T) + bias`` with replicated output.
        ``ssq_out``: leave the per-token sums of squares of the result there (deferred RMSNorm)."""
        self.calls += 1
        from ..models.decoder import _linear_any
        from ..models.weights import QuantizedTensor

        if self.tp_size == 1:
            return _linear_any(x, w, bias=bias, residual=residual, out=residual, ssq_out=ssq_out)
        fused_ok = self.backend == "fused"
        if fused_ok and isinstance(w, QuantizedTensor) and x.is_cuda and x.shape[0] <= _QMV_AR_MAX_M:
            # a handful of rows: bandwidth-bound GEMV with the all-reduce in its epilogue
            y = self.fused.qmv_allreduce(x, w, bias, residual)
            if y is not None:
                if ssq_out is not None:
                    ops.row_ssq(y, ssq_out)
                return y
        if fused_ok and isinstance(w, QuantizedTensor):
            from ..ops import quant
            fused_ok = (x.is_cuda and x.shape[0] <= self.fused.small_m and w.packed.dim() == 2
                        and quant.fused_wq(w, x.shape[0], x.shape[1]) != 0)
        if fused_ok and (x.shape[0] <= self.fused.small_m or _FUSED_PREFILL):
            one_shot = x.shape[0] <= self.fused.small_m
            y = self.fused.gemm_allreduce(x, w, bias, residual, ssq_out=ssq_out if one_shot else None)
            if ssq_out is not None and not one_shot:
                ops.row_ssq(y, ssq_out)
            return y
        first = self.tp_rank == 0
        y = _linear_any(x, w, bias=bias if first else None, residual=residual if first else None)
        y = self.all_reduce(y)
        if ssq_out is not None:
            ops.row_ssq(y, ssq_out)
        return y

    def gather_logits(self, logits_local: torch.Tensor) -> torch.Tensor:
        """[R, V/tp] per rank → [R, V] on every rank."""
        if self.tp_size == 1:
            return logits_local
        R, Vl = logits_local.shape
        out = torch.empty(self.tp_size * R, Vl, dtype=logits_local.dtype, device=logits_local.device)
        dist.all_gather_into_tensor(out, logits_local.contiguous(), group=self.group)
        return out.view(self.tp_size, R, Vl).permute(1, 0, 2).reshape(R, self.tp_size * Vl)

    def lm_head(self, x, w):
        """Vocab-parallel LM head: fused GEMM → all-gather when available."""
        if (self.tp_size > 1 and self.backend == "fused" and x.shape[0] <= self.fused.small_m
                and self.tp_size * w.shape[0] <= self.fused.vocab_cap):
            return self.fused.gemm_allgather(x, w)
        return self.gather_logits(ops.linear(x, w))      # many rows at once (scoring): GEMM + NCCL all-gather

    def embed(self, ids, table, scale, vocab_start: int = 0):
        return ops.embedding(ids, table, scale)

    def barrier(self):
        if self.tp_size > 1:
            dist.barrier(group=self.group)
