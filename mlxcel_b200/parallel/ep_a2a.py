"""Expert-parallel MoE with all-to-all dispatch / combine over peer memory (token-sharded ranks).

Every rank brings its OWN tokens; experts are sharded (expert ``e`` on rank ``e // experts_per_rank``).
``EpAllToAll.moe`` runs one layer: dispatch kernel (permutation fused with the NVLink transfer: rows
are stored straight into the owner's receive area), grouped expert GEMMs over the received rows,
combine kernel (weighted sum fused with the transfer: output rows are loaded straight from the
owner's memory). Kernels and protocol: ``csrc/ep_a2a.cu``. Reference: the expert-parallel path of
src/distributed around ``SwitchGLU`` (src/models/switch_layers.rs:98-220).

The symmetric buffer of one rank holds, at the same offsets on every rank::

    recv  [world * cap, H] bf16    rows received, source s in [s * cap, (s + 1) * cap)
    ret   [world * cap, H] bf16    expert outputs of those rows (read by the sources)
    meta  [world * cap]    int32   expert id per received row
    count [world] int32, dflag [world] uint32, cflag [world] uint32

``cap`` bounds the rows one source may send to one destination (worst case ``T_max * k``).

``EpAllToAll.emulated`` builds ``world`` instances over plain buffers of ONE device. Their stages can
then be run rank after rank in protocol order (all dispatches, all expert stages, all combines), so
that every flag is already set when a kernel looks at it: this is how the single-GPU test checks
the index arithmetic without kernels that wait on one another.
"""
from __future__ import annotations

import ctypes

import torch

from ..ops import _lib
from ..ops import moe as moe_ops

_MAX_RANKS = 8


class _EpCall(ctypes.Structure):
    _fields_ = ([(n, ctypes.c_int) for n in ("rank", "world", "T", "k", "H", "experts_per_rank", "cap")]
                + [("reserved", ctypes.c_uint)]
                + [(n, ctypes.c_ulonglong) for n in ("epoch", "status", "x", "ids", "wts", "residual", "out", "cnt", "ticket",
                                                     "route", "ids_eff", "rowmap", "nrecv", "meta", "count", "dflag", "cflag")]
                + [(n, ctypes.c_ulonglong * _MAX_RANKS) for n in ("recv_peer", "meta_peer", "count_peer",
                                                                  "dflag_peer", "cflag_peer", "ret_peer")])


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class EpAllToAll:
    @staticmethod
    def layout(world: int, hidden: int, cap: int) -> dict:
        rows = world * cap
        off, out = 0, {}
        for name, nbytes in (("recv", rows * hidden * 2), ("ret", rows * hidden * 2), ("meta", rows * 4),
                             ("count", world * 4), ("dflag", world * 4), ("cflag", world * 4)):
            out[name] = off
            off += _align(nbytes)
        out["bytes"] = off
        return out

    @staticmethod
    def required_bytes(world: int, hidden: int, cap: int) -> int:
        return EpAllToAll.layout(world, hidden, cap)["bytes"]

    def __init__(self, rank: int, world: int, peer_bases: list[int], local: torch.Tensor, hidden: int, cap: int,
                 experts_per_rank: int, max_tokens: int, k: int):
        """``local``: this rank's symmetric buffer as a uint8 tensor (at ``peer_bases[rank]``), zeroed."""
        if world > _MAX_RANKS:
            raise ValueError(f"at most {_MAX_RANKS} ranks")
        if hidden % 8:
            raise ValueError("hidden size must be a multiple of 8")
        self.rank, self.world, self.H, self.cap, self.epr = rank, world, hidden, cap, experts_per_rank
        self.max_tokens, self.k = max_tokens, k
        self.lay = EpAllToAll.layout(world, hidden, cap)
        assert local.numel() >= self.lay["bytes"] and local.data_ptr() == peer_bases[rank]
        self.local, self.bases = local, list(peer_bases)
        dev = local.device
        rows = world * cap
        self.recv = local[self.lay["recv"]:self.lay["recv"] + rows * hidden * 2].view(torch.bfloat16).view(rows, hidden)
        self.ret = local[self.lay["ret"]:self.lay["ret"] + rows * hidden * 2].view(torch.bfloat16).view(rows, hidden)
        self.cnt = torch.zeros(world + 2, dtype=torch.int32, device=dev)          # [world] counters, ticket, epoch
        self.route = torch.full((max_tokens * k,), -1, dtype=torch.int32, device=dev)
        # compact list of the receive rows in use (expert id, row index) and their number: the receive
        # area is sized for the worst case, the expert stage only ever touches the rows that arrived
        self.ids_eff = torch.full((rows, 1), -1, dtype=torch.int32, device=dev)
        self.rowmap = torch.zeros(rows, dtype=torch.int32, device=dev)
        self.nrecv = torch.zeros(1, dtype=torch.int32, device=dev)
        self._T = 0
        # dry: a forward pass that must not talk to the other ranks (the warm-up before a CUDA-graph
        # capture is a pass of this rank alone). The exchanges are skipped, the local expert kernels
        # still run (their lazy set-up is what the warm-up is for) and the layer returns its residual.
        self.dry = False
        # expected rows at this rank this step when the caller knows better than "as many as I send"
        # (token counts differ between data-parallel ranks); picks the expert kernels
        self.rows_hint: int | None = None
        self._build_call()

    # ------------------------------------------------------------------ constructors
    @staticmethod
    def from_heap(heap, hidden: int, cap: int, experts_per_rank: int, max_tokens: int, k: int) -> "EpAllToAll":
        """Carve the regions out of a :class:`~mlxcel_b200.parallel.symm.SymmetricHeap` (collective)."""
        nbytes = EpAllToAll.required_bytes(heap.world, hidden, cap)
        off = heap.alloc(nbytes)
        local = heap.buf[off:off + nbytes]
        local.zero_()
        torch.cuda.synchronize(heap.device)
        import torch.distributed as dist
        dist.barrier(group=heap.group)
        return EpAllToAll(heap.rank, heap.world, [b + off for b in heap.peer_base], local, hidden, cap,
                          experts_per_rank, max_tokens, k)

    @staticmethod
    def emulated(world: int, device, hidden: int, cap: int, experts_per_rank: int, max_tokens: int, k: int):
        nbytes = EpAllToAll.required_bytes(world, hidden, cap)
        bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=device) for _ in range(world)]
        bases = [b.data_ptr() for b in bufs]
        return [EpAllToAll(r, world, bases, bufs[r], hidden, cap, experts_per_rank, max_tokens, k)
                for r in range(world)]

    # ------------------------------------------------------------------ stages
    def _build_call(self) -> None:
        """The call record is filled once; a stage only updates the per-call fields."""
        c = _EpCall()
        c.rank, c.world, c.k, c.H = self.rank, self.world, self.k, self.H
        c.experts_per_rank, c.cap = self.epr, self.cap
        c.status = _lib.workspace(self.local.device).data_ptr()
        c.cnt, c.ticket = self.cnt.data_ptr(), self.cnt.data_ptr() + 4 * self.world
        c.epoch = self.cnt.data_ptr() + 4 * (self.world + 1)
        c.route, c.ids_eff = self.route.data_ptr(), self.ids_eff.data_ptr()
        c.rowmap, c.nrecv = self.rowmap.data_ptr(), self.nrecv.data_ptr()
        me = self.bases[self.rank]
        c.meta, c.count = me + self.lay["meta"], me + self.lay["count"]
        c.dflag, c.cflag = me + self.lay["dflag"], me + self.lay["cflag"]
        for r in range(self.world):
            b = self.bases[r]
            c.recv_peer[r], c.ret_peer[r] = b + self.lay["recv"], b + self.lay["ret"]
            c.meta_peer[r], c.count_peer[r] = b + self.lay["meta"], b + self.lay["count"]
            c.dflag_peer[r], c.cflag_peer[r] = b + self.lay["dflag"], b + self.lay["cflag"]
        fn = _lib.load().mx_ep_a2a
        fn.argtypes, fn.restype = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p], ctypes.c_int
        self._c, self._cref, self._fn = c, ctypes.byref(c), fn

    def _call(self, stage: int, x=None, ids=None, wts=None, residual=None, out=None) -> None:
        c = self._c
        c.T = self._T
        c.x = 0 if x is None else x.data_ptr()
        c.ids = 0 if ids is None else ids.data_ptr()
        c.wts = 0 if wts is None else wts.data_ptr()
        c.residual = 0 if residual is None else residual.data_ptr()
        c.out = 0 if out is None else out.data_ptr()
        rc = self._fn(self._cref, stage, _lib.stream())
        _lib.count_launch()
        if rc:
            _lib.check(rc, f"mx_ep_a2a stage {stage}")

    def dispatch(self, x: torch.Tensor, ids: torch.Tensor) -> None:
        """Send every (token, k) row of ``x`` [T, H] to the rank that owns expert ``ids[t, k]``."""
        T, k = ids.shape
        if k != self.k or T > self.max_tokens or x.shape != (T, self.H):
            raise ValueError("dispatch shape does not match the buffers")
        assert x.dtype == torch.bfloat16 and ids.dtype == torch.int32 and x.is_contiguous() and ids.is_contiguous()
        self._T = T
        self._call(0, x=x, ids=ids)

    def expert_stage(self, w_gate_up, w_down, inter: int, act: str, b_gate_up=None, b_down=None,
                     alpha: float = 1.702, limit: float = 7.0) -> None:
        """Wait for every source's rows, run this rank's experts over them, publish the outputs."""
        self._call(1)
        # rows in use are known on the device only; with balanced routing a rank receives about as many
        # rows as it sends, which is what picks the decode (weight-streaming) or prefill expert kernels
        moe_ops.moe_experts_rows(self.recv, self.ids_eff, self.rowmap, self.nrecv, w_gate_up, w_down, inter, act,
                                 b_gate_up, b_down, e_begin=self.rank * self.epr, alpha=alpha, limit=limit,
                                 out=self.ret, rows_hint=max(1, self.rows_hint or self._T * self.k))
        self._call(2)

    def combine(self, wts: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """out[t] = residual[t] + sum_k wts[t, k] * expert output of row (t, k), read from the owners."""
        T = self._T
        assert wts.shape == (T, self.k) and wts.dtype == torch.float32 and wts.is_contiguous()
        out = torch.empty(T, self.H, dtype=torch.bfloat16, device=self.local.device)
        self._call(3, wts=wts, residual=residual, out=out)
        return out

    def moe(self, x, ids, wts, w_gate_up, w_down, inter: int, act: str, b_gate_up=None, b_down=None,
            residual=None, alpha: float = 1.702, limit: float = 7.0) -> torch.Tensor:
        """One expert-parallel MoE layer (collective over the ranks of the heap)."""
        if self.dry:
            self.nrecv.zero_()
            moe_ops.moe_experts_rows(self.recv, self.ids_eff, self.rowmap, self.nrecv, w_gate_up, w_down, inter, act,
                                     b_gate_up, b_down, e_begin=self.rank * self.epr, alpha=alpha, limit=limit,
                                     out=self.ret, rows_hint=max(1, x.shape[0] * self.k))
            return residual.clone() if residual is not None else torch.zeros_like(x)
        self.dispatch(x, ids)
        self.expert_stage(w_gate_up, w_down, inter, act, b_gate_up, b_down, alpha, limit)
        return self.combine(wts, residual)
