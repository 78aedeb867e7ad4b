"""Symmetric heap over NVLink peer memory and the fused compute+collective ops built on it.

One allocation per rank from ``torch.distributed._symmetric_memory`` (CUDA VMM memory whose
handles are exchanged at rendezvous) gives every rank the device addresses of every peer's
buffer. Regions are carved at identical offsets on all ranks, so "the same tensor on rank r" is
``peer_base[r] + offset``. Kernels use plain peer loads/stores and ``red.release.sys`` /
``ld.acquire.sys`` flags on these addresses — never TMA from a peer's memory. Where the
allocation also has an NVSwitch multicast mapping (NVLS), ``mc_base + offset`` names the same
region on ALL ranks at once and the kernels use ``multimem.ld_reduce`` / ``multimem.st`` /
``multimem.red`` on it (``MLXCEL_B200_NVLS=0`` keeps the peer-store protocol).

Channel layout (per fused op kind): 4 control words + 8193 consumed-arrival words (local use) +
8193 arrival flags (written by peers) + an optional double-buffered receive area.
"""
from __future__ import annotations

import ctypes
import math
import os

import torch
import torch.distributed as dist

from ..ops import _lib

_ELEM = {torch.bfloat16: 2, torch.float16: 2, torch.float32: 4, torch.int32: 4, torch.uint8: 1}
_MAX_TILES = 8192
_CTL_WORDS = 16
_CHANNEL_WORDS = _CTL_WORDS + 2 * (_MAX_TILES + 8)


def _align(n: int, a: int = 256) -> int:
    return (n + a - 1) // a * a


class SymmetricHeap:
    def __init__(self, group, device: torch.device, nbytes: int = 0):
        import torch.distributed._symmetric_memory as symm_mem

        self.group, self.device = group, device
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.nbytes = _align(nbytes or (768 << 20), 2 << 20)
        self.buf = symm_mem.empty(self.nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group.group_name if hasattr(group, "group_name") else group)
        self.peer_base = [int(p) for p in self.handle.buffer_ptrs]
        assert self.peer_base[self.rank] == self.buf.data_ptr()
        # NVLS: multicast address of the same buffer (0 when the fabric / driver has no multicast
        # support or the mapping was not created)
        self.mc_base = 0
        if os.environ.get("MLXCEL_B200_NVLS", "1") != "0":
            try:
                mc = int(getattr(self.handle, "multicast_ptr", 0) or 0)
            except Exception:
                mc = 0
            self.mc_base = mc
        # every rank must take the same protocol: all ranks need the mapping
        flag = torch.tensor([1 if self.mc_base else 0], dtype=torch.int32, device=device)
        dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
        if int(flag.item()) == 0:
            self.mc_base = 0
        self.offset = 0
        torch.cuda.synchronize(device)
        dist.barrier(group=group)

    def alloc(self, nbytes: int) -> int:
        """Reserve ``nbytes`` at the same offset on every rank; returns the offset."""
        off = self.offset
        nbytes = _align(nbytes)
        if off + nbytes > self.nbytes:
            raise MemoryError(f"symmetric heap exhausted ({off + nbytes} > {self.nbytes})")
        self.offset = off + nbytes
        return off

    def view(self, offset: int, shape, dtype) -> torch.Tensor:
        n = math.prod(shape) * _ELEM[dtype]
        return self.buf[offset:offset + n].view(dtype).view(*shape)

    def mc_ptr(self, offset: int) -> int:
        """Multicast address of a region (0 without NVLS)."""
        return self.mc_base + offset if self.mc_base else 0

    def peer_ptrs(self, offset: int):
        """ctypes array of this region's address on every rank."""
        arr = (ctypes.c_void_p * self.world)()
        for r in range(self.world):
            arr[r] = self.peer_base[r] + offset
        return arr


class _Channel:
    def __init__(self, heap: SymmetricHeap, recv_bytes: int):
        self.heap = heap
        self.ctl_off = heap.alloc(_CHANNEL_WORDS * 4)
        words = heap.view(self.ctl_off, (_CHANNEL_WORDS,), torch.int32)
        self.ctl = words[:_CTL_WORDS]
        self.expect = words[_CTL_WORDS:_CTL_WORDS + _MAX_TILES + 8]
        self.flags_off = self.ctl_off + 4 * (_CTL_WORDS + _MAX_TILES + 8)
        self.flags_peer = heap.peer_ptrs(self.flags_off)
        self.flags_mc = heap.mc_ptr(self.flags_off)
        self.recv_bytes = recv_bytes
        if recv_bytes:
            self.recv_off = heap.alloc(2 * recv_bytes)
            self.recv_peer = heap.peer_ptrs(self.recv_off)
            self.recv_mc = heap.mc_ptr(self.recv_off)
        else:
            self.recv_off, self.recv_peer, self.recv_mc = 0, None, 0

    def reset(self) -> None:
        self.heap.view(self.ctl_off, (_CHANNEL_WORDS,), torch.int32).zero_()


class FusedOps:
    """GEMM → all-reduce (+bias +residual) and GEMM → all-gather as single kernels."""

    @staticmethod
    def required_bytes(world: int, max_tokens: int = 8192, hidden: int = 8192, vocab: int = 262144,
                       small_m: int = 256) -> int:
        """Heap bytes the channels and buffers below take (what ``SymmetricHeap`` must be sized for)."""
        ctl = _align(_CHANNEL_WORDS * 4)
        one = _align(2 * world * small_m * hidden * 2)
        qmv = _align(2 * world * 8 * hidden * 2)
        tiles = ((max_tokens + 127) // 128) * ((hidden + 255) // 256)
        two = _align(2 * world * ((tiles + world - 1) // world) * 128 * 256 * 2)
        chunks = (max_tokens * hidden + 8191) // 8192
        ar_two = _align(2 * world * ((chunks + world - 1) // world) * 8192 * 2)
        return (6 * ctl + 2 * one + two + ar_two + qmv + _align(max_tokens * hidden * 2) + _align(small_m * vocab * 2)
                + (4 << 20))

    def __init__(self, heap: SymmetricHeap, max_tokens: int = 8192, hidden: int = 8192,
                 vocab: int = 262144, small_m: int = 256):
        self.heap = heap
        W = heap.world
        self.world, self.rank = W, heap.rank
        self.small_m, self.max_tokens, self.hidden = small_m, max_tokens, hidden
        # one-shot: [2][world][small_m * hidden] bf16
        self.one_stride = small_m * hidden
        self.ch_one = _Channel(heap, W * self.one_stride * 2)
        # two-shot: [2][world][ceil(tiles / world) * 128 * 256] bf16 with tiles over max_tokens x hidden
        tiles = ((max_tokens + 127) // 128) * ((hidden + 255) // 256)
        self.two_stride = ((tiles + W - 1) // W) * 128 * 256
        self.ch_two = _Channel(heap, W * self.two_stride * 2)
        self.ch_ag = _Channel(heap, 0)
        # stand-alone all-reduce channels (MoE combine, quantized GEMV partials)
        self.ar_one_stride = small_m * hidden
        self.ch_ar_one = _Channel(heap, W * self.ar_one_stride * 2)
        chunks = (max_tokens * hidden + 8191) // 8192
        self.ar_two_stride = ((chunks + W - 1) // W) * 8192
        self.ch_ar_two = _Channel(heap, W * self.ar_two_stride * 2)
        # quantized GEMV -> all-reduce (up to 8 token rows)
        self.qmv_stride = 8 * hidden
        self.ch_qmv = _Channel(heap, W * self.qmv_stride * 2)
        # replicated residual stream and gathered logits live in the heap
        self.h_off = heap.alloc(max_tokens * hidden * 2)
        self.h_peer = heap.peer_ptrs(self.h_off)
        self.h_mc = heap.mc_ptr(self.h_off)
        self.vocab_cap = vocab
        self.logits_off = heap.alloc(small_m * vocab * 2)
        self.logits_peer = heap.peer_ptrs(self.logits_off)
        self.logits_mc = heap.mc_ptr(self.logits_off)
        self.nvls = bool(heap.mc_base)
        # Transport per algorithm. Two-shot (prefill-sized) reductions and the all-gather go through the
        # switch: each byte leaves a GPU once (measured at 8 ranks, M = 8192: 290 us against 998 us with
        # peer stores and 471 us for GEMM + NCCL). One-shot (decode-sized) reductions stay on peer
        # stores: there every rank needs the whole sum, so in-switch reduction makes each GPU serve
        # its partial to all requesters and moves more bytes than pushing it once per peer (measured at
        # 8 ranks, M = 64: 42 us against 26 us; at 2 ranks 24 against 20).
        # MLXCEL_B200_NVLS_ONESHOT=1 forces the switch for one-shot reductions too.
        import os
        self.nvls_two = self.nvls
        self.nvls_one = self.nvls and os.environ.get("MLXCEL_B200_NVLS_ONESHOT", "0") == "1"
        torch.cuda.synchronize(heap.device)
        dist.barrier(group=heap.group)

    def reset(self) -> None:
        """Zero every channel on all ranks (after a bounded wait reported a failure)."""
        torch.cuda.synchronize(self.heap.device)
        dist.barrier(group=self.heap.group)
        for ch in (self.ch_one, self.ch_two, self.ch_ag, self.ch_ar_one, self.ch_ar_two, self.ch_qmv):
            ch.reset()
        torch.cuda.synchronize(self.heap.device)
        dist.barrier(group=self.heap.group)

    def hidden_buffer(self, tokens: int, hidden: int) -> torch.Tensor:
        return self.heap.view(self.h_off, (tokens, hidden), torch.bfloat16)

    def gemm_allreduce(self, x: torch.Tensor, w: torch.Tensor, bias, residual, ssq_out=None) -> torch.Tensor:
        """``residual + bias + sum_ranks(x_r @ w_r^T)``; the result is bitwise identical on all
        ranks and lives in the symmetric residual buffer."""
        from ..models.weights import QuantizedTensor

        M, K = x.shape
        qt = w if isinstance(w, QuantizedTensor) else None
        N = w.shape[-2] if qt is not None else w.shape[0]
        lib = _lib.load()
        ws = _lib.workspace(x.device)
        out = self.hidden_buffer(M, N)
        if M <= self.small_m:
            ch, mode, stride = self.ch_one, 1, self.one_stride
        else:
            ch, mode, stride = self.ch_two, 2, self.two_stride
        if M > self.max_tokens or N > self.hidden:
            raise ValueError("gemm_allreduce shape exceeds the symmetric buffers")
        res = residual  # read locally by the reducing rank; may alias `out` (in-place update)
        if ssq_out is not None:
            assert mode == 1, "per-tile sums of squares come out of the one-shot epilogue only"
        use_mc = self.nvls_one if mode == 1 else self.nvls_two
        mc = dict(flags_mc=ch.flags_mc, recv_mc=ch.recv_mc, out_mc=self.h_mc) if use_mc else {}
        if qt is not None:
            # packed weights: dequantised by the kernel's transform warps (one-shot all-reduce only),
            # i.e. quantized GEMV/GEMM -> all-reduce in one kernel
            from ..ops import quant
            wq = quant.fused_wq(qt, M, K)
            assert wq and mode == 1, "fused quantized row-parallel GEMM: covered formats, M <= 256"
            w_ptr, ex = quant.quant_extras(qt, wq, ssq_out=ssq_out, **mc)
            ldw = 0
        else:
            w_ptr, ldw = w.data_ptr(), w.stride(0)
            ex = _lib.gemm_extras(ssq_out=ssq_out, **mc)
        rc = lib.mx_gemm_comm(x.data_ptr(), w_ptr, out.data_ptr(), _lib.ptr(bias), _lib.ptr(res),
                              M, N, K, x.stride(0), ldw, out.stride(0),
                              res.stride(0) if res is not None else 0, mode, self.rank, self.world,
                              ch.flags_peer, ch.recv_peer, self.h_peer, ch.ctl.data_ptr(),
                              ch.expect.data_ptr(), self.world * stride, stride, ws.data_ptr(),
                              ws.numel(), _lib.stream(), _lib.ref_or_null(ex))
        _lib.count_launch()
        _lib.check(rc, "mx_gemm_comm")
        return out

    def qmv_allreduce(self, x: torch.Tensor, qt, bias, residual) -> torch.Tensor | None:
        """Row-parallel quantized projection for up to 8 token rows: GEMV over this rank's packed
        shard and the cross-rank sum in one kernel. Returns None when the shape is not covered."""
        from ..ops.quant import _MODE_ID

        M, K = x.shape
        N = qt.shape[-2]
        if M > 8 or qt.bits not in (4, 8) or qt.packed.dim() != 2 or M * N > self.qmv_stride or x.stride(1) != 1:
            return None
        lib = _lib.load()
        ws = _lib.workspace(x.device)
        out = self.hidden_buffer(M, N)
        ch = self.ch_qmv
        mc = (ch.flags_mc or None, ch.recv_mc or None) if self.nvls_one else (None, None)
        rc = lib.mx_qmv_allreduce(x.data_ptr(), qt.packed.data_ptr(), qt.scales.data_ptr(), _lib.ptr(qt.biases),
                                  out.data_ptr(), _lib.ptr(residual), _lib.ptr(bias), M, N, K, qt.bits, qt.group_size,
                                  _MODE_ID[qt.mode], x.stride(0), out.stride(0),
                                  residual.stride(0) if residual is not None else 0, self.rank, self.world,
                                  ch.flags_peer, ch.recv_peer, ch.ctl.data_ptr(), ch.expect.data_ptr(),
                                  self.world * self.qmv_stride, self.qmv_stride, ws.data_ptr(), mc[0], mc[1],
                                  _lib.stream())
        if rc == -9:
            return None
        _lib.count_launch()
        _lib.check(rc, "mx_qmv_allreduce")
        return out

    def all_reduce(self, x: torch.Tensor, residual: torch.Tensor | None = None) -> torch.Tensor:
        """Sum of ``x`` over ranks (+ residual) with the stand-alone peer-memory kernel. Small tensors
        are reduced in place (one-shot), large ones land in the symmetric residual buffer."""
        n = x.numel()
        lib = _lib.load()
        ws = _lib.workspace(x.device)
        x = x.contiguous()
        if n <= self.ar_one_stride:
            ch, mode, stride, out = self.ch_ar_one, 1, self.ar_one_stride, x
        else:
            ch, mode, stride = self.ch_ar_two, 2, self.ar_two_stride
            if x.dim() != 2 or x.shape[0] > self.max_tokens or x.shape[1] > self.hidden:
                raise ValueError("all_reduce shape exceeds the symmetric buffers")
            out = self.hidden_buffer(x.shape[0], x.shape[1])
        mc = (ch.flags_mc, ch.recv_mc, self.h_mc) if (self.nvls_one if mode == 1 else self.nvls_two) else (None, None, None)
        rc = lib.mx_allreduce_comm(x.data_ptr(), _lib.ptr(residual), out.data_ptr(), n, mode, self.rank,
                                   self.world, ch.flags_peer, ch.recv_peer, self.h_peer, ch.ctl.data_ptr(),
                                   ch.expect.data_ptr(), self.world * stride, stride, ws.data_ptr(), _lib.stream(),
                                   *mc)
        _lib.count_launch()
        _lib.check(rc, "mx_allreduce_comm")
        return out

    def gemm_allgather(self, x: torch.Tensor, w: torch.Tensor, bias=None) -> torch.Tensor:
        """Vocab-parallel projection: every rank ends with ``[M, world * N]`` logits."""
        M, K = x.shape
        N = w.shape[0]
        if M > self.small_m or self.world * N > self.vocab_cap:
            raise ValueError("gemm_allgather shape exceeds the symmetric buffers")
        lib = _lib.load()
        ws = _lib.workspace(x.device)
        out = self.heap.view(self.logits_off, (M, self.world * N), torch.bfloat16)
        ch = self.ch_ag
        ex = _lib.gemm_extras(flags_mc=ch.flags_mc, out_mc=self.logits_mc) if self.nvls else None
        rc = lib.mx_gemm_comm(x.data_ptr(), w.data_ptr(), out.data_ptr(), _lib.ptr(bias), None, M, N, K,
                              x.stride(0), w.stride(0), out.stride(0), 0, 3, self.rank, self.world,
                              ch.flags_peer, None, self.logits_peer, ch.ctl.data_ptr(),
                              ch.expect.data_ptr(), 0, 0, ws.data_ptr(), ws.numel(), _lib.stream(),
                              _lib.ref_or_null(ex))
        _lib.count_launch()
        _lib.check(rc, "mx_gemm_comm")
        return out
