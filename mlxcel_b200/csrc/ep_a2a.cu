// Expert-parallel MoE dispatch / combine over peer memory (NVLink), for token-sharded ranks.
//
// Every rank holds its own tokens and a shard of the experts (expert e lives on rank
// e / experts_per_rank). One MoE layer is, per rank:
//
//   ep_dispatch   permutation + transfer in one pass: every (token, k) row is written straight into
//                 the owner rank's receive area with 16-byte peer stores. Source s owns the region
//                 [s * cap, (s + 1) * cap) of every destination, so slot numbers come from a local
//                 counter and nothing is negotiated between ranks. The last CTA publishes the row
//                 counts and raises this rank's flag on every destination (release, system scope).
//   ep_recv       destination side: waits (bounded) for all sources' flags of this epoch and turns the
//                 per-source counts into the expert id of every receive row (-1 for unused rows), which
//                 is what the grouped expert GEMM's alignment kernel consumes.
//   (grouped gate/up + down GEMMs over the received rows, see moe.cu / gemm.cu)
//   ep_ready      raises this rank's "outputs ready" flag on every source.
//   ep_combine    weighted sum + transfer in one pass: waits for the owners' flags, then reads each
//                 (token, k) output row straight out of the owner's memory with 16-byte peer loads and
//                 accumulates w_k * row (+ residual) in registers.
//
// Buffers are reused from layer to layer without double buffering: a rank dispatches epoch n + 1
// only after its combine of epoch n, which needed every owner's ready flag of epoch n, which an
// owner raises after its GEMMs have consumed the receive area; and an owner starts the GEMMs of
// epoch n + 1 only after every source's dispatch flag of n + 1, raised after that source's combine
// of n has read the owner's outputs. Flags carry the epoch number (monotonic, same on all ranks).
// Every wait is bounded and reports through the status word; no TMA touches peer memory.
//
// Reference behaviour: the expert-parallel MoE of src/distributed (all-to-all dispatch / combine
// around SwitchGLU, src/models/switch_layers.rs:98-220).
#include "api.h"
#include "common.cuh"

namespace mx {

constexpr int kEpMaxRanks = 8;
constexpr int kEpThreads = 256;
constexpr int kErrEpOverflow = 203;

struct EpParams {
  int rank, world, T, k, H, experts_per_rank, cap;
  uint32_t epoch;
  int* status;
  // local tensors
  const __nv_bfloat16* x;        // [T, H]
  const int* ids;                // [T, k] global expert ids
  const float* wts;              // [T, k]
  const __nv_bfloat16* residual; // [T, H] or null
  __nv_bfloat16* out;            // [T, H]
  int* cnt;                      // [world] rows sent to each destination (zero between calls)
  uint32_t* ticket;              // CTA completion counter (zero between calls)
  int* route;                    // [T * k]: dst * cap + slot
  int* ids_eff;                  // [world * cap] expert id of every receive row, -1 = unused
  // own symmetric regions
  const int* meta;               // [world * cap] expert ids as written by the sources
  const int* count;              // [world] rows written by each source
  const uint32_t* dflag;         // [world] dispatch flags, one per source
  const uint32_t* cflag;         // [world] ready flags, one per owner
  // the same regions on every rank
  __nv_bfloat16* recv_peer[kEpMaxRanks];
  int* meta_peer[kEpMaxRanks];
  int* count_peer[kEpMaxRanks];
  uint32_t* dflag_peer[kEpMaxRanks];
  uint32_t* cflag_peer[kEpMaxRanks];
  const __nv_bfloat16* ret_peer[kEpMaxRanks];
};

__device__ __forceinline__ void ep_flag_store(uint32_t* addr, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}

__device__ __forceinline__ bool ep_flag_wait(const uint32_t* addr, uint32_t target, int* status) {
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      uint32_t v;
      asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
      if (static_cast<int32_t>(v - target) >= 0) return true;
    }
    if (*reinterpret_cast<volatile int*>(status) != 0) return false;
    if (globaltimer_ns() - t0 > kWaitLimitNs) {
      atomicCAS(status, 0, kErrPeerFlagWait);
      return false;
    }
  }
}

// One warp per (token, k) row, grid-strided.
__global__ void __launch_bounds__(kEpThreads) ep_dispatch_kernel(const EpParams p) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * kEpThreads) >> 5;
  const int vec = p.H >> 3;                       // 16-byte words per row
  for (int e = (blockIdx.x * kEpThreads + threadIdx.x) >> 5; e < p.T * p.k; e += warps) {
    int dst = 0, slot = 0, expert = 0;
    if (lane == 0) {
      expert = p.ids[e];
      dst = expert / p.experts_per_rank;
      if (expert < 0 || dst >= p.world) {
        dst = -1;
        atomicCAS(p.status, 0, kErrBadArgument);
      } else {
        slot = atomicAdd(&p.cnt[dst], 1);
        if (slot >= p.cap) {
          dst = -1;
          atomicCAS(p.status, 0, kErrEpOverflow);
        }
      }
      p.route[e] = dst < 0 ? -1 : dst * p.cap + slot;
    }
    dst = __shfl_sync(0xffffffffu, dst, 0);
    slot = __shfl_sync(0xffffffffu, slot, 0);
    if (dst < 0) continue;
    const size_t row = static_cast<size_t>(p.rank) * p.cap + slot;
    const uint4* src = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>(e / p.k) * p.H);
    uint4* dstp = reinterpret_cast<uint4*>(p.recv_peer[dst] + row * p.H);
    for (int i = lane; i < vec; i += 32) dstp[i] = src[i];
    if (lane == 0) p.meta_peer[dst][row] = expert;
  }
  // last CTA: publish the counts and raise the flags (every CTA's rows are fenced before its ticket)
  __shared__ bool last;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    last = atomicAdd(p.ticket, 1u) == gridDim.x - 1;
  }
  __syncthreads();
  if (!last) return;
  if (threadIdx.x < p.world) {
    const int d = threadIdx.x;
    __threadfence_system();
    const int n = min(atomicAdd(&p.cnt[d], 0), p.cap);
    p.count_peer[d][p.rank] = n;
    p.cnt[d] = 0;
    __threadfence_system();
    ep_flag_store(&p.dflag_peer[d][p.rank], p.epoch);
  }
  if (threadIdx.x == 0) *p.ticket = 0u;
}

// ids_eff[i] = expert of receive row i, or -1 beyond the rows its source wrote this epoch.
__global__ void __launch_bounds__(kEpThreads) ep_recv_kernel(const EpParams p) {
  __shared__ int cnt[kEpMaxRanks];
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    if (!ep_flag_wait(&p.dflag[threadIdx.x], p.epoch, p.status)) ok = 0;
    cnt[threadIdx.x] = *reinterpret_cast<const volatile int*>(&p.count[threadIdx.x]);
  }
  __syncthreads();
  const int total = p.world * p.cap;
  for (int i = blockIdx.x * kEpThreads + threadIdx.x; i < total; i += gridDim.x * kEpThreads) {
    const int s = i / p.cap, slot = i - s * p.cap;
    p.ids_eff[i] = (ok && slot < cnt[s]) ? *reinterpret_cast<const volatile int*>(&p.meta[i]) : -1;
  }
}

__global__ void ep_ready_kernel(const EpParams p) {
  if (threadIdx.x < p.world) {
    __threadfence_system();
    ep_flag_store(&p.cflag_peer[threadIdx.x][p.rank], p.epoch);
  }
}

// One warp per token: out[t] = residual[t] + sum_k w[t, k] * (owner's output row), 8 columns per lane
// and pass.
__global__ void __launch_bounds__(kEpThreads) ep_combine_kernel(const EpParams p) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    if (!ep_flag_wait(&p.cflag[threadIdx.x], p.epoch, p.status)) ok = 0;
  }
  __syncthreads();
  if (!ok) return;
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * kEpThreads) >> 5;
  const int vec = p.H >> 3;
  for (int t = (blockIdx.x * kEpThreads + threadIdx.x) >> 5; t < p.T; t += warps) {
    for (int v0 = lane; v0 < vec; v0 += 32) {
      float acc[8];
      if (p.residual) {
        const uint4 r = reinterpret_cast<const uint4*>(p.residual + static_cast<size_t>(t) * p.H)[v0];
        const __nv_bfloat162* r2 = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __bfloat1622float2(r2[q]);
          acc[2 * q] = f.x, acc[2 * q + 1] = f.y;
        }
      } else {
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[q] = 0.f;
      }
      for (int kk = 0; kk < p.k; ++kk) {
        const int rt = p.route[t * p.k + kk];
        if (rt < 0) continue;
        const int d = rt / p.cap, slot = rt - d * p.cap;
        const float w = p.wts[t * p.k + kk];
        const uint4 y = reinterpret_cast<const uint4*>(p.ret_peer[d] +
                                                       (static_cast<size_t>(p.rank) * p.cap + slot) * p.H)[v0];
        const __nv_bfloat162* y2 = reinterpret_cast<const __nv_bfloat162*>(&y);
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 f = __bfloat1622float2(y2[q]);
          acc[2 * q] += w * f.x, acc[2 * q + 1] += w * f.y;
        }
      }
      uint4 o;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int q = 0; q < 4; ++q) o2[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
      reinterpret_cast<uint4*>(p.out + static_cast<size_t>(t) * p.H)[v0] = o;
    }
  }
}

}  // namespace mx

using namespace mx;

// Plain-C description of one call (pointers as 64-bit integers so that ctypes can fill it).
struct MxEpCall {
  int rank, world, T, k, H, experts_per_rank, cap;
  unsigned int epoch;
  unsigned long long status, x, ids, wts, residual, out, cnt, ticket, route, ids_eff;
  unsigned long long meta, count, dflag, cflag;
  unsigned long long recv_peer[kEpMaxRanks], meta_peer[kEpMaxRanks], count_peer[kEpMaxRanks],
      dflag_peer[kEpMaxRanks], cflag_peer[kEpMaxRanks], ret_peer[kEpMaxRanks];
};

static int ep_fill(const MxEpCall* c, EpParams& p) {
  if (c == nullptr || c->world < 1 || c->world > kEpMaxRanks || c->rank < 0 || c->rank >= c->world) return -1;
  if (c->H <= 0 || c->H % 8 || c->k < 1 || c->cap < 1 || c->experts_per_rank < 1 || c->T < 0) return -1;
  if (static_cast<long long>(c->world) * c->cap > 0x7fffffffLL) return -1;
  p.rank = c->rank, p.world = c->world, p.T = c->T, p.k = c->k, p.H = c->H;
  p.experts_per_rank = c->experts_per_rank, p.cap = c->cap, p.epoch = c->epoch;
  auto ptr = [](unsigned long long v) { return reinterpret_cast<void*>(static_cast<uintptr_t>(v)); };
  p.status = static_cast<int*>(ptr(c->status));
  p.x = static_cast<const __nv_bfloat16*>(ptr(c->x));
  p.ids = static_cast<const int*>(ptr(c->ids));
  p.wts = static_cast<const float*>(ptr(c->wts));
  p.residual = static_cast<const __nv_bfloat16*>(ptr(c->residual));
  p.out = static_cast<__nv_bfloat16*>(ptr(c->out));
  p.cnt = static_cast<int*>(ptr(c->cnt));
  p.ticket = static_cast<uint32_t*>(ptr(c->ticket));
  p.route = static_cast<int*>(ptr(c->route));
  p.ids_eff = static_cast<int*>(ptr(c->ids_eff));
  p.meta = static_cast<const int*>(ptr(c->meta));
  p.count = static_cast<const int*>(ptr(c->count));
  p.dflag = static_cast<const uint32_t*>(ptr(c->dflag));
  p.cflag = static_cast<const uint32_t*>(ptr(c->cflag));
  for (int r = 0; r < c->world; ++r) {
    p.recv_peer[r] = static_cast<__nv_bfloat16*>(ptr(c->recv_peer[r]));
    p.meta_peer[r] = static_cast<int*>(ptr(c->meta_peer[r]));
    p.count_peer[r] = static_cast<int*>(ptr(c->count_peer[r]));
    p.dflag_peer[r] = static_cast<uint32_t*>(ptr(c->dflag_peer[r]));
    p.cflag_peer[r] = static_cast<uint32_t*>(ptr(c->cflag_peer[r]));
    p.ret_peer[r] = static_cast<const __nv_bfloat16*>(ptr(c->ret_peer[r]));
  }
  return 0;
}

static int ep_grid(long long warps_needed) {
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const long long blocks = (warps_needed * 32 + kEpThreads - 1) / kEpThreads;
  return static_cast<int>(blocks < 1 ? 1 : (blocks > 4LL * sms ? 4LL * sms : blocks));
}

// stage 0: dispatch, 1: receive (ids_eff), 2: ready, 3: combine
extern "C" int mx_ep_a2a(const void* call, int stage, void* stream_) {
  EpParams p{};
  const int rc = ep_fill(static_cast<const MxEpCall*>(call), p);
  if (rc) return rc;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  switch (stage) {
    case 0:
      if (p.cnt == nullptr || p.ticket == nullptr || p.route == nullptr) return -1;
      if (p.T > 0 && (p.x == nullptr || p.ids == nullptr)) return -1;   // T == 0 still raises the flags
      return static_cast<int>(launch_kernel(ep_dispatch_kernel, dim3(ep_grid(static_cast<long long>(p.T) * p.k)),
                                            dim3(kEpThreads), 0, stream, p));
    case 1:
      if (p.ids_eff == nullptr) return -1;
      return static_cast<int>(launch_kernel(ep_recv_kernel,
                                            dim3(ep_grid((static_cast<long long>(p.world) * p.cap + 31) / 32)),
                                            dim3(kEpThreads), 0, stream, p));
    case 2:
      return static_cast<int>(launch_kernel(ep_ready_kernel, dim3(1), dim3(32), 0, stream, p));
    case 3:
      if (p.T > 0 && (p.out == nullptr || p.wts == nullptr || p.route == nullptr)) return -1;
      return static_cast<int>(launch_kernel(ep_combine_kernel, dim3(ep_grid(p.T)), dim3(kEpThreads), 0, stream, p));
    default:
      return -1;
  }
}
