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
//                 per-source counts into a COMPACT list of the rows in use: expert id and receive-row
//                 index of each, and their number, all on the device. The receive area is sized for
//                 the worst case (every source sends all its pairs here), so the expert stage must
//                 never walk it whole: its alignment, gather and scatter kernels are bounded by that
//                 number.
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
  uint32_t* epoch;               // local word: number of the current layer call; the dispatch kernel
                                 // advances it, the later stages read it (so a captured CUDA graph
                                 // replays with fresh flag values)
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
  int* ids_eff;                  // [world * cap] expert id of the i-th row in use (compact list)
  int* rowmap;                   // [world * cap] receive-row index of the i-th row in use
  int* nrecv;                    // number of rows in use
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

// A CTA takes kEpRowsPerCta (token, k) rows at a time: its first threads draw the slots, then all
// threads copy the rows as one flat range of 16-byte words (independent loads, peer stores that
// nobody waits for).
constexpr int kEpRowsPerCta = 8;

__global__ void __launch_bounds__(kEpThreads) ep_dispatch_kernel(const EpParams p) {
  __shared__ int s_dst[kEpRowsPerCta], s_slot[kEpRowsPerCta];
  const int vec = p.H >> 3;                       // 16-byte words per row
  const int rows = p.T * p.k;
  for (int e0 = blockIdx.x * kEpRowsPerCta; e0 < rows; e0 += gridDim.x * kEpRowsPerCta) {
    const int n = min(kEpRowsPerCta, rows - e0);
    __syncthreads();                              // the previous batch's slots have been used
    if (threadIdx.x < n) {
      const int e = e0 + threadIdx.x;
      const int expert = p.ids[e];
      int dst = expert / p.experts_per_rank, slot = 0;
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
      s_dst[threadIdx.x] = dst, s_slot[threadIdx.x] = slot;
      if (dst >= 0) p.meta_peer[dst][static_cast<size_t>(p.rank) * p.cap + slot] = expert;
    }
    __syncthreads();
#pragma unroll 4
    for (int i = threadIdx.x; i < n * vec; i += kEpThreads) {
      const int r = i / vec, v = i - r * vec;
      const int dst = s_dst[r];
      if (dst < 0) continue;
      const uint4 w = reinterpret_cast<const uint4*>(p.x + static_cast<size_t>((e0 + r) / p.k) * p.H)[v];
      reinterpret_cast<uint4*>(p.recv_peer[dst] + (static_cast<size_t>(p.rank) * p.cap + s_slot[r]) * p.H)[v] = w;
    }
  }
  // last CTA: publish the counts and raise the flags (every CTA's rows are fenced before its ticket)
  __shared__ bool last;
  __shared__ uint32_t epoch;
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    last = atomicAdd(p.ticket, 1u) == gridDim.x - 1;
    if (last) {
      epoch = *p.epoch + 1u;
      *p.epoch = epoch;
    }
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
    ep_flag_store(&p.dflag_peer[d][p.rank], epoch);
  }
  if (threadIdx.x == 0) *p.ticket = 0u;
}

// Compact list of the rows in use, source after source: entry base[s] + slot is row s * cap + slot.
__global__ void __launch_bounds__(kEpThreads) ep_recv_kernel(const EpParams p) {
  __shared__ int cnt[kEpMaxRanks], base[kEpMaxRanks + 1];
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    if (!ep_flag_wait(&p.dflag[threadIdx.x], *p.epoch, p.status)) ok = 0;
    cnt[threadIdx.x] = min(max(*reinterpret_cast<const volatile int*>(&p.count[threadIdx.x]), 0), p.cap);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int s = 0; s < p.world; ++s) {
      base[s] = acc;
      acc += ok ? cnt[s] : 0;
    }
    base[p.world] = acc;
    if (blockIdx.x == 0) *p.nrecv = acc;
  }
  __syncthreads();
  if (!ok) return;
  for (int s = 0; s < p.world; ++s) {
    for (int slot = blockIdx.x * kEpThreads + threadIdx.x; slot < cnt[s]; slot += gridDim.x * kEpThreads) {
      const int row = s * p.cap + slot;
      p.ids_eff[base[s] + slot] = *reinterpret_cast<const volatile int*>(&p.meta[row]);
      p.rowmap[base[s] + slot] = row;
    }
  }
}

__global__ void ep_ready_kernel(const EpParams p) {
  if (threadIdx.x < p.world) {
    __threadfence_system();
    ep_flag_store(&p.cflag_peer[threadIdx.x][p.rank], *p.epoch);
  }
}

// One thread per 16-byte word of the output: out[t] = residual[t] + sum_k w[t, k] * (owner's output
// row). The k peer loads of a word are issued together (a peer load is a round trip over NVLink, so
// the kernel is shaped for loads in flight, not for work per thread).
constexpr int kEpMaxTopK = 16;

__global__ void __launch_bounds__(kEpThreads) ep_combine_kernel(const EpParams p) {
  __shared__ int ok;
  if (threadIdx.x == 0) ok = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    if (!ep_flag_wait(&p.cflag[threadIdx.x], *p.epoch, p.status)) ok = 0;
  }
  __syncthreads();
  if (!ok) return;
  const int vec = p.H >> 3;
  const long long total = static_cast<long long>(p.T) * vec;
  for (long long i = static_cast<long long>(blockIdx.x) * kEpThreads + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * kEpThreads) {
    const int t = static_cast<int>(i / vec), v0 = static_cast<int>(i - static_cast<long long>(t) * vec);
    uint4 y[kEpMaxTopK];
    float w[kEpMaxTopK];
#pragma unroll
    for (int kk = 0; kk < kEpMaxTopK; ++kk) {
      w[kk] = 0.f;
      y[kk] = make_uint4(0u, 0u, 0u, 0u);
      if (kk < p.k) {
        const int rt = p.route[t * p.k + kk];
        if (rt >= 0) {
          const int d = rt / p.cap, slot = rt - d * p.cap;
          w[kk] = p.wts[t * p.k + kk];
          y[kk] = reinterpret_cast<const uint4*>(p.ret_peer[d] +
                                                 (static_cast<size_t>(p.rank) * p.cap + slot) * p.H)[v0];
        }
      }
    }
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
#pragma unroll
    for (int kk = 0; kk < kEpMaxTopK; ++kk) {
      const __nv_bfloat162* y2 = reinterpret_cast<const __nv_bfloat162*>(&y[kk]);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 f = __bfloat1622float2(y2[q]);
        acc[2 * q] += w[kk] * f.x, acc[2 * q + 1] += w[kk] * f.y;
      }
    }
    uint4 o;
    __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int q = 0; q < 4; ++q) o2[q] = __floats2bfloat162_rn(acc[2 * q], acc[2 * q + 1]);
    reinterpret_cast<uint4*>(p.out + static_cast<size_t>(t) * p.H)[v0] = o;
  }
}

}  // namespace mx

using namespace mx;

// Plain-C description of one call (pointers as 64-bit integers so that ctypes can fill it).
struct MxEpCall {
  int rank, world, T, k, H, experts_per_rank, cap;
  unsigned int reserved;
  unsigned long long epoch, status, x, ids, wts, residual, out, cnt, ticket, route, ids_eff, rowmap, nrecv;
  unsigned long long meta, count, dflag, cflag;
  unsigned long long recv_peer[kEpMaxRanks], meta_peer[kEpMaxRanks], count_peer[kEpMaxRanks],
      dflag_peer[kEpMaxRanks], cflag_peer[kEpMaxRanks], ret_peer[kEpMaxRanks];
};

static int ep_fill(const MxEpCall* c, EpParams& p) {
  if (c == nullptr || c->world < 1 || c->world > kEpMaxRanks || c->rank < 0 || c->rank >= c->world) return -1;
  if (c->H <= 0 || c->H % 8 || c->k < 1 || c->k > kEpMaxTopK || c->cap < 1 || c->experts_per_rank < 1 || c->T < 0) return -1;
  if (static_cast<long long>(c->world) * c->cap > 0x7fffffffLL) return -1;
  p.rank = c->rank, p.world = c->world, p.T = c->T, p.k = c->k, p.H = c->H;
  p.experts_per_rank = c->experts_per_rank, p.cap = c->cap;
  auto ptr = [](unsigned long long v) { return reinterpret_cast<void*>(static_cast<uintptr_t>(v)); };
  p.status = static_cast<int*>(ptr(c->status));
  p.epoch = static_cast<uint32_t*>(ptr(c->epoch));
  if (p.epoch == nullptr || p.status == nullptr) return -1;
  p.x = static_cast<const __nv_bfloat16*>(ptr(c->x));
  p.ids = static_cast<const int*>(ptr(c->ids));
  p.wts = static_cast<const float*>(ptr(c->wts));
  p.residual = static_cast<const __nv_bfloat16*>(ptr(c->residual));
  p.out = static_cast<__nv_bfloat16*>(ptr(c->out));
  p.cnt = static_cast<int*>(ptr(c->cnt));
  p.ticket = static_cast<uint32_t*>(ptr(c->ticket));
  p.route = static_cast<int*>(ptr(c->route));
  p.ids_eff = static_cast<int*>(ptr(c->ids_eff));
  p.rowmap = static_cast<int*>(ptr(c->rowmap));
  p.nrecv = static_cast<int*>(ptr(c->nrecv));
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
      return static_cast<int>(launch_kernel(
          ep_dispatch_kernel,
          dim3(ep_grid((static_cast<long long>(p.T) * p.k + kEpRowsPerCta - 1) / kEpRowsPerCta * (kEpThreads / 32))),
          dim3(kEpThreads), 0, stream, p));
    case 1:
      if (p.ids_eff == nullptr || p.rowmap == nullptr || p.nrecv == nullptr) return -1;
      // a few CTAs: the rows in use are normally a small part of the receive area
      return static_cast<int>(launch_kernel(ep_recv_kernel, dim3(32), dim3(kEpThreads), 0, stream, p));
    case 2:
      return static_cast<int>(launch_kernel(ep_ready_kernel, dim3(1), dim3(32), 0, stream, p));
    case 3:
      if (p.T > 0 && (p.out == nullptr || p.wts == nullptr || p.route == nullptr)) return -1;
      return static_cast<int>(launch_kernel(ep_combine_kernel,
                                            dim3(ep_grid((static_cast<long long>(p.T) * (p.H >> 3) + 31) / 32)),
                                            dim3(kEpThreads), 0, stream, p));
    default:
      return -1;
  }
}
