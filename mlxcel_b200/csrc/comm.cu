// Stand-alone all-reduce over the symmetric heap (peer loads/stores + system-scope flags), for
// partial results that do not come out of the dense GEMM epilogue: the weighted MoE combine under
// expert parallelism and the quantized GEMV under tensor parallelism.
//
// Same channel protocol as the GEMM communication epilogues (see CommParams in gemm.cu): the
// tensor is cut into chunks of kChunkElems bf16; per chunk
//   one-shot (mode 1): push the chunk into every peer's slot [rank], bump the chunk's arrival flag
//     on every peer, wait for `world` arrivals on the own flag, sum the slots in rank order
//     (+ residual) -> out. All ranks end with bitwise identical results.
//   two-shot (mode 2): chunk c is owned by rank c % world: partials go to the owner only, the owner
//     sums (+ residual) and stores the result into every peer's output; a per-call completion
//     counter tells each rank when all chunks have landed.
// With multicast (NVLS) addresses of the channel (flags_mc != NULL) the traffic goes through the
// NVSwitch instead of per-peer stores:
//   one-shot: the chunk is copied into THIS rank's slot 0 (local stores), one multimem.red bumps
//     the chunk flag on every rank, and after `world` arrivals every rank pulls the sum of all
//     replicas with multimem.ld_reduce (fp32 accumulation in the switch).
//   two-shot: chunks stay local the same way, the owner pulls the reduced chunk with
//     multimem.ld_reduce, adds the residual and writes every rank's output with one multimem.st.
// Receive slots are double-buffered by call parity. Waits are bounded and report through `status`.
#include "api.h"
#include "common.cuh"

namespace mx {

constexpr int kArMaxRanks = 8;
constexpr int kArThreads = 256;
constexpr int kChunkElems = kArThreads * 8 * 4;   // 8192 bf16 = 16 KiB per chunk
constexpr int kArMaxChunks = 8192;
constexpr int kArDoneIdx = kArMaxChunks;

struct ArParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* residual;
  __nv_bfloat16* out;
  long long n;               // elements
  int rank, world, mode;
  uint32_t* ctl;
  uint32_t* expect;
  int* status;
  uint32_t* flags_peer[kArMaxRanks];
  __nv_bfloat16* recv_peer[kArMaxRanks];
  __nv_bfloat16* out_peer[kArMaxRanks];
  long long parity_stride, rank_stride;
  int nvls;
  uint32_t* flags_mc;
  __nv_bfloat16* recv_mc;
  __nv_bfloat16* out_mc;
};

__device__ __forceinline__ void ar_signal(uint32_t* addr) {
  asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(addr) : "memory");
}
__device__ __forceinline__ bool ar_wait(const uint32_t* addr, uint32_t target, int* status) {
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

__global__ void __launch_bounds__(kArThreads) allreduce_kernel(const ArParams p) {
  __shared__ int ok_s;
  pdl_trigger();
  pdl_wait();
  const uint32_t parity = *reinterpret_cast<volatile uint32_t*>(p.ctl) & 1u;
  const long long chunks = (p.n + kChunkElems - 1) / kChunkElems;
  const size_t pbase = parity * static_cast<size_t>(p.parity_stride);
  for (long long c = blockIdx.x; c < chunks; c += gridDim.x) {
    const long long e0 = c * kChunkElems;
    const int owner = static_cast<int>(c % p.world);
    // NVLS: every chunk keeps its own place in the local half (slot 0 spans the whole tensor)
    const long long slot_off = (p.mode == 1 || p.nvls) ? e0 : (c / p.world) * kChunkElems;
    // ---- push
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      const long long e = e0 + (static_cast<long long>(it) * kArThreads + threadIdx.x) * 8;
      if (e < p.n) {
        const uint4 v = *reinterpret_cast<const uint4*>(p.x + e);
        const size_t off = pbase + (p.nvls ? 0 : p.rank * static_cast<size_t>(p.rank_stride)) + slot_off + (e - e0);
        if (p.nvls) {
          *reinterpret_cast<uint4*>(p.recv_peer[p.rank] + off) = v;
        } else if (p.mode == 1) {
          for (int pr = 0; pr < p.world; ++pr) *reinterpret_cast<uint4*>(p.recv_peer[pr] + off) = v;
        } else {
          *reinterpret_cast<uint4*>(p.recv_peer[owner] + off) = v;
        }
      }
    }
    __syncthreads();   // then one releasing thread per peer signals (release is cumulative)
    if (p.mode == 1 && p.nvls) {
      if (threadIdx.x == 0) multimem_signal_add(p.flags_mc + c, 1u);
    } else if (p.mode == 1) {
      if (threadIdx.x < p.world) ar_signal(p.flags_peer[threadIdx.x] + c);
    } else if (threadIdx.x == 0) {
      ar_signal(p.flags_peer[owner] + c);
    }
    const bool reducer = (p.mode == 1) || owner == p.rank;
    if (reducer) {
      if (threadIdx.x == 0) {
        const uint32_t target = p.expect[c] + static_cast<uint32_t>(p.world);
        ok_s = ar_wait(p.flags_peer[p.rank] + c, target, p.status) ? 1 : 0;
        p.expect[c] = target;
      }
      __syncthreads();
      if (ok_s) {
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const long long e = e0 + (static_cast<long long>(it) * kArThreads + threadIdx.x) * 8;
          if (e < p.n) {
            float acc[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[j] = 0.f;
            if (p.residual != nullptr) {
              const uint4 r = *reinterpret_cast<const uint4*>(p.residual + e);
              const uint32_t w4[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                acc[2 * j] = bf16_lo(w4[j]);
                acc[2 * j + 1] = bf16_hi(w4[j]);
              }
            }
            if (p.nvls) {
              const uint4 a = multimem_ld_reduce_bf16x8(p.recv_mc + pbase + slot_off + (e - e0));
              const uint32_t w4[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                acc[2 * j] += bf16_lo(w4[j]);
                acc[2 * j + 1] += bf16_hi(w4[j]);
              }
            }
            for (int r = 0; r < (p.nvls ? 0 : p.world); ++r) {
              const uint4 a = __ldcg(reinterpret_cast<const uint4*>(
                  p.recv_peer[p.rank] + pbase + r * static_cast<size_t>(p.rank_stride) + slot_off + (e - e0)));
              const uint32_t w4[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                acc[2 * j] += bf16_lo(w4[j]);
                acc[2 * j + 1] += bf16_hi(w4[j]);
              }
            }
            uint4 o;
            o.x = pack_bf16(acc[0], acc[1]);
            o.y = pack_bf16(acc[2], acc[3]);
            o.z = pack_bf16(acc[4], acc[5]);
            o.w = pack_bf16(acc[6], acc[7]);
            if (p.mode == 1) {
              *reinterpret_cast<uint4*>(p.out + e) = o;
            } else if (p.nvls) {
              multimem_st_16(p.out_mc + e, o);
            } else {
              for (int pr = 0; pr < p.world; ++pr) *reinterpret_cast<uint4*>(p.out_peer[pr] + e) = o;
            }
          }
        }
      }
      if (p.mode == 2) {
        __syncthreads();
        if (p.nvls) {
          if (threadIdx.x == 0) multimem_signal_add(p.flags_mc + kArDoneIdx, 1u);
        } else if (threadIdx.x < p.world) {
          ar_signal(p.flags_peer[threadIdx.x] + kArDoneIdx);
        }
      }
    }
    __syncthreads();
  }
  // ---- per-call completion + call counter
  if (threadIdx.x == 0) {
    const uint32_t per_call = (p.mode == 2) ? static_cast<uint32_t>(chunks) : 0u;
    if (per_call != 0u) {
      const uint32_t target = *reinterpret_cast<volatile uint32_t*>(p.ctl + 2) + per_call;
      ar_wait(p.flags_peer[p.rank] + kArDoneIdx, target, p.status);
    }
    __threadfence();
    const uint32_t prev = atomicAdd(p.ctl + 1, 1u);
    if (prev == gridDim.x - 1) {
      p.ctl[1] = 0u;
      p.ctl[2] += per_call;
      __threadfence();
      atomicAdd(p.ctl, 1u);
    }
  }
}

}  // namespace mx

using namespace mx;

// out = residual + sum over ranks of x (n bf16 elements, n % 8 == 0, 16-byte aligned buffers).
// mode 1: one-shot (out is local); mode 2: two-shot (results land in every out_peer, which must be
// the same heap offset on every rank; `out` is ignored). rank_stride (elements) must hold n for
// mode 1 and ceil(chunks / world) * 8192 for mode 2. status: device status word.
// flags_mc / recv_mc / out_mc: multicast addresses of the same flags / receive area / output, or
// NULL for the peer-store protocol.
extern "C" int mx_allreduce_comm(const void* x, const void* residual, void* out, long long n, int mode,
                                 int rank, int world, const void* const* flags_peer,
                                 const void* const* recv_peer, const void* const* out_peer, void* ctl,
                                 void* expect, long long parity_stride, long long rank_stride,
                                 void* status, void* stream_, void* flags_mc, void* recv_mc,
                                 void* out_mc) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (n <= 0) return 0;
  if (n % 8 || world < 1 || world > kArMaxRanks || rank < 0 || rank >= world) return -1;
  if (mode != 1 && mode != 2) return -1;
  const long long chunks = (n + kChunkElems - 1) / kChunkElems;
  if (chunks > kArMaxChunks) return -5;
  const bool nvls = flags_mc != nullptr && recv_mc != nullptr && (mode == 1 || out_mc != nullptr) &&
                    chunks * kChunkElems <= (mode == 1 ? rank_stride : parity_stride);
  if (mode == 1 && n > rank_stride) return -5;
  if (mode == 2 && !nvls && ((chunks + world - 1) / world) * kChunkElems > rank_stride) return -5;
  ArParams p{};
  p.x = static_cast<const __nv_bfloat16*>(x);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.out = static_cast<__nv_bfloat16*>(out);
  p.n = n;
  p.rank = rank;
  p.world = world;
  p.mode = mode;
  p.ctl = static_cast<uint32_t*>(ctl);
  p.expect = static_cast<uint32_t*>(expect);
  p.status = static_cast<int*>(status);
  for (int r = 0; r < world; ++r) {
    p.flags_peer[r] = static_cast<uint32_t*>(const_cast<void*>(flags_peer[r]));
    p.recv_peer[r] = static_cast<__nv_bfloat16*>(const_cast<void*>(recv_peer[r]));
    p.out_peer[r] = out_peer ? static_cast<__nv_bfloat16*>(const_cast<void*>(out_peer[r])) : nullptr;
  }
  p.parity_stride = parity_stride;
  p.rank_stride = rank_stride;
  p.nvls = nvls ? 1 : 0;
  p.flags_mc = static_cast<uint32_t*>(flags_mc);
  p.recv_mc = static_cast<__nv_bfloat16*>(recv_mc);
  p.out_mc = static_cast<__nv_bfloat16*>(out_mc);
  // every CTA must be resident at once (peers wait on each other's chunks)
  int sms = 148;
  int dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int grid = static_cast<int>(chunks < sms ? chunks : sms);
  return static_cast<int>(launch_kernel(allreduce_kernel, dim3(grid), dim3(kArThreads), 0, stream, p));
}
