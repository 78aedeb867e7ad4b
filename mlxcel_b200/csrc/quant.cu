// MLX checkpoint quantization formats on the GPU: dequantization to bf16 and the
// weight-bandwidth-bound GEMV (decode with a handful of rows).
//
// Formats (as stored by MLX, see the reference's src/lib/mlxcel-core/src/layers.rs:1885-2522 and
// src/lib/mlxcel-core/cpp/mlx_cxx_kernels.cpp:3073-3152):
//   affine  bits in {2,3,4,5,6,8}: values packed LSB-first along the input dimension into uint32
//           words (a contiguous little-endian bit stream, so 3/5/6-bit values may straddle
//           words); one (scale, bias) pair in the activation dtype per `group` inputs per row;
//           w = q * scale + bias.
//   mxfp4   4-bit e2m1 values, one e8m0 (uint8, 2^(s-127)) scale per 32 inputs, no bias.
//   mxfp8   8-bit e4m3 values, one e8m0 scale per 32 inputs.
//
// qmv: one warp per output row, lanes stride the packed row with 16-byte loads, fp32
// accumulation for up to 8 activation rows that share every dequantized weight (the reference's
// qmv / qmv_multirow kernels, overlays/cuda/.../quantized/qmm/qmv.cu:661-728, fold 2..8 rows the
// same way). Larger M goes through dequantize + the tcgen05 GEMM.
#include "api.h"
#include "common.cuh"

namespace mx {

enum QMode : int { kAffine = 0, kMxfp4 = 1, kMxfp8 = 2 };

__device__ __forceinline__ float e8m0_to_float(uint8_t s) {
  // 2^(s - 127); s = 0 maps to 2^-127 (denormal in fp32), s = 255 is NaN by the OCP spec.
  if (s == 255) return __uint_as_float(0x7fc00000u);
  if (s == 0) return __uint_as_float(0x00400000u);
  return __uint_as_float(static_cast<uint32_t>(s) << 23);
}
__device__ __forceinline__ float e2m1_to_float(uint32_t nib) {
  // sign | 2-bit exponent | 1-bit mantissa: {0, .5, 1, 1.5, 2, 3, 4, 6}
  const uint32_t ee = (nib >> 1) & 3u, m = nib & 1u;
  const uint32_t mag = ee ? (((ee + 126u) << 23) | (m << 22)) : (m ? 0x3F000000u : 0u);
  return __uint_as_float(mag | ((nib & 8u) << 28));
}
__device__ __forceinline__ float e4m3_to_float(uint32_t b) {
  const uint32_t sign = (b & 0x80u) << 24;
  const uint32_t exp = (b >> 3) & 0xFu, man = b & 7u;
  float v;
  if (exp == 0) {
    v = static_cast<float>(man) * 0.001953125f;  // subnormal: man * 2^-9
  } else if (exp == 15 && man == 7) {
    v = __uint_as_float(0x7fc00000u);            // NaN (e4m3fn has no inf)
  } else {
    v = __uint_as_float(((exp + 120u) << 23) | (man << 20));
  }
  return __uint_as_float(__float_as_uint(v) | sign);
}

// Value i of a row's little-endian bit stream.
__device__ __forceinline__ uint32_t extract_bits(const uint32_t* row, long long i, int bits) {
  const long long bit = i * bits;
  const long long wi = bit >> 5;
  const int sh = static_cast<int>(bit & 31);
  uint32_t v = row[wi] >> sh;
  if (sh + bits > 32) v |= row[wi + 1] << (32 - sh);
  return v & ((1u << bits) - 1u);
}

__global__ void dequantize_kernel(const uint32_t* __restrict__ w, const void* __restrict__ scales,
                                  const __nv_bfloat16* __restrict__ biases,
                                  __nv_bfloat16* __restrict__ out, long long rows, int K, int bits,
                                  int group, int mode) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  const int per_row = K / 8;
  if (idx >= rows * per_row) return;
  const long long r = idx / per_row;
  const int k0 = static_cast<int>(idx - r * per_row) * 8;
  const int words_per_row = K * bits / 32;
  const uint32_t* row = w + r * words_per_row;
  const int groups_per_row = K / group;
  float sc, bi = 0.f;
  const long long g = r * groups_per_row + k0 / group;
  if (mode == kAffine) {
    sc = __bfloat162float(static_cast<const __nv_bfloat16*>(scales)[g]);
    bi = __bfloat162float(biases[g]);
  } else {
    sc = e8m0_to_float(static_cast<const uint8_t*>(scales)[g]);
  }
  float f[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    const uint32_t q = extract_bits(row, k0 + j, bits);
    float v;
    if (mode == kAffine) v = static_cast<float>(q) * sc + bi;
    else if (mode == kMxfp4) v = e2m1_to_float(q) * sc;
    else v = e4m3_to_float(q) * sc;
    f[j] = v;
  }
  uint4 o;
  o.x = pack_bf16(f[0], f[1]);
  o.y = pack_bf16(f[2], f[3]);
  o.z = pack_bf16(f[4], f[5]);
  o.w = pack_bf16(f[6], f[7]);
  *reinterpret_cast<uint4*>(out + r * K + k0) = o;
}

// 4-bit formats, 32 values (one 16-byte piece, inside one group) per thread: direct nibble
// extraction with the format fixed at compile time and 64 contiguous output bytes per thread. The
// generic kernel above spends its time on per-value bit-stream arithmetic (measured 0.6 TB/s of
// output on 128 stacked experts); expanding a layer's experts before a prefill-sized grouped GEMM
// needs this to run at memory speed.
template <int MODE>
__global__ void __launch_bounds__(256)
dequantize4_kernel(const uint4* __restrict__ w, const void* __restrict__ scales,
                   const __nv_bfloat16* __restrict__ biases, uint4* __restrict__ out, long long pieces,
                   int pieces_per_row, int group) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= pieces) return;
  const long long r = idx / pieces_per_row;
  const int c = static_cast<int>(idx - r * pieces_per_row);
  uint4 pk;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(pk.x), "=r"(pk.y), "=r"(pk.z), "=r"(pk.w) : "l"(w + idx));
  const long long g = r * (static_cast<long long>(pieces_per_row) * 32 / group) + (c * 32) / group;
  float sc, bi = 0.f;
  if (MODE == kAffine) {
    sc = __bfloat162float(static_cast<const __nv_bfloat16*>(scales)[g]);
    bi = __bfloat162float(biases[g]);
  } else {
    sc = e8m0_to_float(static_cast<const uint8_t*>(scales)[g]);
  }
  const uint32_t words[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    float f[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const uint32_t nib = (words[q] >> (4 * j)) & 0xFu;
      f[j] = (MODE == kAffine) ? static_cast<float>(nib) * sc + bi : e2m1_to_float(nib) * sc;
    }
    out[idx * 4 + q] = make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]),
                                  pack_bf16(f[6], f[7]));
  }
}

// ----------------------------------------------------------------------------- qmv
constexpr int kQmvWarps = 8;

// BITS in {4, 8}. One lane consumes one uint4 of packed weights per step:
// 32 values (4-bit) or 16 values (8-bit), all inside one quantization group (group >= 32).
// Dot products of weight row n with M activation rows, lanes striding the packed row. After the
// call every lane holds the warp-reduced sums in acc[0..M).
template <int BITS, int MODE, int M>
__device__ __forceinline__ void qmv_row_dot(const __nv_bfloat16* __restrict__ x, const uint32_t* __restrict__ w,
                                            const void* __restrict__ scales,
                                            const __nv_bfloat16* __restrict__ biases, int n, int K, int group,
                                            int ldx, int lane, float (&acc)[M]) {
  constexpr int VPL = 128 / BITS;  // values per lane per step
  const int words_per_row = K * BITS / 32;
  const uint4* row = reinterpret_cast<const uint4*>(w + static_cast<size_t>(n) * words_per_row);
  const int groups_per_row = K / group;
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = 0.f;
  const int steps = K / VPL;  // uint4 chunks per row
  for (int c = lane; c < steps; c += 32) {
    const uint4 pk = row[c];
    const int k0 = c * VPL;
    const size_t g = static_cast<size_t>(n) * groups_per_row + k0 / group;
    float sc, bi = 0.f;
    if (MODE == kAffine) {
      sc = __bfloat162float(static_cast<const __nv_bfloat16*>(scales)[g]);
      bi = __bfloat162float(biases[g]);
    } else {
      sc = e8m0_to_float(static_cast<const uint8_t*>(scales)[g]);
    }
    const uint32_t words[4] = {pk.x, pk.y, pk.z, pk.w};
    float wv[VPL];
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const uint32_t q = (words[(j * BITS) >> 5] >> ((j * BITS) & 31)) & ((1u << BITS) - 1u);
      if (MODE == kAffine) wv[j] = static_cast<float>(q);
      else if (MODE == kMxfp4) wv[j] = e2m1_to_float(q);
      else wv[j] = e4m3_to_float(q);
    }
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(m) * ldx + k0);
      float dot = 0.f, xs = 0.f;
#pragma unroll
      for (int v = 0; v < VPL / 8; ++v) {
        const uint4 xa = xr[v];
        const uint32_t xw[4] = {xa.x, xa.y, xa.z, xa.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = bf16_lo(xw[j]), b = bf16_hi(xw[j]);
          dot += a * wv[v * 8 + 2 * j] + b * wv[v * 8 + 2 * j + 1];
          xs += a + b;
        }
      }
      // affine: sum_k x_k (q_k s + b) = s * sum x_k q_k + b * sum x_k
      acc[m] += (MODE == kAffine) ? (sc * dot + bi * xs) : sc * dot;
    }
  }
#pragma unroll
  for (int m = 0; m < M; ++m) acc[m] = warp_sum(acc[m]);
}

// BITS in {4, 8}. One lane consumes one uint4 of packed weights per step:
// 32 values (4-bit) or 16 values (8-bit), all inside one quantization group (group >= 32).
template <int BITS, int MODE, int M>
__global__ void __launch_bounds__(kQmvWarps * 32)
qmv_kernel(const __nv_bfloat16* __restrict__ x, const uint32_t* __restrict__ w,
           const void* __restrict__ scales, const __nv_bfloat16* __restrict__ biases,
           __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ residual,
           const __nv_bfloat16* __restrict__ lin_bias, int N, int K, int group, int ldx, int ldo) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * kQmvWarps + warp;
  if (n >= N) return;
  float acc[M];
  qmv_row_dot<BITS, MODE, M>(x, w, scales, biases, n, K, group, ldx, lane, acc);
  if (lane == 0) {
    const float lb = lin_bias ? __bfloat162float(lin_bias[n]) : 0.f;
#pragma unroll
    for (int m = 0; m < M; ++m) {
      float v = acc[m] + lb;
      if (residual) v += __bfloat162float(residual[static_cast<size_t>(m) * ldo + n]);
      out[static_cast<size_t>(m) * ldo + n] = __float2bfloat16(v);
    }
  }
}

// ----------------------------------------------------------------------------- qmv -> all-reduce
// Row-parallel quantized projection at decode batch sizes (M <= 8) under tensor parallelism: the
// GEMV over this rank's K shard and the cross-rank sum of the partial rows in ONE kernel. A block
// computes 8 consecutive output features (one warp each) for all M tokens = one 16-byte piece per
// token. Phase 1 (all of a block's groups): bf16 partials go into this rank's receive half (NVLS)
// or into slot [rank] of every peer (peer stores); the group's flag is bumped on every rank.
// Phase 2: wait for `world` arrivals, pull the sum with multimem.ld_reduce (or add the `world`
// local slots in rank order), add bias and residual, store. Phase 1 never waits, so blocks that
// are not resident yet cannot be waited on by resident ones of the same rank.
// Same channel words as the GEMM epilogues (ctl / expect / flags, receive halves by call parity).
// Replaces the reference's qmv kernels followed by its reduce_sum
// (overlays/cuda/.../quantized/qmm/qmv.cu:661-728, src/distributed/tensor_parallel/llama_runtime.rs:3133).
constexpr int kQmvMaxRanks = 8;
constexpr int kQmvMaxGroups = 8192;
struct QmvCommParams {
  int rank, world, nvls;
  uint32_t* ctl;
  uint32_t* expect;
  int* status;
  uint32_t* flags_peer[kQmvMaxRanks];
  __nv_bfloat16* recv_peer[kQmvMaxRanks];
  uint32_t* flags_mc;
  __nv_bfloat16* recv_mc;
  long long parity_stride, rank_stride;
};

__device__ __forceinline__ bool qmv_wait_flag(const uint32_t* addr, uint32_t target, int* status) {
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

template <int BITS, int MODE, int M>
__global__ void __launch_bounds__(kQmvWarps * 32)
qmv_allreduce_kernel(const __nv_bfloat16* __restrict__ x, const uint32_t* __restrict__ w,
                     const void* __restrict__ scales, const __nv_bfloat16* __restrict__ biases,
                     __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ residual,
                     const __nv_bfloat16* __restrict__ lin_bias, int N, int K, int group, int ldx, int ldo,
                     int ldr, const QmvCommParams cm) {
  __shared__ int ok_s;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int groups = N / kQmvWarps;      // N is a multiple of 8
  pdl_trigger();
  pdl_wait();
  const uint32_t parity = *reinterpret_cast<volatile uint32_t*>(cm.ctl) & 1u;
  const size_t pbase = parity * static_cast<size_t>(cm.parity_stride);
  // ---- phase 1: partial rows -> receive areas, one flag bump per group
  for (int gi = blockIdx.x; gi < groups; gi += gridDim.x) {
    const int n = gi * kQmvWarps + warp;
    float acc[M];
    qmv_row_dot<BITS, MODE, M>(x, w, scales, biases, n, K, group, ldx, lane, acc);
    if (lane == 0) {
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const __nv_bfloat16 v = __float2bfloat16(acc[m]);
        const size_t off = pbase + static_cast<size_t>(m) * N + n;
        if (cm.nvls) {
          // fp32 partial: the switch adds in fp32, nothing is rounded before the cross-rank sum
          reinterpret_cast<float*>(cm.recv_peer[cm.rank] + pbase)[static_cast<size_t>(m) * N + n] = acc[m];
        } else {
          const size_t so = off + cm.rank * static_cast<size_t>(cm.rank_stride);
          for (int pr = 0; pr < cm.world; ++pr) cm.recv_peer[pr][so] = v;
        }
      }
    }
    __syncthreads();   // the block's stores are ordered before the releasing signal below
    if (cm.nvls) {
      if (threadIdx.x == 0) multimem_signal_add(cm.flags_mc + gi, 1u);
    } else if (threadIdx.x < cm.world) {
      asm volatile("red.release.sys.global.add.u32 [%0], 1;" ::"l"(cm.flags_peer[threadIdx.x] + gi) : "memory");
    }
  }
  // ---- phase 2: wait, reduce, finish
  for (int gi = blockIdx.x; gi < groups; gi += gridDim.x) {
    if (threadIdx.x == 0) {
      const uint32_t target = cm.expect[gi] + static_cast<uint32_t>(cm.world);
      ok_s = qmv_wait_flag(cm.flags_peer[cm.rank] + gi, target, cm.status) ? 1 : 0;
      cm.expect[gi] = target;
    }
    __syncthreads();
    if (ok_s && threadIdx.x < M) {
      const int m = threadIdx.x, n0 = gi * kQmvWarps;
      float o[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = 0.f;
      if (cm.nvls) {
        const float* src = reinterpret_cast<const float*>(cm.recv_mc + pbase) + static_cast<size_t>(m) * N + n0;
        const float4 a = multimem_ld_reduce_f32x4(src), b = multimem_ld_reduce_f32x4(src + 4);
        o[0] = a.x, o[1] = a.y, o[2] = a.z, o[3] = a.w, o[4] = b.x, o[5] = b.y, o[6] = b.z, o[7] = b.w;
      } else {
        for (int r = 0; r < cm.world; ++r) {
          const uint4 a = __ldcg(reinterpret_cast<const uint4*>(
              cm.recv_peer[cm.rank] + pbase + r * static_cast<size_t>(cm.rank_stride) + static_cast<size_t>(m) * N + n0));
          const uint32_t w4[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) o[2 * j] += bf16_lo(w4[j]), o[2 * j + 1] += bf16_hi(w4[j]);
        }
      }
      if (lin_bias != nullptr) {
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j] += __bfloat162float(lin_bias[n0 + j]);
      }
      if (residual != nullptr) {
        const uint4 rs = *reinterpret_cast<const uint4*>(residual + static_cast<size_t>(m) * ldr + n0);
        const uint32_t r4[4] = {rs.x, rs.y, rs.z, rs.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) o[2 * j] += bf16_lo(r4[j]), o[2 * j + 1] += bf16_hi(r4[j]);
      }
      uint4 pk;
      pk.x = pack_bf16(o[0], o[1]);
      pk.y = pack_bf16(o[2], o[3]);
      pk.z = pack_bf16(o[4], o[5]);
      pk.w = pack_bf16(o[6], o[7]);
      *reinterpret_cast<uint4*>(out + static_cast<size_t>(m) * ldo + n0) = pk;
    }
    __syncthreads();
  }
  // ---- per-call completion: the last block to finish advances the channel's call counter
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(cm.ctl + 1, 1u);
    if (prev == gridDim.x - 1) {
      cm.ctl[1] = 0u;
      __threadfence();
      atomicAdd(cm.ctl, 1u);
    }
  }
}

template <int BITS, int MODE>
static int launch_qmv(const void* x, const void* w, const void* scales, const void* biases,
                      void* out, const void* residual, const void* lin_bias, int M, int N, int K,
                      int group, int ldx, int ldo, cudaStream_t st) {
  const int grid = (N + kQmvWarps - 1) / kQmvWarps;
#define MX_QMV(M_)                                                                          \
  case M_:                                                                                  \
    qmv_kernel<BITS, MODE, M_><<<grid, kQmvWarps * 32, 0, st>>>(                            \
        static_cast<const __nv_bfloat16*>(x), static_cast<const uint32_t*>(w), scales,      \
        static_cast<const __nv_bfloat16*>(biases), static_cast<__nv_bfloat16*>(out),        \
        static_cast<const __nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(lin_bias), \
        N, K, group, ldx, ldo);                                                             \
    break;
  switch (M) {
    MX_QMV(1) MX_QMV(2) MX_QMV(3) MX_QMV(4) MX_QMV(5) MX_QMV(6) MX_QMV(7) MX_QMV(8)
    default: return -1;
  }
#undef MX_QMV
  return static_cast<int>(cudaGetLastError());
}

}  // namespace mx

using namespace mx;

extern "C" int mx_dequantize(const void* w, const void* scales, const void* biases, void* out,
                             long long N, int K, int bits, int group, int mode, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (N <= 0) return 0;
  if (K % 8 || K % group || (K * bits) % 32) return -1;
  if (mode == kAffine && !(bits == 2 || bits == 3 || bits == 4 || bits == 5 || bits == 6 || bits == 8)) return -1;
  if (mode == kMxfp4 && bits != 4) return -1;
  if (mode == kMxfp8 && bits != 8) return -1;
  if (bits == 4 && K % 32 == 0 && group % 32 == 0 && (mode == kAffine || mode == kMxfp4) &&
      (reinterpret_cast<uintptr_t>(w) & 15) == 0 && (reinterpret_cast<uintptr_t>(out) & 15) == 0) {
    const long long pieces = N * (K / 32);
    const long long nb = (pieces + 255) / 256;
    if (nb > 0x7fffffffll) return -1;
    if (mode == kAffine)
      dequantize4_kernel<kAffine><<<static_cast<int>(nb), 256, 0, stream>>>(
          static_cast<const uint4*>(w), scales, static_cast<const __nv_bfloat16*>(biases), static_cast<uint4*>(out),
          pieces, K / 32, group);
    else
      dequantize4_kernel<kMxfp4><<<static_cast<int>(nb), 256, 0, stream>>>(
          static_cast<const uint4*>(w), scales, static_cast<const __nv_bfloat16*>(biases), static_cast<uint4*>(out),
          pieces, K / 32, group);
    return static_cast<int>(cudaGetLastError());
  }
  const long long total = N * (K / 8);
  const int threads = 256;
  const long long blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffll) return -1;
  dequantize_kernel<<<static_cast<int>(blocks), threads, 0, stream>>>(
      static_cast<const uint32_t*>(w), scales, static_cast<const __nv_bfloat16*>(biases),
      static_cast<__nv_bfloat16*>(out), N, K, bits, group, mode);
  return static_cast<int>(cudaGetLastError());
}

template <int BITS, int MODE>
static int launch_qmv_ar(const void* x, const void* w, const void* scales, const void* biases, void* out,
                         const void* residual, const void* lin_bias, int M, int N, int K, int group, int ldx,
                         int ldo, int ldr, const QmvCommParams& cm, cudaStream_t st) {
  const int groups = N / kQmvWarps;
  int sms = 148, dev = 0;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
#define MX_QMV_AR(M_)                                                                                  \
  case M_: {                                                                                           \
    auto kern = qmv_allreduce_kernel<BITS, MODE, M_>;                                                  \
    int per_sm = 0;                                                                                    \
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kern, kQmvWarps * 32, 0);                   \
    if (per_sm < 1) per_sm = 1;                                                                        \
    /* blocks wait on peers in phase 2: keep the grid within what is resident at once */              \
    const int grid = groups < per_sm * sms ? groups : per_sm * sms;                                    \
    return static_cast<int>(launch_kernel(kern, dim3(grid), dim3(kQmvWarps * 32), 0, st,              \
        static_cast<const __nv_bfloat16*>(x), static_cast<const uint32_t*>(w), scales,                 \
        static_cast<const __nv_bfloat16*>(biases), static_cast<__nv_bfloat16*>(out),                   \
        static_cast<const __nv_bfloat16*>(residual), static_cast<const __nv_bfloat16*>(lin_bias), N, K, \
        group, ldx, ldo, ldr, cm));                                                                    \
  }
  switch (M) {
    MX_QMV_AR(1) MX_QMV_AR(2) MX_QMV_AR(3) MX_QMV_AR(4) MX_QMV_AR(5) MX_QMV_AR(6) MX_QMV_AR(7) MX_QMV_AR(8)
    default: return -1;
  }
#undef MX_QMV_AR
}

// Quantized GEMV -> all-reduce in one kernel (see qmv_allreduce_kernel). Same shape rules as mx_qmv
// plus N % 8 == 0, 16-byte aligned out / residual rows, N / 8 <= 8192 flag words. flags_peer /
// recv_peer: host arrays of `world` device addresses; ctl / expect: this rank's channel words;
// rank_stride >= M * N elements (peer-store protocol: one slot per source rank), parity_stride =
// distance between the two receive halves. flags_mc / recv_mc: multicast addresses or NULL.
// Returns -9 when the shape is not covered (the caller takes the GEMM path).
extern "C" int mx_qmv_allreduce(const void* x, const void* w, const void* scales, const void* biases, void* out,
                                const void* residual, const void* lin_bias, int M, int N, int K, int bits,
                                int group, int mode, int ldx, int ldo, int ldr, int rank, int world,
                                const void* const* flags_peer, const void* const* recv_peer, void* ctl,
                                void* expect, long long parity_stride, long long rank_stride, void* status,
                                void* flags_mc, void* recv_mc, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (M > 8 || (bits != 4 && bits != 8) || world < 1 || world > kQmvMaxRanks || rank < 0 || rank >= world) return -9;
  const int vpl = 128 / bits;
  if (K % vpl || group % vpl || K % group || (ldx % 8) || (N % 8) || (ldo % 8) || (residual && (ldr % 8))) return -9;
  if (N / kQmvWarps > kQmvMaxGroups || static_cast<long long>(M) * N > rank_stride) return -9;
  if (world > 1 && 2ll * M * N > parity_stride) return -9;   // fp32 partials (NVLS) live in the bf16-sized half
  auto mis = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) != 0; };
  if (mis(w) || mis(x) || mis(out) || (residual && mis(residual))) return -9;
  if ((static_cast<long long>(K) * bits / 8) % 16 || (parity_stride % 8) || (rank_stride % 8)) return -9;
  QmvCommParams cm{};
  cm.rank = rank;
  cm.world = world;
  cm.ctl = static_cast<uint32_t*>(ctl);
  cm.expect = static_cast<uint32_t*>(expect);
  cm.status = static_cast<int*>(status);
  for (int r = 0; r < world; ++r) {
    cm.flags_peer[r] = static_cast<uint32_t*>(const_cast<void*>(flags_peer[r]));
    cm.recv_peer[r] = static_cast<__nv_bfloat16*>(const_cast<void*>(recv_peer[r]));
    if (mis(cm.recv_peer[r])) return -9;
  }
  cm.nvls = (flags_mc != nullptr && recv_mc != nullptr && !mis(recv_mc)) ? 1 : 0;
  cm.flags_mc = static_cast<uint32_t*>(flags_mc);
  cm.recv_mc = static_cast<__nv_bfloat16*>(recv_mc);
  cm.parity_stride = parity_stride;
  cm.rank_stride = rank_stride;
  if (mode == kAffine) {
    return bits == 4 ? launch_qmv_ar<4, kAffine>(x, w, scales, biases, out, residual, lin_bias, M, N, K, group, ldx, ldo, ldr, cm, stream)
                     : launch_qmv_ar<8, kAffine>(x, w, scales, biases, out, residual, lin_bias, M, N, K, group, ldx, ldo, ldr, cm, stream);
  }
  if (mode == kMxfp4 && bits == 4)
    return launch_qmv_ar<4, kMxfp4>(x, w, scales, biases, out, residual, lin_bias, M, N, K, group, ldx, ldo, ldr, cm, stream);
  if (mode == kMxfp8 && bits == 8)
    return launch_qmv_ar<8, kMxfp8>(x, w, scales, biases, out, residual, lin_bias, M, N, K, group, ldx, ldo, ldr, cm, stream);
  return -9;
}

// GEMV path of quantized linears (M <= 8, bits in {4, 8}, group >= 128 / bits and K a multiple of
// the per-lane chunk). mode: 0 affine, 1 mxfp4, 2 mxfp8. Returns -9 when the shape needs the
// dequantize + GEMM path instead.
extern "C" int mx_qmv(const void* x, const void* w, const void* scales, const void* biases,
                      void* out, const void* residual, const void* lin_bias, int M, int N, int K,
                      int bits, int group, int mode, int ldx, int ldo, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (M <= 0 || N <= 0) return 0;
  if (M > 8 || (bits != 4 && bits != 8)) return -9;
  const int vpl = 128 / bits;
  if (K % vpl || group % vpl || K % group || (ldx % 8)) return -9;
  if (reinterpret_cast<uintptr_t>(w) & 15 || reinterpret_cast<uintptr_t>(x) & 15) return -9;
  if ((static_cast<long long>(K) * bits / 8) % 16) return -9;
  if (mode == kAffine) {
    return bits == 4 ? launch_qmv<4, kAffine>(x, w, scales, biases, out, residual, lin_bias, M, N, K, group, ldx, ldo, stream)
                     : launch_qmv<8, kAffine>(x, w, scales, biases, out, residual, lin_bias, M, N, K, group, ldx, ldo, stream);
  }
  if (mode == kMxfp4 && bits == 4)
    return launch_qmv<4, kMxfp4>(x, w, scales, biases, out, residual, lin_bias, M, N, K, group, ldx, ldo, stream);
  if (mode == kMxfp8 && bits == 8)
    return launch_qmv<8, kMxfp8>(x, w, scales, biases, out, residual, lin_bias, M, N, K, group, ldx, ldo, stream);
  return -9;
}
