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
  const float tab[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  const float v = tab[nib & 7u];
  return (nib & 8u) ? -v : v;
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

// ----------------------------------------------------------------------------- qmv
constexpr int kQmvWarps = 8;

// BITS in {4, 8}. One lane consumes one uint4 of packed weights per step:
// 32 values (4-bit) or 16 values (8-bit), all inside one quantization group (group >= 32).
template <int BITS, int MODE, int M>
__global__ void __launch_bounds__(kQmvWarps * 32)
qmv_kernel(const __nv_bfloat16* __restrict__ x, const uint32_t* __restrict__ w,
           const void* __restrict__ scales, const __nv_bfloat16* __restrict__ biases,
           __nv_bfloat16* __restrict__ out, const __nv_bfloat16* __restrict__ residual,
           const __nv_bfloat16* __restrict__ lin_bias, int N, int K, int group, int ldx, int ldo) {
  constexpr int VPL = 128 / BITS;  // values per lane per step
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.x * kQmvWarps + warp;
  if (n >= N) return;
  const int words_per_row = K * BITS / 32;
  const uint4* row = reinterpret_cast<const uint4*>(w + static_cast<size_t>(n) * words_per_row);
  const int groups_per_row = K / group;
  float acc[M];
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
  const long long total = N * (K / 8);
  const int threads = 256;
  const long long blocks = (total + threads - 1) / threads;
  if (blocks > 0x7fffffffll) return -1;
  dequantize_kernel<<<static_cast<int>(blocks), threads, 0, stream>>>(
      static_cast<const uint32_t*>(w), scales, static_cast<const __nv_bfloat16*>(biases),
      static_cast<__nv_bfloat16*>(out), N, K, bits, group, mode);
  return static_cast<int>(cudaGetLastError());
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
