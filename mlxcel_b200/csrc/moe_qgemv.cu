// Grouped 4-bit GEMV for mixture-of-experts decode: few rows per expert, packed weights streamed once.
//
// At decode batch sizes an expert receives a handful of token rows (128 requests x top-4 over 128
// experts = 4 rows each), so its matrices are read for almost no arithmetic: the step is bound by
// the bytes of the packed weights. The tensor-core GEMM with its unpack stage pays a fixed
// synchronisation cost per 64-wide k-step for 4 KB of weights and reaches a tenth of the HBM
// bandwidth there. This kernel streams the MLX-packed rows directly (reference: gather_qmm for
// SwitchGLU, src/models/switch_layers.rs:98-220; overlays/cuda/.../quantized/qmm/qmv.cu):
//
//   grid  = (output-feature blocks, local experts); a block whose expert got no rows returns at once,
//           so only routed experts are read.
//   warp  = kFeat output features (gate row + up row each when gated). Lanes stride the packed row
//           in 16-byte pieces (32 weights), `kUnroll` pieces in flight per lane and row.
//   x     = the expert's token rows live in REGISTERS as half2, already in the order the nibble pairs
//           come out of a word ((j, j + 4) of each 8-nibble word), `kTok` tokens per pass; every
//           weight row of the warp reuses them. More tokens = more passes over the block's rows
//           (which then come from L2).
//   math  = two nibbles become one half2 with three integer ops and one exact half2 fix-up
//           (affine: 0x6400 | q is 1024 + q; mxfp4: sign / exponent / mantissa bits land in the
//           half's fields and 2^14 restores the exponent bias), products accumulate in half2 over
//           eight pairs, then in fp32 with the group's scale (and bias * sum(x) for affine).
//   out   = gated: act(gate + b, up + b) in bf16; plain: acc + bias.
#include <cuda_fp16.h>

#include "api.h"
#include "common.cuh"

namespace mx {

constexpr int kGvWarps = 8;     // warps per block
constexpr int kGvFeat = 2;      // output features per warp
constexpr int kGvTok = 2;       // token rows per pass (registers)
constexpr int kGvUnroll = 2;    // 16-byte pieces per lane per slab

__device__ __forceinline__ float gv_e8m0(uint8_t s) {
  if (s == 255) return __uint_as_float(0x7fc00000u);
  if (s == 0) return __uint_as_float(0x00400000u);
  return __uint_as_float(static_cast<uint32_t>(s) << 23);
}

// (nibble j, nibble j + 4) of `w` shifted so that they sit at bits 0..3 and 16..19.
template <int MODE>
__device__ __forceinline__ __half2 gv_pair(uint32_t t) {
  uint32_t h;
  if (MODE == 0) {                       // affine: 1024 + q, then - 1024 (exact)
    h = (t & 0x000F000Fu) | 0x64006400u;
    return __hsub2(*reinterpret_cast<__half2*>(&h), __half2half2(__ushort_as_half(0x6400)));
  }
  // mxfp4 (e2m1): s eem -> half bits s | eem << 9; times 2^14 moves the exponent bias from 15 to 1
  h = ((t & 0x00070007u) << 9) | ((t & 0x00080008u) << 12);
  return __hmul2(*reinterpret_cast<__half2*>(&h), __half2half2(__ushort_as_half(0x7400)));   // 2^14, exact
}

__device__ __forceinline__ float gv_glu(int epi, float g, float u, float alpha, float limit) {
  if (epi == MX_EPI_SWIGLU) return g / (1.f + __expf(-g)) * u;
  if (epi == MX_EPI_GEGLU) {
    const float c = 0.7978845608028654f * (g + 0.044715f * g * g * g);
    return 0.5f * g * (1.f + tanhf(c)) * u;
  }
  g = fminf(g, limit);
  u = fminf(fmaxf(u, -limit), limit);
  return g / (1.f + __expf(-alpha * g)) * (u + 1.f);
}

struct GvParams {
  const __nv_bfloat16* xs;     // [rows, K] rows of expert e are [offsets[e], offsets[e + 1])
  const uint32_t* w;           // [E, N, K / 8]
  const void* scales;          // affine: bf16 [E, N, K / group]; mxfp4: uint8 e8m0
  const __nv_bfloat16* biases; // affine only
  const __nv_bfloat16* lin_bias;  // [E, N] or null
  const __nv_bfloat16* residual;  // [rows, n_out] added by the plain epilogue, or null
  long long ldo, ldr;             // row strides of out / residual (elements)
  const int* offsets;          // [E + 1]
  __nv_bfloat16* out;          // [rows, n_out]
  int E, N, K, group, n_out, epi;
  float alpha, limit;
};

template <int MODE>
__global__ void __launch_bounds__(kGvWarps * 32) moe_qgemv_kernel(const GvParams p) {
  const int e = blockIdx.y;
  const int row0 = p.offsets[e], m_e = p.offsets[e + 1] - row0;
  if (m_e <= 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int f0 = (blockIdx.x * kGvWarps + warp) * kGvFeat;       // first output feature of this warp
  if (f0 >= p.n_out) return;
  const bool gated = p.epi >= MX_EPI_SWIGLU;
  constexpr int kRows = kGvFeat * 2;                              // weight rows per warp (gate + up)
  const int nrows = gated ? kRows : kGvFeat;
  const int pieces = p.K >> 5;                                    // 16-byte pieces (32 weights) per row
  const int words_per_row = p.K >> 3;
  const int groups_per_row = p.K / p.group;
  const size_t ebase = static_cast<size_t>(e) * p.N;

  for (int t0 = 0; t0 < m_e; t0 += kGvTok) {
    float acc[kRows][kGvTok];
#pragma unroll
    for (int r = 0; r < kRows; ++r)
#pragma unroll
      for (int t = 0; t < kGvTok; ++t) acc[r][t] = 0.f;

    for (int slab = 0; slab * 32 * kGvUnroll < pieces; ++slab) {
      // ---- this lane's activations of the slab: kUnroll pieces x 16 half2 per token
      __half2 xr[kGvTok][kGvUnroll][16];
      float xsum[kGvTok][kGvUnroll];
      bool live[kGvUnroll];
#pragma unroll
      for (int u = 0; u < kGvUnroll; ++u) {
        const int c = (slab * kGvUnroll + u) * 32 + lane;
        live[u] = c < pieces;
#pragma unroll
        for (int t = 0; t < kGvTok; ++t) {
          xsum[t][u] = 0.f;
          const bool tok = live[u] && (t0 + t) < m_e;
          const uint4* src = reinterpret_cast<const uint4*>(p.xs + static_cast<size_t>(row0 + t0 + t) * p.K + (c << 5));
#pragma unroll
          for (int q = 0; q < 4; ++q) {                           // 8 activations = one weight word
            uint4 v = make_uint4(0, 0, 0, 0);
            if (tok) v = src[q];
            const float a[8] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y),
                                bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w)};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              xr[t][u][q * 4 + j] = __floats2half2_rn(a[j], a[j + 4]);
              xsum[t][u] += a[j] + a[j + 4];
            }
          }
        }
      }
      // ---- every weight row of the warp against those registers: all loads first (kRows x kUnroll
      //      16-byte pieces in flight per lane), then the arithmetic
      uint4 pk[kRows][kGvUnroll];
      float sc[kRows][kGvUnroll], bi[kRows][kGvUnroll];
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
        const int feat = f0 + (r % kGvFeat);
        const bool row_live = r < nrows && feat < p.n_out;
        const int n = (r < kGvFeat) ? feat : p.n_out + feat;      // gate rows first, then up rows
        const uint4* wrow = reinterpret_cast<const uint4*>(p.w + (ebase + n) * words_per_row);
#pragma unroll
        for (int u = 0; u < kGvUnroll; ++u) {
          const int c = (slab * kGvUnroll + u) * 32 + lane;
          pk[r][u] = make_uint4(0, 0, 0, 0);
          sc[r][u] = bi[r][u] = 0.f;
          if (row_live && live[u]) {
            asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(pk[r][u].x), "=r"(pk[r][u].y), "=r"(pk[r][u].z), "=r"(pk[r][u].w) : "l"(wrow + c));
            const size_t g = (ebase + n) * groups_per_row + (c << 5) / p.group;
            if (MODE == 0) {
              sc[r][u] = __bfloat162float(static_cast<const __nv_bfloat16*>(p.scales)[g]);
              bi[r][u] = __bfloat162float(p.biases[g]);
            } else {
              sc[r][u] = gv_e8m0(static_cast<const uint8_t*>(p.scales)[g]);
            }
          }
        }
      }
#pragma unroll
      for (int r = 0; r < kRows; ++r) {
#pragma unroll
        for (int u = 0; u < kGvUnroll; ++u) {
          const uint32_t words[4] = {pk[r][u].x, pk[r][u].y, pk[r][u].z, pk[r][u].w};
          __half2 h[kGvTok][2];
#pragma unroll
          for (int t = 0; t < kGvTok; ++t) h[t][0] = h[t][1] = __floats2half2_rn(0.f, 0.f);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __half2 wv = gv_pair<MODE>(words[q] >> (4 * j));
#pragma unroll
              for (int t = 0; t < kGvTok; ++t) h[t][q >> 1] = __hfma2(wv, xr[t][u][q * 4 + j], h[t][q >> 1]);
            }
          }
#pragma unroll
          for (int t = 0; t < kGvTok; ++t) {
            const float2 a = __half22float2(h[t][0]), b = __half22float2(h[t][1]);
            const float dot = (a.x + a.y) + (b.x + b.y);
            acc[r][t] += sc[r][u] * dot + bi[r][u] * xsum[t][u];
          }
        }
      }
    }
    // ---- reduce over lanes, finish, store
#pragma unroll
    for (int r = 0; r < kRows; ++r)
#pragma unroll
      for (int t = 0; t < kGvTok; ++t) acc[r][t] = warp_sum(acc[r][t]);
    if (lane < kGvFeat * kGvTok) {
      const int fi = lane % kGvFeat, t = lane / kGvFeat;
      const int feat = f0 + fi;
      if (feat < p.n_out && (t0 + t) < m_e) {
        float g = 0.f, u = 0.f;
#pragma unroll
        for (int r = 0; r < kGvFeat; ++r)
#pragma unroll
          for (int tt = 0; tt < kGvTok; ++tt)
            if (r == fi && tt == t) {
              g = acc[r][tt];
              u = acc[r + kGvFeat][tt];
            }
        float v;
        if (gated) {
          if (p.lin_bias) {
            g += __bfloat162float(p.lin_bias[ebase + feat]);
            u += __bfloat162float(p.lin_bias[ebase + p.n_out + feat]);
          }
          v = gv_glu(p.epi, g, u, p.alpha, p.limit);
        } else {
          v = g + (p.lin_bias ? __bfloat162float(p.lin_bias[ebase + feat]) : 0.f);
          if (p.residual) v += __bfloat162float(p.residual[static_cast<size_t>(row0 + t0 + t) * p.ldr + feat]);
        }
        p.out[static_cast<size_t>(row0 + t0 + t) * p.ldo + feat] = __float2bfloat16(v);
      }
    }
  }
}

}  // namespace mx

// xs [rows, K] grouped by expert through `offsets`; w [E, N, K/8] MLX-packed 4-bit (N = 2 * n_out rows,
// gate then up, when `epi` is a gated activation, else N = n_out). mode: 0 affine (bf16 scales and
// biases per `group`), 1 mxfp4 (e8m0 scales per 32). `residual` (plain epilogue only) and the row
// strides `ldo` / `ldr` (0 = n_out) serve the dense use: E = 1, offsets = {0, M}. Returns -9 for shapes
// it does not cover.
extern "C" int mx_moe_qgemv(const void* xs, const void* w, const void* scales, const void* biases,
                            const void* lin_bias, const int* offsets, void* out, int E, int n_out, int K,
                            int group, int mode, int epi, float alpha, float limit, const void* residual,
                            long long ldo, long long ldr, void* stream_) {
  using namespace mx;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (E <= 0 || n_out <= 0) return 0;
  if (K % 32 || group < 32 || group % 32 || (mode != 0 && mode != 1)) return -9;
  if (mode == 0 && biases == nullptr) return -9;
  if (reinterpret_cast<uintptr_t>(xs) & 15 || reinterpret_cast<uintptr_t>(w) & 15 || (K * 2) % 16) return -9;
  const bool gated = epi >= MX_EPI_SWIGLU;
  if (!gated && epi != MX_EPI_NONE && epi != MX_EPI_BIAS) return -9;
  GvParams p;
  p.xs = static_cast<const __nv_bfloat16*>(xs);
  p.w = static_cast<const uint32_t*>(w);
  p.scales = scales;
  p.biases = static_cast<const __nv_bfloat16*>(biases);
  p.lin_bias = static_cast<const __nv_bfloat16*>(lin_bias);
  p.offsets = offsets;
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.ldo = ldo > 0 ? ldo : n_out;
  p.ldr = ldr > 0 ? ldr : n_out;
  if (gated && residual != nullptr) return -9;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.E = E, p.N = gated ? 2 * n_out : n_out, p.K = K, p.group = group, p.n_out = n_out, p.epi = epi;
  p.alpha = alpha, p.limit = limit;
  const dim3 grid((n_out + kGvWarps * kGvFeat - 1) / (kGvWarps * kGvFeat), E);
  if (grid.y > 65535) return -9;
  cudaError_t err = mode == 0 ? launch_kernel(moe_qgemv_kernel<0>, grid, dim3(kGvWarps * 32), 0, stream, p)
                              : launch_kernel(moe_qgemv_kernel<1>, grid, dim3(kGvWarps * 32), 0, stream, p);
  return static_cast<int>(err);
}
