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
//   warp  = 8 weight rows (8 output features, or 4 features x (gate, up) when gated). Lanes stride the
//           packed rows in 16-byte pieces (32 weights); the 8 rows' pieces are requested together.
//   x     = up to 4 token rows per pass. The block stages a K slab of them in shared memory as
//           half2, already in the order the nibble pairs come out of a word ((j, j + 4) of each
//           8-nibble word); a lane pulls its piece of all 4 tokens into registers once and uses it
//           for the 8 rows. More than 4 rows for an expert = more passes over the block's weight
//           rows (which then come from L2).
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
constexpr int kGvRows = 8;      // weight rows per warp: 8 features, or 4 features x (gate, up) when gated
constexpr int kGvTok = 4;       // token rows per pass
constexpr int kGvSlab = 128;    // 16-byte pieces (32 weights each) of K staged per slab: 4 per lane

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
  // activations of the current token pass and K slab, as half2 in nibble-pair order:
  // xs[token][quarter][piece] (16 bytes each: consecutive lanes read consecutive chunks)
  __shared__ uint4 xs[kGvTok][4][kGvSlab];
  __shared__ float xsum_s[kGvTok][kGvSlab];
  const int e = blockIdx.y;
  const int row0 = p.offsets[e], m_e = p.offsets[e + 1] - row0;
  if (m_e <= 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const bool gated = p.epi >= MX_EPI_SWIGLU;
  const int feats = gated ? kGvRows / 2 : kGvRows;               // output features per warp
  const int f0 = (blockIdx.x * kGvWarps + warp) * feats;
  const int pieces = p.K >> 5;
  const int words_per_row = p.K >> 3;
  const int groups_per_row = p.K / p.group;
  const size_t ebase = static_cast<size_t>(e) * p.N;
  // weight row of local row r: features first (gate), then their up rows
  const uint4* wrow[kGvRows];
  size_t grow[kGvRows];
  bool rlive[kGvRows];
#pragma unroll
  for (int r = 0; r < kGvRows; ++r) {
    const int feat = f0 + (gated ? (r % (kGvRows / 2)) : r);
    rlive[r] = feat < p.n_out;
    const int n = rlive[r] ? ((gated && r >= kGvRows / 2) ? p.n_out + feat : feat) : 0;
    wrow[r] = reinterpret_cast<const uint4*>(p.w + (ebase + n) * words_per_row);
    grow[r] = (ebase + n) * groups_per_row;
  }

  for (int t0 = 0; t0 < m_e; t0 += kGvTok) {
    float acc[kGvRows][kGvTok];
#pragma unroll
    for (int r = 0; r < kGvRows; ++r)
#pragma unroll
      for (int t = 0; t < kGvTok; ++t) acc[r][t] = 0.f;

    for (int s0 = 0; s0 < pieces; s0 += kGvSlab) {
      const int np = min(kGvSlab, pieces - s0);
      __syncthreads();                                            // the previous slab is consumed
      for (int i = threadIdx.x; i < kGvTok * np; i += kGvWarps * 32) {
        const int t = i / np, c = i - t * np;
        uint4 v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) v[q] = make_uint4(0, 0, 0, 0);
        if (t0 + t < m_e) {
          const uint4* src = reinterpret_cast<const uint4*>(p.xs + static_cast<size_t>(row0 + t0 + t) * p.K +
                                                            (static_cast<size_t>(s0 + c) << 5));
#pragma unroll
          for (int q = 0; q < 4; ++q) v[q] = src[q];
        }
        float sum = 0.f;
#pragma unroll
        for (int q = 0; q < 4; ++q) {                             // 8 activations <-> one weight word
          const float a[8] = {bf16_lo(v[q].x), bf16_hi(v[q].x), bf16_lo(v[q].y), bf16_hi(v[q].y),
                              bf16_lo(v[q].z), bf16_hi(v[q].z), bf16_lo(v[q].w), bf16_hi(v[q].w)};
          __half2 h[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            h[j] = __floats2half2_rn(a[j], a[j + 4]);             // nibbles (j, j + 4) of the word
            sum += a[j] + a[j + 4];
          }
          xs[t][q][c] = *reinterpret_cast<uint4*>(h);
        }
        xsum_s[t][c] = sum;
      }
      __syncthreads();
      // ---- this lane's pieces of the slab against the warp's rows
      for (int c = lane; c < np; c += 32) {
        uint4 pk[kGvRows];
        float sc[kGvRows], bi[kGvRows];
#pragma unroll
        for (int r = 0; r < kGvRows; ++r) {
          pk[r] = make_uint4(0, 0, 0, 0);
          sc[r] = bi[r] = 0.f;
          if (rlive[r]) {
            asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(pk[r].x), "=r"(pk[r].y), "=r"(pk[r].z), "=r"(pk[r].w) : "l"(wrow[r] + s0 + c));
            const size_t g = grow[r] + ((s0 + c) << 5) / p.group;
            if (MODE == 0) {
              sc[r] = __bfloat162float(static_cast<const __nv_bfloat16*>(p.scales)[g]);
              bi[r] = __bfloat162float(p.biases[g]);
            } else {
              sc[r] = gv_e8m0(static_cast<const uint8_t*>(p.scales)[g]);
            }
          }
        }
        __half2 xr[kGvTok][16];
        float xsum[kGvTok];
#pragma unroll
        for (int t = 0; t < kGvTok; ++t) {
#pragma unroll
          for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(&xr[t][q * 4]) = xs[t][q][c];
          xsum[t] = xsum_s[t][c];
        }
#pragma unroll
        for (int r = 0; r < kGvRows; ++r) {
          const uint32_t words[4] = {pk[r].x, pk[r].y, pk[r].z, pk[r].w};
          __half2 h[kGvTok][2];
#pragma unroll
          for (int t = 0; t < kGvTok; ++t) h[t][0] = h[t][1] = __floats2half2_rn(0.f, 0.f);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const __half2 wv = gv_pair<MODE>(words[q] >> (4 * j));
#pragma unroll
              for (int t = 0; t < kGvTok; ++t) h[t][q >> 1] = __hfma2(wv, xr[t][q * 4 + j], h[t][q >> 1]);
            }
          }
#pragma unroll
          for (int t = 0; t < kGvTok; ++t) {
            const float2 a = __half22float2(h[t][0]), b = __half22float2(h[t][1]);
            acc[r][t] += sc[r] * ((a.x + a.y) + (b.x + b.y)) + bi[r] * xsum[t];
          }
        }
      }
    }
    // ---- reduce over lanes, finish, store: lane (f, t) writes feature f of token t
#pragma unroll
    for (int r = 0; r < kGvRows; ++r)
#pragma unroll
      for (int t = 0; t < kGvTok; ++t) acc[r][t] = warp_sum(acc[r][t]);
    const int fi = lane % feats, t = lane / feats;
    if (t < kGvTok && f0 + fi < p.n_out && t0 + t < m_e) {
      float g = 0.f, u = 0.f;
#pragma unroll
      for (int r = 0; r < kGvRows; ++r)
#pragma unroll
        for (int tt = 0; tt < kGvTok; ++tt) {
          if (tt == t && r == fi) g = acc[r][tt];
          if (tt == t && r == fi + kGvRows / 2) u = acc[r][tt];
        }
      const int feat = f0 + fi;
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
  const int per_block = kGvWarps * (gated ? kGvRows / 2 : kGvRows);
  const dim3 grid((n_out + per_block - 1) / per_block, E);
  if (grid.y > 65535) return -9;
  cudaError_t err = mode == 0 ? launch_kernel(moe_qgemv_kernel<0>, grid, dim3(kGvWarps * 32), 0, stream, p)
                              : launch_kernel(moe_qgemv_kernel<1>, grid, dim3(kGvWarps * 32), 0, stream, p);
  return static_cast<int>(err);
}
