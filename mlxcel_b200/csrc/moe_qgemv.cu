// Grouped 4-bit weight-streaming kernel for mixture-of-experts decode: few rows per expert, packed
// weights read once, arithmetic on mma.sync.
//
// At decode batch sizes an expert receives a handful of token rows (128 requests x top-4 over 128
// experts = 4 rows each), so its matrices are read for almost no arithmetic and the step is bound by
// the bytes of the packed weights. The tcgen05 GEMM with its unpack stage pays a fixed
// synchronisation cost per 64-wide k-step for 4 KB of weights and reaches a tenth of the HBM
// bandwidth there; a scalar GEMV spends its issue slots on multiply-adds. Here the multiply-adds go
// to the warp-level MMA (m16n8k16, fp16 in, fp32 out: 8 token columns for free) and the issue slots
// go to unpacking (reference: gather_qmm for SwitchGLU, src/models/switch_layers.rs:98-220;
// overlays/cuda/.../quantized/qmm/qmv.cu):
//
//   grid  = (output-feature blocks, local experts); a block whose expert got no rows returns at once,
//           so only routed experts are read.
//   warp  = one 16-row A tile: 8 features x (gate row, up row) when gated, else 16 features. Rows r
//           and r + 8 of the tile belong to the same lane quad, so a gate value and its up value
//           meet in one lane and the gated activation needs no exchange.
//   A     = weights. A lane quad reads the 16-byte pieces (32 weights) of its two rows; the byte
//           holding nibbles (2q, 2q + 1) becomes one half2: mxfp4 through the hardware
//           `cvt.rn.f16x2.e2m1x2`, affine through the 0x6400 | code trick. Eight pieces per row are
//           requested before the first one is used.
//   B     = up to 8 token rows per pass, staged per K slab in shared memory as fp16 (row stride
//           padded so that the 8 x 4 fragment reads of a warp fall into 32 banks).
//   C     = per 32-weight group a fresh fp32 accumulator, folded into the running sum with the
//           group's scale (and bias x sum(x) for affine).
//   out   = gated: act(gate + b, up + b) in bf16; plain: acc + bias (+ residual).
#include <cuda_fp16.h>

#include "api.h"
#include "common.cuh"

namespace mx {

constexpr int kGvWarps = 4;        // warps per block, one 16-row tile each
constexpr int kGvTok = 8;          // token rows per pass (the MMA's n)
constexpr int kGvSlabK = 2048;     // K values staged per slab
constexpr int kGvPad = 8;          // halfs of padding per staged row: stride = 4 words (mod 32 banks)
constexpr int kGvAhead = 8;        // 32-weight pieces per row requested together
constexpr bool kE2m1LowFirst = true;   // cvt.rn.f16x2.e2m1x2: low nibble -> low half

__device__ __forceinline__ float gv_e8m0(uint8_t s) {
  if (s == 255) return __uint_as_float(0x7fc00000u);
  if (s == 0) return __uint_as_float(0x00400000u);
  return __uint_as_float(static_cast<uint32_t>(s) << 23);
}

// Byte `q` of `w` = nibbles (2q, 2q + 1) -> half2 (value 2q in the low half).
template <int MODE>
__device__ __forceinline__ uint32_t gv_byte_to_half2(uint32_t w, int q) {
  const uint32_t b = __byte_perm(w, 0, 0x4440 | q);                // the byte, zero-extended
  if (MODE == 0) {                                                  // affine: 1024 + code, minus 1024
    uint32_t h = ((b * 4097u) & 0x000F000Fu) | 0x64006400u;         // low nibble -> bits 0..3, high -> 16..19
    const __half2 r = __hsub2(*reinterpret_cast<__half2*>(&h), __half2half2(__ushort_as_half(0x6400)));
    return *reinterpret_cast<const uint32_t*>(&r);
  }
  uint32_t d;
  asm("{ .reg .b8 t;\n cvt.u8.u32 t, %1;\n cvt.rn.f16x2.e2m1x2 %0, t;\n }" : "=r"(d) : "r"(b));
  if (!kE2m1LowFirst) d = __byte_perm(d, 0, 0x1032);
  return d;
}

__device__ __forceinline__ void gv_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
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
  __shared__ __align__(16) __half xs[kGvTok][kGvSlabK + kGvPad];
  __shared__ float xsum_s[kGvTok][kGvSlabK / 32];                 // sum of x per 32-weight piece (affine)
  const int e = blockIdx.y;
  const int row0 = p.offsets[e], m_e = p.offsets[e + 1] - row0;
  if (m_e <= 0) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int r = lane >> 2, q = lane & 3;                          // tile row (and r + 8), k quad / token pair
  const bool gated = p.epi >= MX_EPI_SWIGLU;
  const int feats = gated ? 8 : 16;                               // output features per warp
  const int f0 = (blockIdx.x * kGvWarps + warp) * feats;
  // the lane's two weight rows: tile rows r and r + 8
  const int feat_a = f0 + r, feat_b = gated ? f0 + r : f0 + r + 8;
  const bool live_a = feat_a < p.n_out, live_b = feat_b < p.n_out;
  const size_t ebase = static_cast<size_t>(e) * p.N;
  const size_t na = ebase + (live_a ? feat_a : 0), nb = ebase + (live_b ? (gated ? p.n_out + feat_b : feat_b) : 0);
  const int words_per_row = p.K >> 3, groups_per_row = p.K / p.group;
  const uint4* wa = reinterpret_cast<const uint4*>(p.w + na * words_per_row);
  const uint4* wb = reinterpret_cast<const uint4*>(p.w + nb * words_per_row);
  const size_t ga = na * groups_per_row, gb = nb * groups_per_row;

  for (int t0 = 0; t0 < m_e; t0 += kGvTok) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};                          // (row r: tokens 2q, 2q + 1), (row r + 8: same)
    for (int k0 = 0; k0 < p.K; k0 += kGvSlabK) {
      const int ks = min(kGvSlabK, p.K - k0);                     // multiple of 32
      __syncthreads();                                            // the previous slab is consumed
      for (int i = threadIdx.x; i < kGvTok * (ks >> 3); i += kGvWarps * 32) {
        const int t = i / (ks >> 3), c = i - t * (ks >> 3);       // 8 activations per item
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t0 + t < m_e)
          v = *reinterpret_cast<const uint4*>(p.xs + static_cast<size_t>(row0 + t0 + t) * p.K + k0 + c * 8);
        const __half2 h[4] = {__floats2half2_rn(bf16_lo(v.x), bf16_hi(v.x)), __floats2half2_rn(bf16_lo(v.y), bf16_hi(v.y)),
                              __floats2half2_rn(bf16_lo(v.z), bf16_hi(v.z)), __floats2half2_rn(bf16_lo(v.w), bf16_hi(v.w))};
        *reinterpret_cast<uint4*>(&xs[t][c * 8]) = *reinterpret_cast<const uint4*>(h);
      }
      if (MODE == 0) {
        __syncthreads();
        for (int i = threadIdx.x; i < kGvTok * (ks >> 5); i += kGvWarps * 32) {
          const int t = i / (ks >> 5), c = i - t * (ks >> 5);
          float s = 0.f;
#pragma unroll
          for (int j = 0; j < 32; j += 2) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&xs[t][c * 32 + j]));
            s += f.x + f.y;
          }
          xsum_s[t][c] = s;
        }
      }
      __syncthreads();
      // ---- the warp walks the slab's 32-weight pieces, kGvAhead at a time
      const int np = ks >> 5;
      for (int c0 = 0; c0 < np; c0 += kGvAhead) {
        uint4 pa[kGvAhead], pb[kGvAhead];
        float sa[kGvAhead], sb[kGvAhead], ba[kGvAhead], bb[kGvAhead];
#pragma unroll
        for (int u = 0; u < kGvAhead; ++u) {
          const int c = c0 + u;
          const int piece = (k0 >> 5) + c;
          pa[u] = pb[u] = make_uint4(0, 0, 0, 0);
          sa[u] = sb[u] = ba[u] = bb[u] = 0.f;
          if (c < np) {
            if (live_a)
              asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(pa[u].x), "=r"(pa[u].y), "=r"(pa[u].z), "=r"(pa[u].w) : "l"(wa + piece));
            if (live_b)
              asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                           : "=r"(pb[u].x), "=r"(pb[u].y), "=r"(pb[u].z), "=r"(pb[u].w) : "l"(wb + piece));
            const int g = (piece << 5) / p.group;
            if (MODE == 0) {
              sa[u] = __bfloat162float(static_cast<const __nv_bfloat16*>(p.scales)[ga + g]);
              sb[u] = __bfloat162float(static_cast<const __nv_bfloat16*>(p.scales)[gb + g]);
              ba[u] = __bfloat162float(p.biases[ga + g]);
              bb[u] = __bfloat162float(p.biases[gb + g]);
            } else {
              sa[u] = gv_e8m0(static_cast<const uint8_t*>(p.scales)[ga + g]);
              sb[u] = gv_e8m0(static_cast<const uint8_t*>(p.scales)[gb + g]);
            }
          }
        }
#pragma unroll
        for (int u = 0; u < kGvAhead; ++u) {
          const int c = c0 + u;
          if (c < np) {
            const uint32_t wa4[4] = {pa[u].x, pa[u].y, pa[u].z, pa[u].w};
            const uint32_t wb4[4] = {pb[u].x, pb[u].y, pb[u].z, pb[u].w};
            float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int s = 0; s < 2; ++s) {                         // two k16 steps per piece
              uint32_t a[4];
              a[0] = gv_byte_to_half2<MODE>(wa4[2 * s], q);        // row r,     k = 2q, 2q + 1
              a[1] = gv_byte_to_half2<MODE>(wb4[2 * s], q);        // row r + 8, k = 2q, 2q + 1
              a[2] = gv_byte_to_half2<MODE>(wa4[2 * s + 1], q);    // row r,     k = 8 + 2q, ...
              a[3] = gv_byte_to_half2<MODE>(wb4[2 * s + 1], q);    // row r + 8, k = 8 + 2q, ...
              const __half* xrow = &xs[r][c * 32 + s * 16 + 2 * q];   // token r of the pass
              const uint32_t b0 = *reinterpret_cast<const uint32_t*>(xrow);
              const uint32_t b1 = *reinterpret_cast<const uint32_t*>(xrow + 8);
              gv_mma(d, a, b0, b1);
            }
            acc[0] += sa[u] * d[0];
            acc[1] += sa[u] * d[1];
            acc[2] += sb[u] * d[2];
            acc[3] += sb[u] * d[3];
            if (MODE == 0) {
              const float x0 = xsum_s[2 * q][c], x1 = xsum_s[2 * q + 1][c];
              acc[0] += ba[u] * x0;
              acc[1] += ba[u] * x1;
              acc[2] += bb[u] * x0;
              acc[3] += bb[u] * x1;
            }
          }
        }
      }
    }
    // ---- finish and store: this lane holds tokens t0 + 2q, t0 + 2q + 1 of its two rows
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int t = t0 + 2 * q + j;
      if (t >= m_e) continue;
      const size_t orow = static_cast<size_t>(row0 + t);
      if (gated) {
        if (live_a) {
          float g = acc[j], u = acc[2 + j];
          if (p.lin_bias) {
            g += __bfloat162float(p.lin_bias[ebase + feat_a]);
            u += __bfloat162float(p.lin_bias[ebase + p.n_out + feat_a]);
          }
          p.out[orow * p.ldo + feat_a] = __float2bfloat16(gv_glu(p.epi, g, u, p.alpha, p.limit));
        }
      } else {
        if (live_a) {
          float v = acc[j] + (p.lin_bias ? __bfloat162float(p.lin_bias[ebase + feat_a]) : 0.f);
          if (p.residual) v += __bfloat162float(p.residual[orow * p.ldr + feat_a]);
          p.out[orow * p.ldo + feat_a] = __float2bfloat16(v);
        }
        if (live_b) {
          float v = acc[2 + j] + (p.lin_bias ? __bfloat162float(p.lin_bias[ebase + feat_b]) : 0.f);
          if (p.residual) v += __bfloat162float(p.residual[orow * p.ldr + feat_b]);
          p.out[orow * p.ldo + feat_b] = __float2bfloat16(v);
        }
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
  const int per_block = kGvWarps * (gated ? 8 : 16);
  const dim3 grid((n_out + per_block - 1) / per_block, E);
  if (grid.y > 65535) return -9;
  cudaError_t err = mode == 0 ? launch_kernel(moe_qgemv_kernel<0>, grid, dim3(kGvWarps * 32), 0, stream, p)
                              : launch_kernel(moe_qgemv_kernel<1>, grid, dim3(kGvWarps * 32), 0, stream, p);
  return static_cast<int>(err);
}
