// Memory-bound row kernels: residual-add + RMSNorm, per-head RMSNorm, RoPE + paged KV append
// (with optional 8-bit / 4-bit affine KV quantization), embedding gather, gated activations.
//
// Parity targets in the reference: fused_add_rms_norm (src/lib/mlxcelverse/kernels/fused_norm.h:17-77),
// fused_rope_qk_append (src/lib/mlxcelverse/kernels/fused_rope_append.h:17-114) and the per-token
// int8 KV quantizer (src/lib/mlxcel-core/src/cache.rs:366-412). Unlike the reference's append
// kernel this one writes straight into the paged block pool.
#include "api.h"
#include "common.cuh"

namespace mx {

// ----------------------------------------------------------------------------- add + rmsnorm
// One CTA per row; 16-byte vector loads; values stay in registers between the two passes
// (up to 4 vectors per thread), so each row is read once and written once per output.
template <int VPT>
__global__ void add_rmsnorm_kernel(const __nv_bfloat16* __restrict__ x,
                                   const __nv_bfloat16* __restrict__ residual,
                                   const __nv_bfloat16* __restrict__ weight,
                                   __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ residual_out, int dim, float eps,
                                   float w_bias) {
  pdl_trigger();
  pdl_wait();
  const int row = blockIdx.x;
  const int nvec = dim >> 3;
  const uint4* xr = reinterpret_cast<const uint4*>(x + static_cast<size_t>(row) * dim);
  const uint4* rr =
      residual ? reinterpret_cast<const uint4*>(residual + static_cast<size_t>(row) * dim) : nullptr;
  uint4* ro = residual_out
                  ? reinterpret_cast<uint4*>(residual_out + static_cast<size_t>(row) * dim)
                  : nullptr;
  float vals[VPT][8];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      uint4 a = xr[v];
      const uint32_t aw[4] = {a.x, a.y, a.z, a.w};
      float f[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        f[2 * j] = bf16_lo(aw[j]);
        f[2 * j + 1] = bf16_hi(aw[j]);
      }
      if (rr) {
        uint4 b = rr[v];
        const uint32_t bw[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          f[2 * j] += bf16_lo(bw[j]);
          f[2 * j + 1] += bf16_hi(bw[j]);
        }
      }
      if (ro) {
        // The residual stream is kept in bf16; the norm sees the rounded value so that the
        // fused and the unfused paths agree bit for bit.
        uint4 o;
        o.x = pack_bf16(f[0], f[1]);
        o.y = pack_bf16(f[2], f[3]);
        o.z = pack_bf16(f[4], f[5]);
        o.w = pack_bf16(f[6], f[7]);
        ro[v] = o;
        const uint32_t ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          f[2 * j] = bf16_lo(ow[j]);
          f[2 * j + 1] = bf16_hi(ow[j]);
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        vals[i][j] = f[j];
        ss += f[j] * f[j];
      }
    }
  }
  __shared__ float red[32];
  ss = warp_sum(ss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) red[0] = t;
  }
  __syncthreads();
  const float rstd = rsqrtf(red[0] / static_cast<float>(dim) + eps);
  uint4* yr = reinterpret_cast<uint4*>(y + static_cast<size_t>(row) * dim);
  const uint4* wr = reinterpret_cast<const uint4*>(weight);
#pragma unroll
  for (int i = 0; i < VPT; ++i) {
    const int v = threadIdx.x + i * blockDim.x;
    if (v < nvec) {
      uint4 wv = wr[v];
      const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
      float o[8];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        o[2 * j] = vals[i][2 * j] * rstd * (bf16_lo(ww[j]) + w_bias);
        o[2 * j + 1] = vals[i][2 * j + 1] * rstd * (bf16_hi(ww[j]) + w_bias);
      }
      uint4 ov;
      ov.x = pack_bf16(o[0], o[1]);
      ov.y = pack_bf16(o[2], o[3]);
      ov.z = pack_bf16(o[4], o[5]);
      ov.w = pack_bf16(o[6], o[7]);
      yr[v] = ov;
    }
  }
}

// ----------------------------------------------------------------------------- head rmsnorm
// One warp per (token, head).
__global__ void head_rmsnorm_kernel(__nv_bfloat16* __restrict__ x,
                                    const __nv_bfloat16* __restrict__ weight, int tokens, int heads,
                                    int head_dim, long long token_stride, float eps) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= tokens * heads) return;
  const int t = gw / heads, h = gw - t * heads;
  __nv_bfloat16* p = x + static_cast<size_t>(t) * token_stride + static_cast<size_t>(h) * head_dim;
  float ss = 0.f;
  for (int i = lane; i < head_dim; i += 32) {
    float v = __bfloat162float(p[i]);
    ss += v * v;
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / head_dim + eps);
  for (int i = lane; i < head_dim; i += 32)
    p[i] = __float2bfloat16(__bfloat162float(p[i]) * rstd * __bfloat162float(weight[i]));
}

// ----------------------------------------------------------------------------- rope + append
// One warp per (token, head slot); slots are [0,Hq) q heads, [Hq,Hq+Hkv) k heads, then v heads.
// The head's D values are staged in shared memory as fp32 so that any rotary pairing
// (half-split or interleaved, partial rotary) is a plain indexed read.
constexpr int kRopeWarps = 4;
constexpr int kMaxHeadDim = 256;

template <int KV_BITS>
__global__ void rope_append_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                                   const int* __restrict__ slot_mapping,
                                   const float* __restrict__ inv_freq, void* __restrict__ k_pool,
                                   void* __restrict__ v_pool, __nv_bfloat16* __restrict__ k_meta,
                                   __nv_bfloat16* __restrict__ v_meta,
                                   const __nv_bfloat16* __restrict__ q_norm_w,
                                   const __nv_bfloat16* __restrict__ k_norm_w, float norm_eps, int T,
                                   int Hq, int Hkv, int D, int rot_dim, int block_size,
                                   int rope_mode, float mscale, int heads_per_warp) {
  __shared__ float stage[kRopeWarps][kMaxHeadDim];
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = Hq + 2 * Hkv;
  // A warp owns (token, chunk of `heads_per_warp` head slots): the rotation angles depend on the
  // token only, so sin / cos are evaluated once per warp and reused for every head of the chunk.
  const int chunks = (slots + heads_per_warp - 1) / heads_per_warp;
  const long long gw = static_cast<long long>(blockIdx.x) * kRopeWarps + warp;
  if (gw >= static_cast<long long>(T) * chunks) return;
  const int t = static_cast<int>(gw / chunks);
  const int s_begin = static_cast<int>(gw - static_cast<long long>(t) * chunks) * heads_per_warp;
  const int s_end = min(slots, s_begin + heads_per_warp);
  float* st = stage[warp];
  const int slot = slot_mapping[t];
  const int half = rot_dim >> 1;
  float sn[kMaxHeadDim / 64], cs[kMaxHeadDim / 64];
  if (s_begin < Hq + Hkv) {
    const float pos = static_cast<float>(positions[t]);
    int n = 0;
    for (int p = lane; p < half; p += 32, ++n) sincosf(pos * inv_freq[p], &sn[n], &cs[n]);
  }
  for (int s = s_begin; s < s_end; ++s) {
    const bool is_q = s < Hq;
    const bool is_k = !is_q && s < Hq + Hkv;
    const int kvh = is_q ? 0 : (is_k ? s - Hq : s - Hq - Hkv);
    __nv_bfloat16* src = qkv + static_cast<size_t>(t) * slots * D + static_cast<size_t>(s) * D;
    if (!is_q && slot < 0) continue;  // padded token: nothing to append
    __syncwarp();

    float ss = 0.f;
    for (int i = lane; i < D; i += 32) {
      float v = __bfloat162float(src[i]);
      st[i] = v;
      ss += v * v;
    }
    const __nv_bfloat16* nw = is_q ? q_norm_w : (is_k ? k_norm_w : nullptr);
    if (nw != nullptr) {
      ss = warp_sum(ss);
      const float rstd = rsqrtf(ss / D + norm_eps);
      __syncwarp();
      for (int i = lane; i < D; i += 32) {
        // Round through bf16 like an unfused norm would, then rotate in fp32.
        st[i] = __bfloat162float(__float2bfloat16(st[i] * rstd * __bfloat162float(nw[i])));
      }
    }
    __syncwarp();

    if (is_q || is_k) {
      // Each lane rotates pairs p = lane, lane + 32, ...; results go back to the stage.
      float r1[kMaxHeadDim / 64], r2[kMaxHeadDim / 64];
      int n = 0;
      for (int p = lane; p < half; p += 32, ++n) {
        const int i1 = rope_mode == 0 ? p : 2 * p;
        const int i2 = rope_mode == 0 ? p + half : 2 * p + 1;
        const float a = st[i1], b = st[i2];
        r1[n] = (a * cs[n] - b * sn[n]) * mscale;
        r2[n] = (b * cs[n] + a * sn[n]) * mscale;
      }
      __syncwarp();
      n = 0;
      for (int p = lane; p < half; p += 32, ++n) {
        const int i1 = rope_mode == 0 ? p : 2 * p;
        const int i2 = rope_mode == 0 ? p + half : 2 * p + 1;
        st[i1] = r1[n];
        st[i2] = r2[n];
      }
      if (mscale != 1.0f) {
        for (int i = rot_dim + lane; i < D; i += 32) st[i] *= mscale;
      }
      __syncwarp();
    }

    if (is_q) {
      for (int i = lane; i < D; i += 32) src[i] = __float2bfloat16(st[i]);
      continue;
    }

    const int blk = slot / block_size, off = slot - blk * block_size;
    const size_t row = (static_cast<size_t>(blk) * Hkv + kvh) * block_size + off;
    if (KV_BITS == 16) {
      __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(is_k ? k_pool : v_pool) + row * D;
      for (int i = lane; i < D; i += 32) dst[i] = __float2bfloat16(st[i]);
    } else if (KV_BITS == 4) {
      // 4-bit affine, groups of 64 along D: q = round((x - min) / scale), scale = (max - min) / 15;
      // element i of a row lives in byte i / 2 (even elements in the low nibble), D / 2 bytes per row.
      uint8_t* dst = reinterpret_cast<uint8_t*>(is_k ? k_pool : v_pool) + row * (D / 2);
      __nv_bfloat16* meta = (is_k ? k_meta : v_meta) + row * (D / 64) * 2;
      for (int g = 0; g < D / 64; ++g) {
        const float a = st[g * 64 + lane], b = st[g * 64 + 32 + lane];
        float mn = fminf(a, b), mxv = fmaxf(a, b);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
          mxv = fmaxf(mxv, __shfl_xor_sync(0xffffffffu, mxv, o));
        }
        float scale = __bfloat162float(__float2bfloat16((mxv - mn) / 15.0f));
        const float bias = __bfloat162float(__float2bfloat16(mn));
        if (scale == 0.f) scale = 1.0f;
        const float inv = 1.0f / scale;
        const int qa = min(15, max(0, __float2int_rn((a - bias) * inv)));
        const int qb = min(15, max(0, __float2int_rn((b - bias) * inv)));
        // neighbouring lanes share a byte: the even lane stores (own | odd neighbour << 4)
        const int qa_hi = __shfl_down_sync(0xffffffffu, qa, 1);
        const int qb_hi = __shfl_down_sync(0xffffffffu, qb, 1);
        if ((lane & 1) == 0) {
          dst[g * 32 + (lane >> 1)] = static_cast<uint8_t>(qa | (qa_hi << 4));
          dst[g * 32 + 16 + (lane >> 1)] = static_cast<uint8_t>(qb | (qb_hi << 4));
        }
        if (lane == 0) {
          meta[g * 2] = __float2bfloat16(scale);
          meta[g * 2 + 1] = __float2bfloat16(bias);
        }
      }
    } else {
      // 8-bit affine, groups of 64 along D: q = round((x - min) / scale), scale = (max - min) / 255.
      uint8_t* dst = reinterpret_cast<uint8_t*>(is_k ? k_pool : v_pool) + row * D;
      __nv_bfloat16* meta = (is_k ? k_meta : v_meta) + row * (D / 64) * 2;
      for (int g = 0; g < D / 64; ++g) {
        const float a = st[g * 64 + lane], b = st[g * 64 + 32 + lane];
        float mn = fminf(a, b), mxv = fmaxf(a, b);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
          mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
          mxv = fmaxf(mxv, __shfl_xor_sync(0xffffffffu, mxv, o));
        }
        // Scale and bias are stored in bf16; quantize against the rounded values so that
        // dequantization reproduces what the quantizer saw.
        float scale = __bfloat162float(__float2bfloat16((mxv - mn) / 255.0f));
        const float bias = __bfloat162float(__float2bfloat16(mn));
        if (scale == 0.f) scale = 1.0f;
        const float inv = 1.0f / scale;
        const int qa = min(255, max(0, __float2int_rn((a - bias) * inv)));
        const int qb = min(255, max(0, __float2int_rn((b - bias) * inv)));
        dst[g * 64 + lane] = static_cast<uint8_t>(qa);
        dst[g * 64 + 32 + lane] = static_cast<uint8_t>(qb);
        if (lane == 0) {
          meta[g * 2] = __float2bfloat16(scale);
          meta[g * 2 + 1] = __float2bfloat16(bias);
        }
      }
    }
  }
}

// Fast path of rope_append: half-split rotation over the whole head (rot_dim == D), bf16 pool,
// D = 64 or 128. A warp owns (token, chunk of head slots); each lane holds D/32 elements of a
// head in registers (the pair halves p and p + D/2 sit in the same lane), four heads are loaded
// before any is stored so the loads overlap, and sin / cos are evaluated once per warp.
template <int D, bool NORM>
__global__ void rope_append_fast_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                                        const int* __restrict__ slot_mapping,
                                        const float* __restrict__ inv_freq, __nv_bfloat16* __restrict__ k_pool,
                                        __nv_bfloat16* __restrict__ v_pool,
                                        const __nv_bfloat16* __restrict__ q_norm_w,
                                        const __nv_bfloat16* __restrict__ k_norm_w, float norm_eps, int T,
                                        int Hq, int Hkv, int block_size, float mscale, int heads_per_warp) {
  constexpr int E = D / 64;          // elements per lane in each half (1 or 2)
  constexpr int HALF = D / 2;
  constexpr int HB = 4;              // heads in flight
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slots = Hq + 2 * Hkv;
  const int chunks = (slots + heads_per_warp - 1) / heads_per_warp;
  const long long gw = static_cast<long long>(blockIdx.x) * kRopeWarps + warp;
  if (gw >= static_cast<long long>(T) * chunks) return;
  const int t = static_cast<int>(gw / chunks);
  const int s_begin = static_cast<int>(gw - static_cast<long long>(t) * chunks) * heads_per_warp;
  const int s_end = min(slots, s_begin + heads_per_warp);
  const int slot = slot_mapping[t];
  float sn[E], cs[E];
  if (s_begin < Hq + Hkv) {
    const float pos = static_cast<float>(positions[t]);
#pragma unroll
    for (int e = 0; e < E; ++e) sincosf(pos * inv_freq[lane * E + e], &sn[e], &cs[e]);
  }
  [[maybe_unused]] float qw[2][E], kw[2][E];   // norm weights of this lane's elements
  if (NORM) {
#pragma unroll
    for (int e = 0; e < E; ++e) {
      qw[0][e] = q_norm_w ? __bfloat162float(q_norm_w[lane * E + e]) : 1.f;
      qw[1][e] = q_norm_w ? __bfloat162float(q_norm_w[HALF + lane * E + e]) : 1.f;
      kw[0][e] = k_norm_w ? __bfloat162float(k_norm_w[lane * E + e]) : 1.f;
      kw[1][e] = k_norm_w ? __bfloat162float(k_norm_w[HALF + lane * E + e]) : 1.f;
    }
  }
  __nv_bfloat16* row = qkv + static_cast<size_t>(t) * slots * D;
  const int blk = slot >= 0 ? slot / block_size : 0;
  const int off = slot >= 0 ? slot - blk * block_size : 0;
  for (int s0 = s_begin; s0 < s_end; s0 += HB) {
    float a[HB][E], b[HB][E];
#pragma unroll
    for (int i = 0; i < HB; ++i) {
      const int s = s0 + i;
      if (s < s_end) {
        const __nv_bfloat16* src = row + static_cast<size_t>(s) * D + lane * E;
        if constexpr (E == 2) {
          const uint32_t lo = *reinterpret_cast<const uint32_t*>(src);
          const uint32_t hi = *reinterpret_cast<const uint32_t*>(src + HALF);
          a[i][0] = bf16_lo(lo), a[i][1] = bf16_hi(lo);
          b[i][0] = bf16_lo(hi), b[i][1] = bf16_hi(hi);
        } else {
          a[i][0] = __bfloat162float(src[0]);
          b[i][0] = __bfloat162float(src[HALF]);
        }
      }
    }
#pragma unroll
    for (int i = 0; i < HB; ++i) {
      const int s = s0 + i;
      if (s >= s_end) break;
      const bool is_q = s < Hq;
      const bool is_k = !is_q && s < Hq + Hkv;
      if (!is_q && slot < 0) continue;   // padded token: nothing to append
      if (NORM && (is_q ? q_norm_w != nullptr : (is_k && k_norm_w != nullptr))) {
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < E; ++e) ss += a[i][e] * a[i][e] + b[i][e] * b[i][e];
        ss = warp_sum(ss);
        const float rstd = rsqrtf(ss / D + norm_eps);
#pragma unroll
        for (int e = 0; e < E; ++e) {
          // round through bf16 like an unfused norm would, then rotate in fp32
          a[i][e] = __bfloat162float(__float2bfloat16(a[i][e] * rstd * (is_q ? qw[0][e] : kw[0][e])));
          b[i][e] = __bfloat162float(__float2bfloat16(b[i][e] * rstd * (is_q ? qw[1][e] : kw[1][e])));
        }
      }
      float r1[E], r2[E];
#pragma unroll
      for (int e = 0; e < E; ++e) {
        if (is_q || is_k) {
          r1[e] = (a[i][e] * cs[e] - b[i][e] * sn[e]) * mscale;
          r2[e] = (b[i][e] * cs[e] + a[i][e] * sn[e]) * mscale;
        } else {
          r1[e] = a[i][e];
          r2[e] = b[i][e];
        }
      }
      __nv_bfloat16* dst;
      if (is_q) {
        dst = row + static_cast<size_t>(s) * D;
      } else {
        const int kvh = is_k ? s - Hq : s - Hq - Hkv;
        dst = (is_k ? k_pool : v_pool) + ((static_cast<size_t>(blk) * Hkv + kvh) * block_size + off) * D;
      }
      dst += lane * E;
      if constexpr (E == 2) {
        *reinterpret_cast<uint32_t*>(dst) = pack_bf16(r1[0], r1[1]);
        *reinterpret_cast<uint32_t*>(dst + HALF) = pack_bf16(r2[0], r2[1]);
      } else {
        dst[0] = __float2bfloat16(r1[0]);
        dst[HALF] = __float2bfloat16(r2[0]);
      }
    }
  }
}

// The same fast path with 8-byte accesses: a lane holds four adjacent elements of each half of a head,
// so a head takes D / 8 lanes (8 for D = 64, 16 for D = 128) and a warp works on 32 / (D / 8) heads
// at once, two such groups in flight. With 2-byte accesses (D = 64 in the kernel above) an
// 8192-token prefill step of a 64 + 2 x 8 head model took ~450 us for 170 MB of traffic.
template <int D, bool NORM>
__global__ void rope_append_vec_kernel(__nv_bfloat16* __restrict__ qkv, const int* __restrict__ positions,
                                       const int* __restrict__ slot_mapping,
                                       const float* __restrict__ inv_freq, __nv_bfloat16* __restrict__ k_pool,
                                       __nv_bfloat16* __restrict__ v_pool,
                                       const __nv_bfloat16* __restrict__ q_norm_w,
                                       const __nv_bfloat16* __restrict__ k_norm_w, float norm_eps, int T,
                                       int Hq, int Hkv, int block_size, float mscale, int heads_per_warp) {
  constexpr int HALF = D / 2;
  constexpr int V = 4;               // elements per lane in each half
  constexpr int LPH = HALF / V;      // lanes per head
  constexpr int HPI = 32 / LPH;      // heads per warp iteration
  constexpr int IT = 2;              // iterations in flight
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int sub = lane / LPH, j = lane - sub * LPH;
  const int slots = Hq + 2 * Hkv;
  const int chunks = (slots + heads_per_warp - 1) / heads_per_warp;
  const long long gw = static_cast<long long>(blockIdx.x) * kRopeWarps + warp;
  if (gw >= static_cast<long long>(T) * chunks) return;
  const int t = static_cast<int>(gw / chunks);
  const int s_begin = static_cast<int>(gw - static_cast<long long>(t) * chunks) * heads_per_warp;
  const int s_end = min(slots, s_begin + heads_per_warp);
  const int slot = slot_mapping[t];
  float sn[V], cs[V];
  if (s_begin < Hq + Hkv) {
    const float pos = static_cast<float>(positions[t]);
#pragma unroll
    for (int e = 0; e < V; ++e) sincosf(pos * inv_freq[j * V + e], &sn[e], &cs[e]);
  }
  [[maybe_unused]] float qw[2][V], kw[2][V];
  if (NORM) {
#pragma unroll
    for (int e = 0; e < V; ++e) {
      qw[0][e] = q_norm_w ? __bfloat162float(q_norm_w[j * V + e]) : 1.f;
      qw[1][e] = q_norm_w ? __bfloat162float(q_norm_w[HALF + j * V + e]) : 1.f;
      kw[0][e] = k_norm_w ? __bfloat162float(k_norm_w[j * V + e]) : 1.f;
      kw[1][e] = k_norm_w ? __bfloat162float(k_norm_w[HALF + j * V + e]) : 1.f;
    }
  }
  __nv_bfloat16* row = qkv + static_cast<size_t>(t) * slots * D;
  const int blk = slot >= 0 ? slot / block_size : 0;
  const int off = slot >= 0 ? slot - blk * block_size : 0;
  for (int s0 = s_begin; s0 < s_end; s0 += HPI * IT) {
    float a[IT][V], b[IT][V];
#pragma unroll
    for (int i = 0; i < IT; ++i) {
      const int s = s0 + i * HPI + sub;
      uint2 lo = make_uint2(0u, 0u), hi = make_uint2(0u, 0u);
      if (s < s_end) {
        const __nv_bfloat16* src = row + static_cast<size_t>(s) * D + j * V;
        lo = *reinterpret_cast<const uint2*>(src);
        hi = *reinterpret_cast<const uint2*>(src + HALF);
      }
      a[i][0] = bf16_lo(lo.x), a[i][1] = bf16_hi(lo.x), a[i][2] = bf16_lo(lo.y), a[i][3] = bf16_hi(lo.y);
      b[i][0] = bf16_lo(hi.x), b[i][1] = bf16_hi(hi.x), b[i][2] = bf16_lo(hi.y), b[i][3] = bf16_hi(hi.y);
    }
#pragma unroll
    for (int i = 0; i < IT; ++i) {
      const int s = s0 + i * HPI + sub;
      const bool live = s < s_end;
      const bool is_q = s < Hq;
      const bool is_k = !is_q && s < Hq + Hkv;
      if (NORM) {
        // every lane takes part in the shuffles (the heads of a warp differ per lane group)
        float ss = 0.f;
#pragma unroll
        for (int e = 0; e < V; ++e) ss += a[i][e] * a[i][e] + b[i][e] * b[i][e];
#pragma unroll
        for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        if (live && (is_q ? q_norm_w != nullptr : (is_k && k_norm_w != nullptr))) {
          const float rstd = rsqrtf(ss / D + norm_eps);
#pragma unroll
          for (int e = 0; e < V; ++e) {
            a[i][e] = __bfloat162float(__float2bfloat16(a[i][e] * rstd * (is_q ? qw[0][e] : kw[0][e])));
            b[i][e] = __bfloat162float(__float2bfloat16(b[i][e] * rstd * (is_q ? qw[1][e] : kw[1][e])));
          }
        }
      }
      if (!live || (!is_q && slot < 0)) continue;      // padded token: nothing to append
      float r1[V], r2[V];
#pragma unroll
      for (int e = 0; e < V; ++e) {
        if (is_q || is_k) {
          r1[e] = (a[i][e] * cs[e] - b[i][e] * sn[e]) * mscale;
          r2[e] = (b[i][e] * cs[e] + a[i][e] * sn[e]) * mscale;
        } else {
          r1[e] = a[i][e];
          r2[e] = b[i][e];
        }
      }
      __nv_bfloat16* dst;
      if (is_q) {
        dst = row + static_cast<size_t>(s) * D;
      } else {
        const int kvh = is_k ? s - Hq : s - Hq - Hkv;
        dst = (is_k ? k_pool : v_pool) + ((static_cast<size_t>(blk) * Hkv + kvh) * block_size + off) * D;
      }
      dst += j * V;
      *reinterpret_cast<uint2*>(dst) = make_uint2(pack_bf16(r1[0], r1[1]), pack_bf16(r1[2], r1[3]));
      *reinterpret_cast<uint2*>(dst + HALF) = make_uint2(pack_bf16(r2[0], r2[1]), pack_bf16(r2[2], r2[3]));
    }
  }
}

// ----------------------------------------------------------------------------- row sum of squares
// One warp per row: ssq[8 + row] = sum of x[row, :]^2, partial count (word 0) = 1. Starts a chain
// of deferred RMSNorms when the residual stream does not come out of a GEMM epilogue (embedding
// output, an NCCL all-reduce).
__global__ void row_ssq_kernel(const __nv_bfloat16* __restrict__ x, int rows, int dim, long long ldx,
                               float* __restrict__ ssq) {
  pdl_trigger();
  pdl_wait();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + warp;
  if (blockIdx.x == 0 && threadIdx.x == 0) reinterpret_cast<int*>(ssq)[0] = 1;
  if (row >= rows) return;
  const __nv_bfloat16* src = x + static_cast<size_t>(row) * ldx;
  float ss = 0.f;
  for (int i = lane * 8; i < dim; i += 32 * 8) {
    const uint4 a = *reinterpret_cast<const uint4*>(src + i);
    const uint32_t w4[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float lo = bf16_lo(w4[j]), hi = bf16_hi(w4[j]);
      ss += lo * lo + hi * hi;
    }
  }
  ss = warp_sum(ss);
  if (lane == 0) ssq[8 + row] = ss;
}

extern "C" int mx_row_ssq(const void* x, int rows, int dim, long long ldx, void* ssq, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rows <= 0) return 0;
  if (dim % 8 || ldx % 8 || (reinterpret_cast<uintptr_t>(x) & 15)) return -1;
  const int wpb = 4;
  launch_kernel(row_ssq_kernel, dim3((rows + wpb - 1) / wpb), dim3(wpb * 32), 0, stream,
                static_cast<const __nv_bfloat16*>(x), rows, dim, ldx, static_cast<float*>(ssq));
  return static_cast<int>(cudaGetLastError());
}

// ----------------------------------------------------------------------------- embedding
__global__ void embedding_kernel(const int* __restrict__ ids, const __nv_bfloat16* __restrict__ table,
                                 __nv_bfloat16* __restrict__ out, int dim, int vocab, float scale) {
  pdl_trigger();
  pdl_wait();
  const int t = blockIdx.x;
  const int id = ids[t];
  const int nvec = dim >> 3;
  uint4* o = reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * dim);
  if (id < 0 || id >= vocab) {
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) o[v] = make_uint4(0, 0, 0, 0);
    return;
  }
  const uint4* src = reinterpret_cast<const uint4*>(table + static_cast<size_t>(id) * dim);
  for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
    uint4 a = src[v];
    if (scale != 1.0f) {
      uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = pack_bf16(bf16_lo(w[j]) * scale, bf16_hi(w[j]) * scale);
      a = make_uint4(w[0], w[1], w[2], w[3]);
    }
    o[v] = a;
  }
}

// ----------------------------------------------------------------------------- gated act
__global__ void swiglu_kernel(const __nv_bfloat16* __restrict__ gate_up,
                              __nv_bfloat16* __restrict__ out, long long total, int I, int mode,
                              float alpha, float limit) {
  const long long idx = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (idx >= total) return;
  const long long t = idx / I;
  const int i = static_cast<int>(idx - t * I);
  float g = __bfloat162float(gate_up[t * 2 * I + i]);
  float u = __bfloat162float(gate_up[t * 2 * I + I + i]);
  float r;
  if (mode == 0) {
    r = g / (1.0f + __expf(-g)) * u;
  } else if (mode == 1) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    r = 0.5f * g * (1.0f + tanhf(k0 * (g + k1 * g * g * g))) * u;
  } else {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    r = g / (1.0f + __expf(-alpha * g)) * (u + 1.0f);
  }
  out[idx] = __float2bfloat16(r);
}

}  // namespace mx

using namespace mx;

// Switch for the 8-byte-access rope + append kernel (on unless MLXCEL_B200_ROPE_VEC=0 at load).
static int g_rope_vec = 1;
extern "C" void mx_set_rope_vec(int on) { g_rope_vec = on ? 1 : 0; }

extern "C" int mx_add_rmsnorm(const void* x, const void* residual, const void* weight, void* y,
                              void* residual_out, int rows, int dim, float eps, float w_bias,
                              void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (rows <= 0) return 0;
  if (dim % 8 != 0 || dim > 32768) return -1;
  const int nvec = dim / 8;
  int threads = ((nvec + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  const int vpt = (nvec + threads - 1) / threads;
  auto X = static_cast<const __nv_bfloat16*>(x);
  auto R = static_cast<const __nv_bfloat16*>(residual);
  auto W = static_cast<const __nv_bfloat16*>(weight);
  auto Y = static_cast<__nv_bfloat16*>(y);
  auto RO = static_cast<__nv_bfloat16*>(residual_out);
  MX_PREFER_SHARED(add_rmsnorm_kernel<1>);
  MX_PREFER_SHARED(add_rmsnorm_kernel<2>);
  MX_PREFER_SHARED(add_rmsnorm_kernel<4>);
  if (vpt <= 1)
    launch_kernel(add_rmsnorm_kernel<1>, dim3(rows), dim3(threads), 0, stream, X, R, W, Y, RO, dim, eps, w_bias);
  else if (vpt <= 2)
    launch_kernel(add_rmsnorm_kernel<2>, dim3(rows), dim3(threads), 0, stream, X, R, W, Y, RO, dim, eps, w_bias);
  else
    launch_kernel(add_rmsnorm_kernel<4>, dim3(rows), dim3(threads), 0, stream, X, R, W, Y, RO, dim, eps, w_bias);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mx_head_rmsnorm(void* x, const void* weight, int tokens, int heads, int head_dim,
                               long long token_stride, float eps, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long warps = static_cast<long long>(tokens) * heads;
  if (warps <= 0) return 0;
  const int threads = 128;
  const int blocks = static_cast<int>((warps * 32 + threads - 1) / threads);
  head_rmsnorm_kernel<<<blocks, threads, 0, stream>>>(static_cast<__nv_bfloat16*>(x),
                                                      static_cast<const __nv_bfloat16*>(weight),
                                                      tokens, heads, head_dim, token_stride, eps);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mx_rope_append(void* qkv, const int* positions, const int* slot_mapping,
                              const float* inv_freq, void* k_pool, void* v_pool, void* k_meta,
                              void* v_meta, const void* q_norm_w, const void* k_norm_w,
                              float norm_eps, int T, int Hq, int Hkv, int D, int rot_dim,
                              int block_size, int rope_mode, float mscale, int kv_bits,
                              void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (T <= 0) return 0;
  if (D > kMaxHeadDim || D % 2 || rot_dim > D || rot_dim % 2) return -1;
  if ((kv_bits == 8 || kv_bits == 4) && D % 64) return -1;
  if (kv_bits != 16 && kv_bits != 8 && kv_bits != 4) return -1;
  // Few tokens (decode): few heads per warp for parallelism; many tokens (prefill): all heads of a
  // token in one warp so the sin / cos evaluation is shared 40-fold.
  const int slots = Hq + 2 * Hkv;
  int hpw = 1;
  while (hpw < slots && static_cast<long long>(T) * ((slots + hpw - 1) / hpw) > 4096) hpw *= 2;
  if (hpw > slots) hpw = slots;
  const long long warps = static_cast<long long>(T) * ((slots + hpw - 1) / hpw);
  const int blocks = static_cast<int>((warps + kRopeWarps - 1) / kRopeWarps);
  if (kv_bits == 16 && rope_mode == 0 && rot_dim == D && (D == 64 || D == 128)) {
    // register-resident fast path: up to 8 heads per warp (sin / cos shared, 4 heads in flight)
    int h2 = 1;
    while (h2 < 8 && static_cast<long long>(T) * ((slots + h2 - 1) / h2) > 65536) h2 *= 2;
    const long long w2 = static_cast<long long>(T) * ((slots + h2 - 1) / h2);
    const int b2 = static_cast<int>((w2 + kRopeWarps - 1) / kRopeWarps);
    auto Qf = static_cast<__nv_bfloat16*>(qkv);
    auto KP = static_cast<__nv_bfloat16*>(k_pool);
    auto VP = static_cast<__nv_bfloat16*>(v_pool);
    auto QNf = static_cast<const __nv_bfloat16*>(q_norm_w);
    auto KNf = static_cast<const __nv_bfloat16*>(k_norm_w);
    const bool norm = q_norm_w != nullptr || k_norm_w != nullptr;
    const bool aligned8 = ((reinterpret_cast<uintptr_t>(qkv) | reinterpret_cast<uintptr_t>(k_pool) |
                            reinterpret_cast<uintptr_t>(v_pool)) & 7u) == 0;
    if (g_rope_vec && aligned8) {
      // 8-byte accesses: a warp iteration covers 32 / (D / 8) heads, so that is the least a warp owns
      int hv = 32 / (D / 8);
      while (hv < 8 && static_cast<long long>(T) * ((slots + hv - 1) / hv) > 65536) hv *= 2;
      const long long wv = static_cast<long long>(T) * ((slots + hv - 1) / hv);
      const int bv = static_cast<int>((wv + kRopeWarps - 1) / kRopeWarps);
#define MX_ROPE_VEC(D_, N_)                                                                              \
      launch_kernel(rope_append_vec_kernel<D_, N_>, dim3(bv), dim3(kRopeWarps * 32), 0, stream, Qf, positions, \
                    slot_mapping, inv_freq, KP, VP, QNf, KNf, norm_eps, T, Hq, Hkv, block_size, mscale, hv)
      if (D == 128) {
        if (norm) MX_ROPE_VEC(128, true);
        else MX_ROPE_VEC(128, false);
      } else {
        if (norm) MX_ROPE_VEC(64, true);
        else MX_ROPE_VEC(64, false);
      }
#undef MX_ROPE_VEC
      return static_cast<int>(cudaGetLastError());
    }
#define MX_ROPE_FAST(D_, N_)                                                                              \
    launch_kernel(rope_append_fast_kernel<D_, N_>, dim3(b2), dim3(kRopeWarps * 32), 0, stream, Qf, positions, \
                  slot_mapping, inv_freq, KP, VP, QNf, KNf, norm_eps, T, Hq, Hkv, block_size, mscale, h2)
    if (D == 128) {
      if (norm) MX_ROPE_FAST(128, true);
      else MX_ROPE_FAST(128, false);
    } else {
      if (norm) MX_ROPE_FAST(64, true);
      else MX_ROPE_FAST(64, false);
    }
#undef MX_ROPE_FAST
    return static_cast<int>(cudaGetLastError());
  }
  auto Q = static_cast<__nv_bfloat16*>(qkv);
  auto KM = static_cast<__nv_bfloat16*>(k_meta);
  auto VM = static_cast<__nv_bfloat16*>(v_meta);
  auto QN = static_cast<const __nv_bfloat16*>(q_norm_w);
  auto KN = static_cast<const __nv_bfloat16*>(k_norm_w);
  MX_PREFER_SHARED(rope_append_kernel<16>);
  MX_PREFER_SHARED(rope_append_kernel<8>);
  MX_PREFER_SHARED(rope_append_kernel<4>);
  if (kv_bits == 4)
    launch_kernel(rope_append_kernel<4>, dim3(blocks), dim3(kRopeWarps * 32), 0, stream, Q, positions,
                  slot_mapping, inv_freq, k_pool, v_pool, KM, VM, QN, KN, norm_eps, T, Hq, Hkv, D, rot_dim,
                  block_size, rope_mode, mscale, hpw);
  else if (kv_bits == 16)
    launch_kernel(rope_append_kernel<16>, dim3(blocks), dim3(kRopeWarps * 32), 0, stream, Q, positions,
                  slot_mapping, inv_freq, k_pool, v_pool, KM, VM, QN, KN, norm_eps, T, Hq, Hkv, D, rot_dim,
                  block_size, rope_mode, mscale, hpw);
  else
    launch_kernel(rope_append_kernel<8>, dim3(blocks), dim3(kRopeWarps * 32), 0, stream, Q, positions,
                  slot_mapping, inv_freq, k_pool, v_pool, KM, VM, QN, KN, norm_eps, T, Hq, Hkv, D, rot_dim,
                  block_size, rope_mode, mscale, hpw);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mx_embedding(const int* ids, const void* table, void* out, int T, int dim, int vocab,
                            float scale, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (T <= 0) return 0;
  if (dim % 8) return -1;
  int threads = dim / 8;
  if (threads > 256) threads = 256;
  if (threads < 32) threads = 32;
  MX_PREFER_SHARED(embedding_kernel);
  launch_kernel(embedding_kernel, dim3(T), dim3(threads), 0, stream, ids,
                static_cast<const __nv_bfloat16*>(table), static_cast<__nv_bfloat16*>(out), dim, vocab, scale);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mx_swiglu(const void* gate_up, void* out, int T, int I, int mode, float alpha,
                         float limit, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const long long total = static_cast<long long>(T) * I;
  if (total <= 0) return 0;
  const int threads = 256;
  const int blocks = static_cast<int>((total + threads - 1) / threads);
  swiglu_kernel<<<blocks, threads, 0, stream>>>(static_cast<const __nv_bfloat16*>(gate_up),
                                                static_cast<__nv_bfloat16*>(out), total, I, mode,
                                                alpha, limit);
  return static_cast<int>(cudaGetLastError());
}
