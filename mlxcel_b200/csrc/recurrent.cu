// State-space / linear-attention decode kernels and small element-wise ops for the hybrid model
// families (Mamba, Mamba2 / Jamba / Nemotron-H, Qwen3-Next GatedDeltaNet, BitNet).
// All are memory-bound SIMT kernels with fp32 state and accumulation.
//
// Reference counterparts (src/lib/mlxcel-core/cpp/mlx_cxx_kernels.cpp): ssm_update_kernel :679-850,
// mamba1_selective_scan :2680-3021, gated_delta :887-1500, bitlinear_matmul :90-312,
// fused_gelu_tanh_f32 (kernels/gelu_tanh_f32.cpp:117), fused_xielu :338-600,
// fused_add3_layer_norm :4322-4673.
#include "api.h"
#include "common.cuh"

namespace mx {

__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

// ----------------------------------------------------------------------------- Mamba2 step
// state [B, H, Dh, N] fp32 (in place); x [B, H, Dh]; dt [B, H]; A [H]; Bm, C [B, G, N]; D [H];
// y [B, H, Dh]. One warp per (b, h, dh): lanes stride N.
__global__ void ssm_update_kernel(float* __restrict__ state, const __nv_bfloat16* __restrict__ x,
                                  const __nv_bfloat16* __restrict__ dt, const float* __restrict__ A,
                                  const __nv_bfloat16* __restrict__ Bm, const __nv_bfloat16* __restrict__ C,
                                  const float* __restrict__ D, const float* __restrict__ dt_bias,
                                  __nv_bfloat16* __restrict__ y, int B, int H, int Dh, int N, int G,
                                  int dt_softplus) {
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= static_cast<long long>(B) * H * Dh) return;
  const int dh = static_cast<int>(gw % Dh);
  const int h = static_cast<int>((gw / Dh) % H);
  const int b = static_cast<int>(gw / (static_cast<long long>(Dh) * H));
  const int g = h / (H / G);
  float dtv = __bfloat162float(dt[b * H + h]) + (dt_bias ? dt_bias[h] : 0.f);
  if (dt_softplus) dtv = softplus_f(dtv);
  const float dA = __expf(dtv * A[h]);
  const float xv = __bfloat162float(x[(static_cast<size_t>(b) * H + h) * Dh + dh]);
  float* st = state + ((static_cast<size_t>(b) * H + h) * Dh + dh) * N;
  const __nv_bfloat16* bp = Bm + (static_cast<size_t>(b) * G + g) * N;
  const __nv_bfloat16* cp = C + (static_cast<size_t>(b) * G + g) * N;
  float acc = 0.f;
  for (int n = lane; n < N; n += 32) {
    const float s = st[n] * dA + dtv * xv * __bfloat162float(bp[n]);
    st[n] = s;
    acc += s * __bfloat162float(cp[n]);
  }
  acc = warp_sum(acc);
  if (lane == 0) y[(static_cast<size_t>(b) * H + h) * Dh + dh] = __float2bfloat16(acc + (D ? D[h] * xv : 0.f));
}

// ----------------------------------------------------------------------------- Mamba1 scan
// x, dt [B, L, Di]; A [Di, N]; Bm, C [B, L, N]; D [Di]; state [B, Di, N] fp32 in/out; y [B, L, Di].
// One warp per (b, d): lanes own the N state columns (N <= 32), time is walked sequentially.
__global__ void selective_scan_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dt,
                                      const float* __restrict__ A, const __nv_bfloat16* __restrict__ Bm,
                                      const __nv_bfloat16* __restrict__ C, const float* __restrict__ D,
                                      float* __restrict__ state, __nv_bfloat16* __restrict__ y, int B, int L,
                                      int Di, int N, int dt_softplus) {
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= static_cast<long long>(B) * Di) return;
  const int d = static_cast<int>(gw % Di), b = static_cast<int>(gw / Di);
  const bool on = lane < N;
  float s = on ? state[(static_cast<size_t>(b) * Di + d) * N + lane] : 0.f;
  const float a = on ? A[static_cast<size_t>(d) * N + lane] : 0.f;
  for (int t = 0; t < L; ++t) {
    const size_t xi = (static_cast<size_t>(b) * L + t) * Di + d;
    float dtv = __bfloat162float(dt[xi]);
    if (dt_softplus) dtv = softplus_f(dtv);
    const float xv = __bfloat162float(x[xi]);
    const size_t bi = (static_cast<size_t>(b) * L + t) * N + lane;
    float contrib = 0.f;
    if (on) {
      s = __expf(dtv * a) * s + dtv * xv * __bfloat162float(Bm[bi]);
      contrib = s * __bfloat162float(C[bi]);
    }
    contrib = warp_sum(contrib);
    if (lane == 0) y[xi] = __float2bfloat16(contrib + (D ? D[d] * xv : 0.f));
  }
  if (on) state[(static_cast<size_t>(b) * Di + d) * N + lane] = s;
}

// ----------------------------------------------------------------------------- Mamba2 over a ragged batch
// One launch serves every sequence piece of an engine step: decode rows are pieces of one token,
// prefill chunks pieces of many. Piece j covers token rows cu[j] .. cu[j+1]-1 and owns slot
// slots[j] of the state pools; reset[j] != 0 starts it from a zero state (a new sequence).

// Causal depth-wise convolution (width K <= 8) + bias + SiLU. in: rows of `in_stride` elements of
// which the first C are convolved; conv_state [slots, K-1, C] fp32 holds the last K-1 inputs of each
// sequence and is advanced. One thread per (piece, channel); time is walked with the window in
// registers, neighbouring threads read neighbouring channels.
__global__ void causal_conv_varlen_kernel(const __nv_bfloat16* __restrict__ in, int in_stride,
                                          float* __restrict__ conv_state, const int* __restrict__ slots,
                                          const int* __restrict__ cu, const int* __restrict__ reset,
                                          const float* __restrict__ w, const float* __restrict__ bias,
                                          __nv_bfloat16* __restrict__ out, int C, int K, int silu) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int j = blockIdx.y;
  if (c >= C) return;
  const int t0 = cu[j], t1 = cu[j + 1];
  if (t1 <= t0) return;
  float* cs = conv_state + static_cast<size_t>(slots[j]) * (K - 1) * C + c;
  float win[8], wk[8];
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    wk[k] = k < K ? w[static_cast<size_t>(c) * K + k] : 0.f;
    win[k] = (k < K - 1 && !reset[j]) ? cs[static_cast<size_t>(k) * C] : 0.f;
  }
  const float bv = bias ? bias[c] : 0.f;
  for (int t = t0; t < t1; ++t) {
    const float xv = __bfloat162float(in[static_cast<size_t>(t) * in_stride + c]);
    float acc = bv;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (k == K - 1) win[k] = xv;
      if (k < K) acc += wk[k] * win[k];
    }
    if (silu) acc = acc / (1.f + __expf(-acc));
    out[static_cast<size_t>(t) * C + c] = __float2bfloat16(acc);
#pragma unroll
    for (int k = 0; k < 7; ++k)
      if (k < K - 1) win[k] = win[k + 1];
  }
#pragma unroll
  for (int k = 0; k < 7; ++k)
    if (k < K - 1) cs[static_cast<size_t>(k) * C] = win[k];
}

// State-space recurrence  S <- S exp(dt A_h) + dt x (x) B,  y = S C + D_h x  walked over each piece.
// state [slots, H, P, N] fp32; x rows [H*P] at stride x_stride; Bm, Cm rows [G*N] at stride
// bc_stride; dt rows [H] at stride dt_stride; y [T, H*P]. One warp per (piece, h, p): lane l keeps
// state columns l, l+32, ... (N <= 256) in registers for the whole piece.
__global__ void ssm_scan_varlen_kernel(float* __restrict__ state, const int* __restrict__ slots,
                                       const int* __restrict__ cu, const int* __restrict__ reset,
                                       const __nv_bfloat16* __restrict__ x, int x_stride,
                                       const __nv_bfloat16* __restrict__ dt, int dt_stride,
                                       const float* __restrict__ A, const __nv_bfloat16* __restrict__ Bm,
                                       const __nv_bfloat16* __restrict__ Cm, int bc_stride,
                                       const float* __restrict__ D, const float* __restrict__ dt_bias,
                                       __nv_bfloat16* __restrict__ y, int H, int P, int N, int G,
                                       int dt_softplus, float dt_min, float dt_max) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int j = blockIdx.y;
  if (gw >= H * P) return;
  const int h = gw / P, p = gw - h * P, g = h / (H / G);
  const int t0 = cu[j], t1 = cu[j + 1];
  if (t1 <= t0) return;
  float* st = state + ((static_cast<size_t>(slots[j]) * H + h) * P + p) * N;
  float s[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int n = lane + 32 * i;
    s[i] = (n < N && !reset[j]) ? st[n] : 0.f;
  }
  const float a = A[h], dv = D ? D[h] : 0.f, db = dt_bias ? dt_bias[h] : 0.f;
  for (int t = t0; t < t1; ++t) {
    float dtv = __bfloat162float(dt[static_cast<size_t>(t) * dt_stride + h]) + db;
    if (dt_softplus) dtv = softplus_f(dtv);
    dtv = fminf(fmaxf(dtv, dt_min), dt_max);
    const float dA = __expf(dtv * a);
    const float xv = __bfloat162float(x[static_cast<size_t>(t) * x_stride + gw]);
    const __nv_bfloat16* bp = Bm + static_cast<size_t>(t) * bc_stride + g * N;
    const __nv_bfloat16* cp = Cm + static_cast<size_t>(t) * bc_stride + g * N;
    const float dx = dtv * xv;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const int n = lane + 32 * i;
      if (n < N) {
        s[i] = s[i] * dA + dx * __bfloat162float(bp[n]);
        acc += s[i] * __bfloat162float(cp[n]);
      }
    }
    acc = warp_sum(acc);
    if (lane == 0) y[static_cast<size_t>(t) * H * P + gw] = __float2bfloat16(acc + dv * xv);
  }
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int n = lane + 32 * i;
    if (n < N) st[n] = s[i];
  }
}

// out = RMSNorm(y * silu(z)) * weight over rows of `dim`; z rows at stride z_stride. One CTA per row.
__global__ void gated_rmsnorm_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ z,
                                     int z_stride, const __nv_bfloat16* __restrict__ weight,
                                     __nv_bfloat16* __restrict__ out, int dim, float eps) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  float ssq = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float zv = __bfloat162float(z[row * z_stride + i]);
    const float v = __bfloat162float(y[row * dim + i]) * (zv / (1.f + __expf(-zv)));
    ssq += v * v;
  }
  ssq = warp_sum(ssq);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ssq;
  __syncthreads();
  if (threadIdx.x < 32) {
    float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
    t = warp_sum(t);
    if (threadIdx.x == 0) red[0] = rsqrtf(t / dim + eps);
  }
  __syncthreads();
  const float r = red[0];
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float zv = __bfloat162float(z[row * z_stride + i]);
    const float v = __bfloat162float(y[row * dim + i]) * (zv / (1.f + __expf(-zv)));
    out[row * dim + i] = __float2bfloat16(v * r * __bfloat162float(weight[i]));
  }
}

// ----------------------------------------------------------------------------- gated delta rule
// state S [B, Hv, Dk, Dv] fp32 in place; q, k [B, Hv, Dk]; v [B, Hv, Dv]; g (log decay), beta [B, Hv];
// out [B, Hv, Dv]. One CTA per (b, h), thread j owns column j of S (Dv <= 1024).
__global__ void gated_delta_kernel(float* __restrict__ S, const __nv_bfloat16* __restrict__ q,
                                   const __nv_bfloat16* __restrict__ k, const __nv_bfloat16* __restrict__ v,
                                   const float* __restrict__ g, const float* __restrict__ beta,
                                   __nv_bfloat16* __restrict__ out, int Dk, int Dv, float q_scale) {
  extern __shared__ float sh[];   // k [Dk], q [Dk]
  float* ks = sh;
  float* qs = sh + Dk;
  const int bh = blockIdx.x, j = threadIdx.x;
  for (int i = threadIdx.x; i < Dk; i += blockDim.x) {
    ks[i] = __bfloat162float(k[static_cast<size_t>(bh) * Dk + i]);
    qs[i] = __bfloat162float(q[static_cast<size_t>(bh) * Dk + i]) * q_scale;
  }
  __syncthreads();
  if (j >= Dv) return;
  float* col = S + static_cast<size_t>(bh) * Dk * Dv + j;
  const float decay = __expf(g[bh]);
  float mem = 0.f;
  for (int i = 0; i < Dk; ++i) {
    const float s = col[static_cast<size_t>(i) * Dv] * decay;
    col[static_cast<size_t>(i) * Dv] = s;
    mem += s * ks[i];
  }
  const float delta = (__bfloat162float(v[static_cast<size_t>(bh) * Dv + j]) - mem) * beta[bh];
  float o = 0.f;
  for (int i = 0; i < Dk; ++i) {
    const float s = col[static_cast<size_t>(i) * Dv] + ks[i] * delta;
    col[static_cast<size_t>(i) * Dv] = s;
    o += s * qs[i];
  }
  out[static_cast<size_t>(bh) * Dv + j] = __float2bfloat16(o);
}

// ----------------------------------------------------------------------------- BitLinear
// Ternary weights {-1, 0, +1} packed 4 per byte (2 bits each, value = code - 1), [N, K/4];
// out[m, n] = scale * sum_k x[m, k] * w[n, k]. One warp per (m, n).
__global__ void bitlinear_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ w,
                                 __nv_bfloat16* __restrict__ out, int M, int N, int K, float scale) {
  const long long gw = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= static_cast<long long>(M) * N) return;
  const int n = static_cast<int>(gw % N), m = static_cast<int>(gw / N);
  const uint8_t* wr = w + static_cast<size_t>(n) * (K / 4);
  const __nv_bfloat16* xr = x + static_cast<size_t>(m) * K;
  float acc = 0.f;
  for (int c = lane; c < K / 4; c += 32) {
    const uint32_t byte = wr[c];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int code = static_cast<int>((byte >> (2 * j)) & 3u) - 1;
      acc += static_cast<float>(code) * __bfloat162float(xr[c * 4 + j]);
    }
  }
  acc = warp_sum(acc);
  if (lane == 0) out[static_cast<size_t>(m) * N + n] = __float2bfloat16(acc * scale);
}

// ----------------------------------------------------------------------------- element-wise
// mode 0: tanh-GELU; mode 1: xIELU with per-tensor alpha_p, alpha_n, beta, eps.
__global__ void activation_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                  long long n, int mode, float ap, float an, float beta, float eps) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = __bfloat162float(x[i]);
  float r;
  if (mode == 0) {
    r = 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
  } else {
    r = v > 0.f ? ap * v * v + beta * v : an * (expm1f(fminf(v, eps)) - v) + beta * v;
  }
  y[i] = __float2bfloat16(r);
}

// y = LayerNorm(a + b + c) * w + bias; also writes the sum. One CTA per row.
__global__ void add3_layernorm_kernel(const __nv_bfloat16* __restrict__ a, const __nv_bfloat16* __restrict__ b,
                                      const __nv_bfloat16* __restrict__ c, const __nv_bfloat16* __restrict__ w,
                                      const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ sum_out,
                                      __nv_bfloat16* __restrict__ y, int dim, float eps) {
  __shared__ float red[2][32];
  const size_t base = static_cast<size_t>(blockIdx.x) * dim;
  float s1 = 0.f, s2 = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = __bfloat162float(__float2bfloat16(__bfloat162float(a[base + i]) + __bfloat162float(b[base + i]) +
                                                      __bfloat162float(c[base + i])));
    if (sum_out) sum_out[base + i] = __float2bfloat16(v);
    s1 += v;
    s2 += v * v;
  }
  s1 = warp_sum(s1);
  s2 = warp_sum(s2);
  if ((threadIdx.x & 31) == 0) {
    red[0][threadIdx.x >> 5] = s1;
    red[1][threadIdx.x >> 5] = s2;
  }
  __syncthreads();
  if (threadIdx.x < 32) {
    float t1 = threadIdx.x < (blockDim.x >> 5) ? red[0][threadIdx.x] : 0.f;
    float t2 = threadIdx.x < (blockDim.x >> 5) ? red[1][threadIdx.x] : 0.f;
    t1 = warp_sum(t1);
    t2 = warp_sum(t2);
    if (threadIdx.x == 0) {
      red[0][0] = t1;
      red[1][0] = t2;
    }
  }
  __syncthreads();
  const float mean = red[0][0] / dim;
  const float var = fmaxf(red[1][0] / dim - mean * mean, 0.f);
  const float rstd = rsqrtf(var + eps);
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = __bfloat162float(__float2bfloat16(__bfloat162float(a[base + i]) + __bfloat162float(b[base + i]) +
                                                      __bfloat162float(c[base + i])));
    y[base + i] = __float2bfloat16((v - mean) * rstd * __bfloat162float(w[i]) + (bias ? __bfloat162float(bias[i]) : 0.f));
  }
}

}  // namespace mx

using namespace mx;

extern "C" int mx_ssm_update(void* state, const void* x, const void* dt, const void* A, const void* Bm,
                             const void* C, const void* D, const void* dt_bias, void* y, int B, int H, int Dh,
                             int N, int G, int dt_softplus, void* stream) {
  const long long warps = static_cast<long long>(B) * H * Dh;
  if (warps <= 0) return 0;
  if (G <= 0 || H % G) return -1;
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  ssm_update_kernel<<<static_cast<int>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<float*>(state), static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dt),
      static_cast<const float*>(A), static_cast<const __nv_bfloat16*>(Bm), static_cast<const __nv_bfloat16*>(C),
      static_cast<const float*>(D), static_cast<const float*>(dt_bias), static_cast<__nv_bfloat16*>(y), B, H, Dh, N,
      G, dt_softplus);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mx_selective_scan(const void* x, const void* dt, const void* A, const void* Bm, const void* C,
                                 const void* D, void* state, void* y, int B, int L, int Di, int N, int dt_softplus,
                                 void* stream) {
  const long long warps = static_cast<long long>(B) * Di;
  if (warps <= 0 || L <= 0) return 0;
  if (N > 32) return -1;
  const int threads = 128;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  selective_scan_kernel<<<static_cast<int>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(dt), static_cast<const float*>(A),
      static_cast<const __nv_bfloat16*>(Bm), static_cast<const __nv_bfloat16*>(C), static_cast<const float*>(D),
      static_cast<float*>(state), static_cast<__nv_bfloat16*>(y), B, L, Di, N, dt_softplus);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mx_causal_conv_varlen(const void* in, int in_stride, void* conv_state, const void* slots,
                                     const void* cu, const void* reset, const void* w, const void* bias, void* out,
                                     int pieces, int C, int K, int silu, void* stream) {
  if (pieces <= 0 || C <= 0) return 0;
  if (K < 1 || K > 8 || pieces > 65535) return -1;
  const int threads = 128;
  const dim3 grid((C + threads - 1) / threads, pieces);
  causal_conv_varlen_kernel<<<grid, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(in), in_stride, static_cast<float*>(conv_state),
      static_cast<const int*>(slots), static_cast<const int*>(cu), static_cast<const int*>(reset),
      static_cast<const float*>(w), static_cast<const float*>(bias), static_cast<__nv_bfloat16*>(out), C, K, silu);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mx_ssm_scan_varlen(void* state, const void* slots, const void* cu, const void* reset, const void* x,
                                  int x_stride, const void* dt, int dt_stride, const void* A, const void* Bm,
                                  const void* Cm, int bc_stride, const void* D, const void* dt_bias, void* y,
                                  int pieces, int H, int P, int N, int G, int dt_softplus, float dt_min,
                                  float dt_max, void* stream) {
  if (pieces <= 0 || H <= 0 || P <= 0) return 0;
  if (N < 1 || N > 256 || G <= 0 || H % G || pieces > 65535) return -1;
  const int threads = 128;
  const dim3 grid((H * P * 32 + threads - 1) / threads, pieces);
  ssm_scan_varlen_kernel<<<grid, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<float*>(state), static_cast<const int*>(slots), static_cast<const int*>(cu),
      static_cast<const int*>(reset), static_cast<const __nv_bfloat16*>(x), x_stride,
      static_cast<const __nv_bfloat16*>(dt), dt_stride, static_cast<const float*>(A),
      static_cast<const __nv_bfloat16*>(Bm), static_cast<const __nv_bfloat16*>(Cm), bc_stride,
      static_cast<const float*>(D), static_cast<const float*>(dt_bias), static_cast<__nv_bfloat16*>(y), H, P, N, G,
      dt_softplus, dt_min, dt_max);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mx_gated_rmsnorm(const void* y, const void* z, int z_stride, const void* weight, void* out,
                                int rows, int dim, float eps, void* stream) {
  if (rows <= 0 || dim <= 0) return 0;
  gated_rmsnorm_kernel<<<rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(z), z_stride,
      static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(out), dim, eps);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mx_gated_delta_update(void* S, const void* q, const void* k, const void* v, const void* g,
                                     const void* beta, void* out, int BH, int Dk, int Dv, float q_scale,
                                     void* stream) {
  if (BH <= 0) return 0;
  if (Dv > 1024 || Dk > 4096) return -1;
  const int threads = ((Dv + 31) / 32) * 32;
  gated_delta_kernel<<<BH, threads, 2 * Dk * sizeof(float), static_cast<cudaStream_t>(stream)>>>(
      static_cast<float*>(S), static_cast<const __nv_bfloat16*>(q), static_cast<const __nv_bfloat16*>(k),
      static_cast<const __nv_bfloat16*>(v), static_cast<const float*>(g), static_cast<const float*>(beta),
      static_cast<__nv_bfloat16*>(out), Dk, Dv, q_scale);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mx_bitlinear(const void* x, const void* w, void* out, int M, int N, int K, float scale,
                            void* stream) {
  const long long warps = static_cast<long long>(M) * N;
  if (warps <= 0) return 0;
  if (K % 4) return -1;
  const int threads = 256;
  const long long blocks = (warps * 32 + threads - 1) / threads;
  bitlinear_kernel<<<static_cast<int>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const uint8_t*>(w), static_cast<__nv_bfloat16*>(out), M, N, K,
      scale);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mx_activation(const void* x, void* y, long long n, int mode, float ap, float an, float beta,
                             float eps, void* stream) {
  if (n <= 0) return 0;
  const int threads = 256;
  activation_kernel<<<static_cast<int>((n + threads - 1) / threads), threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<__nv_bfloat16*>(y), n, mode, ap, an, beta, eps);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mx_add3_layernorm(const void* a, const void* b, const void* c, const void* w, const void* bias,
                                 void* sum_out, void* y, int rows, int dim, float eps, void* stream) {
  if (rows <= 0) return 0;
  int threads = ((dim + 31) / 32) * 32;
  if (threads > 1024) threads = 1024;
  add3_layernorm_kernel<<<rows, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(a), static_cast<const __nv_bfloat16*>(b), static_cast<const __nv_bfloat16*>(c),
      static_cast<const __nv_bfloat16*>(w), static_cast<const __nv_bfloat16*>(bias),
      static_cast<__nv_bfloat16*>(sum_out), static_cast<__nv_bfloat16*>(y), dim, eps);
  return static_cast<int>(cudaGetLastError());
}
