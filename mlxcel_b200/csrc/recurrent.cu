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
// sequence and is advanced. One thread per (piece, CPT neighbouring channels, chunk of kConvChunk
// steps): the convolution is not recurrent, so time chunks run in parallel. A thread first issues all
// of its chunk's loads (kConvChunk + KT - 1 rows; the taps sit right-aligned in a window of KT so
// that every register index is static), then computes. KT = 4 serves K == 4, KT = 8 any K <= 8;
// CPT = 2 moves channel pairs as 4-byte words. Only the thread of chunk 0 touches the state: it
// reads the old tail and, after its chunk, writes the new one, so no other thread races it.
constexpr int kConvChunk = 16;

template <int KT, int CPT>
__global__ void causal_conv_varlen_kernel(const __nv_bfloat16* __restrict__ in, int in_stride,
                                          float* __restrict__ conv_state, const int* __restrict__ slots,
                                          const int* __restrict__ cu, const int* __restrict__ reset,
                                          const float* __restrict__ w, const float* __restrict__ bias,
                                          __nv_bfloat16* __restrict__ out, int C, int K, int silu) {
  const int c = (blockIdx.x * blockDim.x + threadIdx.x) * CPT;
  const int j = blockIdx.y;
  if (c >= C) return;
  const int t0 = cu[j], t1 = cu[j + 1];
  const int tb = t0 + blockIdx.z * kConvChunk;
  if (tb >= t1) return;
  const bool first = blockIdx.z == 0;
  const bool fresh = reset[j] != 0;
  float* cs = conv_state + static_cast<size_t>(slots[j]) * (K - 1) * C + c;
  const int pad = KT - K;                         // window slots [0, pad) carry zero taps
  constexpr int W = kConvChunk + KT - 1;
  float v[W][CPT], wr[KT][CPT];
#pragma unroll
  for (int m = 0; m < KT; ++m)
#pragma unroll
    for (int e = 0; e < CPT; ++e) wr[m][e] = m >= pad ? w[static_cast<size_t>(c + e) * K + (m - pad)] : 0.f;
  const auto load_row = [&](int tt, float (&dst)[CPT]) {
    const __nv_bfloat16* src = in + static_cast<size_t>(tt) * in_stride + c;
    if constexpr (CPT == 2) {
      const float2 f = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(src));
      dst[0] = f.x, dst[1] = f.y;
    } else {
      dst[0] = __bfloat162float(*src);
    }
  };
  const int base = tb - (KT - 1);                 // v[i] is the input at row base + i
  if (base >= t0 && tb + kConvChunk <= t1) {      // interior chunk: no edge on either side
#pragma unroll
    for (int i = 0; i < W; ++i) {
#pragma unroll
      for (int e = 0; e < CPT; ++e) v[i][e] = 0.f;
      if (i >= pad) load_row(base + i, v[i]);
    }
  } else {
#pragma unroll
    for (int i = 0; i < W; ++i) {
      const int tt = base + i;
#pragma unroll
      for (int e = 0; e < CPT; ++e) v[i][e] = 0.f;
      if (i >= pad && tt < t1) {
        if (tt >= t0) {
          load_row(tt, v[i]);
        } else if (first && !fresh) {
#pragma unroll
          for (int e = 0; e < CPT; ++e) v[i][e] = cs[static_cast<size_t>(tt - t0 + (K - 1)) * C + e];
        }
      }
    }
  }
  float bv[CPT];
#pragma unroll
  for (int e = 0; e < CPT; ++e) bv[e] = bias ? bias[c + e] : 0.f;
#pragma unroll
  for (int sidx = 0; sidx < kConvChunk; ++sidx) {
    const int t = tb + sidx;
    if (t < t1) {
      float acc[CPT];
#pragma unroll
      for (int e = 0; e < CPT; ++e) {
        acc[e] = bv[e];
#pragma unroll
        for (int m = 0; m < KT; ++m) acc[e] += wr[m][e] * v[sidx + m][e];
        if (silu) acc[e] = acc[e] / (1.f + __expf(-acc[e]));
      }
      __nv_bfloat16* dst = out + static_cast<size_t>(t) * C + c;
      if constexpr (CPT == 2) *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(acc[0], acc[1]);
      else *dst = __float2bfloat16(acc[0]);
    }
  }
  if (!first) return;
  // new tail = the K-1 rows before t1; a piece shorter than the tail shifts the old one (reads run
  // ahead of the writes: entry L + m > m)
  const int L = t1 - t0;
  for (int m = 0; m < K - 1; ++m) {
    const int tt = t1 - (K - 1) + m;
    float x[CPT];
    if (tt >= t0) {
      load_row(tt, x);
    } else {
#pragma unroll
      for (int e = 0; e < CPT; ++e) x[e] = fresh ? 0.f : cs[static_cast<size_t>(L + m) * C + e];
    }
#pragma unroll
    for (int e = 0; e < CPT; ++e) cs[static_cast<size_t>(m) * C + e] = x[e];
  }
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

// The same recurrence for pieces of ONE token (decode rows), bandwidth-bound on the state: a warp owns
// kStepRows consecutive rows p of one (piece, head) and lane l the columns 4(l + 32 i) .. +3 of each,
// moved as float4, so that every lane has kStepRows x 2 independent 16-byte loads in flight and dt,
// exp(dt A), B and C are worked out once per warp (N % 4 == 0, N <= 256, P % kStepRows == 0; B and C
// rows 8-byte aligned).
constexpr int kStepRows = 4;

template <int NV>                               // float4 groups per lane: 1 for N <= 128, 2 up to 256
__global__ void ssm_step_vec4_kernel(float* __restrict__ state, const int* __restrict__ slots,
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
  const int ppw = P / kStepRows;
  if (gw >= H * ppw) return;
  const int h = gw / ppw, p0 = (gw - h * ppw) * kStepRows, g = h / (H / G);
  const int t = cu[j];
  if (cu[j + 1] <= t) return;
  float* st = state + ((static_cast<size_t>(slots[j]) * H + h) * P + p0) * N;
  const bool fresh = reset[j] != 0;
  float4 s[kStepRows][NV];
#pragma unroll
  for (int r = 0; r < kStepRows; ++r)
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int n = 4 * (lane + 32 * i);
      s[r][i] = (n < N && !fresh) ? *reinterpret_cast<const float4*>(st + static_cast<size_t>(r) * N + n)
                                  : make_float4(0.f, 0.f, 0.f, 0.f);
    }
  float dtv = __bfloat162float(dt[static_cast<size_t>(t) * dt_stride + h]) + (dt_bias ? dt_bias[h] : 0.f);
  if (dt_softplus) dtv = softplus_f(dtv);
  dtv = fminf(fmaxf(dtv, dt_min), dt_max);
  const float dA = __expf(dtv * A[h]), dv = D ? D[h] : 0.f;
  const __nv_bfloat16* bp = Bm + static_cast<size_t>(t) * bc_stride + g * N;
  const __nv_bfloat16* cp = Cm + static_cast<size_t>(t) * bc_stride + g * N;
  float4 bq[NV], cq[NV];
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int n = 4 * (lane + 32 * i);
    bq[i] = cq[i] = make_float4(0.f, 0.f, 0.f, 0.f);
    if (n < N) {
      const uint2 braw = *reinterpret_cast<const uint2*>(bp + n), craw = *reinterpret_cast<const uint2*>(cp + n);
      const float2 b0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&braw.x));
      const float2 b1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&braw.y));
      const float2 c0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&craw.x));
      const float2 c1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&craw.y));
      bq[i] = make_float4(b0.x, b0.y, b1.x, b1.y);
      cq[i] = make_float4(c0.x, c0.y, c1.x, c1.y);
    }
  }
  const __nv_bfloat16* xr = x + static_cast<size_t>(t) * x_stride + h * P + p0;
  float xv[kStepRows], acc[kStepRows];
#pragma unroll
  for (int r = 0; r < kStepRows; ++r) {
    xv[r] = __bfloat162float(xr[r]);
    const float dx = dtv * xv[r];
    acc[r] = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      s[r][i].x = s[r][i].x * dA + dx * bq[i].x;
      s[r][i].y = s[r][i].y * dA + dx * bq[i].y;
      s[r][i].z = s[r][i].z * dA + dx * bq[i].z;
      s[r][i].w = s[r][i].w * dA + dx * bq[i].w;
      acc[r] += s[r][i].x * cq[i].x + s[r][i].y * cq[i].y + s[r][i].z * cq[i].z + s[r][i].w * cq[i].w;
    }
  }
#pragma unroll
  for (int r = 0; r < kStepRows; ++r)
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int n = 4 * (lane + 32 * i);
      if (n < N) *reinterpret_cast<float4*>(st + static_cast<size_t>(r) * N + n) = s[r][i];
    }
#pragma unroll
  for (int r = 0; r < kStepRows; ++r) acc[r] = warp_sum(acc[r]);
  if (lane < kStepRows) {
    float a = acc[0], xx = xv[0];
#pragma unroll
    for (int r = 1; r < kStepRows; ++r)
      if (lane == r) a = acc[r], xx = xv[r];
    y[static_cast<size_t>(t) * H * P + h * P + p0 + lane] = __float2bfloat16(a + dv * xx);
  }
}

// The same recurrence for long pieces (prefill chunks). It is bound by instruction issue and by the
// shared-memory pipe, not by DRAM, so the layout is a register tile: a thread keeps RPT rows x 4V
// columns of the state, SPLIT neighbouring lanes cover a row's N columns (lane q holds the float4
// column groups q, q + SPLIT, ...), and every B / C word a thread reads from shared memory feeds RPT
// rows. A step is 2N FMAs per row; the row sums are completed with a halving exchange (RPT values
// over SPLIT lanes in log2(RPT) + 2 rounds). A CTA is kScanRows rows of one (piece, head); per chunk
// of kScanChunk steps it stages B, C (shared by the head's rows), x, dt and exp(dt A) in shared memory
// as fp32. RPT = SPLIT / 4, so that a CTA of kScanThreads threads always covers kScanRows rows.
constexpr int kScanChunk = 16;
constexpr int kScanRows = 32;
constexpr int kScanThreads = 128;

template <int N, int SPLIT>
__global__ void __launch_bounds__(kScanThreads)
ssm_scan_rows_kernel(float* __restrict__ state, const int* __restrict__ slots, const int* __restrict__ cu,
                     const int* __restrict__ reset, const __nv_bfloat16* __restrict__ x, int x_stride,
                     const __nv_bfloat16* __restrict__ dt, int dt_stride, const float* __restrict__ A,
                     const __nv_bfloat16* __restrict__ Bm, const __nv_bfloat16* __restrict__ Cm, int bc_stride,
                     const float* __restrict__ D, const float* __restrict__ dt_bias, __nv_bfloat16* __restrict__ y,
                     int H, int P, int G, int dt_softplus, float dt_min, float dt_max) {
  constexpr int RPT = SPLIT / 4;              // rows per thread
  constexpr int V = N / (4 * SPLIT);          // float4 column groups per thread and row
  static_assert(V >= 1 && RPT >= 1 && (kScanThreads / SPLIT) * RPT == kScanRows, "tile shape");
  __shared__ __align__(16) float Bs[kScanChunk * N];
  __shared__ __align__(16) float Cs[kScanChunk * N];
  __shared__ __align__(16) float xs[kScanChunk * kScanRows];
  __shared__ float dts[kScanChunk], dAs[kScanChunk];
  const int row_blocks = (P + kScanRows - 1) / kScanRows;
  const int h = blockIdx.x / row_blocks, rb = blockIdx.x - h * row_blocks, j = blockIdx.y;
  const int grp = threadIdx.x / SPLIT, q = threadIdx.x % SPLIT;
  const int r0 = grp * RPT;                   // first of this thread's rows inside the CTA's rows
  const int p0 = rb * kScanRows + r0;
  const int g = h / (H / G);
  const int t0 = cu[j], t1 = cu[j + 1];
  if (t1 <= t0) return;
  float* st = state + (static_cast<size_t>(slots[j]) * H + h) * P * N;
  float4 s[RPT][V];
  const bool fresh = reset[j] != 0;
#pragma unroll
  for (int k = 0; k < RPT; ++k)
#pragma unroll
    for (int i = 0; i < V; ++i)
      s[k][i] = (p0 + k < P && !fresh)
                    ? *reinterpret_cast<const float4*>(st + static_cast<size_t>(p0 + k) * N + 4 * (i * SPLIT + q))
                    : make_float4(0.f, 0.f, 0.f, 0.f);
  const float a = A[h], dv = D ? D[h] : 0.f, db = dt_bias ? dt_bias[h] : 0.f;
  // the lane that ends up with a row's sum after the exchange below, and where it writes it
  const int my_row = q / (SPLIT / RPT);
  const bool writer = q % (SPLIT / RPT) == 0 && p0 + my_row < P;
  const int HP = H * P;
  __nv_bfloat16* yp = y + static_cast<size_t>(t0) * HP + h * P + p0 + my_row;
  for (int c0 = t0; c0 < t1; c0 += kScanChunk) {
    const int steps = min(kScanChunk, t1 - c0);
    __syncthreads();                          // the previous chunk has been consumed
    for (int i = threadIdx.x; i < steps * N; i += kScanThreads) {
      const int tt = i / N, n = i - tt * N;
      const size_t off = static_cast<size_t>(c0 + tt) * bc_stride + g * N + n;
      Bs[i] = __bfloat162float(Bm[off]);
      Cs[i] = __bfloat162float(Cm[off]);
    }
    for (int i = threadIdx.x; i < steps * kScanRows; i += kScanThreads) {
      const int tt = i / kScanRows, rr = i - tt * kScanRows;
      const int pp = rb * kScanRows + rr;
      xs[i] = pp < P ? __bfloat162float(x[static_cast<size_t>(c0 + tt) * x_stride + h * P + pp]) : 0.f;
    }
    if (threadIdx.x < steps) {
      float dtv = __bfloat162float(dt[static_cast<size_t>(c0 + threadIdx.x) * dt_stride + h]) + db;
      if (dt_softplus) dtv = softplus_f(dtv);
      dtv = fminf(fmaxf(dtv, dt_min), dt_max);
      dts[threadIdx.x] = dtv;
      dAs[threadIdx.x] = __expf(dtv * a);
    }
    __syncthreads();
    for (int tt = 0; tt < steps; ++tt) {
      const float dA = dAs[tt], dtv = dts[tt];
      float xv[RPT], dx[RPT], a0[RPT], a1[RPT], acc[RPT];
      if constexpr (RPT == 4) {
        const float4 x4 = *reinterpret_cast<const float4*>(xs + tt * kScanRows + r0);
        xv[0] = x4.x, xv[1] = x4.y, xv[2] = x4.z, xv[3] = x4.w;
      } else {
#pragma unroll
        for (int k = 0; k < RPT; ++k) xv[k] = xs[tt * kScanRows + r0 + k];
      }
#pragma unroll
      for (int k = 0; k < RPT; ++k) dx[k] = dtv * xv[k], a0[k] = 0.f, a1[k] = 0.f;
      const float4* b4 = reinterpret_cast<const float4*>(Bs + tt * N) + q;
      const float4* c4 = reinterpret_cast<const float4*>(Cs + tt * N) + q;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float4 b = b4[i * SPLIT], c = c4[i * SPLIT];
#pragma unroll
        for (int k = 0; k < RPT; ++k) {
          s[k][i].x = fmaf(s[k][i].x, dA, dx[k] * b.x);
          s[k][i].y = fmaf(s[k][i].y, dA, dx[k] * b.y);
          s[k][i].z = fmaf(s[k][i].z, dA, dx[k] * b.z);
          s[k][i].w = fmaf(s[k][i].w, dA, dx[k] * b.w);
          a0[k] = fmaf(s[k][i].x, c.x, a0[k]);
          a1[k] = fmaf(s[k][i].y, c.y, a1[k]);
          a0[k] = fmaf(s[k][i].z, c.z, a0[k]);
          a1[k] = fmaf(s[k][i].w, c.w, a1[k]);
        }
      }
#pragma unroll
      for (int k = 0; k < RPT; ++k) acc[k] = a0[k] + a1[k];
      // halving exchange: after the round with lane mask m a lane keeps the rows of its half
#pragma unroll
      for (int w = RPT / 2, m = SPLIT / 2; w >= 1; w /= 2, m /= 2) {
        const bool upper = (q & m) != 0;
#pragma unroll
        for (int k = 0; k < w; ++k) {
          const float send = upper ? acc[k] : acc[k + w];
          const float keep = upper ? acc[k + w] : acc[k];
          acc[k] = keep + __shfl_xor_sync(0xffffffffu, send, m);
        }
      }
#pragma unroll
      for (int m = SPLIT / RPT / 2; m >= 1; m /= 2) acc[0] += __shfl_xor_sync(0xffffffffu, acc[0], m);
      float xr = xv[0];
#pragma unroll
      for (int k = 1; k < RPT; ++k)
        if (my_row == k) xr = xv[k];
      if (writer) yp[static_cast<size_t>(tt) * HP] = __float2bfloat16(acc[0] + dv * xr);
    }
    yp += static_cast<size_t>(steps) * HP;
  }
#pragma unroll
  for (int k = 0; k < RPT; ++k)
#pragma unroll
    for (int i = 0; i < V; ++i)
      if (p0 + k < P)
        *reinterpret_cast<float4*>(st + static_cast<size_t>(p0 + k) * N + 4 * (i * SPLIT + q)) = s[k][i];
}

// out = RMSNorm(y * silu(z)) * weight over rows of `dim`; z rows at stride z_stride. One CTA per row.
// Vector variant: 16-byte loads, every thread keeps its (up to 16) gated values in registers, so y and
// z are read once (dim % 8 == 0, dim <= 16 * blockDim, rows of y, z and out 16-byte aligned).
__global__ void __launch_bounds__(512)
gated_rmsnorm_vec_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ z, int z_stride,
                         const __nv_bfloat16* __restrict__ weight, __nv_bfloat16* __restrict__ out, int dim,
                         int groups, float eps) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  const size_t tok = row / groups, grp = row - tok * groups;
  y += row * dim, out += row * dim, z += tok * z_stride + grp * dim, weight += grp * dim;
  float v[2][8];
  float ssq = 0.f;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int i = (threadIdx.x + r * blockDim.x) * 8;
    if (i < dim) {
      const uint4 yr = *reinterpret_cast<const uint4*>(y + i);
      const uint4 zr = *reinterpret_cast<const uint4*>(z + i);
      const __nv_bfloat162* y2 = reinterpret_cast<const __nv_bfloat162*>(&yr);
      const __nv_bfloat162* z2 = reinterpret_cast<const __nv_bfloat162*>(&zr);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 yv = __bfloat1622float2(y2[q]), zv = __bfloat1622float2(z2[q]);
        v[r][2 * q] = yv.x * (zv.x / (1.f + __expf(-zv.x)));
        v[r][2 * q + 1] = yv.y * (zv.y / (1.f + __expf(-zv.y)));
        ssq += v[r][2 * q] * v[r][2 * q] + v[r][2 * q + 1] * v[r][2 * q + 1];
      }
    }
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
  const float rs = red[0];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int i = (threadIdx.x + r * blockDim.x) * 8;
    if (i < dim) {
      const uint4 wr = *reinterpret_cast<const uint4*>(weight + i);
      const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wr);
      uint4 o;
      __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 wv = __bfloat1622float2(w2[q]);
        o2[q] = __floats2bfloat162_rn(v[r][2 * q] * rs * wv.x, v[r][2 * q + 1] * rs * wv.y);
      }
      *reinterpret_cast<uint4*>(out + i) = o;
    }
  }
}

// out = RMSNorm(y * silu(z)) * weight; a token row holds `groups` independently normalised sub-rows
// of `dim` elements (grouped variant of Nemotron-H; groups == 1: the whole row). z token rows at
// stride z_stride. One CTA per sub-row.
__global__ void gated_rmsnorm_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ z,
                                     int z_stride, const __nv_bfloat16* __restrict__ weight,
                                     __nv_bfloat16* __restrict__ out, int dim, int groups, float eps) {
  __shared__ float red[32];
  const size_t row = blockIdx.x;
  const size_t tok = row / groups, grp = row - tok * groups;
  y += row * dim, out += row * dim, z += tok * z_stride + grp * dim, weight += grp * dim;
  float ssq = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float zv = __bfloat162float(z[i]);
    const float v = __bfloat162float(y[i]) * (zv / (1.f + __expf(-zv)));
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
    const float zv = __bfloat162float(z[i]);
    const float v = __bfloat162float(y[i]) * (zv / (1.f + __expf(-zv)));
    out[i] = __float2bfloat16(v * r * __bfloat162float(weight[i]));
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
// mode 0: tanh-GELU; mode 1: xIELU with per-tensor alpha_p, alpha_n, beta, eps; mode 2: relu(x)^2;
// mode 3: erf-GELU; mode 4: SiLU.
__global__ void activation_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y,
                                  long long n, int mode, float ap, float an, float beta, float eps) {
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= n) return;
  const float v = __bfloat162float(x[i]);
  float r;
  if (mode == 0) {
    r = 0.5f * v * (1.f + tanhf(0.7978845608028654f * (v + 0.044715f * v * v * v)));
  } else if (mode == 2) {
    r = v > 0.f ? v * v : 0.f;
  } else if (mode == 3) {
    r = 0.5f * v * (1.f + erff(v * 0.7071067811865476f));
  } else if (mode == 4) {
    r = v / (1.f + __expf(-v));
  } else {
    r = v > 0.f ? ap * v * v + beta * v : an * (expm1f(fminf(v, eps)) - v) + beta * v;
  }
  y[i] = __float2bfloat16(r);
}

// y = LayerNorm(x) * w + bias (bias optional). One CTA per row; the row is read twice (mean, then
// centred variance) from L1/L2.
__global__ void layernorm_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ w,
                                 const __nv_bfloat16* __restrict__ bias, __nv_bfloat16* __restrict__ y, int dim,
                                 float eps) {
  __shared__ float red[33];
  const __nv_bfloat16* xr = x + static_cast<size_t>(blockIdx.x) * dim;
  const auto block_sum = [&](float v) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
      float t = threadIdx.x < (blockDim.x >> 5) ? red[threadIdx.x] : 0.f;
      t = warp_sum(t);
      if (threadIdx.x == 0) red[32] = t;
    }
    __syncthreads();
    return red[32];
  };
  float s = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) s += __bfloat162float(xr[i]);
  const float mean = block_sum(s) / dim;
  float q = 0.f;
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float d = __bfloat162float(xr[i]) - mean;
    q += d * d;
  }
  const float rstd = rsqrtf(block_sum(q) / dim + eps);
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    const float v = (__bfloat162float(xr[i]) - mean) * rstd * __bfloat162float(w[i]);
    y[static_cast<size_t>(blockIdx.x) * dim + i] = __float2bfloat16(v + (bias ? __bfloat162float(bias[i]) : 0.f));
  }
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

// max_len: an upper bound of the longest piece (sizes the grid over time chunks).
extern "C" int mx_causal_conv_varlen(const void* in, int in_stride, void* conv_state, const void* slots,
                                     const void* cu, const void* reset, const void* w, const void* bias, void* out,
                                     int pieces, int max_len, int C, int K, int silu, void* stream) {
  if (pieces <= 0 || C <= 0 || max_len <= 0) return 0;
  const int chunks = (max_len + kConvChunk - 1) / kConvChunk;
  if (K < 1 || K > 8 || pieces > 65535 || chunks > 65535) return -1;
  const int threads = 128;
  const auto al4 = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 4 == 0; };
  const bool pair = C % 2 == 0 && in_stride % 2 == 0 && al4(in) && al4(out);
  const int cpt = pair ? 2 : 1;
  const dim3 grid(((C + cpt - 1) / cpt + threads - 1) / threads, pieces, chunks);
#define MX_CONV(KT, CPT)                                                                                         \
  causal_conv_varlen_kernel<KT, CPT><<<grid, threads, 0, static_cast<cudaStream_t>(stream)>>>(                  \
      static_cast<const __nv_bfloat16*>(in), in_stride, static_cast<float*>(conv_state),                       \
      static_cast<const int*>(slots), static_cast<const int*>(cu), static_cast<const int*>(reset),             \
      static_cast<const float*>(w), static_cast<const float*>(bias), static_cast<__nv_bfloat16*>(out), C, K, silu)
  if (K == 4) {
    if (pair) MX_CONV(4, 2);
    else MX_CONV(4, 1);
  } else {
    if (pair) MX_CONV(8, 2);
    else MX_CONV(8, 1);
  }
#undef MX_CONV
  return static_cast<int>(cudaGetLastError());
}

namespace {

template <int N, int SPLIT>
int launch_scan_rows(float* state, const int* slots, const int* cu, const int* reset, const __nv_bfloat16* x,
                     int x_stride, const __nv_bfloat16* dt, int dt_stride, const float* A, const __nv_bfloat16* Bm,
                     const __nv_bfloat16* Cm, int bc_stride, const float* D, const float* dt_bias, __nv_bfloat16* y,
                     int pieces, int H, int P, int G, int dt_softplus, float dt_min, float dt_max,
                     cudaStream_t stream) {
  const int row_blocks = (P + kScanRows - 1) / kScanRows;
  ssm_scan_rows_kernel<N, SPLIT><<<dim3(H * row_blocks, pieces), kScanThreads, 0, stream>>>(
      state, slots, cu, reset, x, x_stride, dt, dt_stride, A, Bm, Cm, bc_stride, D, dt_bias, y, H, P, G, dt_softplus,
      dt_min, dt_max);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace

// The first n_short pieces hold one token each (decode rows) and take the bandwidth-shaped kernel;
// the others take the row kernel where its shape is covered (N in {16, 32, 64, 128}), else the
// generic warp-per-row kernel.
extern "C" int mx_ssm_scan_varlen(void* state, const void* slots, const void* cu, const void* reset, const void* x,
                                  int x_stride, const void* dt, int dt_stride, const void* A, const void* Bm,
                                  const void* Cm, int bc_stride, const void* D, const void* dt_bias, void* y,
                                  int pieces, int n_short, int H, int P, int N, int G, int dt_softplus, float dt_min,
                                  float dt_max, void* stream) {
  if (pieces <= 0 || H <= 0 || P <= 0) return 0;
  if (N < 1 || N > 256 || G <= 0 || H % G || pieces > 65535 || n_short < 0 || n_short > pieces) return -1;
  auto* st = static_cast<float*>(state);
  const auto* sl = static_cast<const int*>(slots);
  const auto* cup = static_cast<const int*>(cu);
  const auto* rs = static_cast<const int*>(reset);
  const auto* xp = static_cast<const __nv_bfloat16*>(x);
  const auto* dtp = static_cast<const __nv_bfloat16*>(dt);
  const auto* bp = static_cast<const __nv_bfloat16*>(Bm);
  const auto* cp = static_cast<const __nv_bfloat16*>(Cm);
  const auto* Ap = static_cast<const float*>(A);
  const auto* Dp = static_cast<const float*>(D);
  const auto* dbp = static_cast<const float*>(dt_bias);
  auto* yp = static_cast<__nv_bfloat16*>(y);
  auto s = static_cast<cudaStream_t>(stream);
  const int threads = 128;
  const int gx = (H * P * 32 + threads - 1) / threads;
  const bool vec4 = N % 4 == 0 && P % kStepRows == 0 && bc_stride % 4 == 0 && reinterpret_cast<uintptr_t>(Bm) % 8 == 0 &&
                    reinterpret_cast<uintptr_t>(Cm) % 8 == 0 && reinterpret_cast<uintptr_t>(state) % 16 == 0;
  const bool rows_ok = (N == 16 || N == 32 || N == 64 || N == 128) && static_cast<long long>(H) * P < (1 << 26) &&
                       reinterpret_cast<uintptr_t>(state) % 16 == 0;
  int first_generic = 0, n_generic = pieces;      // what is left for the generic kernel
  if (n_short > 0 && vec4) {
    const int gxs = (H * (P / kStepRows) * 32 + threads - 1) / threads;
    if (N <= 128)
      ssm_step_vec4_kernel<1><<<dim3(gxs, n_short), threads, 0, s>>>(st, sl, cup, rs, xp, x_stride, dtp, dt_stride, Ap,
                                                                      bp, cp, bc_stride, Dp, dbp, yp, H, P, N, G,
                                                                      dt_softplus, dt_min, dt_max);
    else
      ssm_step_vec4_kernel<2><<<dim3(gxs, n_short), threads, 0, s>>>(st, sl, cup, rs, xp, x_stride, dtp, dt_stride, Ap,
                                                                      bp, cp, bc_stride, Dp, dbp, yp, H, P, N, G,
                                                                      dt_softplus, dt_min, dt_max);
    first_generic = n_short;
    n_generic = pieces - n_short;
  }
  if (n_generic > 0 && rows_ok && first_generic == n_short) {
    const int np = pieces - n_short;
    int rc = 0;
#define MX_SCAN_ROWS(NN, SP)                                                                                  \
  rc = launch_scan_rows<NN, SP>(st, sl + n_short, cup + n_short, rs + n_short, xp, x_stride, dtp, dt_stride, Ap, \
                                bp, cp, bc_stride, Dp, dbp, yp, np, H, P, G, dt_softplus, dt_min, dt_max, s)
    if (np > 0) {
      if (N == 16) MX_SCAN_ROWS(16, 4);
      else if (N == 32) MX_SCAN_ROWS(32, 8);
      else if (N == 64) MX_SCAN_ROWS(64, 16);
      else MX_SCAN_ROWS(128, 16);
    }
#undef MX_SCAN_ROWS
    if (rc) return rc;
    n_generic = 0;
  }
  if (n_generic > 0) {
    ssm_scan_varlen_kernel<<<dim3(gx, n_generic), threads, 0, s>>>(
        st, sl + first_generic, cup + first_generic, rs + first_generic, xp, x_stride, dtp, dt_stride, Ap, bp, cp,
        bc_stride, Dp, dbp, yp, H, P, N, G, dt_softplus, dt_min, dt_max);
  }
  return static_cast<int>(cudaGetLastError());
}

// rows token rows of groups x dim elements each (y, out contiguous; z token rows at z_stride).
extern "C" int mx_gated_rmsnorm(const void* y, const void* z, int z_stride, const void* weight, void* out,
                                int rows, int dim, int groups, float eps, void* stream) {
  if (rows <= 0 || dim <= 0 || groups <= 0) return 0;
  const auto aligned = [](const void* p) { return reinterpret_cast<uintptr_t>(p) % 16 == 0; };
  const bool vec = dim % 8 == 0 && z_stride % 8 == 0 && dim <= 8192 && aligned(y) && aligned(z) &&
                   aligned(weight) && aligned(out);
  const long long blocks = static_cast<long long>(rows) * groups;
  if (blocks > 0x7fffffffLL) return -1;
  if (vec) {
    const int threads = min(512, ((dim / 8 + 1) / 2 + 31) / 32 * 32);
    gated_rmsnorm_vec_kernel<<<static_cast<int>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(z), z_stride,
        static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(out), dim, groups, eps);
  } else {
    gated_rmsnorm_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16*>(y), static_cast<const __nv_bfloat16*>(z), z_stride,
        static_cast<const __nv_bfloat16*>(weight), static_cast<__nv_bfloat16*>(out), dim, groups, eps);
  }
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

extern "C" int mx_layernorm(const void* x, const void* w, const void* bias, void* y, int rows, int dim, float eps,
                            void* stream) {
  if (rows <= 0 || dim <= 0) return 0;
  int threads = ((dim + 31) / 32) * 32;
  if (threads > 512) threads = 512;
  layernorm_kernel<<<rows, threads, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __nv_bfloat16*>(x), static_cast<const __nv_bfloat16*>(w),
      static_cast<const __nv_bfloat16*>(bias), static_cast<__nv_bfloat16*>(y), dim, eps);
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
