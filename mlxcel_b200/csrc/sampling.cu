// Token selection kernels: greedy argmax, the fused filter + Gumbel-max sampler, history
// penalties and the speculative-decoding verify walk. One CTA per logits row; every pass
// streams the row from L2 with 16-byte loads, nothing is sorted.
//
// top-k / top-p / min-p / typical-p cuts are found by bisection over the order-preserving integer
// image of the float logits (32 rounds, each a count or a probability-mass reduction), so the
// kept set is exact and deterministic, ties included. The draw is softmax-free: argmax of
// logit / T + Gumbel noise from Philox-4x32-10 keyed by (seed, step, element index).
//
// Parity targets in the reference: gumbel_max_sample (src/lib/mlxcelverse/kernels/sampling.h:17-88),
// rejection_sample (src/lib/mlxcelverse/kernels/sampling_rejection.h:17-215), the sampler chain
// order of src/lib/mlxcel-core/src/generate.rs:1296-1340 and the verify walk of
// src/lib/mlxcel-core/src/speculative/mtp/walk.rs:15-95.
#include "api.h"
#include "common.cuh"

namespace mx {

constexpr int kSampThreads = 1024;

template <bool FP32>
__device__ __forceinline__ float load_logit(const void* row, int i) {
  if (FP32) return static_cast<const float*>(row)[i];
  return __bfloat162float(static_cast<const __nv_bfloat16*>(row)[i]);
}

// Order-preserving map float -> uint32 (larger float <=> larger key).
__device__ __forceinline__ uint32_t float_key(float f) {
  const uint32_t u = __float_as_uint(f);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

struct ArgMax {
  float v;
  int i;
};
__device__ __forceinline__ ArgMax argmax_combine(ArgMax a, ArgMax b) {
  if (b.v > a.v || (b.v == a.v && b.i < a.i)) return b;
  return a;
}
__device__ __forceinline__ ArgMax block_argmax(ArgMax a, ArgMax* smem) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    ArgMax b;
    b.v = __shfl_xor_sync(0xffffffffu, a.v, o);
    b.i = __shfl_xor_sync(0xffffffffu, a.i, o);
    a = argmax_combine(a, b);
  }
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) smem[warp] = a;
  __syncthreads();
  if (warp == 0) {
    ArgMax b = (lane < (blockDim.x >> 5)) ? smem[lane] : ArgMax{-INFINITY, 0x7fffffff};
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      ArgMax c;
      c.v = __shfl_xor_sync(0xffffffffu, b.v, o);
      c.i = __shfl_xor_sync(0xffffffffu, b.i, o);
      b = argmax_combine(b, c);
    }
    if (lane == 0) smem[0] = b;
  }
  __syncthreads();
  return smem[0];
}
__device__ __forceinline__ float block_sum(float v, float* smem) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) smem[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = (lane < (blockDim.x >> 5)) ? smem[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) smem[0] = t;
  }
  __syncthreads();
  return smem[0];
}

// NaN logits are treated as -inf so that a poisoned row still yields a valid token.
__device__ __forceinline__ float sane(float v) { return (v == v) ? v : -INFINITY; }

template <bool FP32>
__global__ void __launch_bounds__(kSampThreads)
argmax_kernel(const void* __restrict__ logits, long long row_stride, int* __restrict__ out, int V) {
  __shared__ ArgMax red[32];
  pdl_trigger();
  pdl_wait();
  const char* base = static_cast<const char*>(logits) +
                     static_cast<size_t>(blockIdx.x) * row_stride * (FP32 ? 4 : 2);
  ArgMax best{-INFINITY, 0x7fffffff};
  if (!FP32 && (reinterpret_cast<uintptr_t>(base) & 15) == 0) {
    const uint4* v4 = reinterpret_cast<const uint4*>(base);
    const int nvec = V >> 3;
    for (int v = threadIdx.x; v < nvec; v += blockDim.x) {
      const uint4 a = v4[v];
      const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        best = argmax_combine(best, ArgMax{sane(bf16_lo(w[j])), v * 8 + 2 * j});
        best = argmax_combine(best, ArgMax{sane(bf16_hi(w[j])), v * 8 + 2 * j + 1});
      }
    }
    for (int i = (nvec << 3) + threadIdx.x; i < V; i += blockDim.x)
      best = argmax_combine(best, ArgMax{sane(load_logit<false>(base, i)), i});
  } else {
    for (int i = threadIdx.x; i < V; i += blockDim.x)
      best = argmax_combine(best, ArgMax{sane(load_logit<FP32>(base, i)), i});
  }
  best = block_argmax(best, red);
  if (threadIdx.x == 0) out[blockIdx.x] = best.i == 0x7fffffff ? 0 : best.i;
}

// ----------------------------------------------------------------------------- Philox
__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
  const uint32_t M0 = 0xD2511F53u, M1 = 0xCD9E8D57u, W0 = 0x9E3779B9u, W1 = 0xBB67AE85u;
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(M0, c[0]), lo0 = M0 * c[0];
    const uint32_t hi1 = __umulhi(M1, c[2]), lo1 = M1 * c[2];
    const uint32_t n0 = hi1 ^ c[1] ^ k0, n1 = lo1, n2 = hi0 ^ c[3] ^ k1, n3 = lo0;
    c[0] = n0;
    c[1] = n1;
    c[2] = n2;
    c[3] = n3;
    k0 += W0;
    k1 += W1;
  }
}
// Uniform in (0, 1): (x + 0.5) / 2^32.
__device__ __forceinline__ float u01(uint32_t x) {
  return (static_cast<float>(x >> 8) + 0.5f) * (1.0f / 16777216.0f);
}

template <bool FP32>
__global__ void __launch_bounds__(kSampThreads)
sample_kernel(const void* __restrict__ logits, long long row_stride,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ min_p,
              const float* __restrict__ typical_p, const float* __restrict__ top_n_sigma,
              const unsigned long long* __restrict__ seeds,
              const unsigned long long* __restrict__ steps, int* __restrict__ out_tokens,
              float* __restrict__ out_logprob, int V) {
  __shared__ ArgMax red_a[32];
  __shared__ float red_f[32];
  const int b = blockIdx.x;
  const void* row = static_cast<const char*>(logits) + static_cast<size_t>(b) * row_stride * (FP32 ? 4 : 2);
  const float T = temperature ? temperature[b] : 0.f;
  const int k = top_k ? top_k[b] : 0;
  const float tp = top_p ? top_p[b] : 1.f;
  const float mp = min_p ? min_p[b] : 0.f;
  const float typ = typical_p ? typical_p[b] : 1.f;
  const float nsig = top_n_sigma ? top_n_sigma[b] : 0.f;

  // pass 1: max
  ArgMax best{-INFINITY, 0x7fffffff};
  for (int i = threadIdx.x; i < V; i += blockDim.x)
    best = argmax_combine(best, ArgMax{sane(load_logit<FP32>(row, i)), i});
  best = block_argmax(best, red_a);
  const float m = best.v;
  // pass 2: partition function of the untempered distribution
  float z = 0.f;
  for (int i = threadIdx.x; i < V; i += blockDim.x) z += __expf(sane(load_logit<FP32>(row, i)) - m);
  z = block_sum(z, red_f);
  const bool greedy = !(T > 0.f) || k == 1;
  if (greedy) {
    if (threadIdx.x == 0) {
      out_tokens[b] = best.i == 0x7fffffff ? 0 : best.i;
      if (out_logprob) out_logprob[b] = -__logf(z);
    }
    return;
  }

  // thresholds (keys); a token is kept when float_key(logit) >= thr
  uint32_t thr = 0u;
  float kept_mass = z;  // in units of exp(l - m)
  if (k > 0 && k < V) {
    uint32_t prefix = 0u;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = prefix | (1u << bit);
      float cnt = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x)
        cnt += (float_key(sane(load_logit<FP32>(row, i))) >= cand) ? 1.f : 0.f;
      cnt = block_sum(cnt, red_f);
      if (cnt >= static_cast<float>(k)) prefix = cand;
    }
    thr = prefix;
    float mass = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float l = sane(load_logit<FP32>(row, i));
      if (float_key(l) >= thr) mass += __expf(l - m);
    }
    kept_mass = block_sum(mass, red_f);
  }
  if (tp < 1.f) {
    const float need = tp * kept_mass;
    uint32_t prefix = 0u;
    for (int bit = 31; bit >= 0; --bit) {
      const uint32_t cand = prefix | (1u << bit);
      float mass = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float l = sane(load_logit<FP32>(row, i));
        const uint32_t key = float_key(l);
        if (key >= cand && key >= thr) mass += __expf(l - m);
      }
      mass = block_sum(mass, red_f);
      if (mass >= need) prefix = cand;
    }
    thr = max(thr, prefix);
  }
  if (mp > 0.f) {
    const uint32_t key = float_key(m + __logf(mp));
    thr = max(thr, key);
  }
  if (nsig > 0.f) {
    // top-n-sigma: keep logits within nsig standard deviations (unbiased, over the finite logits of
    // the whole row) of the maximum
    float s1 = 0.f, s2 = 0.f, cnt = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float l = sane(load_logit<FP32>(row, i));
      if (l > -INFINITY) {
        const float d = l - m;
        s1 += d, s2 += d * d, cnt += 1.f;
      }
    }
    s1 = block_sum(s1, red_f);
    s2 = block_sum(s2, red_f);
    cnt = block_sum(cnt, red_f);
    if (cnt > 1.5f) {
      const float var = fmaxf(0.f, (s2 - s1 * s1 / cnt) / (cnt - 1.f));
      thr = max(thr, float_key(m - nsig * sqrtf(var)));
    }
  }
  // Never filter out the most likely token.
  thr = min(thr, float_key(m));

  // typical-p (locally typical sampling) on the distribution that survived the filters above:
  // tokens are ranked by |(-log p) - H| and the smallest set reaching typical_p of the mass is
  // kept. The cut is found by bisection over the bit pattern of that (non-negative) deviation.
  float typ_logzk = 0.f, typ_ent = 0.f;
  uint32_t typ_cut = 0xFFFFFFFFu;
  const bool use_typ = typ < 1.f;
  if (use_typ) {
    float zk = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float l = sane(load_logit<FP32>(row, i));
      if (float_key(l) >= thr && l > -INFINITY) zk += __expf(l - m);
    }
    zk = block_sum(zk, red_f);
    typ_logzk = __logf(zk);
    float ent = 0.f;
    for (int i = threadIdx.x; i < V; i += blockDim.x) {
      const float l = sane(load_logit<FP32>(row, i));
      if (float_key(l) >= thr && l > -INFINITY) {
        const float lp = l - m - typ_logzk;
        ent -= __expf(lp) * lp;
      }
    }
    typ_ent = block_sum(ent, red_f);
    // largest cut with mass{dev < cut} < typ; then mass{dev <= cut} >= typ
    uint32_t cut = 0u;
    for (int bit = 30; bit >= 0; --bit) {
      const uint32_t cand = cut | (1u << bit);
      float mass = 0.f;
      for (int i = threadIdx.x; i < V; i += blockDim.x) {
        const float l = sane(load_logit<FP32>(row, i));
        if (float_key(l) >= thr && l > -INFINITY) {
          const float lp = l - m - typ_logzk;
          if (__float_as_uint(fabsf(-lp - typ_ent)) < cand) mass += __expf(lp);
        }
      }
      mass = block_sum(mass, red_f);
      if (mass < typ) cut = cand;
    }
    typ_cut = cut;
  }

  // draw: argmax(l / T + gumbel)
  const unsigned long long seed = seeds ? seeds[b] : 0ull;
  const unsigned long long step = steps ? steps[b] : 0ull;
  const float invT = 1.0f / T;
  ArgMax pick{-INFINITY, 0x7fffffff};
  const int ngroups = (V + 3) >> 2;
  for (int gidx = threadIdx.x; gidx < ngroups; gidx += blockDim.x) {
    uint32_t c[4] = {static_cast<uint32_t>(gidx), 0u, static_cast<uint32_t>(step),
                     static_cast<uint32_t>(step >> 32)};
    philox4x32_10(c, static_cast<uint32_t>(seed), static_cast<uint32_t>(seed >> 32));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = gidx * 4 + j;
      if (i < V) {
        const float l = sane(load_logit<FP32>(row, i));
        bool in = float_key(l) >= thr && l > -INFINITY;
        if (in && use_typ)
          in = __float_as_uint(fabsf(-(l - m - typ_logzk) - typ_ent)) <= typ_cut || i == best.i;
        if (in) {
          const float g = -__logf(-__logf(u01(c[j])));
          pick = argmax_combine(pick, ArgMax{l * invT + g, i});
        }
      }
    }
  }
  pick = block_argmax(pick, red_a);
  if (threadIdx.x == 0) {
    const int tok = pick.i == 0x7fffffff ? (best.i == 0x7fffffff ? 0 : best.i) : pick.i;
    out_tokens[b] = tok;
    if (out_logprob) out_logprob[b] = sane(load_logit<FP32>(row, tok)) - m - __logf(z);
  }
}

// ----------------------------------------------------------------------------- penalties
// One CTA per row. A history position applies the penalty when it is the first occurrence of
// its token; its count is the number of occurrences in the window.
template <bool FP32>
__global__ void penalties_kernel(void* __restrict__ logits, long long row_stride,
                                 const int* __restrict__ history, int max_hist,
                                 const float* __restrict__ rep, const float* __restrict__ freq,
                                 const float* __restrict__ pres, int V) {
  const int b = blockIdx.x;
  const int* h = history + static_cast<size_t>(b) * max_hist;
  const float rp = rep ? rep[b] : 1.f, fp = freq ? freq[b] : 0.f, pp = pres ? pres[b] : 0.f;
  if (rp == 1.f && fp == 0.f && pp == 0.f) return;
  char* row = static_cast<char*>(logits) + static_cast<size_t>(b) * row_stride * (FP32 ? 4 : 2);
  for (int i = threadIdx.x; i < max_hist; i += blockDim.x) {
    const int tok = h[i];
    if (tok < 0 || tok >= V) continue;
    bool first = true;
    int count = 0;
    for (int j = 0; j < max_hist; ++j) {
      if (h[j] == tok) {
        if (j < i) {
          first = false;
          break;
        }
        ++count;
      }
    }
    if (!first) continue;
    float l = load_logit<FP32>(row, tok);
    if (rp != 1.f) l = l > 0.f ? l / rp : l * rp;
    l -= fp * static_cast<float>(count) + pp;
    if (FP32) reinterpret_cast<float*>(row)[tok] = l;
    else reinterpret_cast<__nv_bfloat16*>(row)[tok] = __float2bfloat16(l);
  }
}

// ----------------------------------------------------------------------------- verify walk
__global__ void verify_walk_kernel(const int* __restrict__ target, const int* __restrict__ draft,
                                   int* __restrict__ accept_len, int* __restrict__ next_token, int B,
                                   int K) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b >= B) return;
  int a = 0;
  while (a < K - 1 && draft[b * (K - 1) + a] == target[b * K + a]) ++a;
  accept_len[b] = a;
  next_token[b] = target[b * K + a];
}

}  // namespace mx

using namespace mx;

extern "C" int mx_argmax(const void* logits, int logits_fp32, long long row_stride, int* out, int B,
                         int V, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (B <= 0) return 0;
  MX_PREFER_SHARED(argmax_kernel<true>);
  MX_PREFER_SHARED(argmax_kernel<false>);
  if (logits_fp32)
    return static_cast<int>(launch_kernel(argmax_kernel<true>, dim3(B), dim3(kSampThreads), 0, stream, logits,
                                          row_stride, out, V));
  return static_cast<int>(launch_kernel(argmax_kernel<false>, dim3(B), dim3(kSampThreads), 0, stream, logits,
                                        row_stride, out, V));
}

extern "C" long long mx_sample_scratch_floats(int, int) { return 0; }

extern "C" int mx_sample(const void* logits, int logits_fp32, long long row_stride,
                         const float* temperature, const int* top_k, const float* top_p,
                         const float* min_p, const float* typical_p, const float* top_n_sigma,
                         const unsigned long long* seeds, const unsigned long long* steps,
                         int* out_tokens, float* out_logprob, int B, int V, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (B <= 0) return 0;
  if (logits_fp32)
    sample_kernel<true><<<B, kSampThreads, 0, stream>>>(logits, row_stride, temperature, top_k,
                                                        top_p, min_p, typical_p, top_n_sigma, seeds,
                                                        steps, out_tokens, out_logprob, V);
  else
    sample_kernel<false><<<B, kSampThreads, 0, stream>>>(logits, row_stride, temperature, top_k,
                                                         top_p, min_p, typical_p, top_n_sigma, seeds,
                                                         steps, out_tokens, out_logprob, V);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mx_apply_penalties(void* logits, int logits_fp32, long long row_stride,
                                  const int* history, int max_hist, const float* rep,
                                  const float* freq, const float* pres, int B, int V,
                                  void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (B <= 0 || max_hist <= 0) return 0;
  if (max_hist > 4096) return -1;
  if (logits_fp32)
    penalties_kernel<true><<<B, 256, 0, stream>>>(logits, row_stride, history, max_hist, rep, freq,
                                                  pres, V);
  else
    penalties_kernel<false><<<B, 256, 0, stream>>>(logits, row_stride, history, max_hist, rep, freq,
                                                   pres, V);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mx_spec_verify(const void* logits, int logits_fp32, long long row_stride,
                              const int* draft, int* target_tokens, int* accept_len,
                              int* next_token, int B, int K, int V, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (B <= 0 || K <= 0) return 0;
  int rc = mx_argmax(logits, logits_fp32, row_stride, target_tokens, B * K, V, stream_);
  if (rc != 0) return rc;
  verify_walk_kernel<<<(B + 127) / 128, 128, 0, stream>>>(target_tokens, draft, accept_len,
                                                          next_token, B, K);
  return static_cast<int>(cudaGetLastError());
}
