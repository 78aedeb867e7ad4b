// Mixture-of-experts routing and token permutation.
//
//   mx_moe_route        router logits [T, E] -> top-k expert ids + weights. mode 0: softmax over
//                       all experts, then top-k (optionally renormalised; Qwen-MoE). mode 1: top-k
//                       on the logits, then softmax over the k selected logits (Mixtral, GPT-OSS:
//                       src/models/gpt_oss.rs:402-446 of the reference).
//   mx_moe_align        counts the (token, slot) pairs routed to each LOCAL expert
//                       [e_begin, e_end), builds exclusive offsets and the permutation that sorts
//                       pairs by expert (stable in token order, so results are deterministic).
//   mx_moe_gather_rows  xs[r, :] = x[sorted_token[r], :]
//   mx_moe_combine      out[t, :] = (residual[t, :]) + sum_slots w[t, slot] * y[row(t, slot), :]
//                       in fp32 (the reference's moe_weighted_sum, src/models/switch_layers.rs:2180).
// Under expert parallelism tokens are replicated (attention is tensor parallel), so "dispatch" is
// this local gather and "combine" ends in the all-reduce of the partial outputs.
#include "api.h"
#include "common.cuh"

namespace mx {

constexpr int kMaxTopK = 16;

// One warp per token.
__global__ void moe_route_kernel(const __nv_bfloat16* __restrict__ logits, int* __restrict__ ids,
                                 float* __restrict__ wts, int T, int E, int k, int mode,
                                 int norm_topk) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  const __nv_bfloat16* row = logits + static_cast<size_t>(t) * E;
  // each lane owns experts lane, lane+32, ... (E <= 512 -> <= 16 per lane)
  float v[16];
  int cnt = 0;
  float mx_all = -INFINITY;
  for (int e = lane; e < E; e += 32) {
    float x = __bfloat162float(row[e]);
    if (!(x == x)) x = -INFINITY;
    v[cnt++] = x;
    mx_all = fmaxf(mx_all, x);
  }
  mx_all = warp_max(mx_all);
  float denom = 0.f;
  if (mode == 0) {
    for (int i = 0; i < cnt; ++i) denom += __expf(v[i] - mx_all);
    denom = warp_sum(denom);
  }
  float sel_v[kMaxTopK];
  int sel_e[kMaxTopK];
  for (int s = 0; s < k; ++s) {
    // argmax over the remaining experts (ties: lowest expert id)
    float best = -INFINITY;
    int best_e = 0x7fffffff;
    for (int i = 0; i < cnt; ++i) {
      const int e = lane + 32 * i;
      if (v[i] > best) {
        best = v[i];
        best_e = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
      if (ob > best || (ob == best && oe < best_e)) {
        best = ob;
        best_e = oe;
      }
    }
    if (best_e == 0x7fffffff) best_e = s;  // nothing left above -inf: fall back to expert s
    sel_v[s] = best;
    sel_e[s] = best_e;
    // remove the winner from further rounds (-inf is below every remaining candidate)
    if ((best_e & 31) == lane && best_e < E) v[best_e >> 5] = -INFINITY;
  }
  if (lane == 0) {
    float w[kMaxTopK];
    float sum = 0.f;
    if (mode == 0) {
      for (int s = 0; s < k; ++s) {
        w[s] = __expf(sel_v[s] - mx_all) / denom;
        sum += w[s];
      }
      if (norm_topk && sum > 0.f)
        for (int s = 0; s < k; ++s) w[s] /= sum;
    } else {
      const float m = sel_v[0];
      for (int s = 0; s < k; ++s) {
        w[s] = __expf(sel_v[s] - m);
        sum += w[s];
      }
      for (int s = 0; s < k; ++s) w[s] /= sum;
    }
    for (int s = 0; s < k; ++s) {
      ids[static_cast<size_t>(t) * k + s] = sel_e[s];
      wts[static_cast<size_t>(t) * k + s] = w[s];
    }
  }
}

// Single CTA: histogram -> exclusive scan -> stable scatter. T * k pairs are at most a few
// tens of thousands (8192 tokens x top-8), which one 1024-thread CTA sorts in microseconds.
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ topk_ids, int* __restrict__ expert_offsets,
                 int* __restrict__ sorted_pair, int* __restrict__ sorted_token, int pairs, int k,
                 int e_begin, int e_end, const int* __restrict__ n_pairs_dev,
                 const int* __restrict__ token_map) {
  extern __shared__ int sh[];
  // n_pairs_dev: the pair count lives on the device (at most ``pairs``); token_map: the row of x that
  // token i stands for (a compacted list of rows of a larger buffer)
  if (n_pairs_dev) pairs = min(pairs, max(*n_pairs_dev, 0));
  const int El = e_end - e_begin;
  int* count = sh;            // [El]
  int* cursor = sh + El;      // [El]
  for (int i = threadIdx.x; i < El; i += blockDim.x) count[i] = 0;
  __syncthreads();
  for (int i = threadIdx.x; i < pairs; i += blockDim.x) {
    const int e = topk_ids[i];
    if (e >= e_begin && e < e_end) atomicAdd(&count[e - e_begin], 1);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int i = 0; i < El; ++i) {
      expert_offsets[i] = acc;
      cursor[i] = acc;
      acc += count[i];
    }
    expert_offsets[El] = acc;
  }
  __syncthreads();
  // Stable scatter: a warp walks its contiguous slice in order; warps are ordered by a second
  // pass over per-warp counts would cost more than it saves, so the scatter is done by one warp
  // per expert instead: warp w handles experts w, w + nwarps, ... scanning all pairs in order.
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
  for (int el = warp; el < El; el += nwarps) {
    const int e = e_begin + el;
    int pos = cursor[el];
    for (int base = 0; base < pairs; base += 32) {
      const int i = base + lane;
      const bool hit = i < pairs && topk_ids[i] == e;
      const unsigned m = __ballot_sync(0xffffffffu, hit);
      if (hit) {
        const int r = pos + __popc(m & ((1u << lane) - 1u));
        sorted_pair[r] = i;
        sorted_token[r] = token_map ? token_map[i / k] : i / k;
      }
      pos += __popc(m);
    }
  }
}

// The same result (stable in token order) for up to kAlignFastMaxExperts local experts, without the
// scatter's scan of all pairs per expert: warp w owns a contiguous slice of the pairs, counts its
// pairs per expert, a scan over (expert, warp) gives every warp its first row of every expert, and
// the warp then walks its slice once, 32 pairs per step, ranking equal experts inside a step with
// __match_any_sync. 32768 pairs over 128 experts: 32 steps per warp instead of 4096.
constexpr int kAlignFastMaxExperts = 256;
constexpr int kAlignBatch = 8;

__global__ void __launch_bounds__(1024)
moe_align_fast_kernel(const int* __restrict__ topk_ids, int* __restrict__ expert_offsets,
                      int* __restrict__ sorted_pair, int* __restrict__ sorted_token, int pairs, int k,
                      int e_begin, int e_end, const int* __restrict__ n_pairs_dev,
                      const int* __restrict__ token_map) {
  extern __shared__ int sh[];
  const int El = e_end - e_begin;
  if (n_pairs_dev) pairs = min(pairs, max(*n_pairs_dev, 0));
  int* wcount = sh;                    // [32][El]: pairs of warp w for expert e, then its first row
  int* total = sh + 32 * El;           // [El]
  for (int i = threadIdx.x; i < 32 * El; i += blockDim.x) wcount[i] = 0;
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int chunk = ((pairs + 31) / 32 + 31) / 32 * 32;      // per warp, a multiple of 32
  const int begin = warp * chunk, end = min(pairs, begin + chunk);
  int* mine = wcount + warp * El;
  // kAlignBatch steps per batch: their expert ids are loaded together (independent loads, one trip to
  // memory), then the steps run in order
  for (int base0 = begin; base0 < end; base0 += 32 * kAlignBatch) {
    int eb[kAlignBatch];
#pragma unroll
    for (int u = 0; u < kAlignBatch; ++u) {
      const int i = base0 + u * 32 + lane;
      eb[u] = i < end ? topk_ids[i] : -1;
    }
#pragma unroll
    for (int u = 0; u < kAlignBatch; ++u) {
      if (base0 + u * 32 >= end) break;                      // warp-uniform
      const int e = eb[u];
      const bool hit = e >= e_begin && e < e_end;
      const int key = hit ? e - e_begin : El + lane;         // lanes without a local expert match nobody
      const unsigned m = __match_any_sync(0xffffffffu, key);
      if (hit && (m & ((1u << lane) - 1u)) == 0u) mine[key] += __popc(m);   // lowest lane of each group
      __syncwarp();
    }
  }
  __syncthreads();
  for (int e = threadIdx.x; e < El; e += blockDim.x) {
    int acc = 0;
    for (int w = 0; w < 32; ++w) acc += wcount[w * El + e];
    total[e] = acc;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int e = 0; e < El; ++e) {
      expert_offsets[e] = acc;
      const int t = total[e];
      total[e] = acc;
      acc += t;
    }
    expert_offsets[El] = acc;
  }
  __syncthreads();
  for (int e = threadIdx.x; e < El; e += blockDim.x) {
    int run = total[e];
    for (int w = 0; w < 32; ++w) {
      const int c = wcount[w * El + e];
      wcount[w * El + e] = run;
      run += c;
    }
  }
  __syncthreads();
  for (int base0 = begin; base0 < end; base0 += 32 * kAlignBatch) {
    int eb[kAlignBatch];
#pragma unroll
    for (int u = 0; u < kAlignBatch; ++u) {
      const int i = base0 + u * 32 + lane;
      eb[u] = i < end ? topk_ids[i] : -1;
    }
#pragma unroll
    for (int u = 0; u < kAlignBatch; ++u) {
      if (base0 + u * 32 >= end) break;                      // warp-uniform
      const int i = base0 + u * 32 + lane;
      const int e = eb[u];
      const bool hit = e >= e_begin && e < e_end;
      const int key = hit ? e - e_begin : El + lane;
      const unsigned m = __match_any_sync(0xffffffffu, key);
      const unsigned before = m & ((1u << lane) - 1u);
      int r = 0;
      if (hit) r = mine[key] + __popc(before);
      __syncwarp();                                          // everybody has read the cursor
      if (hit) {
        sorted_pair[r] = i;
        sorted_token[r] = token_map ? token_map[i / k] : i / k;
        if (before == 0u) mine[key] += __popc(m);
      }
      __syncwarp();
    }
  }
}

__global__ void moe_gather_rows_kernel(const __nv_bfloat16* __restrict__ x,
                                       const int* __restrict__ sorted_token,
                                       const int* __restrict__ total_rows,
                                       __nv_bfloat16* __restrict__ out, int dim) {
  const int total = *total_rows;
  for (int r = blockIdx.x; r < total; r += gridDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(x + static_cast<size_t>(sorted_token[r]) * dim);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(r) * dim);
    for (int v = threadIdx.x; v < dim / 8; v += blockDim.x) dst[v] = src[v];
  }
}

// out[sorted_token[r], :] = y[r, :] for the rows in use (the inverse of the gather when every token
// has one pair, as the receive rows of the all-to-all path do: nothing is summed, unused rows of
// ``out`` are left alone).
__global__ void moe_scatter_rows_kernel(const __nv_bfloat16* __restrict__ y,
                                        const int* __restrict__ sorted_token,
                                        const int* __restrict__ total_rows,
                                        __nv_bfloat16* __restrict__ out, int dim) {
  const int total = *total_rows;
  for (int r = blockIdx.x; r < total; r += gridDim.x) {
    const uint4* src = reinterpret_cast<const uint4*>(y + static_cast<size_t>(r) * dim);
    uint4* dst = reinterpret_cast<uint4*>(out + static_cast<size_t>(sorted_token[r]) * dim);
    for (int v = threadIdx.x; v < dim / 8; v += blockDim.x) dst[v] = src[v];
  }
}

// inv_row[pair] = sorted row of the pair or -1 (not routed to a local expert)
__global__ void moe_invert_kernel(const int* __restrict__ sorted_pair,
                                  const int* __restrict__ total_rows, int* __restrict__ inv_row,
                                  int pairs) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < pairs) inv_row[i] = -1;
}
__global__ void moe_invert_fill_kernel(const int* __restrict__ sorted_pair,
                                       const int* __restrict__ total_rows,
                                       int* __restrict__ inv_row) {
  const int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r < *total_rows) inv_row[sorted_pair[r]] = r;
}

__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y,
                                   const int* __restrict__ inv_row, const float* __restrict__ wts,
                                   __nv_bfloat16* __restrict__ out,
                                   const __nv_bfloat16* __restrict__ residual, int k, int dim,
                                   int accumulate) {
  const int t = blockIdx.x;
  for (int v = threadIdx.x; v < dim / 8; v += blockDim.x) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    const __nv_bfloat16* base = nullptr;
    if (residual) base = residual;
    else if (accumulate) base = out;
    if (base) {
      const uint4 a = *reinterpret_cast<const uint4*>(base + static_cast<size_t>(t) * dim + v * 8);
      const uint32_t w4[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] = bf16_lo(w4[j]);
        acc[2 * j + 1] = bf16_hi(w4[j]);
      }
    }
    for (int s = 0; s < k; ++s) {
      const int r = inv_row[static_cast<size_t>(t) * k + s];
      if (r < 0) continue;
      const float w = wts[static_cast<size_t>(t) * k + s];
      const uint4 a = *reinterpret_cast<const uint4*>(y + static_cast<size_t>(r) * dim + v * 8);
      const uint32_t w4[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        acc[2 * j] += w * bf16_lo(w4[j]);
        acc[2 * j + 1] += w * bf16_hi(w4[j]);
      }
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]);
    o.y = pack_bf16(acc[2], acc[3]);
    o.z = pack_bf16(acc[4], acc[5]);
    o.w = pack_bf16(acc[6], acc[7]);
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(t) * dim + v * 8) = o;
  }
}

}  // namespace mx

using namespace mx;

// Switch for the slice-per-warp alignment kernel (on unless MLXCEL_B200_MOE_ALIGN_FAST=0 at load).
static int g_align_fast = 1;
extern "C" void mx_set_moe_align_fast(int on) { g_align_fast = on ? 1 : 0; }

extern "C" int mx_moe_route(const void* logits, int* topk_ids, float* topk_w, int T, int E, int k,
                            int mode, int norm_topk, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (T <= 0) return 0;
  if (E > 512 || k > kMaxTopK || k > E || k < 1) return -1;
  const int threads = 128;
  const int blocks = (T * 32 + threads - 1) / threads;
  moe_route_kernel<<<blocks, threads, 0, stream>>>(static_cast<const __nv_bfloat16*>(logits), topk_ids,
                                                   topk_w, T, E, k, mode, norm_topk);
  return static_cast<int>(cudaGetLastError());
}

// expert_offsets: [E_local + 1]; sorted_row doubles as sorted_pair (pair index = t * k + slot).
extern "C" int mx_moe_align(const int* topk_ids, int* expert_offsets, int* sorted_row,
                            int* sorted_token, int T, int k, int E, int e_begin, int e_end,
                            void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  (void)E;
  const int El = e_end - e_begin;
  if (El <= 0 || El > 4096) return -1;
  if (g_align_fast && El <= kAlignFastMaxExperts)
    moe_align_fast_kernel<<<1, 1024, 33 * El * sizeof(int), stream>>>(topk_ids, expert_offsets, sorted_row,
                                                                     sorted_token, T * k, k, e_begin, e_end,
                                                                     nullptr, nullptr);
  else
    moe_align_kernel<<<1, 1024, 2 * El * sizeof(int), stream>>>(topk_ids, expert_offsets, sorted_row,
                                                                sorted_token, T * k, k, e_begin, e_end,
                                                                nullptr, nullptr);
  return static_cast<int>(cudaGetLastError());
}

// As mx_moe_align with the number of (token, slot) pairs read on the device (n_pairs_dev, at most
// max_tokens * k) and, optionally, sorted_token[r] = token_map[token] instead of the token's index.
extern "C" int mx_moe_align_n(const int* topk_ids, const int* n_pairs_dev, const int* token_map,
                              int* expert_offsets, int* sorted_row, int* sorted_token, int max_tokens,
                              int k, int e_begin, int e_end, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int El = e_end - e_begin;
  if (El <= 0 || El > 4096 || n_pairs_dev == nullptr) return -1;
  if (g_align_fast && El <= kAlignFastMaxExperts)
    moe_align_fast_kernel<<<1, 1024, 33 * El * sizeof(int), stream>>>(topk_ids, expert_offsets, sorted_row,
                                                                     sorted_token, max_tokens * k, k, e_begin,
                                                                     e_end, n_pairs_dev, token_map);
  else
    moe_align_kernel<<<1, 1024, 2 * El * sizeof(int), stream>>>(topk_ids, expert_offsets, sorted_row,
                                                                sorted_token, max_tokens * k, k, e_begin,
                                                                e_end, n_pairs_dev, token_map);
  return static_cast<int>(cudaGetLastError());
}

// rows: upper bound of the row count (grid size); the true count is read from total_rows on
// the device (= expert_offsets[E_local]), so no host synchronisation is needed.
extern "C" int mx_moe_gather_rows_n(const void* x, const int* sorted_token, const int* total_rows,
                                    void* out, int max_rows, int dim, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (max_rows <= 0) return 0;
  if (dim % 8) return -1;
  moe_gather_rows_kernel<<<min(max_rows, 148 * 16), 128, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(x), sorted_token, total_rows, static_cast<__nv_bfloat16*>(out), dim);
  return static_cast<int>(cudaGetLastError());
}

extern "C" int mx_moe_scatter_rows_n(const void* y, const int* sorted_token, const int* total_rows,
                                     void* out, int max_rows, int dim, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (max_rows <= 0) return 0;
  if (dim % 8) return -1;
  moe_scatter_rows_kernel<<<min(max_rows, 148 * 16), 128, 0, stream>>>(
      static_cast<const __nv_bfloat16*>(y), sorted_token, total_rows, static_cast<__nv_bfloat16*>(out), dim);
  return static_cast<int>(cudaGetLastError());
}

// inv_row: [T * k] scratch (pair -> sorted row or -1), filled here.
extern "C" int mx_moe_combine_n(const void* y, const int* sorted_pair, const int* total_rows,
                                int* inv_row, const float* topk_w, void* out, const void* residual,
                                int T, int k, int dim, int max_rows, int accumulate, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (T <= 0) return 0;
  if (dim % 8) return -1;
  const int pairs = T * k;
  moe_invert_kernel<<<(pairs + 255) / 256, 256, 0, stream>>>(sorted_pair, total_rows, inv_row, pairs);
  if (max_rows > 0)
    moe_invert_fill_kernel<<<(max_rows + 255) / 256, 256, 0, stream>>>(sorted_pair, total_rows, inv_row);
  moe_combine_kernel<<<T, 128, 0, stream>>>(static_cast<const __nv_bfloat16*>(y), inv_row, topk_w,
                                            static_cast<__nv_bfloat16*>(out),
                                            static_cast<const __nv_bfloat16*>(residual), k, dim,
                                            accumulate);
  return static_cast<int>(cudaGetLastError());
}
