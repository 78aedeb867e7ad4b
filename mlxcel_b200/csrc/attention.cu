// Paged attention over the block pool [num_blocks, Hkv, block_size, D].
//
//  * paged_decode_kernel: one query token per sequence. A CTA owns (sequence, kv head, KV split)
//    and serves all G = Hq / Hkv query heads of that kv head so K and V are read once. Each warp
//    walks 32-token chunks: score phase is token-parallel (a lane owns one key row and reads it
//    with 16-byte loads, q comes from shared memory as broadcast reads), value phase is
//    dim-parallel (a lane owns D/32 output dims). Online softmax per warp in the exp2 domain,
//    warps merge in shared memory, KV splits merge in the last CTA to arrive for the
//    (sequence, kv head) pair (arrival counter in scratch, returned to zero).
//  * paged_prefill_kernel: chunked causal prefill. A CTA owns 128 (token, head-in-group) query
//    rows of one kv head and streams 64-token K/V tiles from the pool through shared memory.
//
// Both support sliding windows, attention sinks (a per-head logit that only enters the softmax
// denominator), logit soft-capping and 8-bit affine K/V (group 64) dequantized on load.
//
// Parity targets in the reference: paged_attention_decode_v2_partial + merge_states
// (src/lib/mlxcelverse/kernels/paged_attention_v2.cpp:286-459, paged_attention_v2_merge.cpp:113),
// the vector SDPA kernels of its MLX overlay (scaled_dot_product_attention.cu:65-397) and its
// chunked causal attention (src/lib/mlxcel-core/src/layers.rs:5798).
#include "api.h"
#include "common.cuh"

namespace mx {

constexpr float kLog2e = 1.4426950408889634f;

// ============================================================================= decode
constexpr int kDecWarps = 4;
constexpr int kDecThreads = kDecWarps * 32;

struct DecodeParams {
  const __nv_bfloat16* q;
  long long q_stride;
  const void* k_pool;
  const void* v_pool;
  const __nv_bfloat16* k_meta;
  const __nv_bfloat16* v_meta;
  const int* block_tables;
  const int* context_lens;
  const float* sinks;
  __nv_bfloat16* out;
  float* scratch_o;    // [B, Hkv, splits, G, D]
  float* scratch_ml;   // [B, Hkv, splits, G, 2]
  int* counters;       // [B * Hkv]
  int B, Hq, Hkv, block_size, max_blocks, window, num_splits;
  float scale_log2, softcap;
};

// Loads 8 consecutive elements of a K/V row as floats.
template <int KV_BITS>
__device__ __forceinline__ void load8(const void* pool, size_t elem_off, float (&f)[8]) {
  if (KV_BITS == 16) {
    const uint4 a = *reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(pool) + elem_off);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      f[2 * j] = bf16_lo(w[j]);
      f[2 * j + 1] = bf16_hi(w[j]);
    }
  } else if (KV_BITS == 4) {
    // two values per byte, even element in the low nibble: 8 elements = one 32-bit word
    const uint32_t w = *reinterpret_cast<const uint32_t*>(static_cast<const uint8_t*>(pool) + (elem_off >> 1));
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = static_cast<float>((w >> (4 * j)) & 0xFu);
  } else {
    const uint2 a = *reinterpret_cast<const uint2*>(static_cast<const uint8_t*>(pool) + elem_off);
    const uint32_t w[2] = {a.x, a.y};
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = static_cast<float>((w[j >> 2] >> (8 * (j & 3))) & 0xFFu);
  }
}

template <int D, int G, int KV_BITS>
__global__ void __launch_bounds__(kDecThreads)
paged_decode_kernel(const DecodeParams p) {
  constexpr int DPL = D / 32;  // output dims per lane
  __shared__ float q_s[G][D];                    // pre-scaled q (fp32)
  __shared__ float qsum_s[G][D / 64 > 0 ? D / 64 : 1];
  __shared__ float p_s[kDecWarps][G][32];        // probabilities of the current chunk
  __shared__ int row_s[kDecWarps][32];           // pool row of each token of the chunk (-1 = none)
  __shared__ float m_s[kDecWarps][G], l_s[kDecWarps][G];
  __shared__ float o_s[kDecWarps][G][D];
  __shared__ int last_s;

  const int split = blockIdx.x % p.num_splits;
  const int bh = blockIdx.x / p.num_splits;
  const int h = bh % p.Hkv, b = bh / p.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = p.context_lens[b];
  int begin = 0;
  if (p.window > 0 && len > p.window) begin = len - p.window;
  // Split the visible range [begin, len) into num_splits pieces of whole 32-token chunks.
  const int span = len - begin;
  int per = (span + p.num_splits - 1) / p.num_splits;
  per = ((per + 31) / 32) * 32;
  const int t0 = begin + split * per;
  const int t1 = min(len, t0 + per);

  for (int i = threadIdx.x; i < G * D; i += kDecThreads) {
    const int g = i / D, d = i - g * D;
    q_s[g][d] = __bfloat162float(p.q[static_cast<size_t>(b) * p.q_stride + (h * G + g) * D + d]) *
                p.scale_log2;
  }
  __syncthreads();
  if (KV_BITS == 8) {
    for (int i = threadIdx.x; i < G * (D / 64); i += kDecThreads) {
      const int g = i / (D / 64), grp = i - g * (D / 64);
      float s = 0.f;
      for (int d = 0; d < 64; ++d) s += q_s[g][grp * 64 + d];
      qsum_s[g][grp] = s;
    }
    __syncthreads();
  }

  float m_run[G], l_run[G], acc[G][DPL];
#pragma unroll
  for (int g = 0; g < G; ++g) {
    m_run[g] = -INFINITY;
    l_run[g] = 0.f;
#pragma unroll
    for (int j = 0; j < DPL; ++j) acc[g][j] = 0.f;
  }

  const int* table = p.block_tables + static_cast<size_t>(b) * p.max_blocks;
  for (int c0 = t0 + warp * 32; c0 < t1; c0 += kDecWarps * 32) {
    // ---- score phase: lane = token
    const int tok = c0 + lane;
    const bool valid = tok < t1;
    float s[G];
#pragma unroll
    for (int g = 0; g < G; ++g) s[g] = 0.f;
    int row = -1;
    if (valid) {
      const int blk = table[tok / p.block_size];
      row = (blk * p.Hkv + h) * p.block_size + (tok % p.block_size);
      const size_t base = static_cast<size_t>(row) * D;
      if (KV_BITS == 16) {
#pragma unroll 4
        for (int d0 = 0; d0 < D; d0 += 8) {
          float kf[8];
          load8<16>(p.k_pool, base + d0, kf);
#pragma unroll
          for (int g = 0; g < G; ++g) {
            const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][d0]);
            const float4 qb = *reinterpret_cast<const float4*>(&q_s[g][d0 + 4]);
            s[g] += kf[0] * qa.x + kf[1] * qa.y + kf[2] * qa.z + kf[3] * qa.w + kf[4] * qb.x +
                    kf[5] * qb.y + kf[6] * qb.z + kf[7] * qb.w;
          }
        }
      } else {
        const __nv_bfloat16* meta = p.k_meta + static_cast<size_t>(row) * (D / 64) * 2;
#pragma unroll
        for (int grp = 0; grp < D / 64; ++grp) {
          float part[G];
#pragma unroll
          for (int g = 0; g < G; ++g) part[g] = 0.f;
#pragma unroll 2
          for (int d0 = grp * 64; d0 < grp * 64 + 64; d0 += 8) {
            float kf[8];
            load8<KV_BITS>(p.k_pool, base + d0, kf);
#pragma unroll
            for (int g = 0; g < G; ++g) {
              const float4 qa = *reinterpret_cast<const float4*>(&q_s[g][d0]);
              const float4 qb = *reinterpret_cast<const float4*>(&q_s[g][d0 + 4]);
              part[g] += kf[0] * qa.x + kf[1] * qa.y + kf[2] * qa.z + kf[3] * qa.w + kf[4] * qb.x +
                         kf[5] * qb.y + kf[6] * qb.z + kf[7] * qb.w;
            }
          }
          const float sc = __bfloat162float(meta[grp * 2]);
          const float bi = __bfloat162float(meta[grp * 2 + 1]);
#pragma unroll
          for (int g = 0; g < G; ++g) s[g] += sc * part[g] + bi * qsum_s[g][grp];
        }
      }
    }
    row_s[warp][lane] = row;
    // ---- online softmax over the chunk
    float scale_old[G];
#pragma unroll
    for (int g = 0; g < G; ++g) {
      float sv = s[g];
      if (p.softcap > 0.f) {
        // s is in the log2 domain; cap in the natural domain.
        const float nat = sv / kLog2e;
        sv = p.softcap * tanhf(nat / p.softcap) * kLog2e;
      }
      if (!valid) sv = -INFINITY;
      const float cmax = warp_max(sv);
      const float m_new = fmaxf(m_run[g], cmax);
      const float pr = (valid && m_new > -INFINITY) ? exp2f(sv - m_new) : 0.f;
      const float csum = warp_sum(pr);
      scale_old[g] = (m_run[g] > -INFINITY) ? exp2f(m_run[g] - m_new) : 0.f;
      l_run[g] = l_run[g] * scale_old[g] + csum;
      m_run[g] = m_new;
      p_s[warp][g][lane] = pr;
    }
    __syncwarp();
#pragma unroll
    for (int g = 0; g < G; ++g)
#pragma unroll
      for (int j = 0; j < DPL; ++j) acc[g][j] *= scale_old[g];
    // ---- value phase: lane = DPL consecutive dims
    const int nt = min(32, t1 - c0);
    for (int t = 0; t < nt; ++t) {
      const int vrow = row_s[warp][t];
      float vf[DPL];
      if (KV_BITS == 16) {
        const __nv_bfloat16* vp =
            static_cast<const __nv_bfloat16*>(p.v_pool) + static_cast<size_t>(vrow) * D + lane * DPL;
        if (DPL == 4) {
          const uint2 a = *reinterpret_cast<const uint2*>(vp);
          vf[0] = bf16_lo(a.x);
          vf[1] = bf16_hi(a.x);
          vf[2] = bf16_lo(a.y);
          vf[3] = bf16_hi(a.y);
        } else if (DPL == 2) {
          const uint32_t a = *reinterpret_cast<const uint32_t*>(vp);
          vf[0] = bf16_lo(a);
          vf[1] = bf16_hi(a);
        } else {
#pragma unroll
          for (int j = 0; j < DPL; ++j) vf[j] = __bfloat162float(vp[j]);
        }
      } else {
        const uint8_t* vp = static_cast<const uint8_t*>(p.v_pool) + static_cast<size_t>(vrow) * D + lane * DPL;
        const int grp = (lane * DPL) / 64;
        const __nv_bfloat16* meta = p.v_meta + static_cast<size_t>(vrow) * (D / 64) * 2 + grp * 2;
        const float sc = __bfloat162float(meta[0]), bi = __bfloat162float(meta[1]);
#pragma unroll
        for (int j = 0; j < DPL; ++j) vf[j] = static_cast<float>(vp[j]) * sc + bi;
      }
#pragma unroll
      for (int g = 0; g < G; ++g) {
        const float pr = p_s[warp][g][t];
#pragma unroll
        for (int j = 0; j < DPL; ++j) acc[g][j] += pr * vf[j];
      }
    }
    __syncwarp();
  }

  // ---- merge warps
#pragma unroll
  for (int g = 0; g < G; ++g) {
    if (lane == 0) {
      m_s[warp][g] = m_run[g];
      l_s[warp][g] = l_run[g];
    }
#pragma unroll
    for (int j = 0; j < DPL; ++j) o_s[warp][g][lane * DPL + j] = acc[g][j];
  }
  __syncthreads();
  const size_t part_idx = (static_cast<size_t>(b) * p.Hkv + h) * p.num_splits + split;
  float* part_o = p.scratch_o + part_idx * (G * D);
  float* part_ml = p.scratch_ml + part_idx * (G * 2);
  for (int i = threadIdx.x; i < G * D; i += kDecThreads) {
    const int g = i / D, d = i - g * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) m = fmaxf(m, m_s[w][g]);
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < kDecWarps; ++w) {
      const float sc = (m_s[w][g] > -INFINITY) ? exp2f(m_s[w][g] - m) : 0.f;
      l += l_s[w][g] * sc;
      o += o_s[w][g][d] * sc;
    }
    if (p.num_splits == 1) {
      if (p.sinks != nullptr) {
        const float sk = p.sinks[h * G + g] * kLog2e;
        const float m2 = fmaxf(m, sk);
        const float sc = (m > -INFINITY) ? exp2f(m - m2) : 0.f;
        l = l * sc + exp2f(sk - m2);
        o *= sc;
      }
      const float r = l > 0.f ? o / l : 0.f;
      p.out[static_cast<size_t>(b) * p.Hq * D + (h * G + g) * D + d] = __float2bfloat16(r);
    } else {
      part_o[i] = o;
      if (d == 0) {
        part_ml[g * 2] = m;
        part_ml[g * 2 + 1] = l;
      }
    }
  }
  if (p.num_splits == 1) return;

  // ---- merge splits in the last CTA to arrive
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(&p.counters[bh], 1);
    const int last = prev == p.num_splits - 1;
    if (last) atomicExch(&p.counters[bh], 0);
    last_s = last;
  }
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  const size_t base_idx = (static_cast<size_t>(b) * p.Hkv + h) * p.num_splits;
  for (int i = threadIdx.x; i < G * D; i += kDecThreads) {
    const int g = i / D, d = i - g * D;
    float m = -INFINITY;
    for (int s2 = 0; s2 < p.num_splits; ++s2)
      m = fmaxf(m, __ldcg(&p.scratch_ml[(base_idx + s2) * (G * 2) + g * 2]));
    float sk = 0.f;
    if (p.sinks != nullptr) {
      sk = p.sinks[h * G + g] * kLog2e;
      m = fmaxf(m, sk);
    }
    float l = 0.f, o = 0.f;
    for (int s2 = 0; s2 < p.num_splits; ++s2) {
      const float ms = __ldcg(&p.scratch_ml[(base_idx + s2) * (G * 2) + g * 2]);
      const float ls = __ldcg(&p.scratch_ml[(base_idx + s2) * (G * 2) + g * 2 + 1]);
      const float sc = (ms > -INFINITY) ? exp2f(ms - m) : 0.f;
      l += ls * sc;
      o += __ldcg(&p.scratch_o[(base_idx + s2) * (G * D) + i]) * sc;
    }
    if (p.sinks != nullptr) l += exp2f(sk - m);
    const float r = l > 0.f ? o / l : 0.f;
    p.out[static_cast<size_t>(b) * p.Hq * D + (h * G + g) * D + d] = __float2bfloat16(r);
  }
}

// ============================================================================= prefill
constexpr int kPfWarps = 8;
constexpr int kPfThreads = kPfWarps * 32;
constexpr int kPfRows = kPfWarps * 16;  // 128 (token, head-in-group) rows per CTA
constexpr int kPfKv = 64;               // keys per tile

struct PrefillParams {
  const __nv_bfloat16* q;
  long long q_stride;
  const void* k_pool;
  const void* v_pool;
  const __nv_bfloat16* k_meta;
  const __nv_bfloat16* v_meta;
  const int* block_tables;
  const int* cu_q;
  const int* context_lens;
  const float* sinks;
  __nv_bfloat16* out;
  int num_seqs, Hq, Hkv, block_size, max_blocks, window, tiles_per_seq;
  float scale_log2, softcap;
};

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(addr));
}
__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                               uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, "
      "{%8, %9}, {%0, %1, %2, %3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr, bool pred) {
  const int sz = pred ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gptr), "r"(sz)
               : "memory");
}
// 4-, 8- or 16-byte asynchronous copy (cache-all variant: the only one that takes sizes below 16);
// a false predicate zero-fills the destination.
template <int BYTES>
__device__ __forceinline__ void cp_async_small(uint32_t smem_addr, const void* gptr, bool pred) {
  const int sz = pred ? BYTES : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], %2, %3;" ::"r"(smem_addr), "l"(gptr), "n"(BYTES), "r"(sz)
               : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Shared tiles are [rows][D] bf16 with the 16-byte chunk index XOR-swizzled by (row & 7).
template <int D>
__device__ __forceinline__ uint32_t swz(int row, int chunk) {
  return static_cast<uint32_t>(row * (D * 2) + ((chunk ^ (row & 7)) << 4));
}

template <int D, int G, int KV_BITS>
__global__ void __launch_bounds__(kPfThreads)
paged_prefill_kernel(const PrefillParams p) {
  constexpr int CH = D / 8;          // 16-byte chunks per row
  constexpr int TOK_PER_CTA = kPfRows / G;
  extern __shared__ __align__(128) uint8_t pf_smem[];
  uint8_t* q_sm = pf_smem;                              // [128][D]
  uint8_t* k_sm = q_sm + kPfRows * D * 2;               // 2 x [64][D]
  uint8_t* v_sm = k_sm + 2 * kPfKv * D * 2;             // 2 x [64][D]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int tile = blockIdx.x % p.tiles_per_seq;
  const int sh = blockIdx.x / p.tiles_per_seq;
  const int h = sh % p.Hkv, s = sh / p.Hkv;
  const int q0 = p.cu_q[s], q_len = p.cu_q[s + 1] - q0;
  const int tok0 = tile * TOK_PER_CTA;
  if (tok0 >= q_len) return;
  const int ctx = p.context_lens[s];
  const int pos_base = ctx - q_len;  // absolute position of query token 0
  const int* table = p.block_tables + static_cast<size_t>(s) * p.max_blocks;

  // ---- Q tile -> shared
  for (int i = threadIdx.x; i < kPfRows * CH; i += kPfThreads) {
    const int r = i / CH, c = i - r * CH;
    const int tok = tok0 + r / G, hq = h * G + (r % G);
    const bool ok = tok < q_len;
    const __nv_bfloat16* src =
        p.q + static_cast<size_t>(q0 + (ok ? tok : 0)) * p.q_stride + hq * D + c * 8;
    cp_async16(smem_u32(q_sm) + swz<D>(r, c), src, ok);
  }
  cp_async_commit();

  // Keys visible to this CTA: up to the last query token of the tile.
  const int last_tok = min(q_len, tok0 + TOK_PER_CTA) - 1;
  const int kv_end = pos_base + last_tok + 1;
  int kv_begin = 0;
  if (p.window > 0) kv_begin = max(0, pos_base + tok0 - p.window + 1);
  kv_begin = (kv_begin / kPfKv) * kPfKv;
  const int n_tiles = (kv_end - kv_begin + kPfKv - 1) / kPfKv;

  auto load_kv = [&](int t, int buf) {
    const int key0 = kv_begin + t * kPfKv;
    uint8_t* ks = k_sm + buf * kPfKv * D * 2;
    uint8_t* vs = v_sm + buf * kPfKv * D * 2;
    for (int i = threadIdx.x; i < kPfKv * CH; i += kPfThreads) {
      const int r = i / CH, c = i - r * CH;
      const int key = key0 + r;
      const bool ok = key < kv_end;
      const int blk = ok ? table[key / p.block_size] : 0;
      const size_t row = (static_cast<size_t>(blk) * p.Hkv + h) * p.block_size + (ok ? key % p.block_size : 0);
      if (KV_BITS == 16) {
        cp_async16(smem_u32(ks) + swz<D>(r, c),
                   static_cast<const __nv_bfloat16*>(p.k_pool) + row * D + c * 8, ok);
        cp_async16(smem_u32(vs) + swz<D>(r, c),
                   static_cast<const __nv_bfloat16*>(p.v_pool) + row * D + c * 8, ok);
      } else {
        float kf[8], vf[8];
        uint4 ko = make_uint4(0, 0, 0, 0), vo = make_uint4(0, 0, 0, 0);
        if (ok) {
          load8<KV_BITS>(p.k_pool, row * D + c * 8, kf);
          load8<KV_BITS>(p.v_pool, row * D + c * 8, vf);
          const int grp = (c * 8) / 64;
          const __nv_bfloat16* km = p.k_meta + row * (D / 64) * 2 + grp * 2;
          const __nv_bfloat16* vm = p.v_meta + row * (D / 64) * 2 + grp * 2;
          const float ksc = __bfloat162float(km[0]), kbi = __bfloat162float(km[1]);
          const float vsc = __bfloat162float(vm[0]), vbi = __bfloat162float(vm[1]);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            kf[j] = kf[j] * ksc + kbi;
            vf[j] = vf[j] * vsc + vbi;
          }
          ko = make_uint4(pack_bf16(kf[0], kf[1]), pack_bf16(kf[2], kf[3]), pack_bf16(kf[4], kf[5]),
                          pack_bf16(kf[6], kf[7]));
          vo = make_uint4(pack_bf16(vf[0], vf[1]), pack_bf16(vf[2], vf[3]), pack_bf16(vf[4], vf[5]),
                          pack_bf16(vf[6], vf[7]));
        }
        *reinterpret_cast<uint4*>(ks + swz<D>(r, c)) = ko;
        *reinterpret_cast<uint4*>(vs + swz<D>(r, c)) = vo;
      }
    }
    cp_async_commit();
  };

  if (n_tiles > 0) load_kv(0, 0);

  // Per-thread rows: r_lo = warp*16 + lane/4, r_hi = r_lo + 8
  const int r_lo = warp * 16 + (lane >> 2), r_hi = r_lo + 8;
  const int tq_lo = tok0 + r_lo / G, tq_hi = tok0 + r_hi / G;
  const int pos_lo = pos_base + tq_lo, pos_hi = pos_base + tq_hi;
  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;

  for (int t = 0; t < n_tiles; ++t) {
    const int buf = t & 1;
    if (t + 1 < n_tiles) {
      load_kv(t + 1, buf ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const uint32_t ks = smem_u32(k_sm + buf * kPfKv * D * 2);
    const uint32_t vs = smem_u32(v_sm + buf * kPfKv * D * 2);
    const uint32_t qs = smem_u32(q_sm);
    const int key0 = kv_begin + t * kPfKv;

    // ---- S = Q K^T (16 x 64 per warp)
    float sacc[kPfKv / 8][4];
#pragma unroll
    for (int i = 0; i < kPfKv / 8; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a[4];
      {
        const int row = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int chunk = kk * 2 + (lane >> 4);
        ldmatrix_x4(a, qs + swz<D>(row, chunk));
      }
#pragma unroll
      for (int nt = 0; nt < kPfKv / 16; ++nt) {
        uint32_t bfr[4];
        const int row = nt * 16 + (lane & 7) + (lane >> 4) * 8;
        const int chunk = kk * 2 + ((lane >> 3) & 1);
        ldmatrix_x4(bfr, ks + swz<D>(row, chunk));
        mma_bf16_16816(sacc[nt * 2], a, bfr[0], bfr[1]);
        mma_bf16_16816(sacc[nt * 2 + 1], a, bfr[2], bfr[3]);
      }
    }
    // ---- mask + online softmax
    float tmax_lo = -INFINITY, tmax_hi = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < kPfKv / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
        const int pos = (e < 2) ? pos_lo : pos_hi;
        float v = sacc[nt][e] * p.scale_log2;
        if (p.softcap > 0.f) v = p.softcap * tanhf(v / (kLog2e * p.softcap)) * kLog2e;
        const bool vis = key <= pos && key < kv_end && (p.window <= 0 || key > pos - p.window);
        v = vis ? v : -INFINITY;
        sacc[nt][e] = v;
        if (e < 2) tmax_lo = fmaxf(tmax_lo, v);
        else tmax_hi = fmaxf(tmax_hi, v);
      }
    }
    tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 1));
    tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 2));
    tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 1));
    tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 2));
    const float mn_lo = fmaxf(m_lo, tmax_lo), mn_hi = fmaxf(m_hi, tmax_hi);
    const float sc_lo = (m_lo > -INFINITY) ? exp2f(m_lo - mn_lo) : 0.f;
    const float sc_hi = (m_hi > -INFINITY) ? exp2f(m_hi - mn_hi) : 0.f;
    m_lo = mn_lo;
    m_hi = mn_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
    for (int nt = 0; nt < kPfKv / 8; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mref = (e < 2) ? mn_lo : mn_hi;
        const float pr = (mref > -INFINITY) ? exp2f(sacc[nt][e] - mref) : 0.f;
        sacc[nt][e] = pr;
        if (e < 2) sum_lo += pr;
        else sum_hi += pr;
      }
    }
    l_lo = l_lo * sc_lo + sum_lo;
    l_hi = l_hi * sc_hi + sum_hi;
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      o_acc[i][0] *= sc_lo;
      o_acc[i][1] *= sc_lo;
      o_acc[i][2] *= sc_hi;
      o_acc[i][3] *= sc_hi;
    }
    // ---- O += P V
#pragma unroll
    for (int kk = 0; kk < kPfKv / 16; ++kk) {
      uint32_t a[4];
      a[0] = pack_bf16(sacc[2 * kk][0], sacc[2 * kk][1]);
      a[1] = pack_bf16(sacc[2 * kk][2], sacc[2 * kk][3]);
      a[2] = pack_bf16(sacc[2 * kk + 1][0], sacc[2 * kk + 1][1]);
      a[3] = pack_bf16(sacc[2 * kk + 1][2], sacc[2 * kk + 1][3]);
#pragma unroll
      for (int nt = 0; nt < D / 16; ++nt) {
        uint32_t bfr[4];
        const int row = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
        const int chunk = nt * 2 + (lane >> 4);
        ldmatrix_x4_trans(bfr, vs + swz<D>(row, chunk));
        mma_bf16_16816(o_acc[nt * 2], a, bfr[0], bfr[1]);
        mma_bf16_16816(o_acc[nt * 2 + 1], a, bfr[2], bfr[3]);
      }
    }
    __syncthreads();
  }

  // ---- finalize
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  float osc_lo = 1.f, osc_hi = 1.f;
  if (p.sinks != nullptr) {
    const float sk_lo = p.sinks[h * G + (r_lo % G)] * kLog2e;
    const float sk_hi = p.sinks[h * G + (r_hi % G)] * kLog2e;
    const float m2_lo = fmaxf(m_lo, sk_lo), m2_hi = fmaxf(m_hi, sk_hi);
    osc_lo = (m_lo > -INFINITY) ? exp2f(m_lo - m2_lo) : 0.f;
    osc_hi = (m_hi > -INFINITY) ? exp2f(m_hi - m2_hi) : 0.f;
    l_lo = l_lo * osc_lo + exp2f(sk_lo - m2_lo);
    l_hi = l_hi * osc_hi + exp2f(sk_hi - m2_hi);
  }
  const float inv_lo = l_lo > 0.f ? osc_lo / l_lo : 0.f;
  const float inv_hi = l_hi > 0.f ? osc_hi / l_hi : 0.f;
  if (tq_lo < q_len) {
    __nv_bfloat16* dst = p.out + static_cast<size_t>(q0 + tq_lo) * p.Hq * D + (h * G + r_lo % G) * D;
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
      *reinterpret_cast<uint32_t*>(dst + i * 8 + (lane & 3) * 2) =
          pack_bf16(o_acc[i][0] * inv_lo, o_acc[i][1] * inv_lo);
  }
  if (tq_hi < q_len) {
    __nv_bfloat16* dst = p.out + static_cast<size_t>(q0 + tq_hi) * p.Hq * D + (h * G + r_hi % G) * D;
#pragma unroll
    for (int i = 0; i < D / 8; ++i)
      *reinterpret_cast<uint32_t*>(dst + i * 8 + (lane & 3) * 2) =
          pack_bf16(o_acc[i][2] * inv_hi, o_acc[i][3] * inv_hi);
  }
}

// ============================================================================= decode (tensor core)
// Flash-decoding with GQA packing: the G query heads of one kv head form the rows of a 16-row
// MMA tile, so K and V are read once per kv head and the score / value products run on tensor
// cores (mma.sync m16n8k16; the kernel is bound by the KV stream, not by math).
// A CTA owns (sequence, kv head, KV split). Its 4 warps are independent streams: warp w takes
// the 16-key groups w, w+4, ... of the split, each through its own 3-stage cp.async ring in
// shared memory (no CTA-wide barrier inside the loop), keeps its own online-softmax state and
// the warps merge once at the end.
constexpr int kDmWarps = 4;
constexpr int kDmThreads = kDmWarps * 32;
constexpr int kDmStages = 3;
constexpr int kDmKeys = 16;  // keys per group (one MMA k-step of P V)

template <int D, int KV_BITS, bool BS16>
__global__ void __launch_bounds__(kDmThreads)
paged_decode_mma_kernel(const DecodeParams p, const int G) {
  constexpr int CH = D / 8;
  constexpr int TILE_BYTES = kDmKeys * D * 2;            // one K (or V) group in bf16
  constexpr int STAGE_BYTES = 2 * TILE_BYTES;            // K + V
  constexpr int WARP_BYTES = kDmStages * STAGE_BYTES;
  // Quantized pools: a ring stage holds the RAW group (K codes, V codes, K and V scale/offset
  // pairs), fetched with cp.async like the bf16 tiles so that the ring keeps several groups in
  // flight; the group being consumed is expanded to bf16 into one tile pair per warp that sits
  // behind the ring. (Expanding at load time, with plain loads, serialised every group on its own
  // memory latency: 225 us instead of 57 us for the bf16 pool on 64 x 1152 keys.)
  constexpr int RAW_ROW = D * KV_BITS / 8;               // code bytes per key
  constexpr int META_ROW = (D / 64) * 4;                 // (scale, offset) bf16 pairs per key
  constexpr int RAW_STAGE = ((2 * kDmKeys * (RAW_ROW + META_ROW)) + 127) / 128 * 128;
  constexpr bool kQuant = KV_BITS != 16;
  static_assert(!kQuant || kDmStages * RAW_STAGE + STAGE_BYTES <= WARP_BYTES, "raw ring + expanded tile fit the ring");
  extern __shared__ __align__(128) uint8_t dm_smem[];
  uint8_t* q_sm = dm_smem;                               // [16][D] bf16 (swizzled)
  uint8_t* kv_sm = dm_smem + 16 * D * 2;                 // 4 warps x stages x (K, V)
  __shared__ float m_s[kDmWarps][16], l_s[kDmWarps][16];
  __shared__ int last_s;
  pdl_trigger();

  const int split = blockIdx.x % p.num_splits;
  const int bh = blockIdx.x / p.num_splits;
  const int h = bh % p.Hkv, b = bh / p.Hkv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int len = p.context_lens[b];
  int begin = 0;
  if (p.window > 0 && len > p.window) begin = len - p.window;
  const int g_begin = begin / kDmKeys;                          // first key group
  const int g_end = (len + kDmKeys - 1) / kDmKeys;              // one past the last key group
  const int n_groups = max(0, g_end - g_begin);
  int per = (n_groups + p.num_splits - 1) / p.num_splits;
  per = ((per + kDmWarps - 1) / kDmWarps) * kDmWarps;
  const int s_begin = g_begin + split * per;
  const int s_end = min(g_end, s_begin + per);
  const int* table = p.block_tables + static_cast<size_t>(b) * p.max_blocks;

  // Context lengths and block tables are step inputs (uploaded by copies, never written by a
  // kernel of the step) and every key but the newest is already in the pool: the head of this
  // CTA's KV stream is requested into L2 while the previous kernel (the one that appends the
  // newest key and writes q) is still running. L2 is the coherence point, so the newest key is
  // seen by the loads below whether or not its line was prefetched early.
  if constexpr (BS16 && KV_BITS == 16) {
    constexpr int kPrefetchGroups = 8;
    const int grp = s_begin + static_cast<int>(threadIdx.x);
    if (threadIdx.x < kPrefetchGroups && grp < s_end) {
      const size_t row16 = (static_cast<size_t>(table[grp]) * p.Hkv + h) * kDmKeys;
      bulk_prefetch_l2(static_cast<const __nv_bfloat16*>(p.k_pool) + row16 * D, TILE_BYTES);
      bulk_prefetch_l2(static_cast<const __nv_bfloat16*>(p.v_pool) + row16 * D, TILE_BYTES);
    }
  }
  pdl_wait();

  // ---- Q tile (rows >= G are zero)
  for (int i = threadIdx.x; i < 16 * CH; i += kDmThreads) {
    const int r = i / CH, c = i - r * CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < G)
      v = *reinterpret_cast<const uint4*>(p.q + static_cast<size_t>(b) * p.q_stride +
                                          static_cast<size_t>(h * G + r) * D + c * 8);
    *reinterpret_cast<uint4*>(q_sm + swz<D>(r, c)) = v;
  }
  __syncthreads();
  uint32_t qf[D / 16][4];
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
    const int chunk = kk * 2 + (lane >> 4);
    ldmatrix_x4(qf[kk], smem_u32(q_sm) + swz<D>(row, chunk));
  }

  uint8_t* my_sm = kv_sm + warp * WARP_BYTES;
  // Per-lane constants of the load pattern: chunk i = lane + 32 * it covers row i / CH,
  // 16-byte column i % CH of the 16 x D tile.
  auto load_group = [&](int grp, int stage, int blk16) {
    // grp: key group index (16 keys); blk16: pool block of the group when block_size == 16.
    uint8_t* ks = my_sm + stage * STAGE_BYTES;
    uint8_t* vs = ks + TILE_BYTES;
    if (grp < s_end) {
      const size_t row16 = (static_cast<size_t>(blk16) * p.Hkv + h) * kDmKeys;
      const int rows_ok = len - grp * kDmKeys;  // rows below this index hold real keys
      if constexpr (!kQuant) {
#pragma unroll
        for (int it = 0; it < (kDmKeys * CH) / 32; ++it) {
          const int i = lane + it * 32;
          const int r = i / CH, c = i - r * CH;
          const bool ok = r < rows_ok;
          size_t row;
          if (BS16) {
            row = row16 + r;
          } else {
            const int key = grp * kDmKeys + r;
            const int blk = ok ? table[key / p.block_size] : 0;
            row = (static_cast<size_t>(blk) * p.Hkv + h) * p.block_size + (ok ? key % p.block_size : 0);
          }
          cp_async16(smem_u32(ks) + swz<D>(r, c),
                     static_cast<const __nv_bfloat16*>(p.k_pool) + row * D + c * 8, ok);
          cp_async16(smem_u32(vs) + swz<D>(r, c),
                     static_cast<const __nv_bfloat16*>(p.v_pool) + row * D + c * 8, ok);
        }
      }
      if constexpr (kQuant) {
        // raw stage: [K codes 16 x RAW_ROW][V codes][K meta 16 x META_ROW][V meta]
        uint8_t* raw = my_sm + stage * RAW_STAGE;
        constexpr int CHQ = RAW_ROW / 16;                // 16-byte pieces of codes per key
#pragma unroll
        for (int it = 0; it < (kDmKeys * CHQ + 31) / 32; ++it) {
          const int i = lane + it * 32;
          if (i < kDmKeys * CHQ) {
            const int r = i / CHQ, c = i - r * CHQ;
            const bool ok = r < rows_ok;
            size_t row;
            if (BS16) {
              row = row16 + r;
            } else {
              const int key = grp * kDmKeys + r;
              const int blk = ok ? table[key / p.block_size] : 0;
              row = (static_cast<size_t>(blk) * p.Hkv + h) * p.block_size + (ok ? key % p.block_size : 0);
            }
            cp_async16(smem_u32(raw) + r * RAW_ROW + c * 16,
                       static_cast<const uint8_t*>(p.k_pool) + row * RAW_ROW + c * 16, ok);
            cp_async16(smem_u32(raw) + kDmKeys * RAW_ROW + r * RAW_ROW + c * 16,
                       static_cast<const uint8_t*>(p.v_pool) + row * RAW_ROW + c * 16, ok);
          }
        }
        {
          const int r = lane & 15;
          const bool ok = r < rows_ok;
          size_t row;
          if (BS16) {
            row = row16 + r;
          } else {
            const int key = grp * kDmKeys + r;
            const int blk = ok ? table[key / p.block_size] : 0;
            row = (static_cast<size_t>(blk) * p.Hkv + h) * p.block_size + (ok ? key % p.block_size : 0);
          }
          const uint8_t* src = reinterpret_cast<const uint8_t*>(lane < 16 ? p.k_meta : p.v_meta) + row * META_ROW;
          const uint32_t dst = smem_u32(raw) + 2 * kDmKeys * RAW_ROW + (lane < 16 ? 0 : kDmKeys * META_ROW) + r * META_ROW;
          cp_async_small<META_ROW>(dst, src, ok);
        }
      }
    }
    cp_async_commit();
  };
  // Block-table entries are fetched one ring slot ahead of the loads that need them.
  auto table_at = [&](int grp) -> int { return (BS16 && grp < s_end) ? table[grp] : 0; };

  float m_lo = -INFINITY, m_hi = -INFINITY, l_lo = 0.f, l_hi = 0.f;
  float o_acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f;

  const int first = s_begin + warp;
#pragma unroll
  for (int s = 0; s < kDmStages - 1; ++s)
    load_group(first + s * kDmWarps, s, table_at(first + s * kDmWarps));
  int blk_next = table_at(first + (kDmStages - 1) * kDmWarps);

  int stage = 0;
  for (int grp = first; grp < s_end; grp += kDmWarps) {
    {
      int ls = stage + kDmStages - 1;
      if (ls >= kDmStages) ls -= kDmStages;
      load_group(grp + (kDmStages - 1) * kDmWarps, ls, blk_next);
      blk_next = table_at(grp + kDmStages * kDmWarps);
    }
    cp_async_wait<kDmStages - 1>();
    __syncwarp();
    uint32_t ks = smem_u32(my_sm + stage * STAGE_BYTES);
    if constexpr (kQuant) {
      // expand the raw group of this stage into the warp's bf16 tile pair
      const uint8_t* raw = my_sm + stage * RAW_STAGE;
      uint8_t* tile = my_sm + kDmStages * RAW_STAGE;
#pragma unroll
      for (int kv = 0; kv < 2; ++kv) {
        const uint8_t* codes = raw + kv * kDmKeys * RAW_ROW;
        const uint8_t* meta = raw + 2 * kDmKeys * RAW_ROW + kv * kDmKeys * META_ROW;
        uint8_t* dst = tile + kv * TILE_BYTES;
#pragma unroll
        for (int it = 0; it < (kDmKeys * CH) / 32; ++it) {
          const int i = lane + it * 32;
          const int r = i / CH, c = i - r * CH;
          float f[8];
          if (KV_BITS == 8) {
            const uint2 a = *reinterpret_cast<const uint2*>(codes + r * RAW_ROW + c * 8);
            const uint32_t w[2] = {a.x, a.y};
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = static_cast<float>((w[j >> 2] >> (8 * (j & 3))) & 0xFFu);
          } else {
            const uint32_t w = *reinterpret_cast<const uint32_t*>(codes + r * RAW_ROW + c * 4);
#pragma unroll
            for (int j = 0; j < 8; ++j) f[j] = static_cast<float>((w >> (4 * j)) & 0xFu);
          }
          const uint32_t m = *reinterpret_cast<const uint32_t*>(meta + r * META_ROW + ((c * 8) / 64) * 4);
          const float sc = bf16_lo(m), bi = bf16_hi(m);
#pragma unroll
          for (int j = 0; j < 8; ++j) f[j] = f[j] * sc + bi;
          *reinterpret_cast<uint4*>(dst + swz<D>(r, c)) =
              make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
        }
      }
      __syncwarp();
      ks = smem_u32(tile);
    }
    const uint32_t vs = ks + TILE_BYTES;
    float sacc[2][4];
#pragma unroll
    for (int i = 0; i < 2; ++i) sacc[i][0] = sacc[i][1] = sacc[i][2] = sacc[i][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t bfr[4];
      const int row = (lane & 7) + (lane >> 4) * 8;
      const int chunk = kk * 2 + ((lane >> 3) & 1);
      ldmatrix_x4(bfr, ks + swz<D>(row, chunk));
      mma_bf16_16816(sacc[0], qf[kk], bfr[0], bfr[1]);
      mma_bf16_16816(sacc[1], qf[kk], bfr[2], bfr[3]);
    }
    const int key0 = grp * kDmKeys;
    float tmax_lo = -INFINITY, tmax_hi = -INFINITY;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int key = key0 + nt * 8 + (lane & 3) * 2 + (e & 1);
        float v = sacc[nt][e] * p.scale_log2;
        if (p.softcap > 0.f) v = p.softcap * tanhf(v / (kLog2e * p.softcap)) * kLog2e;
        v = (key >= begin && key < len) ? v : -INFINITY;
        sacc[nt][e] = v;
        if (e < 2) tmax_lo = fmaxf(tmax_lo, v);
        else tmax_hi = fmaxf(tmax_hi, v);
      }
    }
    tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 1));
    tmax_lo = fmaxf(tmax_lo, __shfl_xor_sync(0xffffffffu, tmax_lo, 2));
    tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 1));
    tmax_hi = fmaxf(tmax_hi, __shfl_xor_sync(0xffffffffu, tmax_hi, 2));
    const float mn_lo = fmaxf(m_lo, tmax_lo), mn_hi = fmaxf(m_hi, tmax_hi);
    const float sc_lo = (m_lo > -INFINITY) ? exp2f(m_lo - mn_lo) : 0.f;
    const float sc_hi = (m_hi > -INFINITY) ? exp2f(m_hi - mn_hi) : 0.f;
    m_lo = mn_lo;
    m_hi = mn_hi;
    float sum_lo = 0.f, sum_hi = 0.f;
#pragma unroll
    for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float mref = (e < 2) ? mn_lo : mn_hi;
        const float pr = (mref > -INFINITY) ? exp2f(sacc[nt][e] - mref) : 0.f;
        sacc[nt][e] = pr;
        if (e < 2) sum_lo += pr;
        else sum_hi += pr;
      }
    }
    l_lo = l_lo * sc_lo + sum_lo;
    l_hi = l_hi * sc_hi + sum_hi;
    // The running maximum settles after the first groups: skip the 64-register rescale
    // whenever no row of the warp moved its maximum.
    if (__any_sync(0xffffffffu, sc_lo != 1.0f || sc_hi != 1.0f)) {
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        o_acc[i][0] *= sc_lo;
        o_acc[i][1] *= sc_lo;
        o_acc[i][2] *= sc_hi;
        o_acc[i][3] *= sc_hi;
      }
    }
    uint32_t a[4];
    a[0] = pack_bf16(sacc[0][0], sacc[0][1]);
    a[1] = pack_bf16(sacc[0][2], sacc[0][3]);
    a[2] = pack_bf16(sacc[1][0], sacc[1][1]);
    a[3] = pack_bf16(sacc[1][2], sacc[1][3]);
#pragma unroll
    for (int nt = 0; nt < D / 16; ++nt) {
      uint32_t bfr[4];
      const int row = (lane & 7) + ((lane >> 3) & 1) * 8;
      const int chunk = nt * 2 + (lane >> 4);
      ldmatrix_x4_trans(bfr, vs + swz<D>(row, chunk));
      mma_bf16_16816(o_acc[nt * 2], a, bfr[0], bfr[1]);
      mma_bf16_16816(o_acc[nt * 2 + 1], a, bfr[2], bfr[3]);
    }
    if (++stage == kDmStages) stage = 0;
  }
  cp_async_wait<0>();

  // ---- merge the 4 warps (the KV ring is reused as an fp32 [warp][16][D] buffer)
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 1);
  l_lo += __shfl_xor_sync(0xffffffffu, l_lo, 2);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 1);
  l_hi += __shfl_xor_sync(0xffffffffu, l_hi, 2);
  __syncthreads();
  float* o_s = reinterpret_cast<float*>(kv_sm);
  {
    const int r_lo = lane >> 2, r_hi = r_lo + 8;
    if ((lane & 3) == 0) {
      m_s[warp][r_lo] = m_lo;
      l_s[warp][r_lo] = l_lo;
      m_s[warp][r_hi] = m_hi;
      l_s[warp][r_hi] = l_hi;
    }
#pragma unroll
    for (int i = 0; i < D / 8; ++i) {
      const int col = i * 8 + (lane & 3) * 2;
      float* dlo = o_s + (warp * 16 + r_lo) * D + col;
      float* dhi = o_s + (warp * 16 + r_hi) * D + col;
      dlo[0] = o_acc[i][0];
      dlo[1] = o_acc[i][1];
      dhi[0] = o_acc[i][2];
      dhi[1] = o_acc[i][3];
    }
  }
  __syncthreads();
  const size_t part_idx = (static_cast<size_t>(b) * p.Hkv + h) * p.num_splits + split;
  float* part_o = p.scratch_o + part_idx * (static_cast<size_t>(G) * D);
  float* part_ml = p.scratch_ml + part_idx * (static_cast<size_t>(G) * 2);
  for (int i = threadIdx.x; i < G * D; i += kDmThreads) {
    const int g = i / D, d = i - g * D;
    float m = -INFINITY;
#pragma unroll
    for (int w = 0; w < kDmWarps; ++w) m = fmaxf(m, m_s[w][g]);
    float l = 0.f, o = 0.f;
#pragma unroll
    for (int w = 0; w < kDmWarps; ++w) {
      const float sc = (m_s[w][g] > -INFINITY) ? exp2f(m_s[w][g] - m) : 0.f;
      l += l_s[w][g] * sc;
      o += o_s[(w * 16 + g) * D + d] * sc;
    }
    if (p.num_splits == 1) {
      if (p.sinks != nullptr) {
        const float sk = p.sinks[h * G + g] * kLog2e;
        const float m2 = fmaxf(m, sk);
        const float sc = (m > -INFINITY) ? exp2f(m - m2) : 0.f;
        l = l * sc + exp2f(sk - m2);
        o *= sc;
      }
      const float r = l > 0.f ? o / l : 0.f;
      p.out[static_cast<size_t>(b) * p.Hq * D + (h * G + g) * D + d] = __float2bfloat16(r);
    } else {
      part_o[i] = o;
      if (d == 0) {
        part_ml[g * 2] = m;
        part_ml[g * 2 + 1] = l;
      }
    }
  }
  if (p.num_splits == 1) return;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int prev = atomicAdd(&p.counters[bh], 1);
    const int last = prev == p.num_splits - 1;
    if (last) atomicExch(&p.counters[bh], 0);
    last_s = last;
  }
  __syncthreads();
  if (!last_s) return;
  __threadfence();
  const size_t base_idx = (static_cast<size_t>(b) * p.Hkv + h) * p.num_splits;
  for (int i = threadIdx.x; i < G * D; i += kDmThreads) {
    const int g = i / D, d = i - g * D;
    float m = -INFINITY;
    for (int s2 = 0; s2 < p.num_splits; ++s2)
      m = fmaxf(m, __ldcg(&p.scratch_ml[(base_idx + s2) * (G * 2) + g * 2]));
    float sk = 0.f;
    if (p.sinks != nullptr) {
      sk = p.sinks[h * G + g] * kLog2e;
      m = fmaxf(m, sk);
    }
    float l = 0.f, o = 0.f;
    for (int s2 = 0; s2 < p.num_splits; ++s2) {
      const float ms = __ldcg(&p.scratch_ml[(base_idx + s2) * (G * 2) + g * 2]);
      const float ls = __ldcg(&p.scratch_ml[(base_idx + s2) * (G * 2) + g * 2 + 1]);
      const float sc = (ms > -INFINITY) ? exp2f(ms - m) : 0.f;
      l += ls * sc;
      o += __ldcg(&p.scratch_o[(base_idx + s2) * (static_cast<size_t>(G) * D) + i]) * sc;
    }
    if (p.sinks != nullptr) l += exp2f(sk - m);
    const float r = l > 0.f ? o / l : 0.f;
    p.out[static_cast<size_t>(b) * p.Hq * D + (h * G + g) * D + d] = __float2bfloat16(r);
  }
}

template <int D, int KV_BITS, bool BS16>
static int launch_decode_mma_bs(const DecodeParams& p, int G, int grid, cudaStream_t st) {
  constexpr int smem = 16 * D * 2 + kDmWarps * kDmStages * 2 * kDmKeys * D * 2;
  static_assert(kDmWarps * kDmStages * 2 * kDmKeys * D * 2 >= kDmWarps * 16 * D * 4, "merge buffer");
  auto kern = paged_decode_mma_kernel<D, KV_BITS, BS16>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout,
                         cudaSharedmemCarveoutMaxShared);
    configured = true;
  }
  return static_cast<int>(launch_kernel(kern, dim3(grid), dim3(kDmThreads), smem, st, p, G));
}

template <int D, int KV_BITS>
static int launch_decode_mma(const DecodeParams& p, int G, int grid, cudaStream_t st) {
  if (p.block_size == kDmKeys) return launch_decode_mma_bs<D, KV_BITS, true>(p, G, grid, st);
  return launch_decode_mma_bs<D, KV_BITS, false>(p, G, grid, st);
}

// ----------------------------------------------------------------------------- dispatch
template <int KV_BITS>
static int launch_decode(const DecodeParams& p, int D, int G, int grid, cudaStream_t st) {
#define MX_DEC(D_, G_)                                                         \
  if (D == D_ && G == G_) {                                                    \
    paged_decode_kernel<D_, G_, KV_BITS><<<grid, kDecThreads, 0, st>>>(p);     \
    return static_cast<int>(cudaGetLastError());                               \
  }
  MX_DEC(128, 1) MX_DEC(128, 2) MX_DEC(128, 4) MX_DEC(128, 8)
  MX_DEC(64, 1) MX_DEC(64, 2) MX_DEC(64, 4) MX_DEC(64, 8)
  MX_DEC(256, 1) MX_DEC(256, 2) MX_DEC(256, 4) MX_DEC(256, 8)      // Gemma-class heads
#undef MX_DEC
  return -1;
}

template <int D, int G, int KV_BITS>
static int launch_prefill_one(const PrefillParams& p, int grid, cudaStream_t st) {
  constexpr int smem = (kPfRows + 4 * kPfKv) * D * 2;
  auto kern = paged_prefill_kernel<D, G, KV_BITS>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    prefer_max_shared(kern);
    configured = true;
  }
  kern<<<grid, kPfThreads, smem, st>>>(p);
  return static_cast<int>(cudaGetLastError());
}

template <int KV_BITS>
static int launch_prefill(const PrefillParams& p, int D, int G, int grid, cudaStream_t st) {
#define MX_PF(D_, G_) \
  if (D == D_ && G == G_) return launch_prefill_one<D_, G_, KV_BITS>(p, grid, st);
  MX_PF(128, 1) MX_PF(128, 2) MX_PF(128, 4) MX_PF(128, 8)
  MX_PF(64, 1) MX_PF(64, 2) MX_PF(64, 4) MX_PF(64, 8)
  MX_PF(256, 1) MX_PF(256, 2) MX_PF(256, 4) MX_PF(256, 8)          // Gemma-class heads
#undef MX_PF
  return -1;
}

}  // namespace mx

using namespace mx;

extern "C" long long mx_paged_decode_scratch_floats(int B, int Hq, int D, int num_splits) {
  // o partials + (m, l) pairs + one counter per (sequence, kv head) (<= B * Hq ints)
  return static_cast<long long>(B) * Hq * num_splits * (D + 2) + static_cast<long long>(B) * Hq + 64;
}

extern "C" int mx_paged_decode(const void* q, long long q_stride, const void* k_pool,
                               const void* v_pool, const void* k_meta, const void* v_meta,
                               const int* block_tables, const int* context_lens, const float* sinks,
                               void* out, float* scratch, int B, int Hq, int Hkv, int D,
                               int block_size, int max_blocks, int window, float scale,
                               float softcap, int kv_bits, int num_splits, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (B <= 0) return 0;
  if (Hq % Hkv) return -1;
  if (num_splits < 1) num_splits = 1;
  const int G = Hq / Hkv;
  DecodeParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_stride;
  p.k_pool = k_pool;
  p.v_pool = v_pool;
  p.k_meta = static_cast<const __nv_bfloat16*>(k_meta);
  p.v_meta = static_cast<const __nv_bfloat16*>(v_meta);
  p.block_tables = block_tables;
  p.context_lens = context_lens;
  p.sinks = sinks;
  p.out = static_cast<__nv_bfloat16*>(out);
  // scratch layout: counters first (they must stay zero between calls), then (m,l), then o.
  p.counters = reinterpret_cast<int*>(scratch);
  const size_t n_cnt = ((static_cast<size_t>(B) * Hkv + 63) / 64) * 64;
  p.scratch_ml = scratch + n_cnt;
  p.scratch_o = p.scratch_ml + static_cast<size_t>(B) * Hkv * num_splits * G * 2;
  p.B = B;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.block_size = block_size;
  p.max_blocks = max_blocks;
  p.window = window;
  p.num_splits = num_splits;
  p.scale_log2 = scale * kLog2e;
  p.softcap = softcap;
  const int grid = B * Hkv * num_splits;
  if (G <= 16 && (D == 128 || D == 64) && block_size % 16 == 0 && (q_stride % 8) == 0 &&
      (reinterpret_cast<uintptr_t>(q) & 15) == 0) {
    if (kv_bits == 16)
      return D == 128 ? launch_decode_mma<128, 16>(p, G, grid, stream)
                      : launch_decode_mma<64, 16>(p, G, grid, stream);
    if (kv_bits == 8)
      return D == 128 ? launch_decode_mma<128, 8>(p, G, grid, stream)
                      : launch_decode_mma<64, 8>(p, G, grid, stream);
    if (kv_bits == 4)
      return D == 128 ? launch_decode_mma<128, 4>(p, G, grid, stream)
                      : launch_decode_mma<64, 4>(p, G, grid, stream);
    return -1;
  }
  if (kv_bits == 16) return launch_decode<16>(p, D, G, grid, stream);
  if (kv_bits == 8) return launch_decode<8>(p, D, G, grid, stream);
  return -1;
}

extern "C" int mx_paged_prefill(const void* q, long long q_stride, const void* k_pool,
                                const void* v_pool, const void* k_meta, const void* v_meta,
                                const int* block_tables, const int* cu_q, const int* context_lens,
                                const float* sinks, void* out, int num_seqs, int total_q,
                                int max_q_len, int Hq, int Hkv, int D, int block_size,
                                int max_blocks, int window, float scale, float softcap, int kv_bits,
                                void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (num_seqs <= 0 || total_q <= 0) return 0;
  if (Hq % Hkv) return -1;
  const int G = Hq / Hkv;
  if (kPfRows % G) return -1;
  PrefillParams p{};
  p.q = static_cast<const __nv_bfloat16*>(q);
  p.q_stride = q_stride;
  p.k_pool = k_pool;
  p.v_pool = v_pool;
  p.k_meta = static_cast<const __nv_bfloat16*>(k_meta);
  p.v_meta = static_cast<const __nv_bfloat16*>(v_meta);
  p.block_tables = block_tables;
  p.cu_q = cu_q;
  p.context_lens = context_lens;
  p.sinks = sinks;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.num_seqs = num_seqs;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.block_size = block_size;
  p.max_blocks = max_blocks;
  p.window = window;
  const int tok_per_cta = kPfRows / G;
  p.tiles_per_seq = (max_q_len + tok_per_cta - 1) / tok_per_cta;
  p.scale_log2 = scale * kLog2e;
  p.softcap = softcap;
  const long long grid = static_cast<long long>(num_seqs) * Hkv * p.tiles_per_seq;
  if (grid > 0x7fffffffll) return -1;
  if (kv_bits == 16) return launch_prefill<16>(p, D, G, static_cast<int>(grid), stream);
  if (kv_bits == 8) return launch_prefill<8>(p, D, G, static_cast<int>(grid), stream);
  if (kv_bits == 4) return launch_prefill<4>(p, D, G, static_cast<int>(grid), stream);
  return -1;
}
