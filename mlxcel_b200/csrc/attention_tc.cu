// Chunked causal prefill attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA).
//
// A CTA owns 128 consecutive query tokens of one query head and walks the visible keys of the
// paged KV pool in tiles of 128 keys (8 pool blocks of 16):
//
//   warp 0     TMA producer: Q once; per KV tile the eight K and eight V block slabs of the pool
//              (each [16 keys][D] bf16, contiguous per (block, kv head)) land as 128-byte-swizzled
//              shared-memory tiles, lanes 0-7 issuing one block each
//   warp 1     MMA issuer: S = Q K^T (M=128, N=128, K=D) into one of two TMEM score buffers, then
//              O += P V (M=128, N=D, K=128 keys) with P read from shared memory and V consumed
//              MN-major, exactly as it sits in the pool
//   warps 2-5  softmax, one thread per query row: tcgen05.ld the scores, mask, running max with
//              lazy rescaling (O in TMEM is rescaled only when a row maximum grows by more than
//              2^8, the final normalisation uses the same stale maximum, so the result is exact),
//              P = exp2(...) written as the bf16 A operand of the next MMA, and the epilogue
//
// S is double-buffered, so the score MMA of tile j+1 runs while the softmax of tile j does.
// Every wait is bounded and reports through the status word.
//
// Replaces the reference's cuDNN SDPA prefill (mlx/backend/cuda/scaled_dot_product_attention.cpp in
// its MLX overlay) and `chunked_causal_attention` (src/lib/mlxcel-core/src/layers.rs:5798).
#include "api.h"
#include "common.cuh"

namespace mx {

bool make_tensor_map_bf16(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols,
                          uint64_t ld, uint32_t box_rows, uint32_t box_cols);

constexpr int kTcRows = 128;      // query rows per CTA (UMMA M)
constexpr int kTcKeys = 128;      // keys per tile
constexpr int kTcThreads = 192;
constexpr int kTcStages = 2;
constexpr int kTcBlock = 16;      // pool block size this kernel is written for
constexpr float kRescaleThreshold = 8.0f;   // log2 units

enum : int { kErrAttnProducer = 401, kErrAttnMma = 402, kErrAttnSoftmax = 403 };

struct TcPrefillParams {
  const int* block_tables;
  const int* cu_q;
  const int* context_lens;
  const float* sinks;
  __nv_bfloat16* out;
  int* status;
  int num_seqs, Hq, Hkv, max_blocks, window, tiles_per_seq;
  float scale_log2;
};

template <int D>
__global__ void __launch_bounds__(kTcThreads, 1)
paged_prefill_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                        const __grid_constant__ CUtensorMap map_v, const TcPrefillParams p) {
  constexpr int DC = D / 64;                          // 64-column (128-byte) sub-tiles per row
  constexpr int SUB_BYTES = 128 * 128;                // one [128 rows][64 cols] sub-tile
  constexpr int Q_BYTES = DC * SUB_BYTES;
  constexpr int K_BYTES = DC * SUB_BYTES;             // [128 keys][D]
  constexpr int V_BYTES = DC * SUB_BYTES;
  constexpr int P_BYTES = 2 * SUB_BYTES;              // [128 rows][128 keys]
  constexpr int S_COLS = kTcKeys;                     // fp32 columns of one score buffer
  constexpr int O_COL = 2 * S_COLS;                   // first TMEM column of O
  constexpr uint32_t TMEM_COLS = 512;
  static_assert(D == 64 || D == 128, "head dim");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  uint8_t* q_sm = smem;
  uint8_t* k_sm = q_sm + Q_BYTES;                     // kTcStages x K_BYTES
  uint8_t* v_sm = k_sm + kTcStages * K_BYTES;         // kTcStages x V_BYTES
  uint8_t* p_sm = v_sm + kTcStages * V_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(p_sm + P_BYTES);
  uint64_t* q_full = bars;                // 1
  uint64_t* k_full = bars + 1;            // [stages]
  uint64_t* v_full = k_full + kTcStages;  // [stages]
  uint64_t* kv_empty = v_full + kTcStages;   // [stages]
  uint64_t* s_full = kv_empty + kTcStages;   // [2]
  uint64_t* s_empty = s_full + 2;            // [2]
  uint64_t* p_full = s_empty + 2;            // 1
  uint64_t* pv_done = p_full + 1;            // 1
  uint64_t* k_empty = pv_done + 1;           // [stages] K tile consumed (after the score MMA)
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(k_empty + kTcStages);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  // ---- which tile (heavy tiles, i.e. late tokens, first)
  const int tile = p.tiles_per_seq - 1 - static_cast<int>(blockIdx.x % p.tiles_per_seq);
  const int sh = blockIdx.x / p.tiles_per_seq;
  const int hq = sh % p.Hq, s = sh / p.Hq;
  const int hkv = hq / (p.Hq / p.Hkv);
  const int q0 = p.cu_q[s], q_len = p.cu_q[s + 1] - q0;
  const int tok0 = tile * kTcRows;
  if (tok0 >= q_len) return;   // whole CTA leaves before any barrier / TMEM use
  const int ctx = p.context_lens[s];
  const int pos_base = ctx - q_len;   // absolute position of query token 0
  const int rows_valid = min(kTcRows, q_len - tok0);
  const int kv_end = pos_base + tok0 + rows_valid;   // one past the last visible key
  int kv_begin = 0;
  if (p.window > 0) kv_begin = max(0, pos_base + tok0 - p.window + 1);
  kv_begin = (kv_begin / kTcKeys) * kTcKeys;
  const int n_tiles = (kv_end - kv_begin + kTcKeys - 1) / kTcKeys;
  const int last_block = (ctx - 1) / kTcBlock;   // last pool block the sequence owns

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
    mbar_init(q_full, 1);
    for (int i = 0; i < kTcStages; ++i) {
      mbar_init(&k_full[i], 1);
      mbar_init(&v_full[i], 1);
      mbar_init(&kv_empty[i], 1);
      mbar_init(&k_empty[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&s_full[i], 1);
      mbar_init(&s_empty[i], 4);
    }
    mbar_init(p_full, 4);
    mbar_init(pv_done, 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;
  pdl_trigger();
  pdl_wait();   // q and the newest keys come from the previous kernels of the step

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    const int* table = p.block_tables + static_cast<size_t>(s) * p.max_blocks;
    const uint64_t pol_q = l2_policy_evict_first();
    const uint64_t pol_kv = l2_policy_evict_last();   // re-read by the other heads / token tiles
    if (lane == 0) {
      mbar_expect_tx(q_full, Q_BYTES);
      for (int c = 0; c < DC; ++c)
        tma_load_2d(q_sm + c * SUB_BYTES, &map_q, q_full, hq * D + c * 64, q0 + tok0, pol_q);
    }
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      // The K tile of a stage is free as soon as its score MMA has run, the V tile only after the
      // P V MMA of the same key tile: K of tile j + stages is requested a whole softmax earlier.
      // one pool block per lane; blocks past the sequence's last one repeat it (masked keys, but
      // the values multiplied by P = 0 must be finite)
      int row0 = 0;
      if (lane < kTcKeys / kTcBlock) {
        const int b = min((kv_begin + j * kTcKeys) / kTcBlock + lane, last_block);
        row0 = (table[b] * p.Hkv + hkv) * kTcBlock;
      }
      if (lane == 0) {
        ok = mbar_wait(&k_empty[stage], phase ^ 1u, p.status, kErrAttnProducer);
        if (ok) mbar_expect_tx(&k_full[stage], K_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      if (lane < kTcKeys / kTcBlock) {
        uint8_t* kd = k_sm + stage * K_BYTES + lane * (kTcBlock * 128);
        for (int c = 0; c < DC; ++c) tma_load_2d(kd + c * SUB_BYTES, &map_k, &k_full[stage], c * 64, row0, pol_kv);
      }
      if (lane == 0) {
        ok = mbar_wait(&kv_empty[stage], phase ^ 1u, p.status, kErrAttnProducer);
        if (ok) mbar_expect_tx(&v_full[stage], V_BYTES);
      }
      ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
      if (!ok) break;
      if (lane < kTcKeys / kTcBlock) {
        uint8_t* vd = v_sm + stage * V_BYTES + lane * (kTcBlock * 128);
        for (int c = 0; c < DC; ++c) tma_load_2d(vd + c * SUB_BYTES, &map_v, &v_full[stage], c * 64, row0, pol_kv);
      }
      __syncwarp();
      if (++stage == kTcStages) {
        stage = 0;
        phase ^= 1u;
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_bf16(kTcKeys, false, false);   // N = keys
      constexpr uint32_t idesc_pv = umma_idesc_bf16(D, false, true);          // N = D, V is MN-major
      bool ok = mbar_wait(q_full, 0, p.status, kErrAttnMma);
      auto issue_qk = [&](int j) -> bool {
        const int stage = j % kTcStages;
        const uint32_t kv_phase = static_cast<uint32_t>(j / kTcStages) & 1u;
        const int sb = j & 1;
        const uint32_t s_phase = static_cast<uint32_t>(j >> 1) & 1u;
        if (!mbar_wait(&k_full[stage], kv_phase, p.status, kErrAttnMma)) return false;
        if (!mbar_wait(&s_empty[sb], s_phase ^ 1u, p.status, kErrAttnMma)) return false;
        tc_fence_after_sync();
        const uint32_t qa = smem_u32(q_sm), kb = smem_u32(k_sm + stage * K_BYTES);
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * SUB_BYTES + (kk & 3) * 32;
          umma_bf16(tmem_base + sb * S_COLS, umma_desc_k_sw128(qa + off), umma_desc_k_sw128(kb + off),
                    idesc_qk, kk > 0 ? 1u : 0u);
        }
        umma_commit(&k_empty[stage]);   // the K tile may be refilled
        umma_commit(&s_full[sb]);
        return true;
      };
      if (ok) ok = issue_qk(0);
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) ok = issue_qk(j + 1);   // scores of the next tile under this softmax
        if (!ok) break;
        const int stage = j % kTcStages;
        const uint32_t kv_phase = static_cast<uint32_t>(j / kTcStages) & 1u;
        if (!mbar_wait(&v_full[stage], kv_phase, p.status, kErrAttnMma)) break;
        if (!mbar_wait(p_full, static_cast<uint32_t>(j) & 1u, p.status, kErrAttnMma)) break;
        tc_fence_after_sync();
        const uint32_t pa = smem_u32(p_sm), vb = smem_u32(v_sm + stage * V_BYTES);
#pragma unroll
        for (int kk = 0; kk < kTcKeys / 16; ++kk) {
          const uint64_t da = umma_desc_k_sw128(pa + (kk >> 2) * SUB_BYTES + (kk & 3) * 32);
          const uint64_t db = umma_desc_mn_sw128(vb + kk * (16 * 128), SUB_BYTES, 1024);
          umma_bf16(tmem_base + O_COL, da, db, idesc_pv, (j > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&kv_empty[stage]);   // the V tile of this stage is consumed
        umma_commit(pv_done);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    const int q4 = warp & 3;
    const int row = q4 * 32 + lane;                 // query row == TMEM lane
    const uint32_t lane_addr = tmem_base + (static_cast<uint32_t>(q4 * 32) << 16);
    const int qpos = pos_base + tok0 + row;         // absolute position of this row's token
    float m_used = -INFINITY;   // the maximum the stored exponentials refer to (scaled, log2 units)
    float l = 0.f;
    bool ok = true;
    for (int j = 0; j < n_tiles && ok; ++j) {
      const int sb = j & 1;
      const uint32_t s_phase = static_cast<uint32_t>(j >> 1) & 1u;
      ok = mbar_wait(&s_full[sb], s_phase, p.status, kErrAttnSoftmax);
      if (!ok) break;
      tc_fence_after_sync();
      const int key0 = kv_begin + j * kTcKeys;
      // Only tiles that cross the diagonal, the window edge or the end need the mask.
      const bool need_mask = (key0 + kTcKeys - 1 > pos_base + tok0) ||
                             (p.window > 0 && key0 < pos_base + tok0 + kTcRows - p.window);
      int lo = 0, hi = kTcKeys;   // valid key columns of this row: [lo, hi)
      if (need_mask) {
        hi = min(kTcKeys, qpos - key0 + 1);
        if (p.window > 0) lo = max(0, qpos - p.window + 1 - key0);
      }
      float sv[kTcKeys];
#pragma unroll
      for (int c = 0; c < kTcKeys / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(lane_addr + sb * S_COLS + c * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) sv[c * 32 + i] = __uint_as_float(r[i]) * p.scale_log2;
      }
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(&s_empty[sb]);   // the score buffer may be overwritten
      float mx = -INFINITY;
      if (need_mask) {
#pragma unroll
        for (int i = 0; i < kTcKeys; ++i) {
          if (i < lo || i >= hi) sv[i] = -INFINITY;
          mx = fmaxf(mx, sv[i]);
        }
      } else {
#pragma unroll
        for (int i = 0; i < kTcKeys; ++i) mx = fmaxf(mx, sv[i]);
      }
      // lazy rescaling: keep the old reference maximum unless the row grew past it by 2^8
      float alpha = 1.0f;
      bool rescale = false;
      if (mx > m_used + kRescaleThreshold || m_used == -INFINITY) {
        if (mx > -INFINITY) {
          alpha = (m_used == -INFINITY) ? 0.0f : exp2f(m_used - mx);
          rescale = (m_used != -INFINITY);
          m_used = mx;
        }
      }
      // O and the P buffer belong to the previous tile's P V until that MMA has finished.
      if (j > 0) {
        ok = mbar_wait(pv_done, static_cast<uint32_t>(j - 1) & 1u, p.status, kErrAttnSoftmax);
        if (!ok) break;
        tc_fence_after_sync();
      }
      if (__any_sync(0xffffffffu, rescale)) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t r[32];
          tmem_ld_32x32(lane_addr + O_COL + c * 32, r);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) r[i] = __float_as_uint(__uint_as_float(r[i]) * alpha);
          tmem_st_32x32(lane_addr + O_COL + c * 32, r);
        }
        tmem_st_wait();
      }
      l *= alpha;
      // P = exp2(s - m) as bf16, K-major with the 128-byte swizzle (row = query, 16-byte chunk
      // index XOR (row & 7) inside each 64-key sub-tile)
      float sum = 0.f;
      const float mref = (m_used == -INFINITY) ? 0.f : m_used;
#pragma unroll
      for (int c8 = 0; c8 < kTcKeys / 8; ++c8) {
        float e[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          e[i] = exp2f(sv[c8 * 8 + i] - mref);   // exp2(-inf) = 0 for masked keys
          sum += e[i];
        }
        uint4 pk;
        pk.x = pack_bf16(e[0], e[1]);
        pk.y = pack_bf16(e[2], e[3]);
        pk.z = pack_bf16(e[4], e[5]);
        pk.w = pack_bf16(e[6], e[7]);
        const int sub = c8 >> 3, ch = c8 & 7;
        *reinterpret_cast<uint4*>(p_sm + sub * SUB_BYTES + row * 128 + ((ch ^ (row & 7)) << 4)) = pk;
      }
      l += sum;
      fence_proxy_async_smem();   // generic-proxy writes of P -> visible to the MMA's async proxy
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) mbar_arrive(p_full);
    }
    // ---- epilogue: O / l -> out (one row of D bf16 per thread)
    if (ok && n_tiles > 0) {
      ok = mbar_wait(pv_done, static_cast<uint32_t>(n_tiles - 1) & 1u, p.status, kErrAttnSoftmax);
    }
    if (ok) {
      tc_fence_after_sync();
      float osc = 1.0f;
      if (p.sinks != nullptr) {
        const float sk = p.sinks[hq] * 1.4426950408889634f;
        const float m2 = fmaxf(m_used, sk);
        osc = (m_used > -INFINITY) ? exp2f(m_used - m2) : 0.f;
        l = l * osc + exp2f(sk - m2);
      }
      const float inv = l > 0.f ? osc / l : 0.f;
      __nv_bfloat16* dst = p.out + static_cast<size_t>(q0 + tok0 + row) * p.Hq * D + hq * D;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t r[32];
        tmem_ld_32x32(lane_addr + O_COL + c * 32, r);
        tmem_ld_wait();
        if (row < rows_valid) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 pk;
            pk.x = pack_bf16(__uint_as_float(r[i]) * inv, __uint_as_float(r[i + 1]) * inv);
            pk.y = pack_bf16(__uint_as_float(r[i + 2]) * inv, __uint_as_float(r[i + 3]) * inv);
            pk.z = pack_bf16(__uint_as_float(r[i + 4]) * inv, __uint_as_float(r[i + 5]) * inv);
            pk.w = pack_bf16(__uint_as_float(r[i + 6]) * inv, __uint_as_float(r[i + 7]) * inv);
            *reinterpret_cast<uint4*>(dst + c * 32 + i) = pk;
          }
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int D>
static int launch_prefill_tc(const CUtensorMap& mq, const CUtensorMap& mk, const CUtensorMap& mv,
                             const TcPrefillParams& p, int grid, cudaStream_t stream) {
  constexpr int DC = D / 64;
  constexpr int SUB = 128 * 128;
  const int smem = DC * SUB * (1 + 2 * kTcStages) + 2 * SUB + 1024 + 256;
  auto kern = paged_prefill_tc_kernel<D>;
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    prefer_max_shared(kern);
    configured = true;
  }
  return static_cast<int>(launch_kernel(kern, dim3(grid), dim3(kTcThreads), smem, stream, mq, mk, mv, p));
}

}  // namespace mx

using namespace mx;

// Tensor-core chunked prefill over a bf16 paged pool with 16-token blocks, D = 64 or 128.
// Returns -10 when the configuration is not covered (the caller then uses mx_paged_prefill).
// `q` rows are `q_stride` elements apart (16-byte aligned, q_stride % 8 == 0); `pool_blocks` is
// the number of blocks in k_pool / v_pool; `status` is the device status word.
extern "C" int mx_paged_prefill_tc(const void* q, long long q_stride, const void* k_pool, const void* v_pool,
                                   long long pool_blocks, const int* block_tables, const int* cu_q,
                                   const int* context_lens, const float* sinks, void* out, int num_seqs,
                                   int total_q, int max_q_len, int Hq, int Hkv, int D, int block_size,
                                   int max_blocks, int window, float scale, void* status, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (num_seqs <= 0 || total_q <= 0) return 0;
  if (block_size != kTcBlock || (D != 64 && D != 128) || Hq % Hkv) return -10;
  if ((q_stride % 8) || (reinterpret_cast<uintptr_t>(q) & 15) || (reinterpret_cast<uintptr_t>(out) & 15))
    return -10;
  TcPrefillParams p{};
  p.block_tables = block_tables;
  p.cu_q = cu_q;
  p.context_lens = context_lens;
  p.sinks = sinks;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.status = static_cast<int*>(status);
  p.num_seqs = num_seqs;
  p.Hq = Hq;
  p.Hkv = Hkv;
  p.max_blocks = max_blocks;
  p.window = window;
  p.tiles_per_seq = (max_q_len + kTcRows - 1) / kTcRows;
  p.scale_log2 = scale * 1.4426950408889634f;
  const long long grid = static_cast<long long>(num_seqs) * Hq * p.tiles_per_seq;
  if (grid > 0x7fffffffll) return -1;
  CUtensorMap mq, mk, mv;
  // q: [total_q rows, Hq * D] with row stride q_stride; box = 128 rows x 64 columns
  if (!make_tensor_map_bf16(&mq, q, static_cast<uint64_t>(total_q), static_cast<uint64_t>(Hq) * D,
                            static_cast<uint64_t>(q_stride), kTcRows, 64))
    return -4;
  // pools: [blocks * Hkv * 16 rows, D]; box = one block slab (16 rows) x 64 columns
  const uint64_t pool_rows = static_cast<uint64_t>(pool_blocks) * Hkv * kTcBlock;
  if (!make_tensor_map_bf16(&mk, k_pool, pool_rows, D, D, kTcBlock, 64)) return -4;
  if (!make_tensor_map_bf16(&mv, v_pool, pool_rows, D, D, kTcBlock, 64)) return -4;
  if (D == 64) return launch_prefill_tc<64>(mq, mk, mv, p, static_cast<int>(grid), stream);
  return launch_prefill_tc<128>(mq, mk, mv, p, static_cast<int>(grid), stream);
}
