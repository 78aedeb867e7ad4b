// Dense bf16 GEMM for sm_100a: out[M, N] = epilogue(x[M, K] @ w[N, K]^T).
//
// One persistent CTA per SM, 6 warps with fixed roles:
//   warp 0     TMA producer: brings 64-wide K slices of both operands into a ring of
//              128-byte-swizzled shared-memory stages (cp.async.bulk.tensor, mbarrier tx count)
//   warp 1     MMA issuer: one thread issues tcgen05.mma (M = 128, N = BN, K = 16) into one of
//              two TMEM accumulators and commits stage/accumulator barriers
//   warps 2-5  epilogue: tcgen05.ld the accumulator (one TMEM lane = one thread), apply
//              bias / residual / gated activation, store bf16 or fp32
// The two TMEM accumulators let the epilogue of tile i overlap the main loop of tile i+1.
//
// Two operand placements share the kernel:
//   token-rows-on-lanes  (prefill, M large): lanes = 128 tokens, columns = BN features
//   weight-rows-on-lanes (decode, M <= 256): lanes = 128 features, columns = BN tokens, so a
//     16..128-token batch still fills the 128-lane MMA; split-K spreads the weight stream over
//     all SMs, partial tiles go to an fp32 workspace and the last CTA to arrive for a tile
//     reduces them in split order (deterministic) and applies the epilogue.
// Gated epilogues keep gate and up in two accumulators fed by two weight tiles (rows n and
// glu_offset + n) so no weight interleaving is needed at load time.
//
// Replaces the reference's cuBLASLt call (mlx/backend/cuda/matmul.cpp:133 in its MLX overlay)
// and the compiled swiglu graph that follows it (src/lib/mlxcel-core/src/layers.rs:4407).
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "api.h"
#include "common.cuh"

namespace mx {

constexpr int kBK = 64;          // K elements per stage (128 bytes of bf16)
constexpr int kLaneRows = 128;   // UMMA M
constexpr int kMaxStages = 8;
constexpr int kGemmThreads = 192;
constexpr int kCtrlBytes = 256 + 256 * 4;   // barriers + per-token scales of a tile (BN <= 256)
constexpr int kSplitDepartOffset = MX_WS_COUNTER_BYTES / 8;   // second half of the counter area

constexpr int kMaxRanks = 8;
constexpr int kCommMaxTiles = 8192;   // per-tile arrival flags of one channel
constexpr int kCommDoneIdx = kCommMaxTiles;  // flag index of the per-call completion counter

// Communication epilogues (one channel = control words + flags + receive area in a symmetric
// heap, i.e. the same offsets are valid on every rank and `*_peer[r]` are rank r's addresses).
//   COMM 1  one-shot all-reduce (weight-rows-on-lanes tiles, small M): every rank pushes its
//           bf16 partial tile into every peer's receive slot, bumps the tile's arrival flag on
//           each peer, waits for `world` arrivals on its own flag and sums the slots in rank
//           order (+ bias + residual), so all ranks hold bitwise identical results.
//   COMM 2  two-shot all-reduce (token-rows-on-lanes tiles, large M): tile t is owned by rank
//           (t + t / 152) % world; partial tiles go to the owner only, the owner reduces (+ bias + residual)
//           and stores the finished tile into every peer's output buffer; a per-call completion
//           counter tells each rank when all tiles have landed.
//   COMM 3  all-gather: the tile is stored into every peer's output at column offset rank * N.
// Receive areas are double-buffered by call parity: a peer can be at most one call ahead.
struct CommParams {
  int rank, world;
  uint32_t* ctl;      // local: [0] calls completed, [1] finished-CTA counter, [2] completion target
  uint32_t* expect;   // local: per-tile arrival target already consumed
  uint32_t* flags_peer[kMaxRanks];
  __nv_bfloat16* recv_peer[kMaxRanks];
  __nv_bfloat16* out_peer[kMaxRanks];
  long long parity_stride;  // elements between the two receive halves
  long long rank_stride;    // elements between source-rank slots
  // NVLS variants (nvls != 0): multicast addresses of the same flags / receive area / output.
  //   COMM 1: the partial stays, in fp32, in THIS rank's receive half (one slot, no per-source
  //           slots), one multimem.red bumps the tile's flag on every rank, and after `world`
  //           arrivals each rank pulls the fp32 sum of all replicas with multimem.ld_reduce instead
  //           of 7 peer pushes and an 8-way local sum. No bf16 rounding before the cross-rank sum.
  //   COMM 2: partial tiles stay local (slot = tile), the owner pulls the reduced tile with
  //           multimem.ld_reduce and writes the finished tile to every rank with one multimem.st.
  //   COMM 3: the logits tile is written to every rank's gathered output with multimem.st.
  // TMA never touches these addresses; all multimem accesses are plain ld / st / red forms.
  int nvls;
  uint32_t* flags_mc;
  __nv_bfloat16* recv_mc;
  __nv_bfloat16* out_mc;
};

// Release at system scope: the writes of the whole CTA are ordered before the flag update when
// the CTA meets at a barrier first and one thread then signals (release is cumulative over what
// the barrier made visible to the signalling thread). One releasing thread per peer replaces a
// system-scope fence in every thread, which cost several microseconds per tile.
__device__ __forceinline__ void signal_add_sys(uint32_t* addr, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t load_acquire_sys(const uint32_t* addr) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}
// Bounded wait until *addr >= target (wrap-safe). Records kErrPeerFlagWait on time-out.
__device__ __forceinline__ bool wait_flag_ge(const uint32_t* addr, uint32_t target, int* status) {
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
#pragma unroll 1
    for (int i = 0; i < 64; ++i) {
      if (static_cast<int32_t>(load_acquire_sys(addr) - target) >= 0) return true;
    }
    if (status != nullptr && *reinterpret_cast<volatile int*>(status) != 0) return false;
    if (globaltimer_ns() - t0 > kWaitLimitNs) {
      if (status != nullptr) atomicCAS(status, 0, kErrPeerFlagWait);
      return false;
    }
  }
}

struct GemmParams {
  void* out;
  const __nv_bfloat16* bias;
  const __nv_bfloat16* residual;
  float* partials;
  int* counters;
  int* status;
  int M, N, K;
  int ldo, ldr;
  int glu_offset;
  int splits, kb_per_split, num_kb;
  int tiles_lane, tiles_col;
  int stages;
  int raster_gm;        // dense tile order: lane tiles per panel (0 = column-major walk)
  // Quantized weights (WQ != 0): per-group scales (bf16 for affine, e8m0 bytes for mxfp4), affine
  // biases, group size (32 / 64 / 128), groups per weight row, number of weight rows.
  const void* q_scales;
  const __nv_bfloat16* q_biases;
  int q_group, q_groups_per_row, q_rows;
  int q_tiles_per_group;   // grouped: re-tiled row tiles per expert (gate tiles then up tiles when gated)
  int q_glu_tiles;         // tile distance from a gate tile to its up tile
  // Deferred RMSNorm (see mx_gemm_set_row_norm). ssq buffers: word 0 = number of partial sums per
  // token, word 1 = tokens per partial row (ld), data from word 8: partial p of token t at
  // 8 + p * ld + t.
  const float* ssq_in;  // consumer: every output row t is scaled by rsqrt(sum_p ssq / K_norm + eps)
  float* ssq_out;       // producer: per (feature tile, token) sum of squares of the bf16 results
  float ssq_eps, ssq_inv_dim;
  int vec_ok;           // 16-byte vector epilogue allowed (N, strides and base addresses aligned)
  unsigned long long* trace;   // optional per-CTA phase timestamps (see MX_WS_TRACE_OFFSET)
  int l2_prefetch_kb;   // k-blocks of weights (beyond the smem ring) to prefetch into L2 before the wait
  int epilogue;
  int out_fp32;
  float glu_alpha, glu_limit;
  CommParams comm;
  // grouped (per-expert) mode: rows [group_offsets[e], group_offsets[e+1]) of x use the weight
  // rows [e * w_group_rows, ...) and bias [e * bias_group_stride, ...)
  const int* group_offsets;
  int num_groups;
  int w_group_rows;
  int bias_group_stride;
};

// One unit of work of the persistent tile loop, in tensor-map coordinates and output indices.
struct WorkItem {
  int tile, split;
  int lane_row0, col_row0;   // first row of the lane-side / column-side operand tile
  int out_tok0, tok_valid;   // first output token row of the tile and how many are real
  int feat0, feat_valid;     // first output feature of the tile and how many are real
  int bias_off;
  int q_tile;                // quantized weights: index of the lane tile in the re-tiled blocks
};
struct GroupCursor {
  int e = 0, base = 0;
};

// Maps the linear work index to a tile. Dense: (tile, split) over a fixed grid of tiles. Grouped:
// feature tile fastest, then token tiles of expert 0, 1, ... (tile counts come from the device
// offsets, so every role advances the same running cursor). Returns false past the end.
template <int BN, bool SWAP, bool GROUPED>
__device__ __forceinline__ bool decode_work(const GemmParams& p, int w, GroupCursor& cur, WorkItem& it) {
  if constexpr (!GROUPED) {
    if (w >= p.tiles_lane * p.tiles_col * p.splits) return false;
    it.tile = w / p.splits;
    it.split = w - it.tile * p.splits;
    int lane_t, col_t;
    if (p.raster_gm > 0) {
      // Tiles are walked in panels of raster_gm lane tiles x all column tiles, lane tile fastest:
      // the panel's rows of the lane operand stay in L2 while the column operand streams past
      // once per panel (instead of the whole lane operand being re-read for every few column tiles).
      const int per_panel = p.raster_gm * p.tiles_col;
      const int g = it.tile / per_panel, r = it.tile - g * per_panel;
      const int lanes = min(p.raster_gm, p.tiles_lane - g * p.raster_gm);
      lane_t = g * p.raster_gm + r % lanes;
      col_t = r / lanes;
    } else {
      lane_t = it.tile % p.tiles_lane;
      col_t = it.tile / p.tiles_lane;
    }
    it.lane_row0 = lane_t * kLaneRows;
    it.col_row0 = col_t * BN;
    it.bias_off = 0;
    it.q_tile = lane_t;
    if (SWAP) {
      it.feat0 = it.lane_row0;
      it.feat_valid = p.N - it.feat0;
      it.out_tok0 = it.col_row0;
      it.tok_valid = p.M - it.out_tok0;
    } else {
      it.out_tok0 = it.lane_row0;
      it.tok_valid = p.M - it.out_tok0;
      it.feat0 = it.col_row0;
      it.feat_valid = p.N - it.feat0;
    }
    return true;
  } else {
    constexpr int TOK_TILE = SWAP ? BN : kLaneRows;
    constexpr int FEAT_TILE = SWAP ? kLaneRows : BN;
    const int F = (p.N + FEAT_TILE - 1) / FEAT_TILE;
    const int f = w % F, g = w / F;
    while (cur.e < p.num_groups) {
      const int rows = p.group_offsets[cur.e + 1] - p.group_offsets[cur.e];
      const int cnt = (rows + TOK_TILE - 1) / TOK_TILE;
      if (g < cur.base + cnt) break;
      cur.base += cnt;
      ++cur.e;
    }
    if (cur.e >= p.num_groups) return false;
    const int e = cur.e;
    it.tile = w;
    it.split = 0;
    it.out_tok0 = p.group_offsets[e] + (g - cur.base) * TOK_TILE;
    it.tok_valid = p.group_offsets[e + 1] - it.out_tok0;
    it.feat0 = f * FEAT_TILE;
    it.feat_valid = p.N - it.feat0;
    it.bias_off = e * p.bias_group_stride;
    it.q_tile = e * p.q_tiles_per_group + f;
    const int w_row = e * p.w_group_rows + it.feat0;
    it.lane_row0 = SWAP ? w_row : it.out_tok0;
    it.col_row0 = SWAP ? it.out_tok0 : w_row;
    return true;
  }
}

// Gated activations, all of the form num * sigmoid(z) * mult, written branch-light with fast
// exp / divide (relative error ~1e-6, far below bf16 rounding) so the epilogue stays a few dozen
// instructions: epilogue code runs once per tile and is instruction-fetch bound.
//   SwiGLU:          silu(g) * u
//   GeGLU (tanh):    0.5 g (1 + tanh(k0 (g + k1 g^3))) u  ==  g sigmoid(2 k0 (g + k1 g^3)) u
//   clipped SwiGLU:  g' sigmoid(alpha g') (u' + 1), g' = min(g, limit), u' = clamp(u, +-limit)
__device__ __forceinline__ float act_glu(int epilogue, float g, float u, float alpha, float limit) {
  float z = g;
  if (epilogue == MX_EPI_GEGLU) {
    const float k0 = 0.7978845608028654f, k1 = 0.044715f;
    z = 2.0f * k0 * (g + k1 * g * g * g);
  } else if (epilogue == MX_EPI_CLIPPED_SWIGLU) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit) + 1.0f;
    z = alpha * g;
  }
  return __fdividef(g, 1.0f + __expf(-z)) * u;
}

// Owner rank of a tile in the two-shot all-reduce. A persistent CTA walks tiles b, b + grid,
// b + 2 grid, ...; with `tile % world` and an even grid it would own either all or none of them
// (the owner's epilogue is the heavy one). The extra term shifts ownership by one every 152 tiles
// (152 is a multiple of every supported world size, so the `world` tiles of an aligned group
// still have distinct owners and `tile / world` stays a valid slot index per owner).
__device__ __forceinline__ int comm2_owner(int tile, int world) { return (tile + tile / 152) % world; }

// Owner-side reduction of the two-shot all-reduce for one token row: features [j0, j0 + 8 NQ) of
// the tile (bounded by nfeat), partials of `world` <= WMAX ranks at `base + r * rank_stride`.
template <int NQ, int WMAX>
__device__ __forceinline__ void comm2_reduce_span(const __nv_bfloat16* base, long long rank_stride, int world,
                                                  const __nv_bfloat16* bias_n, const __nv_bfloat16* res_n,
                                                  __nv_bfloat16* const* out_peer, size_t off0, int j0,
                                                  int nfeat) {
  uint4 a[NQ][WMAX];
  uint4 rs[NQ];
#pragma unroll
  for (int q = 0; q < NQ; ++q) {
    const int j = j0 + q * 8;
    if (j < nfeat) {
#pragma unroll
      for (int r = 0; r < WMAX; ++r)
        if (r < world)
          a[q][r] = __ldcg(reinterpret_cast<const uint4*>(base + r * static_cast<size_t>(rank_stride) + j));
      if (res_n != nullptr) rs[q] = *reinterpret_cast<const uint4*>(res_n + j);
    }
  }
#pragma unroll
  for (int q = 0; q < NQ; ++q) {
    const int j = j0 + q * 8;
    if (j >= nfeat) break;
    float o[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = 0.f;
#pragma unroll
    for (int r = 0; r < WMAX; ++r) {
      if (r < world) {
        const uint32_t w4[4] = {a[q][r].x, a[q][r].y, a[q][r].z, a[q][r].w};
#pragma unroll
        for (int i = 0; i < 4; ++i) o[2 * i] += bf16_lo(w4[i]), o[2 * i + 1] += bf16_hi(w4[i]);
      }
    }
    if (bias_n != nullptr) {
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] += __bfloat162float(bias_n[j + i]);
    }
    if (res_n != nullptr) {
      const uint32_t w4[4] = {rs[q].x, rs[q].y, rs[q].z, rs[q].w};
#pragma unroll
      for (int i = 0; i < 4; ++i) o[2 * i] += bf16_lo(w4[i]), o[2 * i + 1] += bf16_hi(w4[i]);
    }
    uint4 pk;
    pk.x = pack_bf16(o[0], o[1]);
    pk.y = pack_bf16(o[2], o[3]);
    pk.z = pack_bf16(o[4], o[5]);
    pk.w = pack_bf16(o[6], o[7]);
    for (int pr = 0; pr < world; ++pr) *reinterpret_cast<uint4*>(out_peer[pr] + off0 + j) = pk;
  }
}

// ----------------------------------------------------------------------------- weight dequantisation
// One thread turns the packed bytes of ONE weight row of a k-block (64 values) into the 128-byte
// row of the swizzled bf16 MMA tile. Values are q * scale + bias in fp32, rounded once to bf16
// (the semantics of the stand-alone dequantiser). (s0, b0) applies to values 0..31, (s1, b1) to
// 32..63 (equal unless the group size is 32).
__device__ __forceinline__ float e2m1_value(uint32_t nib) {
  const uint32_t mag = nib & 7u, e = mag >> 1, m = mag & 1u;
  const uint32_t bits = e ? (((e + 126u) << 23) | (m << 22)) : (m ? 0x3F000000u : 0u);
  return __uint_as_float(bits | ((nib & 8u) << 28));
}
// `half` selects values 0..31 (chunks 0..3) or 32..63 (chunks 4..7) of the row; sc / bi are the
// scale and bias of that half.
template <int WQ>
__device__ __forceinline__ void dequant_half_row_to_tile(const uint8_t* pk_row, int half, float sc, float bi,
                                                         __nv_bfloat16 sb, __nv_bfloat16 bb, uint8_t* tile,
                                                         int r) {
  uint8_t* dst = tile + r * 128;
  if constexpr (WQ == 1) {
    // affine 4-bit on packed bf16 pairs: (w >> 4i) & 0x000F000F | 0x43004300 is the bf16 pair
    // (128 + n_i, 128 + n_{i+4}); minus 128 is exact, then one fused multiply-add per pair
    // (q * scale + bias, rounded once to bf16), and byte permutes restore the value order.
    const uint4 v = *reinterpret_cast<const uint4*>(pk_row + half * 16);
    const uint32_t wds[4] = {v.x, v.y, v.z, v.w};
    const __nv_bfloat162 s2 = __halves2bfloat162(sb, sb), b2 = __halves2bfloat162(bb, bb);
    const uint32_t k128 = 0x43004300u;
    const __nv_bfloat162 c128 = *reinterpret_cast<const __nv_bfloat162*>(&k128);
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      uint32_t pr[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint32_t raw = ((wds[cc] >> (4 * i)) & 0x000F000Fu) | k128;
        __nv_bfloat162 x = *reinterpret_cast<const __nv_bfloat162*>(&raw);
        x = __hfma2(__hsub2(x, c128), s2, b2);
        pr[i] = *reinterpret_cast<uint32_t*>(&x);   // (n_i, n_{i+4})
      }
      uint4 o;
      o.x = __byte_perm(pr[0], pr[1], 0x5410);   // (n0, n1)
      o.y = __byte_perm(pr[2], pr[3], 0x5410);   // (n2, n3)
      o.z = __byte_perm(pr[0], pr[1], 0x7632);   // (n4, n5)
      o.w = __byte_perm(pr[2], pr[3], 0x7632);   // (n6, n7)
      const int c = half * 4 + cc;
      *reinterpret_cast<uint4*>(dst + ((c ^ (r & 7)) << 4)) = o;
    }
    return;
  }
  if constexpr (WQ == 2) {   // 8-bit: 32 bytes per half, chunk = 8 bytes
    uint32_t wds[8];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const uint4 v = *reinterpret_cast<const uint4*>(pk_row + half * 32 + i * 16);
      wds[4 * i] = v.x, wds[4 * i + 1] = v.y, wds[4 * i + 2] = v.z, wds[4 * i + 3] = v.w;
    }
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const int c = half * 4 + cc;
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t q = (wds[2 * cc + (j >> 2)] >> (8 * (j & 3))) & 0xFFu;
        f[j] = __uint_as_float(0x4B000000u | q) - 8388608.0f;   // exact int -> float without I2F
        f[j] = f[j] * sc + bi;
      }
      uint4 o;
      o.x = pack_bf16(f[0], f[1]), o.y = pack_bf16(f[2], f[3]), o.z = pack_bf16(f[4], f[5]), o.w = pack_bf16(f[6], f[7]);
      *reinterpret_cast<uint4*>(dst + ((c ^ (r & 7)) << 4)) = o;
    }
  } else {                   // 4-bit: 16 bytes per half, chunk = one word, nibbles LSB first
    const uint4 v = *reinterpret_cast<const uint4*>(pk_row + half * 16);
    const uint32_t wds[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int cc = 0; cc < 4; ++cc) {
      const int c = half * 4 + cc;
      float f[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const uint32_t q = (wds[cc] >> (4 * j)) & 0xFu;
        if constexpr (WQ == 3) {
          f[j] = e2m1_value(q) * sc;
        } else {
          f[j] = __uint_as_float(0x4B000000u | q) - 8388608.0f;
          f[j] = f[j] * sc + bi;
        }
      }
      uint4 o;
      o.x = pack_bf16(f[0], f[1]), o.y = pack_bf16(f[2], f[3]), o.z = pack_bf16(f[4], f[5]), o.w = pack_bf16(f[6], f[7]);
      *reinterpret_cast<uint4*>(dst + ((c ^ (r & 7)) << 4)) = o;
    }
  }
}
__device__ __forceinline__ float e8m0_scale(uint8_t sv) {
  if (sv == 255) return __uint_as_float(0x7fc00000u);
  if (sv == 0) return __uint_as_float(0x00400000u);
  return __uint_as_float(static_cast<uint32_t>(sv) << 23);
}

// WQ: weight format of the lane operand. 0 = bf16 (TMA writes the swizzled MMA tile directly);
// otherwise the packed checkpoint bytes are staged by TMA and four extra "transform" warps
// dequantise them into the swizzled bf16 tile that the MMA reads (weight-rows-on-lanes only):
// 1 = affine 4-bit, 2 = affine 8-bit (q * scale + bias per group), 3 = mxfp4 (e2m1 * 2^(s-127)).
__host__ __device__ constexpr int wq_bits(int wq) { return (wq == 2) ? 8 : 4; }
// Rows of one re-tiled block: 128 weight rows of 64 * bits / 8 bytes, followed by the block's scales
// ([2 halves][128 rows]) and, for the affine formats, biases, stored as extra rows of the same
// width so that one TMA box brings values and scales together.
__host__ __device__ constexpr int wq_block_rows(int wq) {
  return 128 + (wq == 3 ? 256 : 1024) / (64 * wq_bits(wq) / 8);
}
__host__ __device__ constexpr int gemm_threads(int wq) { return wq != 0 ? kGemmThreads + 128 : kGemmThreads; }

template <int BN, bool SWAP, bool GLU, int COMM, bool GROUPED, int WQ = 0>
__global__ void __launch_bounds__(gemm_threads(WQ), 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap map_lane,
                 const __grid_constant__ CUtensorMap map_col, const GemmParams p) {
  constexpr int LANE_TILES = (SWAP && GLU) ? 2 : 1;
  constexpr int COL_TILES = (!SWAP && GLU) ? 2 : 1;
  constexpr int LANE_BYTES = kLaneRows * kBK * 2;
  constexpr int COL_BYTES = BN * kBK * 2;
  constexpr int PK_ROW_BYTES = WQ != 0 ? kBK * wq_bits(WQ) / 8 : 0;   // packed bytes of one row per k-block
  constexpr int PK_ROWS = WQ != 0 ? wq_block_rows(WQ) : 0;   // weight rows + scale / bias rows
  constexpr int PK_BYTES = PK_ROWS * PK_ROW_BYTES;
  static_assert(PK_BYTES % 256 == 0, "re-tiled blocks are loaded as rows of 256 bytes");
  // stages start on 1024-byte boundaries (the swizzled MMA tiles need that alignment)
  constexpr int STAGE_BYTES = (LANE_TILES * (LANE_BYTES + PK_BYTES) + COL_TILES * COL_BYTES + 1023) / 1024 * 1024;
  constexpr int RAW_BYTES = LANE_TILES * PK_BYTES + COL_TILES * COL_BYTES;   // what TMA brings when WQ
  static_assert(WQ == 0 || SWAP, "quantized weights: weight-rows-on-lanes tiles only");
  constexpr int ACC_COLS = GLU ? 2 * BN : BN;
  constexpr int TMEM_COLS = (2 * ACC_COLS <= 32)    ? 32
                            : (2 * ACC_COLS <= 64)  ? 64
                            : (2 * ACC_COLS <= 128) ? 128
                            : (2 * ACC_COLS <= 256) ? 256
                                                    : 512;
  constexpr int CW = (BN >= 32) ? 32 : 16;  // columns per tcgen05.ld
  static_assert(BN % CW == 0 && BN >= 16 && BN <= 256, "unsupported BN");
  static_assert(2 * ACC_COLS <= 512, "accumulators exceed TMEM");
  static_assert(COMM == 0 || !GLU, "communication epilogues are for plain projections");
  static_assert(COMM == 0 || !GROUPED, "grouped GEMMs have no communication epilogue");
  static_assert(COMM != 1 || SWAP, "one-shot all-reduce uses weight-rows-on-lanes tiles");
  static_assert(COMM != 2 || !SWAP, "two-shot all-reduce uses token-rows-on-lanes tiles");
  static_assert(COMM != 3 || SWAP, "all-gather epilogue uses weight-rows-on-lanes tiles");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) &
                                             ~static_cast<uintptr_t>(1023));
  constexpr int STAGING_BYTES = SWAP ? BN * kLaneRows * 4 : 0;   // epilogue transpose tile (fp32)
  [[maybe_unused]] float* staging = reinterpret_cast<float*>(smem + p.stages * STAGE_BYTES);
  uint8_t* ctrl = smem + p.stages * STAGE_BYTES + STAGING_BYTES;
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(ctrl);
  uint64_t* empty_bar = full_bar + kMaxStages;
  uint64_t* tmem_full = empty_bar + kMaxStages;
  uint64_t* tmem_empty = tmem_full + 2;
  [[maybe_unused]] uint64_t* raw_full = tmem_empty + 2;   // WQ: packed weights + activations landed
  uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(raw_full + kMaxStages);
  int* last_flag = reinterpret_cast<int*>(tmem_ptr + 1);
  [[maybe_unused]] float* scale_sm = reinterpret_cast<float*>(ctrl + 256);   // per-token row scales of the tile

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  unsigned long long* const trace =
      (p.trace != nullptr && blockIdx.x < MX_WS_TRACE_MAX_CTAS) ? p.trace + blockIdx.x * 16 : nullptr;
  auto stamp = [&](int slot) {
    if (trace != nullptr) trace[slot] = globaltimer_ns();
  };

  // producer state set up by thread 0 before the CTA-wide sync (it is also the producer thread)
  [[maybe_unused]] uint64_t pol_lane = 0, pol_col = 0;
  [[maybe_unused]] int pre = 0;   // ring stages whose weight tiles are already in flight
  auto load_lane = [&](uint8_t* s, uint64_t* bar, int kb, int row0, [[maybe_unused]] int qtile) {
    if constexpr (WQ != 0) {
      // packed bytes of 128 weight rows for this k-block (byte-typed tensor map, no swizzle)
      // The packed weights were re-tiled at load time: (128-row tile, k-block) -> one contiguous
      // block of 128 x PK_ROW_BYTES bytes, so a box is a single 4 / 8 KB run in DRAM (row-major
      // checkpoint rows would give 128 separate 32-byte pieces per box).
      uint8_t* pk = s + LANE_TILES * LANE_BYTES + COL_TILES * COL_BYTES;
      // (the tensor map views the contiguous blocks as rows of 256 bytes: few, wide TMA requests)
      constexpr int BOX_ROWS = PK_BYTES / 256;
      tma_load_2d(pk, &map_lane, bar, 0, (qtile * p.num_kb + kb) * BOX_ROWS, pol_lane);
      if (LANE_TILES == 2)
        tma_load_2d(pk + PK_BYTES, &map_lane, bar, 0, ((qtile + p.q_glu_tiles) * p.num_kb + kb) * BOX_ROWS, pol_lane);
    } else {
      tma_load_2d(s, &map_lane, bar, kb * kBK, row0, pol_lane);
      if (LANE_TILES == 2) tma_load_2d(s + LANE_BYTES, &map_lane, bar, kb * kBK, row0 + p.glu_offset, pol_lane);
    }
  };
  // barrier the TMA loads of a stage complete on: the MMA's when the tile is ready as loaded,
  // the transform warps' when the weights still have to be dequantised
  auto load_bar = [&](int stage) -> uint64_t* { return WQ != 0 ? &raw_full[stage] : &full_bar[stage]; };
  constexpr int TX_BYTES = WQ != 0 ? RAW_BYTES : LANE_TILES * LANE_BYTES + COL_TILES * COL_BYTES;
  auto load_col = [&](uint8_t* s, uint64_t* bar, int kb, int row0) {
    uint8_t* sc = s + LANE_TILES * LANE_BYTES;
    tma_load_2d(sc, &map_col, bar, kb * kBK, row0, pol_col);
    if (COL_TILES == 2) tma_load_2d(sc + COL_BYTES, &map_col, bar, kb * kBK, row0 + p.glu_offset, pol_col);
  };
  if (threadIdx.x == 0) {
    stamp(0);
    tma_prefetch_desc(&map_lane);
    tma_prefetch_desc(&map_col);
    for (int s = 0; s < p.stages; ++s) {
      mbar_init(&full_bar[s], WQ != 0 ? 8 : 1);
      mbar_init(&empty_bar[s], 1);
      if constexpr (WQ != 0) mbar_init(&raw_full[s], 1);
    }
    mbar_init(&tmem_full[0], 1);
    mbar_init(&tmem_full[1], 1);
    mbar_init(&tmem_empty[0], 4);
    mbar_init(&tmem_empty[1], 4);
    fence_mbar_init();
    // Weights are streamed once (evict first); activations are re-read by every tile.
    const uint64_t pol_w = l2_policy_evict_first();
    const uint64_t pol_x = l2_policy_evict_last();
    pol_lane = SWAP ? pol_w : pol_x;
    pol_col = SWAP ? pol_x : pol_w;
    // Weights never depend on the previous kernel: the weight tiles of the first ring of stages
    // are requested before waiting for it, so the weight stream of this GEMM starts while the
    // previous kernel is still in its tail / epilogue. Activation tiles follow after the wait.
    if constexpr (!GROUPED) {
      GroupCursor c0;
      WorkItem it0;
      if (decode_work<BN, SWAP, false>(p, blockIdx.x, c0, it0)) {
        const int kb0 = it0.split * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        pre = min(p.stages, kb1 - kb0);
        for (int i = 0; i < pre; ++i) {
          mbar_expect_tx(load_bar(i), TX_BYTES);
          uint8_t* s = smem + i * STAGE_BYTES;
          if (SWAP) load_lane(s, load_bar(i), kb0 + i, it0.lane_row0, it0.q_tile);
          else load_col(s, load_bar(i), kb0 + i, it0.col_row0);
        }
        // The rest of this CTA's weight slice (up to a budget) goes to L2: HBM keeps streaming
        // through the previous kernels' epilogues and the small kernels in between, and the
        // main loop below then runs out of the 126 MB L2 instead of waiting on DRAM.
        if constexpr (SWAP && WQ == 0) {
          const int kbe = min(kb1, kb0 + pre + p.l2_prefetch_kb);
          for (int kb = kb0 + pre; kb < kbe; ++kb) {
            tma_prefetch_l2_2d(&map_lane, kb * kBK, it0.lane_row0);
            if (LANE_TILES == 2) tma_prefetch_l2_2d(&map_lane, kb * kBK, it0.lane_row0 + p.glu_offset);
          }
        }
      }
    }
  }
  if (warp == 1) {
    tmem_alloc(tmem_ptr, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_ptr;
  // Everything above touched only this CTA's shared memory / TMEM. The next kernel of the stream
  // may be scheduled from here on; each role below waits for the PREVIOUS kernel (pdl_wait) right
  // before its first access to memory that kernel may have written.
  pdl_trigger();
  if (threadIdx.x == 0) stamp(1);

  // Quantized weights: packed block (staged by TMA, scales and biases in its trailing rows) ->
  // swizzled bf16 MMA tile, for all k-blocks of one work item. Eight warps take part (the four
  // transform warps and the four epilogue warps, which are idle during the main loop): thread =
  // (weight row, half of its 64 values); all eight arrive on full_bar per stage.
  [[maybe_unused]] auto transform_item = [&](const WorkItem& it, int half, int r, int& stage, uint32_t& phase) -> bool {
    if constexpr (WQ != 0) {
      const int kb0 = it.split * p.kb_per_split;
      const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
      for (int kb = kb0; kb < kb1; ++kb) {
        if (!mbar_wait(&raw_full[stage], phase, p.status, kErrMmaWaitFull)) return false;
        uint8_t* st = smem + stage * STAGE_BYTES;
        const uint8_t* pk = st + LANE_TILES * LANE_BYTES + COL_TILES * COL_BYTES;
#pragma unroll
        for (int lt = 0; lt < LANE_TILES; ++lt) {
          const uint8_t* blk = pk + lt * PK_BYTES;
          const uint8_t* ex = blk + kLaneRows * PK_ROW_BYTES;   // [2 halves][128 rows] scales, then biases
          if constexpr (WQ == 3) {
            dequant_half_row_to_tile<WQ>(blk + r * PK_ROW_BYTES, half, e8m0_scale(ex[half * kLaneRows + r]), 0.f,
                                         __nv_bfloat16(), __nv_bfloat16(), st + lt * LANE_BYTES, r);
          } else {
            const __nv_bfloat16* sp = reinterpret_cast<const __nv_bfloat16*>(ex);
            const __nv_bfloat16 sb = sp[half * kLaneRows + r], bb = sp[(2 + half) * kLaneRows + r];
            dequant_half_row_to_tile<WQ>(blk + r * PK_ROW_BYTES, half, __bfloat162float(sb), __bfloat162float(bb),
                                         sb, bb, st + lt * LANE_BYTES, r);
          }
        }
        fence_proxy_async_smem();   // generic-proxy writes -> visible to the MMA's async proxy
        __syncwarp();
        if ((threadIdx.x & 31) == 0) mbar_arrive(&full_bar[stage]);
        if (++stage == p.stages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
    return true;
  };

  if (warp == 0) {
    // ------------------------------------------------------------------ TMA producer
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      GroupCursor cur;
      WorkItem it;
      pdl_wait();
      int seq = 0;
      for (int w = blockIdx.x; ok && decode_work<BN, SWAP, GROUPED>(p, w, cur, it); w += gridDim.x) {
        const int kb0 = it.split * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        const int lane_row0 = it.lane_row0, col_row0 = it.col_row0;
        for (int kb = kb0; kb < kb1; ++kb, ++seq) {
          uint8_t* s = smem + stage * STAGE_BYTES;
          if (seq < pre) {
            // weight tile already in flight: only the activation tile is missing
            if (SWAP) load_col(s, load_bar(stage), kb, col_row0);
            else load_lane(s, load_bar(stage), kb, lane_row0, it.q_tile);
          } else {
            if (!mbar_wait(&empty_bar[stage], phase ^ 1u, p.status, kErrProducerWait)) {
              ok = false;
              break;
            }
            mbar_expect_tx(load_bar(stage), TX_BYTES);
            load_lane(s, load_bar(stage), kb, lane_row0, it.q_tile);
            load_col(s, load_bar(stage), kb, col_row0);
          }
          if (seq == 0) stamp(2);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      // Gated, token-rows-on-lanes: the gate and up weight tiles sit back to back in the stage
      // (2 x BN rows of one K-major operand), so ONE MMA of N = 2 BN fills both accumulators.
      constexpr bool kWideGlu = GLU && !SWAP && 2 * BN <= 256;
      constexpr uint32_t idesc = umma_idesc_bf16(kWideGlu ? 2 * BN : BN, false, false);
      if constexpr (GROUPED) pdl_wait();   // the tile schedule reads expert offsets written upstream
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      GroupCursor cur;
      WorkItem it;
      for (int w = blockIdx.x; ok && decode_work<BN, SWAP, GROUPED>(p, w, cur, it); w += gridDim.x) {
        const int kb0 = it.split * p.kb_per_split;
        const int kb1 = min(p.num_kb, kb0 + p.kb_per_split);
        if (!mbar_wait(&tmem_empty[acc], acc_phase ^ 1u, p.status, kErrMmaWaitTmem)) break;
        tc_fence_after_sync();
        const uint32_t d0 = tmem_base + acc * ACC_COLS;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(&full_bar[stage], phase, p.status, kErrMmaWaitFull)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          if (kb == kb0 && w == static_cast<int>(blockIdx.x)) stamp(3);
          const uint32_t sa = smem_u32(smem + stage * STAGE_BYTES);
          const uint32_t sb = sa + LANE_TILES * LANE_BYTES;
#pragma unroll
          for (int kk = 0; kk < kBK / 16; ++kk) {
            const uint32_t accum = (kb > kb0 || kk > 0) ? 1u : 0u;
            const uint64_t da = umma_desc_k_sw128(sa + kk * 32);
            const uint64_t db = umma_desc_k_sw128(sb + kk * 32);
            umma_bf16(d0, da, db, idesc, accum);
            if (GLU && !kWideGlu) {
              if (SWAP) {
                const uint64_t da2 = umma_desc_k_sw128(sa + LANE_BYTES + kk * 32);
                umma_bf16(d0 + BN, da2, db, idesc, accum);
              } else {
                const uint64_t db2 = umma_desc_k_sw128(sb + COL_BYTES + kk * 32);
                umma_bf16(d0 + BN, da, db2, idesc, accum);
              }
            }
          }
          umma_commit(&empty_bar[stage]);
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (!ok) break;
        umma_commit(&tmem_full[acc]);
        stamp(4);
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
    }
    __syncwarp();
  } else if (WQ != 0 && warp >= 6) {
    // ------------------------------------------------------------------ transform (first halves)
    if constexpr (WQ != 0) {
      if constexpr (GROUPED) pdl_wait();   // the tile schedule reads expert offsets written upstream
      const int r = static_cast<int>(threadIdx.x) - kGemmThreads;
      int stage = 0;
      uint32_t phase = 0;
      GroupCursor cur;
      WorkItem it;
      for (int w = blockIdx.x; decode_work<BN, SWAP, GROUPED>(p, w, cur, it); w += gridDim.x)
        if (!transform_item(it, 0, r, stage, phase)) break;
    }
  } else {
    // ------------------------------------------------------------------ epilogue (128 threads)
    const int q = warp & 3;              // TMEM lane quarter this warp may read
    const int row = q * 32 + lane;       // accumulator row (TMEM lane) of this thread
    const int epi_tid = threadIdx.x - 64;
    int acc = 0;
    uint32_t acc_phase = 0;
    const bool glu = GLU;
    pdl_wait();   // bias / residual / workspace / channel words below may come from the previous kernel
    [[maybe_unused]] uint32_t comm_parity = 0;
    if constexpr (COMM != 0) comm_parity = *reinterpret_cast<volatile uint32_t*>(p.comm.ctl) & 1u;
    GroupCursor cur;
    WorkItem it;
    [[maybe_unused]] int t_stage = 0;
    [[maybe_unused]] uint32_t t_phase = 0;
    for (int w = blockIdx.x; decode_work<BN, SWAP, GROUPED>(p, w, cur, it); w += gridDim.x) {
      const int tile = it.tile, split = it.split;
      if constexpr (WQ != 0) {
        // second halves of this item's weight rows (these warps have nothing else to do until the
        // accumulator is ready)
        if (!transform_item(it, 1, epi_tid, t_stage, t_phase)) break;
      }
      // Deferred RMSNorm, consumer side: this GEMM reads the un-normalised residual stream (the
      // norm weight is folded into W) and scales every output row by the row's 1/rms, summed here
      // from the partial sums the producing kernel left, while the main loop is still running.
      [[maybe_unused]] float row_scale = 1.0f;   // token-rows-on-lanes: this thread's token
      if (p.ssq_in != nullptr) {
        const int parts = reinterpret_cast<const int*>(p.ssq_in)[0];
        const int ld = reinterpret_cast<const int*>(p.ssq_in)[1];
        const float* data = p.ssq_in + 8;
        if constexpr (SWAP) {
          named_bar_sync(1, 128);   // the previous item's readers of scale_sm are done
          for (int c = epi_tid; c < BN; c += 128) {
            const int t = it.out_tok0 + c;
            float ss = 0.f;
            if (c < it.tok_valid)
              for (int pp = 0; pp < parts; ++pp) ss += __ldcg(data + static_cast<size_t>(pp) * ld + t);
            scale_sm[c] = rsqrtf(ss * p.ssq_inv_dim + p.ssq_eps);
          }
          named_bar_sync(1, 128);
        } else {
          float ss = 0.f;
          if (row < it.tok_valid)
            for (int pp = 0; pp < parts; ++pp)
              ss += __ldcg(data + static_cast<size_t>(pp) * ld + it.out_tok0 + row);
          row_scale = rsqrtf(ss * p.ssq_inv_dim + p.ssq_eps);
        }
      }
      if (!mbar_wait(&tmem_full[acc], acc_phase, p.status, kErrEpilogueWait)) break;
      tc_fence_after_sync();
      if (epi_tid == 0) stamp(5);
      const uint32_t taddr = tmem_base + (static_cast<uint32_t>(q * 32) << 16) + acc * ACC_COLS;
      bool reduce_from_ws = false;   // split-K: final values come from the parked partials
      bool split_ok = true;          // false when the wait for the other splits timed out
      float* ws_tile = nullptr;
      if (p.splits > 1) {
        // Stage 1: park this split's partial tile (column-major: 128 rows contiguous).
        ws_tile = p.partials + static_cast<size_t>(tile) * p.splits * (kLaneRows * ACC_COLS);
        float* mine = ws_tile + static_cast<size_t>(split) * (kLaneRows * ACC_COLS);
#pragma unroll 1
        for (int c = 0; c < ACC_COLS / CW; ++c) {
          uint32_t r[CW];
          if constexpr (CW == 32) tmem_ld_32x32(taddr + c * CW, r);
          else tmem_ld_32x16(taddr + c * CW, r);
          tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < CW; ++j) mine[(c * CW + j) * kLaneRows + row] = __uint_as_float(r[j]);
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_empty[acc]);
        __threadfence();
        named_bar_sync(1, 128);
        // Every split CTA of the tile reduces and finishes its own share of the token rows, so
        // the tail after the last MMA is one round of loads instead of a whole-tile reduction by
        // the last arriver. All split CTAs of a tile are resident together (the host keeps
        // tiles x splits within one wave), so waiting on the arrival counter cannot deadlock.
        if (epi_tid == 0) {
          atomicAdd(&p.counters[tile], 1);
          *last_flag = wait_flag_ge(reinterpret_cast<const uint32_t*>(&p.counters[tile]),
                                    static_cast<uint32_t>(p.splits), p.status)
                           ? 1
                           : 0;
        }
        named_bar_sync(1, 128);
        reduce_from_ws = true;
        split_ok = (*last_flag != 0);
        __threadfence();
      }

      // Stage 2: final values -> epilogue -> global.
      // lane_idx: output token (token-rows-on-lanes) or output feature (weight-rows-on-lanes)
      const int lane_idx = (SWAP ? it.feat0 : it.out_tok0) + row;
      const bool row_ok = row < (SWAP ? it.feat_valid : it.tok_valid);
      const __nv_bfloat16* bias_p = p.bias ? p.bias + it.bias_off : nullptr;
      if constexpr (SWAP) {
        // The accumulator arrives transposed (thread = output feature, columns = tokens) while the
        // output is token-major. Phase A turns the tile around through shared memory ([token][128
        // features] fp32); phase B walks it with 8 consecutive features per thread, so residual
        // loads, global stores and peer pushes are 16-byte vectors. (Two-byte strided stores issued
        // straight from the accumulator layout were measured at ~100 ns each: 10 us per tile.)
        // Split-K partials are parked in exactly the phase-B layout, so the reducing CTA skips
        // phase A and sums them straight from the workspace.
        const int toks = min(BN, it.tok_valid);
        if (!reduce_from_ws) {
          float bias_g = 0.f, bias_u = 0.f;
          if (COMM != 1 && bias_p != nullptr && row_ok) {
            bias_g = __bfloat162float(bias_p[lane_idx]);
            if (glu) bias_u = __bfloat162float(bias_p[p.glu_offset + lane_idx]);
          }
          // narrow chunks when gated: the activation code is fetched once and re-run from the
          // instruction cache instead of being unrolled 32 times
          constexpr int CA = GLU ? 16 : CW;
#pragma unroll 1
          for (int c = 0; c < BN / CA; ++c) {
            uint32_t r[CA];
            float v[CA];
            if constexpr (CA == 32) tmem_ld_32x32(taddr + c * CA, r);
            else tmem_ld_32x16(taddr + c * CA, r);
            tmem_ld_wait();
            if (p.ssq_in != nullptr) {
#pragma unroll
              for (int j = 0; j < CA; ++j) v[j] = __uint_as_float(r[j]) * scale_sm[c * CA + j] + bias_g;
            } else {
#pragma unroll
              for (int j = 0; j < CA; ++j) v[j] = __uint_as_float(r[j]) + bias_g;
            }
            if (glu) {
              if constexpr (CA == 32) tmem_ld_32x32(taddr + BN + c * CA, r);
              else tmem_ld_32x16(taddr + BN + c * CA, r);
              tmem_ld_wait();
              if (p.ssq_in != nullptr) {
#pragma unroll
                for (int j = 0; j < CA; ++j) r[j] = __float_as_uint(__uint_as_float(r[j]) * scale_sm[c * CA + j]);
              }
#pragma unroll
              for (int j = 0; j < CA; ++j)
                v[j] = act_glu(p.epilogue, v[j], __uint_as_float(r[j]) + bias_u, p.glu_alpha, p.glu_limit);
            }
#pragma unroll
            for (int j = 0; j < CA; ++j) staging[(c * CA + j) * kLaneRows + row] = v[j];
          }
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[acc]);
          named_bar_sync(1, 128);
        }
        if (epi_tid == 0) stamp(8);
        const int seg = epi_tid & 15, tsub = epi_tid >> 4;   // 16 feature segments x 8 tokens per pass
        const int nl = seg * 8;
        const int n = it.feat0 + nl;
        const int nvalid = min(8, it.feat_valid - nl);
        const bool vec = p.vec_ok != 0 && nvalid == 8;
        // Token rows of the tile this CTA finishes: all of them, or its share under split-K.
        int t_begin = 0, t_end = toks;
        if (reduce_from_ws) {
          const int per = (toks + p.splits - 1) / p.splits;
          t_begin = min(toks, split * per);
          t_end = split_ok ? min(toks, t_begin + per) : t_begin;
        }
        constexpr int PU = GLU ? 1 : 2;   // token rows per thread whose loads are in flight together

        // (token rows tl0 + 8 g + tsub, features n .. n+7) after bias / activation
        auto tile_values = [&](int tl0, float(&o)[PU][8]) {
          if (!reduce_from_ws) {
#pragma unroll
            for (int g = 0; g < PU; ++g) {
              const int tl = tl0 + g * 8 + tsub;
              if (tl < t_end) {
                const float4 a = *reinterpret_cast<const float4*>(staging + tl * kLaneRows + nl);
                const float4 b = *reinterpret_cast<const float4*>(staging + tl * kLaneRows + nl + 4);
                o[g][0] = a.x, o[g][1] = a.y, o[g][2] = a.z, o[g][3] = a.w;
                o[g][4] = b.x, o[g][5] = b.y, o[g][6] = b.z, o[g][7] = b.w;
              }
            }
            return;
          }
          // Split-K: the partials of all splits for these rows are requested together (four
          // splits per batch) and summed in split order, so the result is deterministic.
          float u[PU][8];
#pragma unroll
          for (int g = 0; g < PU; ++g)
#pragma unroll
            for (int j = 0; j < 8; ++j) o[g][j] = 0.f, u[g][j] = 0.f;
#pragma unroll 1
          for (int s0 = 0; s0 < p.splits; s0 += 4) {
            float4 a[PU][4], b[PU][4];
            [[maybe_unused]] float4 c4[PU][4], d4[PU][4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float* part = ws_tile + static_cast<size_t>(s0 + k) * (kLaneRows * ACC_COLS);
#pragma unroll
              for (int g = 0; g < PU; ++g) {
                const int tl = tl0 + g * 8 + tsub;
                if (s0 + k < p.splits && tl < t_end) {
                  a[g][k] = __ldcg(reinterpret_cast<const float4*>(part + tl * kLaneRows + nl));
                  b[g][k] = __ldcg(reinterpret_cast<const float4*>(part + tl * kLaneRows + nl + 4));
                  if (glu) {
                    c4[g][k] = __ldcg(reinterpret_cast<const float4*>(part + (BN + tl) * kLaneRows + nl));
                    d4[g][k] = __ldcg(reinterpret_cast<const float4*>(part + (BN + tl) * kLaneRows + nl + 4));
                  }
                }
              }
            }
#pragma unroll
            for (int k = 0; k < 4; ++k) {
#pragma unroll
              for (int g = 0; g < PU; ++g) {
                const int tl = tl0 + g * 8 + tsub;
                if (s0 + k < p.splits && tl < t_end) {
                  o[g][0] += a[g][k].x, o[g][1] += a[g][k].y, o[g][2] += a[g][k].z, o[g][3] += a[g][k].w;
                  o[g][4] += b[g][k].x, o[g][5] += b[g][k].y, o[g][6] += b[g][k].z, o[g][7] += b[g][k].w;
                  if (glu) {
                    u[g][0] += c4[g][k].x, u[g][1] += c4[g][k].y, u[g][2] += c4[g][k].z, u[g][3] += c4[g][k].w;
                    u[g][4] += d4[g][k].x, u[g][5] += d4[g][k].y, u[g][6] += d4[g][k].z, u[g][7] += d4[g][k].w;
                  }
                }
              }
            }
          }
          if (p.ssq_in != nullptr) {
#pragma unroll
            for (int g = 0; g < PU; ++g) {
              const int tl = tl0 + g * 8 + tsub;
              const float sc = tl < t_end ? scale_sm[tl] : 1.0f;
#pragma unroll
              for (int j = 0; j < 8; ++j) o[g][j] *= sc, u[g][j] *= sc;
            }
          }
#pragma unroll
          for (int g = 0; g < PU; ++g) {
            if (COMM != 1 && bias_p != nullptr) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                if (j < nvalid) {
                  o[g][j] += __bfloat162float(bias_p[n + j]);
                  if (glu) u[g][j] += __bfloat162float(bias_p[p.glu_offset + n + j]);
                }
              }
            }
            if (glu) {
#pragma unroll
              for (int j = 0; j < 8; ++j)
                o[g][j] = act_glu(p.epilogue, o[g][j], u[g][j], p.glu_alpha, p.glu_limit);
            }
          }
        };
        auto add_bf16x8 = [&](const __nv_bfloat16* src, float(&o)[8]) {
          if (vec) {
            const uint4 a = *reinterpret_cast<const uint4*>(src);
            const uint32_t w4[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              o[2 * j] += bf16_lo(w4[j]);
              o[2 * j + 1] += bf16_hi(w4[j]);
            }
          } else {
            for (int j = 0; j < nvalid; ++j) o[j] += __bfloat162float(src[j]);
          }
        };
        auto store_bf16x8 = [&](__nv_bfloat16* dst, const float(&o)[8]) {
          if (vec) {
            uint4 pk;
            pk.x = pack_bf16(o[0], o[1]);
            pk.y = pack_bf16(o[2], o[3]);
            pk.z = pack_bf16(o[4], o[5]);
            pk.w = pack_bf16(o[6], o[7]);
            *reinterpret_cast<uint4*>(dst) = pk;
          } else {
            for (int j = 0; j < nvalid; ++j) dst[j] = __float2bfloat16(o[j]);
          }
        };
        auto store_out = [&](size_t off, const float(&o)[8]) {
          if (p.out_fp32) {
            float* dst = reinterpret_cast<float*>(p.out) + off;
            if (vec) {
              reinterpret_cast<float4*>(dst)[0] = make_float4(o[0], o[1], o[2], o[3]);
              reinterpret_cast<float4*>(dst)[1] = make_float4(o[4], o[5], o[6], o[7]);
            } else {
              for (int j = 0; j < nvalid; ++j) dst[j] = o[j];
            }
          } else {
            store_bf16x8(reinterpret_cast<__nv_bfloat16*>(p.out) + off, o);
          }
        };


        // Deferred RMSNorm, producer side: sum of squares of the bf16 results of (token tl, this
        // tile's 128 features), reduced over the 16 threads that share the token row and written
        // as one partial per (feature tile, token); the consumer adds the partials in tile order,
        // so the norm is deterministic and identical on every rank. Requires N % 128 == 0 (every
        // thread of the warp takes part in the shuffles).
        auto emit_ssq = [&](int tl, const float(&o)[8]) {
          float sq = 0.f;
          if (tl < t_end) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              const float r = p.out_fp32 ? o[j] : __bfloat162float(__float2bfloat16(o[j]));
              sq += r * r;
            }
          }
          sq += __shfl_xor_sync(0xffffffffu, sq, 8);
          sq += __shfl_xor_sync(0xffffffffu, sq, 4);
          sq += __shfl_xor_sync(0xffffffffu, sq, 2);
          sq += __shfl_xor_sync(0xffffffffu, sq, 1);
          if (seg == 0 && tl < t_end) {
            const int ld = reinterpret_cast<const int*>(p.ssq_out)[1];
            p.ssq_out[8 + static_cast<size_t>(it.feat0 / kLaneRows) * ld + it.out_tok0 + tl] = sq;
          }
        };
        if (p.ssq_out != nullptr && tile == 0 && split == 0 && epi_tid == 0)
          reinterpret_cast<int*>(p.ssq_out)[0] = p.tiles_lane;

        if (nvalid > 0) {
#pragma unroll 1
          for (int tl0 = t_begin; tl0 < t_end; tl0 += 8 * PU) {
            float o[PU][8];
            tile_values(tl0, o);
            if constexpr (COMM == 0) {
              // every residual load of the batch is issued before the first store: `out` may alias
              // `residual`, and interleaving them would serialise one memory latency per token
              if (!glu && p.residual != nullptr) {
#pragma unroll
                for (int g = 0; g < PU; ++g) {
                  const int tl = tl0 + g * 8 + tsub;
                  if (tl < t_end)
                    add_bf16x8(p.residual + static_cast<size_t>(it.out_tok0 + tl) * p.ldr + n, o[g]);
                }
              }
#pragma unroll
              for (int g = 0; g < PU; ++g) {
                const int tl = tl0 + g * 8 + tsub;
                if (tl < t_end) store_out(static_cast<size_t>(it.out_tok0 + tl) * p.ldo + n, o[g]);
              }
              if (p.ssq_out != nullptr) {
#pragma unroll
                for (int g = 0; g < PU; ++g) emit_ssq(tl0 + g * 8 + tsub, o[g]);
              }
            } else if constexpr (COMM == 1) {
              // bf16 partial (no bias / residual yet) into every peer's slot [rank]; with NVLS it
              // stays in this rank's own receive half and the peers pull the sum through the switch
              const size_t base = comm_parity * static_cast<size_t>(p.comm.parity_stride) +
                                  (p.comm.nvls ? 0 : p.comm.rank * static_cast<size_t>(p.comm.rank_stride));
#pragma unroll
              for (int g = 0; g < PU; ++g) {
                const int tl = tl0 + g * 8 + tsub;
                if (tl < t_end) {
                  const size_t off = base + static_cast<size_t>(it.out_tok0 + tl) * p.N + n;
                  if (p.comm.nvls) {
                    // fp32 partials (the switch adds them in fp32 and returns fp32): the only rounding
                    // on this path is the final one to bf16. The half holds world * rank_stride bf16
                    // elements, M * N floats fit (checked on the host).
                    float* dstf = reinterpret_cast<float*>(p.comm.recv_peer[p.comm.rank] +
                                                           comm_parity * static_cast<size_t>(p.comm.parity_stride)) +
                                  static_cast<size_t>(it.out_tok0 + tl) * p.N + n;
                    reinterpret_cast<float4*>(dstf)[0] = make_float4(o[g][0], o[g][1], o[g][2], o[g][3]);
                    reinterpret_cast<float4*>(dstf)[1] = make_float4(o[g][4], o[g][5], o[g][6], o[g][7]);
                  } else {
                    for (int pr = 0; pr < p.comm.world; ++pr) store_bf16x8(p.comm.recv_peer[pr] + off, o[g]);
                  }
                }
              }
            } else {  // COMM == 3: logits tile (+ bias) into every peer's gathered output
#pragma unroll
              for (int g = 0; g < PU; ++g) {
                const int tl = tl0 + g * 8 + tsub;
                if (tl < t_end) {
                  const size_t off = static_cast<size_t>(it.out_tok0 + tl) * p.ldo +
                                     static_cast<size_t>(p.comm.rank) * p.N + n;
                  if (p.comm.nvls && vec) {
                    uint4 pk;
                    pk.x = pack_bf16(o[g][0], o[g][1]);
                    pk.y = pack_bf16(o[g][2], o[g][3]);
                    pk.z = pack_bf16(o[g][4], o[g][5]);
                    pk.w = pack_bf16(o[g][6], o[g][7]);
                    multimem_st_16(p.comm.out_mc + off, pk);   // one store, the switch writes every rank
                  } else {
                    for (int pr = 0; pr < p.comm.world; ++pr) store_bf16x8(p.comm.out_peer[pr] + off, o[g]);
                  }
                }
              }
            }
          }
        }
        if (epi_tid == 0) stamp(9);
        if constexpr (COMM == 0) {
          named_bar_sync(1, 128);   // the staging tile is rewritten by the next work item
        } else if constexpr (COMM == 1) {
          const CommParams& cm = p.comm;
          named_bar_sync(1, 128);
          if (epi_tid == 0) stamp(11);
          if (cm.nvls) {
            if (epi_tid == 0) multimem_signal_add(cm.flags_mc + tile, 1u);
          } else if (epi_tid < cm.world) {
            signal_add_sys(cm.flags_peer[epi_tid] + tile, 1u);
          }
          // one signal per peer from every split CTA of the tile; expect[] advances once per call
          // (by this CTA when the tile is not split, else by the last split CTA to leave, below)
          const uint32_t comm_target = cm.expect[tile] + static_cast<uint32_t>(cm.world * p.splits);
          if (epi_tid == 0) {
            const bool ok = wait_flag_ge(cm.flags_peer[cm.rank] + tile, comm_target, p.status);
            if (p.splits == 1) cm.expect[tile] = comm_target;
            *last_flag = ok ? 1 : 0;
          }
          named_bar_sync(1, 128);
          if (epi_tid == 0) stamp(10);
          // bias + residual + store (+ sums of squares) of G token rows per thread
          auto finish_rows = [&](int tl0, auto& o) {
            constexpr int G = static_cast<int>(sizeof(o) / sizeof(o[0]));
            if (bias_p != nullptr) {
#pragma unroll
              for (int g = 0; g < G; ++g) {
                if (tl0 + g * 8 + tsub < t_end) {
#pragma unroll
                  for (int j = 0; j < 8; ++j)
                    if (j < nvalid) o[g][j] += __bfloat162float(bias_p[n + j]);
                }
              }
            }
            if (p.residual != nullptr) {
#pragma unroll
              for (int g = 0; g < G; ++g) {
                const int tl = tl0 + g * 8 + tsub;
                if (tl < t_end)
                  add_bf16x8(p.residual + static_cast<size_t>(it.out_tok0 + tl) * p.ldr + n, o[g]);
              }
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
              const int tl = tl0 + g * 8 + tsub;
              if (tl < t_end) store_out(static_cast<size_t>(it.out_tok0 + tl) * p.ldo + n, o[g]);
            }
            if (p.ssq_out != nullptr) {
#pragma unroll
              for (int g = 0; g < G; ++g) emit_ssq(tl0 + g * 8 + tsub, o[g]);
            }
          };
          if (*last_flag != 0 && nvalid > 0 && cm.nvls) {
            // the switch adds the `world` replicas of each float in fp32; two 16-byte requests per
            // token row, two token rows per thread in flight (one NVLink round trip per batch)
            const float* basef = reinterpret_cast<const float*>(cm.recv_mc + comm_parity * static_cast<size_t>(cm.parity_stride));
            constexpr int GRPN = 2;
#pragma unroll 1
            for (int tl0 = t_begin; tl0 < t_end; tl0 += 8 * GRPN) {
              float4 a[GRPN][2];
#pragma unroll
              for (int g = 0; g < GRPN; ++g) {
                const int tl = tl0 + g * 8 + tsub;
                a[g][0] = a[g][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (tl < t_end) {
                  const float* src = basef + static_cast<size_t>(it.out_tok0 + tl) * p.N + n;
                  a[g][0] = multimem_ld_reduce_f32x4(src);
                  a[g][1] = multimem_ld_reduce_f32x4(src + 4);
                }
              }
              float o[GRPN][8];
#pragma unroll
              for (int g = 0; g < GRPN; ++g) {
                o[g][0] = a[g][0].x, o[g][1] = a[g][0].y, o[g][2] = a[g][0].z, o[g][3] = a[g][0].w;
                o[g][4] = a[g][1].x, o[g][5] = a[g][1].y, o[g][6] = a[g][1].z, o[g][7] = a[g][1].w;
              }
              finish_rows(tl0, o);
            }
          } else if (*last_flag != 0 && nvalid > 0) {
            // every rank sums the same bf16 partials in rank order: bitwise identical results
            const __nv_bfloat16* base = cm.recv_peer[cm.rank] +
                                        comm_parity * static_cast<size_t>(cm.parity_stride);
            constexpr int GRPC = 2;
#pragma unroll 1
            for (int tl0 = t_begin; tl0 < t_end; tl0 += 8 * GRPC) {
              float o[GRPC][8];
#pragma unroll
              for (int g = 0; g < GRPC; ++g) {
#pragma unroll
                for (int j = 0; j < 8; ++j) o[g][j] = 0.f;
                const int tl = tl0 + g * 8 + tsub;
                if (tl < t_end) {
                  const __nv_bfloat16* src = base + static_cast<size_t>(it.out_tok0 + tl) * p.N + n;
                  if (vec) {
                    uint4 a[kMaxRanks];
#pragma unroll
                    for (int r = 0; r < kMaxRanks; ++r)
                      if (r < cm.world)
                        a[r] = __ldcg(reinterpret_cast<const uint4*>(src + r * static_cast<size_t>(cm.rank_stride)));
#pragma unroll
                    for (int r = 0; r < kMaxRanks; ++r) {
                      if (r < cm.world) {
                        const uint32_t w4[4] = {a[r].x, a[r].y, a[r].z, a[r].w};
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                          o[g][2 * j] += bf16_lo(w4[j]);
                          o[g][2 * j + 1] += bf16_hi(w4[j]);
                        }
                      }
                    }
                  } else {
                    for (int r = 0; r < cm.world; ++r)
                      for (int j = 0; j < nvalid; ++j) {
                        const unsigned short raw = __ldcg(reinterpret_cast<const unsigned short*>(
                            src + r * static_cast<size_t>(cm.rank_stride) + j));
                        o[g][j] += __uint_as_float(static_cast<uint32_t>(raw) << 16);
                      }
                  }
                }
              }
              finish_rows(tl0, o);
            }
          }
        } else {  // COMM == 3
          const CommParams& cm = p.comm;
          named_bar_sync(1, 128);
          if (cm.nvls) {
            if (epi_tid == 0) multimem_signal_add(cm.flags_mc + kCommDoneIdx, 1u);
          } else if (epi_tid < cm.world) {
            signal_add_sys(cm.flags_peer[epi_tid] + kCommDoneIdx, 1u);
          }
        }
        if (p.splits > 1) {
          // Leave the tile: the last split CTA to get here (all of them have read the partials
          // and the arrival counter by then) re-arms the counters for the next launch.
          if constexpr (COMM != 0) named_bar_sync(1, 128);
          if (epi_tid == 0) {
            const int prev = atomicAdd(&p.counters[kSplitDepartOffset + tile], 1);
            if (prev == p.splits - 1) {
              p.counters[tile] = 0;
              p.counters[kSplitDepartOffset + tile] = 0;
              if constexpr (COMM == 1)
                p.comm.expect[tile] += static_cast<uint32_t>(p.comm.world * p.splits);
            }
          }
        }
      } else {
        float ssq_acc = 0.f;   // deferred RMSNorm, producer side: this token row over the tile's features
#pragma unroll 1
        for (int c = 0; c < BN / CW; ++c) {
          float v[CW], u[CW];
          if (!reduce_from_ws) {
            uint32_t r[CW];
            if constexpr (CW == 32) tmem_ld_32x32(taddr + c * CW, r);
            else tmem_ld_32x16(taddr + c * CW, r);
            tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < CW; ++j) v[j] = __uint_as_float(r[j]);
            if (glu) {
              if constexpr (CW == 32) tmem_ld_32x32(taddr + BN + c * CW, r);
              else tmem_ld_32x16(taddr + BN + c * CW, r);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < CW; ++j) u[j] = __uint_as_float(r[j]);
            }
          } else {
#pragma unroll
            for (int j = 0; j < CW; ++j) {
              v[j] = 0.f;
              u[j] = 0.f;
            }
            for (int s = 0; s < p.splits; ++s) {
              const float* part = ws_tile + static_cast<size_t>(s) * (kLaneRows * ACC_COLS);
#pragma unroll
              for (int j = 0; j < CW; ++j) {
                v[j] += __ldcg(&part[(c * CW + j) * kLaneRows + row]);
                if (glu) u[j] += __ldcg(&part[(BN + c * CW + j) * kLaneRows + row]);
              }
            }
          }
          if (row_ok) {
            if constexpr (COMM == 2) {
              // partial tile row -> the owner's slot [rank][tile / world]
              // (NVLS: the partial tile stays in this rank's own receive half, slot = tile; the
              // owner pulls the sum of all ranks' slots through the switch)
              const int owner = comm2_owner(tile, p.comm.world);
              __nv_bfloat16* dst =
                  p.comm.nvls
                      ? p.comm.recv_peer[p.comm.rank] + comm_parity * static_cast<size_t>(p.comm.parity_stride) +
                            static_cast<size_t>(tile) * (kLaneRows * BN) + static_cast<size_t>(row) * BN + c * CW
                      : p.comm.recv_peer[owner] + comm_parity * static_cast<size_t>(p.comm.parity_stride) +
                            p.comm.rank * static_cast<size_t>(p.comm.rank_stride) +
                            static_cast<size_t>(tile / p.comm.world) * (kLaneRows * BN) +
                            static_cast<size_t>(row) * BN + c * CW;
#pragma unroll
              for (int j8 = 0; j8 < CW; j8 += 8) {
                uint4 pk;
                pk.x = pack_bf16(v[j8 + 0], v[j8 + 1]);
                pk.y = pack_bf16(v[j8 + 2], v[j8 + 3]);
                pk.z = pack_bf16(v[j8 + 4], v[j8 + 5]);
                pk.w = pack_bf16(v[j8 + 6], v[j8 + 7]);
                *reinterpret_cast<uint4*>(dst + j8) = pk;
              }
            } else {
              // thread = token m, columns = features
              const int m = lane_idx;
              const int nl0 = c * CW;  // first feature of the chunk inside the tile
              // The residual of the whole chunk is fetched with 16-byte loads before the first
              // store (`out` may alias it, so loads issued between stores would each wait out a
              // full memory latency).
              const bool res_vec = !glu && p.residual != nullptr && p.vec_ok != 0 && nl0 + CW <= it.feat_valid;
              uint4 rs[CW / 8];
              if (res_vec) {
                const __nv_bfloat16* rp = p.residual + static_cast<size_t>(m) * p.ldr + it.feat0 + nl0;
#pragma unroll
                for (int q8 = 0; q8 < CW / 8; ++q8) rs[q8] = *reinterpret_cast<const uint4*>(rp + q8 * 8);
              }
#pragma unroll
              for (int j8 = 0; j8 < CW; j8 += 8) {
                const int nl = nl0 + j8;
                const int n = it.feat0 + nl;
                if (nl >= it.feat_valid) break;
                float o[8];
                const bool full8 = (nl + 8 <= it.feat_valid);
                float rv[8];
                if (res_vec) {
                  const uint32_t w4[4] = {rs[j8 / 8].x, rs[j8 / 8].y, rs[j8 / 8].z, rs[j8 / 8].w};
#pragma unroll
                  for (int j = 0; j < 4; ++j) rv[2 * j] = bf16_lo(w4[j]), rv[2 * j + 1] = bf16_hi(w4[j]);
                }
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                  float val = v[j8 + j] * row_scale;
                  const bool in = full8 || (nl + j < it.feat_valid);
                  if (glu) {
                    float g = val, uu = u[j8 + j] * row_scale;
                    if (bias_p != nullptr && in) {
                      g += __bfloat162float(bias_p[n + j]);
                      uu += __bfloat162float(bias_p[p.glu_offset + n + j]);
                    }
                    val = act_glu(p.epilogue, g, uu, p.glu_alpha, p.glu_limit);
                  } else {
                    if (bias_p != nullptr && in) val += __bfloat162float(bias_p[n + j]);
                    if (res_vec)
                      val += rv[j];
                    else if (p.residual != nullptr && in)
                      val += __bfloat162float(p.residual[static_cast<size_t>(m) * p.ldr + n + j]);
                  }
                  o[j] = val;
                  if (p.ssq_out != nullptr && in) {
                    const float r = p.out_fp32 ? val : __bfloat162float(__float2bfloat16(val));
                    ssq_acc += r * r;
                  }
                }
                const size_t off = static_cast<size_t>(m) * p.ldo + n;
                if (p.out_fp32) {
                  float* dst = reinterpret_cast<float*>(p.out) + off;
                  if (full8 && ((off & 3) == 0)) {
                    reinterpret_cast<float4*>(dst)[0] = make_float4(o[0], o[1], o[2], o[3]);
                    reinterpret_cast<float4*>(dst)[1] = make_float4(o[4], o[5], o[6], o[7]);
                  } else {
                    for (int j = 0; j < 8 && nl + j < it.feat_valid; ++j) dst[j] = o[j];
                  }
                } else {
                  __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + off;
                  if (full8 && ((off & 7) == 0)) {
                    uint4 pk;
                    pk.x = pack_bf16(o[0], o[1]);
                    pk.y = pack_bf16(o[2], o[3]);
                    pk.z = pack_bf16(o[4], o[5]);
                    pk.w = pack_bf16(o[6], o[7]);
                    *reinterpret_cast<uint4*>(dst) = pk;
                  } else {
                    for (int j = 0; j < 8 && nl + j < it.feat_valid; ++j) dst[j] = __float2bfloat16(o[j]);
                  }
                }
              }
            }
          }
        }
        if (!reduce_from_ws) {
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(&tmem_empty[acc]);
        }
        if (COMM == 0 && p.ssq_out != nullptr) {
          const int ld = reinterpret_cast<const int*>(p.ssq_out)[1];
          if (row_ok) p.ssq_out[8 + static_cast<size_t>(it.feat0 / BN) * ld + it.out_tok0 + row] = ssq_acc;
          if (tile == 0 && epi_tid == 0) reinterpret_cast<int*>(p.ssq_out)[0] = p.tiles_col;
        }
      }
      if constexpr (COMM == 2) {
        const CommParams& cm = p.comm;
        const int owner = comm2_owner(tile, cm.world);
        named_bar_sync(1, 128);
        if (epi_tid == 0) signal_add_sys(cm.flags_peer[owner] + tile, 1u);
        if (owner == cm.rank) {
          if (epi_tid == 0) {
            const uint32_t target = cm.expect[tile] + static_cast<uint32_t>(cm.world);
            const bool ok = wait_flag_ge(cm.flags_peer[cm.rank] + tile, target, p.status);
            cm.expect[tile] = target;
            *last_flag = ok ? 1 : 0;
          }
          named_bar_sync(1, 128);
          const int m = lane_idx;
          if (*last_flag != 0 && cm.nvls) {
            // The tile slot is one contiguous [128][BN] bf16 array on every rank: the 128 threads
            // walk it in 16-byte pieces (a warp reads 512 contiguous bytes per request), eight
            // pieces per thread in flight; the switch returns the fp32-accumulated sum of the
            // replicas, bias and residual are added, and one multimem.st writes every rank's output.
            const __nv_bfloat16* base = cm.recv_mc + comm_parity * static_cast<size_t>(cm.parity_stride) +
                                        static_cast<size_t>(tile) * (kLaneRows * BN);
            constexpr int PIECES = kLaneRows * BN / 8;       // 16-byte pieces of the tile
            constexpr int PER_ROW = BN / 8;
            constexpr int UNR = 8;
            const int rows_valid = min(kLaneRows, it.tok_valid);
            const int nfeat = min(BN, it.feat_valid);
#pragma unroll 1
            for (int i0 = epi_tid; i0 < rows_valid * PER_ROW; i0 += 128 * UNR) {
              uint4 a[UNR];
#pragma unroll
              for (int u = 0; u < UNR; ++u) {
                const int i = i0 + u * 128;
                a[u] = make_uint4(0u, 0u, 0u, 0u);
                if (i < rows_valid * PER_ROW && i < PIECES && (i % PER_ROW) * 8 < nfeat)
                  a[u] = multimem_ld_reduce_bf16x8(base + static_cast<size_t>(i) * 8);
              }
#pragma unroll
              for (int u = 0; u < UNR; ++u) {
                const int i = i0 + u * 128;
                const int r = i / PER_ROW, j = (i % PER_ROW) * 8;
                if (i < rows_valid * PER_ROW && j < nfeat) {
                  const uint32_t w4[4] = {a[u].x, a[u].y, a[u].z, a[u].w};
                  float o[8];
#pragma unroll
                  for (int q4 = 0; q4 < 4; ++q4) o[2 * q4] = bf16_lo(w4[q4]), o[2 * q4 + 1] = bf16_hi(w4[q4]);
                  if (p.bias != nullptr) {
#pragma unroll
                    for (int q8 = 0; q8 < 8; ++q8) o[q8] += __bfloat162float(p.bias[it.feat0 + j + q8]);
                  }
                  const size_t tok = static_cast<size_t>(it.out_tok0 + r);
                  if (p.residual != nullptr) {
                    const uint4 rs = *reinterpret_cast<const uint4*>(p.residual + tok * p.ldr + it.feat0 + j);
                    const uint32_t r4[4] = {rs.x, rs.y, rs.z, rs.w};
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4) o[2 * q4] += bf16_lo(r4[q4]), o[2 * q4 + 1] += bf16_hi(r4[q4]);
                  }
                  uint4 pk;
                  pk.x = pack_bf16(o[0], o[1]);
                  pk.y = pack_bf16(o[2], o[3]);
                  pk.z = pack_bf16(o[4], o[5]);
                  pk.w = pack_bf16(o[6], o[7]);
                  multimem_st_16(cm.out_mc + tok * p.ldo + it.feat0 + j, pk);
                }
              }
            }
          } else if (*last_flag != 0 && row_ok) {
            const __nv_bfloat16* base = cm.recv_peer[cm.rank] +
                                        comm_parity * static_cast<size_t>(cm.parity_stride) +
                                        static_cast<size_t>(tile / cm.world) * (kLaneRows * BN) +
                                        static_cast<size_t>(row) * BN;
            // NQ 8-feature chunks x up to WMAX ranks of partials are requested together (8 loads
            // of 16 bytes in flight), then summed in rank order, finished and pushed to every peer.
            const __nv_bfloat16* bias_n = p.bias != nullptr ? p.bias + it.feat0 : nullptr;
            const __nv_bfloat16* res_n =
                p.residual != nullptr ? p.residual + static_cast<size_t>(m) * p.ldr + it.feat0 : nullptr;
            const size_t off0 = static_cast<size_t>(m) * p.ldo + it.feat0;
            const int nfeat = min(BN, it.feat_valid);
            if (cm.world <= 2) {
              for (int j0 = 0; j0 < nfeat; j0 += 32)
                comm2_reduce_span<4, 2>(base, cm.rank_stride, cm.world, bias_n, res_n, cm.out_peer, off0, j0, nfeat);
            } else if (cm.world <= 4) {
              for (int j0 = 0; j0 < nfeat; j0 += 16)
                comm2_reduce_span<2, 4>(base, cm.rank_stride, cm.world, bias_n, res_n, cm.out_peer, off0, j0, nfeat);
            } else {
              for (int j0 = 0; j0 < nfeat; j0 += 8)
                comm2_reduce_span<1, 8>(base, cm.rank_stride, cm.world, bias_n, res_n, cm.out_peer, off0, j0, nfeat);
            }
          }
          named_bar_sync(1, 128);
          if (cm.nvls) {
            if (epi_tid == 0) multimem_signal_add(cm.flags_mc + kCommDoneIdx, 1u);
          } else if (epi_tid < cm.world) {
            signal_add_sys(cm.flags_peer[epi_tid] + kCommDoneIdx, 1u);
          }
        }
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }
    if constexpr (COMM != 0) {
      // Per-call completion: every tile of every rank has landed here before the kernel ends,
      // then the last CTA to finish advances the channel's call counter.
      if (epi_tid == 0) {
        const CommParams& cm = p.comm;
        const uint32_t tiles = static_cast<uint32_t>(p.tiles_lane * p.tiles_col);
        const uint32_t per_call =
            (COMM == 2) ? tiles : (COMM == 3 ? tiles * static_cast<uint32_t>(p.splits) * cm.world : 0u);
        if (per_call != 0u) {
          const uint32_t target = *reinterpret_cast<volatile uint32_t*>(cm.ctl + 2) + per_call;
          wait_flag_ge(cm.flags_peer[cm.rank] + kCommDoneIdx, target, p.status);
        }
        __threadfence();
        const uint32_t prev = atomicAdd(cm.ctl + 1, 1u);
        if (prev == gridDim.x - 1) {
          cm.ctl[1] = 0u;
          cm.ctl[2] += per_call;
          __threadfence();
          atomicAdd(cm.ctl, 1u);
        }
      }
    }
  }

  // ------------------------------------------------------------------ teardown
  if (threadIdx.x == 64) stamp(6);
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, TMEM_COLS);
    if (lane == 0) stamp(7);
  }
}

// ----------------------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) ==
            cudaSuccess &&
        qres == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<EncodeTiledFn>(sym);
    }
  });
  return fn;
}

struct MapKey {
  const void* ptr;
  uint64_t rows, cols, ld;
  uint32_t box_rows, box_cols;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && rows == o.rows && cols == o.cols && ld == o.ld &&
           box_rows == o.box_rows && box_cols == o.box_cols;
  }
};
struct MapKeyHash {
  size_t operator()(const MapKey& k) const {
    size_t h = reinterpret_cast<size_t>(k.ptr);
    h = h * 1000003u ^ k.rows;
    h = h * 1000003u ^ k.cols;
    h = h * 1000003u ^ k.ld;
    h = h * 1000003u ^ (static_cast<size_t>(k.box_rows) << 16 | k.box_cols);
    return h;
  }
};

// 2-D bf16 row-major tensor [rows, cols] with leading dimension ld (elements); box is
// {box_cols (inner, 64 = 128 bytes), box_rows}; 128-byte swizzle; out-of-range reads give 0.
bool make_tensor_map_bf16(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t cols,
                          uint64_t ld, uint32_t box_rows, uint32_t box_cols) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key{ptr, rows, cols, ld, box_rows, box_cols};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return true;
    }
  }
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return false;
  cuuint64_t gdim[2] = {cols, rows};
  cuuint64_t gstride[1] = {ld * 2};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), gdim, gstride,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 65536) cache.clear();
  cache.emplace(key, *out);
  return true;
}

// 2-D byte tensor [rows, row_bytes] with row stride ld_bytes; box {box_bytes (inner, multiple of
// 16), box_rows}; no swizzle (packed quantized weights, unpacked by the transform warps).
bool make_tensor_map_u8(CUtensorMap* out, const void* ptr, uint64_t rows, uint64_t row_bytes,
                        uint64_t ld_bytes, uint32_t box_rows, uint32_t box_bytes) {
  static std::mutex mu;
  static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> cache;
  MapKey key{ptr, rows, row_bytes, ld_bytes, box_rows, box_bytes};
  {
    std::lock_guard<std::mutex> g(mu);
    auto it = cache.find(key);
    if (it != cache.end()) {
      *out = it->second;
      return true;
    }
  }
  EncodeTiledFn enc = get_encode_fn();
  if (enc == nullptr) return false;
  cuuint64_t gdim[2] = {row_bytes, rows};
  cuuint64_t gstride[1] = {ld_bytes};
  cuuint32_t box[2] = {box_bytes, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(out, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), gdim, gstride, box, estr,
                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return false;
  std::lock_guard<std::mutex> g(mu);
  if (cache.size() > 65536) cache.clear();
  cache.emplace(key, *out);
  return true;
}

// Tuning knob: resident CTAs per SM for the small-M weight-streaming path. With 2, the stage ring
// of each CTA is halved and twice as many (shorter) split-K pieces are in flight, so one CTA's
// prologue / epilogue latency overlaps the other's main loop.
int gemm_ctas_per_sm() {
  static const int v = [] {
    const char* e = getenv("MLXCEL_B200_GEMM_CTAS_PER_SM");
    const int n = e ? atoi(e) : 1;
    return n == 2 ? 2 : 1;
  }();
  return v;
}

int device_sm_count() {
  static int sms[64] = {0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) return 148;
  if (sms[dev] == 0) {
    int n = 0;
    cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    sms[dev] = n > 0 ? n : 148;
  }
  return sms[dev];
}

constexpr int ACC_COLS_HOST(int bn, bool glu) { return glu ? 2 * bn : bn; }

template <int BN, bool SWAP, bool GLU, int COMM = 0, bool GROUPED = false, int WQ = 0>
static int launch_gemm(const CUtensorMap& ml, const CUtensorMap& mc, GemmParams p, int grid,
                       cudaStream_t stream) {
  constexpr int LANE_TILES = (SWAP && GLU) ? 2 : 1;
  constexpr int COL_TILES = (!SWAP && GLU) ? 2 : 1;
  constexpr int PK_BYTES = WQ != 0 ? wq_block_rows(WQ) * kBK * wq_bits(WQ) / 8 : 0;
  constexpr int STAGE_BYTES =
      (LANE_TILES * (kLaneRows * kBK * 2 + PK_BYTES) + COL_TILES * BN * kBK * 2 + 1023) / 1024 * 1024;
  constexpr int STAGING_BYTES = SWAP ? BN * kLaneRows * 4 : 0;
  constexpr int kSmemBudget = 227 * 1024 - 1024 /*align*/ - kCtrlBytes - STAGING_BYTES;
  int stages = kSmemBudget / STAGE_BYTES;
  if (SWAP && COMM == 0 && !GROUPED && gemm_ctas_per_sm() == 2 && 2 * (2 * ACC_COLS_HOST(BN, GLU)) <= 512) {
    const int half = (227 * 1024 / 2 - 2048 - 1024 - kCtrlBytes - STAGING_BYTES) / STAGE_BYTES;
    if (half >= 3) stages = half;
  }
  if (stages > kMaxStages) stages = kMaxStages;
  {
    // Tuning knob: cap the stage count (shared-memory footprint) from the environment.
    static const int cap = [] {
      const char* e = getenv("MLXCEL_B200_GEMM_STAGES");
      return e ? atoi(e) : 0;
    }();
    if (cap >= 2 && stages > cap) stages = cap;
  }
  {
    // Opt-in (MLXCEL_B200_GEMM_OVERLAP=1): cap the ring so that two consecutive small-M GEMMs fit
    // on an SM together and the next one prefetches weights while this one drains. Measured
    // neutral-to-slower than a deep ring on Llama-8B decode, hence off by default.
    static const bool overlap = [] {
      const char* e = getenv("MLXCEL_B200_GEMM_OVERLAP");
      return e != nullptr && e[0] == '1';
    }();
    if (overlap && SWAP && !GROUPED && BN <= 64 && gemm_ctas_per_sm() == 1) {
      const int cap2 = GLU ? 3 : 4;
      if (stages > cap2) stages = cap2;
    }
  }
  if (stages < 2) return -3;
  p.stages = stages;
  {
    static const int gm = [] {
      const char* e = getenv("MLXCEL_B200_GEMM_RASTER");
      return e != nullptr ? atoi(e) : 16;
    }();
    p.raster_gm = (!SWAP && !GROUPED && gm > 0 && p.tiles_lane > gm) ? gm : 0;
  }
  {
    static const bool trace_on = [] {
      const char* e = getenv("MLXCEL_B200_GEMM_TRACE");
      return e != nullptr && e[0] == '1';
    }();
    // status, counters and partials share one allocation: the trace area sits between them
    p.trace = (trace_on && p.status != nullptr)
                  ? reinterpret_cast<unsigned long long*>(reinterpret_cast<uint8_t*>(p.status) +
                                                          (MX_WS_TRACE_OFFSET - MX_WS_STATUS_OFFSET))
                  : nullptr;
  }
  {
    static const int l2_kb = [] {
      const char* e = getenv("MLXCEL_B200_GEMM_L2_PREFETCH_KB");
      return e != nullptr ? atoi(e) : 0;
    }();
    p.l2_prefetch_kb = (SWAP && !GROUPED && pdl_enabled()) ? (l2_kb * 1024) / (LANE_TILES * kLaneRows * kBK * 2) : 0;
  }
  const int smem = stages * STAGE_BYTES + STAGING_BYTES + 1024 + kCtrlBytes;
  {
    auto al16 = [](const void* q) { return (reinterpret_cast<uintptr_t>(q) & 15) == 0; };
    bool ok = (p.N % 8 == 0) && (p.ldo % 8 == 0) && al16(p.out) &&
              (p.residual == nullptr || (p.ldr % 8 == 0 && al16(p.residual)));
    if (COMM != 0) {
      ok = ok && (p.comm.parity_stride % 8 == 0) && (p.comm.rank_stride % 8 == 0);
      for (int r = 0; r < p.comm.world; ++r) ok = ok && al16(p.comm.recv_peer[r]) && al16(p.comm.out_peer[r]);
    }
    p.vec_ok = ok ? 1 : 0;
    if (COMM != 0 && p.comm.nvls) {
      // the multimem forms move 16 bytes: they need the vector layout and aligned multicast addresses
      bool mc_ok = ok && p.comm.flags_mc != nullptr && (COMM == 3 || al16(p.comm.recv_mc)) &&
                   (COMM == 1 || al16(p.comm.out_mc));
      if (COMM == 1)
        mc_ok = mc_ok && p.comm.recv_mc != nullptr && (p.N % 8 == 0) &&
                2ll * p.M * p.N <= p.comm.parity_stride;   // fp32 partials in the bf16-sized half
      if (COMM == 2)
        mc_ok = mc_ok && p.comm.recv_mc != nullptr && p.comm.out_mc != nullptr &&
                static_cast<long long>(p.tiles_lane) * p.tiles_col * kLaneRows * BN <= p.comm.parity_stride;
      if (COMM == 3) mc_ok = mc_ok && p.comm.out_mc != nullptr;
      if (!mc_ok) p.comm.nvls = 0;
    }
  }
  auto kern = gemm_bf16_kernel<BN, SWAP, GLU, COMM, GROUPED, WQ>;
  // function attributes are per device: a process that drives several GPUs sets them on each
  static bool configured[64] = {false};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64) dev = 0;
  if (!configured[dev]) {
    cudaError_t e =
        cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return static_cast<int>(e);
    prefer_max_shared(kern);
    configured[dev] = true;
  }
  return static_cast<int>(launch_kernel(kern, dim3(grid), dim3(gemm_threads(WQ)), smem, stream, ml, mc, p));
}

}  // namespace mx

using namespace mx;

extern "C" long long mx_gemm_workspace_bytes(void) { return 64ll << 20; }

namespace {
// Deferred RMSNorm request of one call (MxGemmExtras) -> launch parameters.
//   ssq_in  (consumer): the GEMM input is an un-normalised residual stream whose norm weight was
//           folded into W; every output row t is multiplied by rsqrt(sum_p ssq_in[p][t] * inv_dim +
//           eps) before bias / activation.
//   ssq_out (producer): besides its result the GEMM leaves, per (128- or 256-feature tile, token),
//           the sum of squares of that part of the result row, for the next consumer.
// Buffer layout (fp32 words): [0] partial count (written by the producer), [1] tokens per partial
// row (set by the owner of the buffer), data from word 8. No counterpart in the reference, where
// the norm is its own kernel (src/lib/mlxcel-core/cpp/fused_norm.cpp).
int take_row_norm(mx::GemmParams& p, const MxGemmExtras* ex, bool swap, int N, int comm_mode) {
  if (ex == nullptr) return 0;
  p.ssq_in = static_cast<const float*>(ex->ssq_in);
  p.ssq_out = static_cast<float*>(ex->ssq_out);
  p.ssq_eps = ex->ssq_eps;
  p.ssq_inv_dim = ex->ssq_inv_dim;
  if (p.ssq_out != nullptr) {
    if (comm_mode == 2 || comm_mode == 3) return -6;   // producers: plain and one-shot all-reduce only
    if (swap && (N % 128) != 0) return -6;
  }
  if (p.ssq_in != nullptr && comm_mode != 0) return -6;
  return 0;
}
struct QuantArgs {
  int group = 0, wq = 0;
};
// Quantized weights of one call (MxGemmExtras.wq != 0): `w` then points to the weights RE-TILED
// for this kernel (built once at load time from the checkpoint tensors,
// mlxcel_b200.ops.quant.tile_for_gemm): block (t, kb) holds 128 rows x (64 * bits / 8) bytes of
// packed values (rows zero-padded to a multiple of 128), then the block's scales [2 halves of the
// k-block][128 rows] and, for affine, biases, as extra rows of the same width; blocks are ordered
// [row tile t][k-block kb]. One TMA box brings a whole block; ldw is ignored. The kernel
// dequantises the blocks in its transform warps (M <= 256 only; the call returns -9 for larger M,
// which the caller serves by dequantise + GEMM).
// wq: 1 affine 4-bit, 2 affine 8-bit, 3 mxfp4 (e2m1 values, e8m0 scale bytes).
// Replaces the reference's qmm / qmv kernels for M > 8 (mlx/backend/cuda/quantized/qmm_*.cu in its
// MLX overlay) with a tcgen05 path.
QuantArgs take_quant(const MxGemmExtras* ex) {
  QuantArgs q;
  if (ex != nullptr) {
    q.group = ex->q_group;
    q.wq = ex->wq;
  }
  return q;
}
}  // namespace

extern "C" int mx_gemm_bf16(const void* x, const void* w, void* out, const void* bias,
                            const void* residual, int M, int N, int K, int ldx, int ldw, int ldo,
                            int ldr, int epilogue, int out_fp32, int glu_offset, float glu_alpha,
                            float glu_limit, void* workspace, long long ws_bytes, int force_mode,
                            int force_splits, void* stream_, const MxGemmExtras* extras) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const QuantArgs quant = take_quant(extras);
  if (M <= 0 || N <= 0 || K <= 0) return -1;
  if ((K % 8) || (ldx % 8) || (quant.wq == 0 && (ldw % 8))) return -1;
  if ((reinterpret_cast<uintptr_t>(x) & 15) || (reinterpret_cast<uintptr_t>(w) & 15)) return -1;
  if (workspace == nullptr || ws_bytes < MX_WS_PARTIAL_OFFSET) return -2;
  if (quant.wq != 0) {
    if (M > 256 || force_mode == 1) return -9;   // large M: dequantise + GEMM is the better split
    if (K % kBK || quant.wq < 1 || quant.wq > 3) return -1;
  }
  const bool glu = epilogue == MX_EPI_SWIGLU || epilogue == MX_EPI_GEGLU ||
                   epilogue == MX_EPI_CLIPPED_SWIGLU;
  const bool swap = force_mode == 2 || (force_mode == 0 && M <= 256);
  const int w_rows = glu ? (glu_offset + N) : N;

  GemmParams p{};
  p.out = out;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = (epilogue == MX_EPI_RESIDUAL) ? static_cast<const __nv_bfloat16*>(residual) : nullptr;
  if (epilogue == MX_EPI_NONE) p.bias = nullptr;
  p.status = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + MX_WS_STATUS_OFFSET);
  p.counters = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + MX_WS_COUNTER_OFFSET);
  p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + MX_WS_PARTIAL_OFFSET);
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldo = ldo;
  p.ldr = ldr;
  p.glu_offset = glu_offset;
  p.epilogue = epilogue;
  p.out_fp32 = out_fp32;
  p.glu_alpha = glu_alpha;
  p.glu_limit = glu_limit;
  p.num_kb = (K + kBK - 1) / kBK;
  p.splits = 1;
  p.kb_per_split = p.num_kb;
  if (const int rn = take_row_norm(p, extras, swap, N, 0); rn != 0) return rn;
  p.q_group = quant.group;
  p.q_groups_per_row = quant.wq != 0 ? K / quant.group : 0;
  p.q_rows = w_rows;
  p.q_glu_tiles = glu ? glu_offset / kLaneRows : 0;

  const int sms = device_sm_count();
  int bn;
  if (swap) {
    bn = (M <= 16) ? 16 : (M <= 32) ? 32 : (M <= 64) ? 64 : 128;
    p.tiles_lane = (N + kLaneRows - 1) / kLaneRows;
    p.tiles_col = (M + bn - 1) / bn;
    const int tiles = p.tiles_lane * p.tiles_col;
    const int acc_cols = glu ? 2 * bn : bn;
    const int per_sm = (gemm_ctas_per_sm() == 2 && 4 * acc_cols <= 512) ? 2 : 1;
    int splits = force_splits > 0 ? force_splits : (per_sm * sms) / tiles;
    if (splits > p.num_kb / 4) splits = p.num_kb / 4;
    if (splits > 16) splits = 16;
    if (splits < 1) splits = 1;
    const long long ws_floats = (ws_bytes - MX_WS_PARTIAL_OFFSET) / 4;
    while (splits > 1 && (static_cast<long long>(tiles) * splits * kLaneRows * acc_cols > ws_floats ||
                          tiles > MX_WS_COUNTER_BYTES / 8 ||
                          static_cast<long long>(tiles) * splits > static_cast<long long>(per_sm) * sms))
      --splits;
    p.kb_per_split = (p.num_kb + splits - 1) / splits;
    p.splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;
  } else {
    bn = glu ? 128 : (N > 128 ? 256 : 128);
    p.tiles_lane = (M + kLaneRows - 1) / kLaneRows;
    p.tiles_col = (N + bn - 1) / bn;
  }
  const long long total = static_cast<long long>(p.tiles_lane) * p.tiles_col * p.splits;
  const int cap = (swap && gemm_ctas_per_sm() == 2 && 4 * (glu ? 2 * bn : bn) <= 512) ? 2 * sms : sms;
  const int grid = static_cast<int>(total < cap ? total : cap);

  CUtensorMap map_x, map_w;
  const uint32_t x_box = swap ? bn : kLaneRows;
  const uint32_t w_box = swap ? kLaneRows : bn;
  if (!make_tensor_map_bf16(&map_x, x, M, K, ldx, x_box, kBK)) return -4;
  if (quant.wq != 0) {
    const int bits = wq_bits(quant.wq);
    // tiled weights: [ceil(w_rows / 128) * K / 64 blocks][128 rows][pkb bytes], fully contiguous
    const uint64_t pkb = static_cast<uint64_t>(kBK) * bits / 8;
    const uint32_t brows = static_cast<uint32_t>(wq_block_rows(quant.wq) * pkb / 256);   // 256-byte rows per block
    const uint64_t trows = static_cast<uint64_t>((w_rows + kLaneRows - 1) / kLaneRows) * p.num_kb * brows;
    if (glu && (glu_offset % kLaneRows)) return -9;
    if (!make_tensor_map_u8(&map_w, w, trows, 256, 256, brows, 256)) return -4;
#define MX_QLAUNCH(BN_, GLU_)                                                                        \
    switch (quant.wq) {                                                                                \
      case 1: return launch_gemm<BN_, true, GLU_, 0, false, 1>(map_w, map_x, p, grid, stream);         \
      case 2: return launch_gemm<BN_, true, GLU_, 0, false, 2>(map_w, map_x, p, grid, stream);         \
      default: return launch_gemm<BN_, true, GLU_, 0, false, 3>(map_w, map_x, p, grid, stream);        \
    }
    if (glu) {
      switch (bn) {
        case 16: MX_QLAUNCH(16, true);
        case 32: MX_QLAUNCH(32, true);
        case 64: MX_QLAUNCH(64, true);
        default: MX_QLAUNCH(128, true);
      }
    } else {
      switch (bn) {
        case 16: MX_QLAUNCH(16, false);
        case 32: MX_QLAUNCH(32, false);
        case 64: MX_QLAUNCH(64, false);
        default: MX_QLAUNCH(128, false);
      }
    }
#undef MX_QLAUNCH
  }
  if (!make_tensor_map_bf16(&map_w, w, w_rows, K, ldw, w_box, kBK)) return -4;
  const CUtensorMap& ml = swap ? map_w : map_x;
  const CUtensorMap& mc = swap ? map_x : map_w;

#define MX_LAUNCH(BN_, SWAP_, GLU_) return launch_gemm<BN_, SWAP_, GLU_>(ml, mc, p, grid, stream)
  if (swap) {
    if (glu) {
      switch (bn) {
        case 16: MX_LAUNCH(16, true, true);
        case 32: MX_LAUNCH(32, true, true);
        case 64: MX_LAUNCH(64, true, true);
        default: MX_LAUNCH(128, true, true);
      }
    } else {
      switch (bn) {
        case 16: MX_LAUNCH(16, true, false);
        case 32: MX_LAUNCH(32, true, false);
        case 64: MX_LAUNCH(64, true, false);
        default: MX_LAUNCH(128, true, false);
      }
    }
  } else {
    if (glu) MX_LAUNCH(128, false, true);
    if (bn == 256) MX_LAUNCH(256, false, false);
    MX_LAUNCH(128, false, false);
  }
#undef MX_LAUNCH
}

// Fused GEMM + collective over a symmetric heap (see CommParams). mode: 1 one-shot all-reduce
// (M <= 256), 2 two-shot all-reduce, 3 all-gather of the output columns (M <= 256).
// `flags_peer`, `recv_peer`, `out_peer` are host arrays of `world` device addresses (the same
// heap offset on every rank); `ctl` (4 words) and `expect` (8193 words) are this rank's
// control words of the channel; all of them start at zero.
//   mode 1: result rows go to `out` (local, ldo), residual/bias are added after the reduction.
//   mode 2: result tiles are stored into every out_peer (ldo), so `out_peer[rank]` must be the
//           local view of the replicated output (it may alias `residual`).
//   mode 3: out_peer[r][t, rank * N + n]; N is this rank's column count.
extern "C" int mx_gemm_comm(const void* x, const void* w, void* out, const void* bias,
                            const void* residual, int M, int N, int K, int ldx, int ldw, int ldo,
                            int ldr, int mode, int rank, int world, const void* const* flags_peer,
                            const void* const* recv_peer, const void* const* out_peer, void* ctl,
                            void* expect, long long parity_stride, long long rank_stride,
                            void* workspace, long long ws_bytes, void* stream_, const MxGemmExtras* extras) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const QuantArgs quant = take_quant(extras);
  if (M <= 0 || N <= 0 || K <= 0 || world < 1 || world > kMaxRanks || rank < 0 || rank >= world)
    return -1;
  if ((K % 8) || (ldx % 8) || (quant.wq == 0 && (ldw % 8)) || (N % 8) || (ldo % 8)) return -1;
  if (quant.wq != 0) {
    // quantized row-parallel projection -> all-reduce in one kernel (one-shot only)
    if (mode != 1) return -9;
    if (K % kBK || quant.wq < 1 || quant.wq > 3) return -1;
  }
  if (workspace == nullptr || ws_bytes < MX_WS_PARTIAL_OFFSET) return -2;
  if ((mode == 1 || mode == 3) && M > 256) return -1;
  if (mode < 1 || mode > 3) return -1;
  const bool swap = mode != 2;

  GemmParams p{};
  p.out = out;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.residual = static_cast<const __nv_bfloat16*>(residual);
  p.status = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + MX_WS_STATUS_OFFSET);
  p.counters = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + MX_WS_COUNTER_OFFSET);
  p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + MX_WS_PARTIAL_OFFSET);
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldo = ldo;
  p.ldr = ldr;
  p.epilogue = residual ? MX_EPI_RESIDUAL : (bias ? MX_EPI_BIAS : MX_EPI_NONE);
  p.num_kb = (K + kBK - 1) / kBK;
  p.splits = 1;
  p.kb_per_split = p.num_kb;
  p.comm.rank = rank;
  p.comm.world = world;
  p.comm.ctl = static_cast<uint32_t*>(ctl);
  p.comm.expect = static_cast<uint32_t*>(expect);
  for (int r = 0; r < world; ++r) {
    p.comm.flags_peer[r] = static_cast<uint32_t*>(const_cast<void*>(flags_peer[r]));
    p.comm.recv_peer[r] = recv_peer ? static_cast<__nv_bfloat16*>(const_cast<void*>(recv_peer[r])) : nullptr;
    p.comm.out_peer[r] = out_peer ? static_cast<__nv_bfloat16*>(const_cast<void*>(out_peer[r])) : nullptr;
  }
  p.comm.parity_stride = parity_stride;
  p.comm.rank_stride = rank_stride;
  if (const int rn = take_row_norm(p, extras, swap, N, mode); rn != 0) return rn;
  if (extras != nullptr && extras->flags_mc != nullptr) {
    p.comm.nvls = 1;   // withdrawn in launch_gemm when the layout does not allow 16-byte multimem accesses
    p.comm.flags_mc = static_cast<uint32_t*>(extras->flags_mc);
    p.comm.recv_mc = static_cast<__nv_bfloat16*>(extras->recv_mc);
    p.comm.out_mc = static_cast<__nv_bfloat16*>(extras->out_mc);
  }
  p.q_group = quant.group;
  p.q_groups_per_row = quant.wq != 0 ? K / quant.group : 0;
  p.q_rows = N;

  const int sms = device_sm_count();
  int bn;
  if (swap) {
    bn = (M <= 16) ? 16 : (M <= 32) ? 32 : (M <= 64) ? 64 : 128;
    p.tiles_lane = (N + kLaneRows - 1) / kLaneRows;
    p.tiles_col = (M + bn - 1) / bn;
    const int tiles = p.tiles_lane * p.tiles_col;
    int splits = sms / tiles;
    if (splits > p.num_kb / 4) splits = p.num_kb / 4;
    if (splits > 16) splits = 16;
    if (splits < 1) splits = 1;
    const long long ws_floats = (ws_bytes - MX_WS_PARTIAL_OFFSET) / 4;
    while (splits > 1 && static_cast<long long>(tiles) * splits * kLaneRows * bn > ws_floats) --splits;
    p.kb_per_split = (p.num_kb + splits - 1) / splits;
    p.splits = (p.num_kb + p.kb_per_split - 1) / p.kb_per_split;
    if (mode == 1 && static_cast<long long>(M) * N > rank_stride) return -5;
  } else {
    bn = N > 128 ? 256 : 128;
    p.tiles_lane = (M + kLaneRows - 1) / kLaneRows;
    p.tiles_col = (N + bn - 1) / bn;
    const long long slots = (static_cast<long long>(p.tiles_lane) * p.tiles_col + world - 1) / world;
    if (slots * kLaneRows * bn > rank_stride) return -5;
  }
  if (p.tiles_lane * p.tiles_col > kCommMaxTiles) return -5;
  const long long total = static_cast<long long>(p.tiles_lane) * p.tiles_col * p.splits;
  // Every CTA must be resident at once: peers wait on each other's tiles.
  const int grid = static_cast<int>(total < sms ? total : sms);

  CUtensorMap map_x, map_w;
  const uint32_t x_box = swap ? bn : kLaneRows;
  const uint32_t w_box = swap ? kLaneRows : bn;
  if (!make_tensor_map_bf16(&map_x, x, M, K, ldx, x_box, kBK)) return -4;
  if (quant.wq != 0) {
    const int bits = wq_bits(quant.wq);
    const uint64_t pkb = static_cast<uint64_t>(kBK) * bits / 8;
    const uint32_t brows = static_cast<uint32_t>(wq_block_rows(quant.wq) * pkb / 256);
    const uint64_t trows = static_cast<uint64_t>((N + kLaneRows - 1) / kLaneRows) * p.num_kb * brows;
    if (!make_tensor_map_u8(&map_w, w, trows, 256, 256, brows, 256)) return -4;
#define MX_QCLAUNCH(BN_)                                                                              \
    switch (quant.wq) {                                                                                \
      case 1: return launch_gemm<BN_, true, false, 1, false, 1>(map_w, map_x, p, grid, stream);        \
      case 2: return launch_gemm<BN_, true, false, 1, false, 2>(map_w, map_x, p, grid, stream);        \
      default: return launch_gemm<BN_, true, false, 1, false, 3>(map_w, map_x, p, grid, stream);       \
    }
    switch (bn) {
      case 16: MX_QCLAUNCH(16);
      case 32: MX_QCLAUNCH(32);
      case 64: MX_QCLAUNCH(64);
      default: MX_QCLAUNCH(128);
    }
#undef MX_QCLAUNCH
  }
  if (!make_tensor_map_bf16(&map_w, w, N, K, ldw, w_box, kBK)) return -4;
  const CUtensorMap& ml = swap ? map_w : map_x;
  const CUtensorMap& mc = swap ? map_x : map_w;
  if (mode == 1) {
    switch (bn) {
      case 16: return launch_gemm<16, true, false, 1>(ml, mc, p, grid, stream);
      case 32: return launch_gemm<32, true, false, 1>(ml, mc, p, grid, stream);
      case 64: return launch_gemm<64, true, false, 1>(ml, mc, p, grid, stream);
      default: return launch_gemm<128, true, false, 1>(ml, mc, p, grid, stream);
    }
  } else if (mode == 3) {
    switch (bn) {
      case 16: return launch_gemm<16, true, false, 3>(ml, mc, p, grid, stream);
      case 32: return launch_gemm<32, true, false, 3>(ml, mc, p, grid, stream);
      case 64: return launch_gemm<64, true, false, 3>(ml, mc, p, grid, stream);
      default: return launch_gemm<128, true, false, 3>(ml, mc, p, grid, stream);
    }
  }
  if (bn == 256) return launch_gemm<256, false, false, 2>(ml, mc, p, grid, stream);
  return launch_gemm<128, false, false, 2>(ml, mc, p, grid, stream);
}


// Grouped (per-expert) GEMM: rows [off[e], off[e+1]) of x are multiplied by expert e's weight
// matrix w[e] ([E, N or 2N, K] contiguous) with the same tcgen05 kernel; the tile schedule is
// derived on the device from `expert_offsets` ([E + 1] ints in device memory), so the host never
// needs the routing result. `max_rows` bounds the row count of x / out (allocation size) and
// `avg_rows_hint` (rows per expert the caller expects) picks the operand placement: few rows per
// expert stream the expert weights through the MMA lanes (decode), many rows put tokens on lanes.
extern "C" int mx_grouped_gemm_bf16(const void* x, const void* w, void* out, const void* bias,
                                    const int* expert_offsets, int E, int N, int K, int max_rows,
                                    int epilogue, int glu_offset, float glu_alpha, float glu_limit,
                                    void* workspace, long long ws_bytes, void* stream_,
                                    const MxGemmExtras* extras) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const QuantArgs quant = take_quant(extras);
  if (E <= 0 || N <= 0 || K <= 0 || max_rows <= 0) return 0;
  if ((K % 8) || (N % 8)) return -1;
  if (workspace == nullptr || ws_bytes < MX_WS_PARTIAL_OFFSET) return -2;
  const bool glu = epilogue == MX_EPI_SWIGLU || epilogue == MX_EPI_GEGLU ||
                   epilogue == MX_EPI_CLIPPED_SWIGLU;
  const int w_group_rows = glu ? (glu_offset + N) : N;
  GemmParams p{};
  p.out = out;
  p.bias = (epilogue == MX_EPI_NONE) ? nullptr : static_cast<const __nv_bfloat16*>(bias);
  p.status = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + MX_WS_STATUS_OFFSET);
  p.counters = reinterpret_cast<int*>(static_cast<uint8_t*>(workspace) + MX_WS_COUNTER_OFFSET);
  p.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + MX_WS_PARTIAL_OFFSET);
  p.M = max_rows;
  p.N = N;
  p.K = K;
  p.ldo = N;
  p.glu_offset = glu_offset;
  p.epilogue = epilogue;
  p.glu_alpha = glu_alpha;
  p.glu_limit = glu_limit;
  p.num_kb = (K + kBK - 1) / kBK;
  p.splits = 1;
  p.kb_per_split = p.num_kb;
  p.group_offsets = expert_offsets;
  p.num_groups = E;
  p.w_group_rows = w_group_rows;
  p.bias_group_stride = w_group_rows;
  const int avg = (max_rows + E - 1) / E;
  const bool swap = avg <= 96;
  const int bn = swap ? (avg <= 16 ? 16 : avg <= 32 ? 32 : 64) : (glu ? 128 : (N > 128 ? 256 : 128));
  const int grid = device_sm_count();
  CUtensorMap map_x, map_w;
  const uint32_t x_box = swap ? bn : kLaneRows;
  const uint32_t w_box = swap ? kLaneRows : bn;
  if (!make_tensor_map_bf16(&map_x, x, max_rows, K, K, x_box, kBK)) return -4;
  if (quant.wq != 0) {
    // Expert weights as re-tiled packed blocks (see mx_gemm_set_quant): per expert ceil(N / 128)
    // row tiles, the gate tiles followed by the up tiles when gated. Few rows per expert only
    // (decode); the caller dequantises for the token-rows-on-lanes case.
    if (!swap || (K % kBK) || (quant.wq != 1 && quant.wq != 3)) return -9;
    const int tN = (N + kLaneRows - 1) / kLaneRows;
    p.q_tiles_per_group = glu ? 2 * tN : tN;
    p.q_glu_tiles = glu ? tN : 0;
    const int bits = wq_bits(quant.wq);
    const uint64_t pkb = static_cast<uint64_t>(kBK) * bits / 8;
    const uint32_t brows = static_cast<uint32_t>(wq_block_rows(quant.wq) * pkb / 256);
    const uint64_t trows = static_cast<uint64_t>(E) * p.q_tiles_per_group * p.num_kb * brows;
    if (!make_tensor_map_u8(&map_w, w, trows, 256, 256, brows, 256)) return -4;
#define MX_GQLAUNCH(BN_, GLU_)                                                                        \
    if (quant.wq == 1) return launch_gemm<BN_, true, GLU_, 0, true, 1>(map_w, map_x, p, grid, stream); \
    return launch_gemm<BN_, true, GLU_, 0, true, 3>(map_w, map_x, p, grid, stream)
    if (glu) {
      if (bn == 16) { MX_GQLAUNCH(16, true); }
      if (bn == 32) { MX_GQLAUNCH(32, true); }
      MX_GQLAUNCH(64, true);
    }
    if (bn == 16) { MX_GQLAUNCH(16, false); }
    if (bn == 32) { MX_GQLAUNCH(32, false); }
    MX_GQLAUNCH(64, false);
#undef MX_GQLAUNCH
  }
  if (!make_tensor_map_bf16(&map_w, w, static_cast<uint64_t>(E) * w_group_rows, K, K, w_box, kBK))
    return -4;
  const CUtensorMap& ml = swap ? map_w : map_x;
  const CUtensorMap& mc = swap ? map_x : map_w;
#define MX_GLAUNCH(BN_, SWAP_, GLU_) return launch_gemm<BN_, SWAP_, GLU_, 0, true>(ml, mc, p, grid, stream)
  if (swap) {
    if (glu) {
      if (bn == 16) MX_GLAUNCH(16, true, true);
      if (bn == 32) MX_GLAUNCH(32, true, true);
      MX_GLAUNCH(64, true, true);
    }
    if (bn == 16) MX_GLAUNCH(16, true, false);
    if (bn == 32) MX_GLAUNCH(32, true, false);
    MX_GLAUNCH(64, true, false);
  }
  if (glu) MX_GLAUNCH(128, false, true);
  if (bn == 256) MX_GLAUNCH(256, false, false);
  MX_GLAUNCH(128, false, false);
#undef MX_GLAUNCH
}
