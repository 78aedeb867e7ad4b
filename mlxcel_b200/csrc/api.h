// C ABI of libmlxcel_b200.so. Every function takes raw device pointers and a CUDA stream
// (as void*), launches asynchronously on that stream and returns 0 on success, a negative
// value for a rejected argument, or a positive cudaError_t from the launch.
//
// Workspace convention: kernels that need scratch memory (split-K partial sums, tile
// counters, the device status word) receive one caller-owned buffer `workspace` of
// `ws_bytes` bytes laid out as
//   [0, 256)            device status word (int) + padding; 0 = no error
//   [256, 256 + 64 KiB) tile arrival counters (int), must be zero before the first use and
//                       are returned to zero by every kernel that completes
//   [128 KiB, ws_bytes) fp32 partial tiles
// The buffer must be zero-initialised once by the caller.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define MX_WS_STATUS_OFFSET 0
#define MX_WS_COUNTER_OFFSET 256
#define MX_WS_COUNTER_BYTES 65536
#define MX_WS_PARTIAL_OFFSET 131072
/* Phase timestamps of the last GEMM launch (MLXCEL_B200_GEMM_TRACE=1): 16 x uint64 (globaltimer ns)
 * per CTA: entry, set-up done, first loads issued, first tile landed, last MMA committed,
 * accumulator ready, results stored, exit; [8] vector epilogue begins, [9] its stores / peer pushes issued,
 * [10] all peers' partials arrived (fused all-reduce). No counterpart in the reference. */
#define MX_WS_TRACE_OFFSET 98304
#define MX_WS_TRACE_MAX_CTAS 256

// Epilogues of mx_gemm_bf16.
#define MX_EPI_NONE 0
#define MX_EPI_BIAS 1            // out = acc + bias[n]
#define MX_EPI_RESIDUAL 2        // out = acc + residual[m, n] (+ bias[n] when bias != NULL)
#define MX_EPI_SWIGLU 3          // out = silu(acc_gate) * acc_up
#define MX_EPI_GEGLU 4           // out = gelu_tanh(acc_gate) * acc_up
#define MX_EPI_CLIPPED_SWIGLU 5  // gpt-oss: (min(g,l)) * sigmoid(a*g) * (clamp(u,-l,l) + 1)

// Optional per-call extras of the GEMM entry points (pass NULL for a plain dense GEMM). Everything a
// call needs travels in its own arguments: there is no per-thread or per-process pending state, so
// several host threads (e.g. the engines of a multi-model router) can launch GEMMs concurrently.
typedef struct MxGemmExtras {
  // Quantized weights: `w` = packed weights re-tiled for the kernel (see gemm.cu), ldw ignored.
  // wq: 0 dense bf16, 1 affine 4-bit, 2 affine 8-bit, 3 mxfp4; q_group: elements per scale group.
  // The call returns -9 when M > 256 (use dequantise + GEMM).
  int wq;
  int q_group;
  // Deferred RMSNorm: scale output rows by the 1/rms that `ssq_in` describes (consumer) and / or
  // leave per-tile sums of squares of the result in `ssq_out` (producer). Either may be NULL.
  const void* ssq_in;
  void* ssq_out;
  float ssq_eps;
  float ssq_inv_dim;
  // mx_gemm_comm only: multicast (NVLS) addresses of the channel's flags, its receive area and the
  // replicated output. flags_mc == NULL selects the peer-store protocol.
  void* flags_mc;
  void* recv_mc;
  void* out_mc;
} MxGemmExtras;

// out[M, N] = epilogue(x[M, K] @ w[N(+N), K]^T). bf16 operands, fp32 accumulation on the
// 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM, operand tiles brought by TMA).
// For the gated epilogues `w` holds gate rows at [0, N) and up rows at [glu_offset, glu_offset + N).
// K, ldx, ldw must be multiples of 8. force_mode: 0 auto, 1 token-rows-on-lanes, 2 weight-rows-on-lanes.
int mx_gemm_bf16(const void* x, const void* w, void* out, const void* bias, const void* residual,
                 int M, int N, int K, int ldx, int ldw, int ldo, int ldr, int epilogue,
                 int out_fp32, int glu_offset, float glu_alpha, float glu_limit, void* workspace,
                 long long ws_bytes, int force_mode, int force_splits, void* stream,
                 const MxGemmExtras* extras);

/* Sum of squares of every row of x [rows, dim] (bf16) as a one-partial ssq buffer (see MxGemmExtras). */
int mx_row_ssq(const void* x, int rows, int dim, long long ldx, void* ssq, void* stream);

// Fused GEMM + collective over a symmetric heap of peer-mapped memory (tensor parallelism).
// mode 1: one-shot all-reduce (M <= 256): out = residual + bias + sum over ranks of x_r @ w_r^T.
// mode 2: two-shot all-reduce (any M): tile owners reduce and store into every out_peer.
// mode 3: all-gather of output columns (M <= 256): out_peer[r][t, rank * N + n].
// flags_peer / recv_peer / out_peer: host arrays of `world` device addresses of the same heap
// offset on each rank; ctl (16 words) / expect (8200 words): this rank's channel words (zeroed).
// With extras->flags_mc set the cross-rank traffic goes through NVSwitch multicast (multimem
// ld_reduce / st / red) instead of per-peer stores; results are then equal across ranks up to the
// switch's fp32 summation order instead of bitwise equal.
int mx_gemm_comm(const void* x, const void* w, void* out, const void* bias, const void* residual,
                 int M, int N, int K, int ldx, int ldw, int ldo, int ldr, int mode, int rank,
                 int world, const void* const* flags_peer, const void* const* recv_peer,
                 const void* const* out_peer, void* ctl, void* expect, long long parity_stride,
                 long long rank_stride, void* workspace, long long ws_bytes, void* stream,
                 const MxGemmExtras* extras);

// Stand-alone all-reduce over the symmetric heap (same channel protocol as mx_gemm_comm):
// out = residual + sum over ranks of x, n bf16 elements. mode 1 one-shot (local out), mode 2
// two-shot (results stored into every out_peer). status: device status word (int).
// flags_mc / recv_mc / out_mc: NVLS multicast addresses of the channel (NULL = peer stores).
int mx_allreduce_comm(const void* x, const void* residual, void* out, long long n, int mode, int rank,
                      int world, const void* const* flags_peer, const void* const* recv_peer,
                      const void* const* out_peer, void* ctl, void* expect, long long parity_stride,
                      long long rank_stride, void* status, void* stream, void* flags_mc, void* recv_mc,
                      void* out_mc);

// Quantized GEMV -> all-reduce in one kernel (M <= 8 tokens; bits 4 / 8; mode 0 affine, 1 mxfp4,
// 2 mxfp8): out = residual + bias + sum over ranks of x_r @ dequant(w_r)^T. Channel arguments as in
// mx_allreduce_comm. Returns -9 for shapes it does not cover.
int mx_qmv_allreduce(const void* x, const void* w, const void* scales, const void* biases, void* out,
                     const void* residual, const void* lin_bias, int M, int N, int K, int bits, int group,
                     int mode, int ldx, int ldo, int ldr, int rank, int world,
                     const void* const* flags_peer, const void* const* recv_peer, void* ctl, void* expect,
                     long long parity_stride, long long rank_stride, void* status, void* flags_mc,
                     void* recv_mc, void* stream);

// Bytes of workspace the no-scratch-allocation path needs at most for mx_gemm_bf16.
long long mx_gemm_workspace_bytes(void);

// h = x + residual (when residual != NULL; written to residual_out), y = rmsnorm(h) * (w + w_bias).
// rows x dim bf16; one row per CTA group. eps as given; w_bias = 1.0 for Gemma-style norms.
int mx_add_rmsnorm(const void* x, const void* residual, const void* weight, void* y,
                   void* residual_out, int rows, int dim, float eps, float w_bias, void* stream);

// Per-head RMSNorm over the last dimension of [tokens, heads, head_dim] (Qwen3 q/k norm), in place.
int mx_head_rmsnorm(void* x, const void* weight, int tokens, int heads, int head_dim,
                    long long token_stride, float eps, void* stream);

// RoPE on q and k (in place on q; k written roped into the paged pool) + KV append.
// qkv: [T, (Hq + 2 Hkv) * D] bf16. positions: [T] int32. slot_mapping: [T] int64/int32 slot
// index (= block_id * block_size + offset); negative slots are skipped.
// inv_freq: [D/2] fp32 (already scaled for llama3 / yarn), mscale multiplies q and k after
// rotation. rope_mode: 0 = half-split (non-traditional), 1 = interleaved (traditional).
// k_pool / v_pool layout: [num_blocks, Hkv, block_size, D] (bf16, kv_bits = 16) or int8 with
// per (token, head, group of 64) scale+bias sidecars (kv_bits = 8) of layout
// [num_blocks, Hkv, block_size, D/64, 2] bf16.
// q_norm_w / k_norm_w: optional per-head RMSNorm weights [D] applied before RoPE (Qwen3).
// 0 selects the 2/4-byte-access form of the register-resident rope + append kernel.
void mx_set_rope_vec(int on);
int mx_rope_append(void* qkv, const int* positions, const int* slot_mapping, const float* inv_freq,
                   void* k_pool, void* v_pool, void* k_meta, void* v_meta, const void* q_norm_w,
                   const void* k_norm_w, float norm_eps, int T, int Hq, int Hkv, int D,
                   int rot_dim, int block_size, int rope_mode, float mscale, int kv_bits,
                   void* stream);

// Paged decode attention (one query token per sequence), split-KV with an in-kernel merge.
// q: rows of [Hq * D] bf16 with stride q_stride elements; out: [B, Hq * D] bf16.
// block_tables: [B, max_blocks] int32; context_lens: [B] int32 (tokens visible, including the
// one just appended). window > 0 limits attention to the last `window` tokens; sinks: optional
// [Hq] fp32 logits added to the softmax denominator. scratch: fp32 buffer of
// mx_paged_decode_scratch_floats(B, Hq, D, max_splits) floats.
int mx_paged_decode(const void* q, long long q_stride, const void* k_pool, const void* v_pool,
                    const void* k_meta, const void* v_meta, const int* block_tables,
                    const int* context_lens, const float* sinks, void* out, float* scratch,
                    int B, int Hq, int Hkv, int D, int block_size, int max_blocks, int window,
                    float scale, float softcap, int kv_bits, int num_splits, void* stream);
long long mx_paged_decode_scratch_floats(int B, int Hq, int D, int num_splits);

// Chunked causal prefill attention over the paged KV pool. Sequence s owns query rows
// [cu_q[s], cu_q[s+1]) of q (row stride q_stride) which are the LAST q_len tokens of its
// context_lens[s] visible tokens. K/V are read from the pool (they were appended first).
int mx_paged_prefill(const void* q, long long q_stride, const void* k_pool, const void* v_pool,
                     const void* k_meta, const void* v_meta, const int* block_tables,
                     const int* cu_q, const int* context_lens, const float* sinks, void* out,
                     int num_seqs, int total_q, int max_q_len, int Hq, int Hkv, int D,
                     int block_size, int max_blocks, int window, float scale, float softcap,
                     int kv_bits, void* stream);

// Same contract on the tcgen05 / TMEM / TMA path: bf16 pool with 16-token blocks, D = 64 or 128,
// no soft cap. Returns -10 when the configuration is not covered (use mx_paged_prefill then).
// pool_blocks: blocks in k_pool / v_pool; status: the device status word (bounded waits report
// there). No counterpart in the reference, whose prefill attention is cuDNN SDPA.
int mx_paged_prefill_tc(const void* q, long long q_stride, const void* k_pool, const void* v_pool,
                        long long pool_blocks, const int* block_tables, const int* cu_q,
                        const int* context_lens, const float* sinks, void* out, int num_seqs,
                        int total_q, int max_q_len, int Hq, int Hkv, int D, int block_size,
                        int max_blocks, int window, float scale, void* status, void* stream);

// Embedding gather: out[t, :] = table[ids[t], :] (bf16), ids outside [0, vocab) give zeros.
int mx_embedding(const int* ids, const void* table, void* out, int T, int dim, int vocab,
                 float scale, void* stream);

// Greedy argmax over [B, V] logits (bf16 or fp32) -> int32 tokens (ties: lowest index).
int mx_argmax(const void* logits, int logits_fp32, long long row_stride, int* out, int B, int V,
              void* stream);

// Fused sampler over [B, V] logits. Per-row parameters: temperature (0 = greedy), top_k
// (0 = off), top_p (1 = off), min_p (0 = off), top_n_sigma (0 = off; optional array), typical_p
// (1 = off; optional array). Chain: top-k -> top-p -> min-p -> top-n-sigma on the untempered
// softmax, then typical-p on what survived; the draw uses Gumbel-max noise from a
// Philox-4x32-10 stream keyed by (seed[row], step[row]). out_logprob: optional [B].
int mx_sample(const void* logits, int logits_fp32, long long row_stride, const float* temperature,
              const int* top_k, const float* top_p, const float* min_p, const float* typical_p,
              const float* top_n_sigma, const unsigned long long* seeds,
              const unsigned long long* steps, int* out_tokens, float* out_logprob, int B, int V,
              void* stream);
long long mx_sample_scratch_floats(int B, int V);

// Repetition / frequency / presence penalties applied in place to fp32 or bf16 logits, given
// per-row token histories [B, max_hist] (int32, -1 padded).
int mx_apply_penalties(void* logits, int logits_fp32, long long row_stride, const int* history,
                       int max_hist, const float* rep, const float* freq, const float* pres, int B,
                       int V, void* stream);

// Speculative verify: target argmax over [B, K, V] logits vs draft tokens [B, K-1];
// accept_len[b] = first mismatch index, next_token[b] = target token at that index,
// target_tokens: [B, K].
int mx_spec_verify(const void* logits, int logits_fp32, long long row_stride, const int* draft,
                   int* target_tokens, int* accept_len, int* next_token, int B, int K, int V,
                   void* stream);

// Affine group-quantized (MLX layout) matmul: out[M, N] = x[M, K] @ dequant(w)[N, K]^T.
// w: uint32 [N, K * bits / 32], scales/biases bf16 [N, K / group]. bits in {4, 8}.
// M <= 16 uses the GEMV kernel (weights read once for all rows); larger M dequantizes tiles
// into shared memory and runs tcgen05 MMAs.
int mx_qmm_affine(const void* x, const void* w, const void* scales, const void* biases,
                  void* out, const void* residual, int M, int N, int K, int bits, int group,
                  int ldx, int ldo, void* workspace, long long ws_bytes, void* stream);

// Dequantize affine / mxfp4 / mxfp8 weights to bf16 (load-time and test helper).
// mode: 0 affine, 1 mxfp4 (e2m1 + e8m0 per 32), 2 mxfp8 (e4m3 + e8m0 per 32).
int mx_dequantize(const void* w, const void* scales, const void* biases, void* out, long long N,
                  int K, int bits, int group, int mode, void* stream);

// SiLU(gate) * up on a fused [T, 2I] tensor -> [T, I] (used by unfused fallbacks and MoE).
int mx_swiglu(const void* gate_up, void* out, int T, int I, int mode, float alpha, float limit,
              void* stream);

// MoE router: logits [T, E] (bf16) -> top-k expert ids [T, k] int32 and weights [T, k] fp32.
// mode 0: softmax over all experts then top-k (renormalised when norm_topk != 0);
// mode 1: top-k on logits then softmax over the k logits (gpt-oss / mixtral).
int mx_moe_route(const void* logits, int* topk_ids, float* topk_w, int T, int E, int k, int mode,
                 int norm_topk, void* stream);

// MoE token permutation helpers: count tokens per expert, exclusive scan, scatter rows.
// 0 selects the scan-per-expert form of the alignment kernel (always used above 256 local experts).
void mx_set_moe_align_fast(int on);
int mx_moe_align(const int* topk_ids, int* expert_offsets, int* sorted_row, int* sorted_token,
                 int T, int k, int E, int e_begin, int e_end, void* stream);
// The same with the pair count read on the device (*n_pairs_dev <= max_tokens * k) and, when
// token_map is given, sorted_token[r] = token_map[token] (tokens are a compacted list of rows).
int mx_moe_align_n(const int* topk_ids, const int* n_pairs_dev, const int* token_map, int* expert_offsets,
                   int* sorted_row, int* sorted_token, int max_tokens, int k, int e_begin, int e_end,
                   void* stream);
// out[sorted_token[r]] = y[r] for r < *total_rows (inverse of the gather for one pair per token).
int mx_moe_scatter_rows_n(const void* y, const int* sorted_token, const int* total_rows, void* out,
                          int max_rows, int dim, void* stream);
// Rows are bounded by `max_rows` on the host; the true row count is read on the device from
// total_rows (= expert_offsets[E_local]) so the MoE block needs no host synchronisation.
int mx_moe_gather_rows_n(const void* x, const int* sorted_token, const int* total_rows, void* out,
                         int max_rows, int dim, void* stream);
// out[t] = (residual[t] | out[t] when accumulate) + sum_slots w[t, slot] * y[row(t, slot)];
// inv_row: [T * k] int scratch.
int mx_moe_combine_n(const void* y, const int* sorted_pair, const int* total_rows, int* inv_row,
                     const float* topk_w, void* out, const void* residual, int T, int k, int dim,
                     int max_rows, int accumulate, void* stream);

// Grouped GEMM over experts: for expert e rows [off[e], off[e+1]) of x use w[e] ([E, N, K]).
int mx_grouped_gemm_bf16(const void* x, const void* w, void* out, const void* bias,
                         const int* expert_offsets, int E, int N, int K, int max_rows,
                         int epilogue, int glu_offset, float glu_alpha, float glu_limit,
                         void* workspace, long long ws_bytes, void* stream, const MxGemmExtras* extras);

// Reads and clears the device status word of a workspace (host-synchronous).
int mx_read_status(void* workspace, int clear);

// Library / build information.
const char* mx_build_info(void);


// Grouped 4-bit GEMV over MLX-packed expert weights for decode-sized groups (few rows per expert).
// -9 = shape not covered (the caller falls back to the grouped GEMM).
int mx_moe_qgemv(const void* xs, const void* w, const void* scales, const void* biases, const void* lin_bias,
                 const int* offsets, void* out, int E, int n_out, int K, int group, int mode, int epi,
                 float alpha, float limit, const void* residual, long long ldo, long long ldr, void* stream);
#ifdef __cplusplus
}
#endif
