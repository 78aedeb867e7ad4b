// Allocation-free entry point of the kernel library.
//
// This entry point has no counterpart in the reference implementation: it exists for callers
// that are not able to allocate device memory themselves — for example a host that embeds the
// library behind a fixed memory plan and is handed only its input and output buffers, a
// plugin that runs inside another runtime's allocator-locked section, or a real-time loop in
// which an allocation (and the device synchronisation it may imply) is off limits.
//
// mx_gemm_bf16_static computes out[M, N] = epilogue(x[M, K] @ w[N, K]^T) exactly like
// mx_gemm_bf16 for small token counts (the weight-streaming split-K path), but instead of a
// caller-provided workspace it uses a fixed scratch array that lives inside the library image:
// MX_STATIC_SCRATCH_BYTES of device memory on every GPU that loads the library, held until
// the process exits. The caller passes only inputs and outputs.
//
// Rules of use:
//  * Limits: M <= MX_STATIC_MAX_M, N <= MX_STATIC_MAX_N, K <= MX_STATIC_MAX_K. Anything
//    larger is refused with MX_STATIC_ERR_TOO_LARGE and nothing is launched.
//  * The first call on each device looks up the device address of the scratch array
//    (cudaGetSymbolAddress, with that device current) and clears its control words. That first
//    call synchronises with the device, so make it before any stream capture begins.
//  * Every call shares the one scratch array and the array keeps what the previous call left
//    in it. Each call re-clears, on the caller's stream, the words that have to start at zero
//    (the tile counters; the status word is kept until mx_gemm_bf16_static_status clears it).
//    Two calls whose kernels overlap on the GPU (different streams, no ordering between them)
//    race on the scratch: order them on one stream or with events.
//  * The function calls no cudaMalloc / cudaFree and no allocating library routine.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

#define MX_STATIC_SCRATCH_BYTES (131072 + (8 << 20))
#define MX_STATIC_MAX_M 256
#define MX_STATIC_MAX_N 262144
#define MX_STATIC_MAX_K 65536

#define MX_STATIC_ERR_TOO_LARGE (-70)   // a dimension exceeds the limits above
#define MX_STATIC_ERR_SYMBOL (-71)      // the scratch array's device address could not be resolved
#define MX_STATIC_ERR_ARGUMENT (-72)    // null pointer, misaligned operand or non-positive size

// epilogue: MX_EPI_* of api.h. For gated epilogues `w` holds gate rows [0, N) and up rows
// [glu_offset, glu_offset + N). Returns 0, one of the MX_STATIC_ERR_* codes, a negative
// mx_gemm_bf16 argument code, or a positive cudaError_t.
int mx_gemm_bf16_static(const void* x, const void* w, void* out, const void* bias,
                        const void* residual, int M, int N, int K, int ldx, int ldw, int ldo,
                        int ldr, int epilogue, int out_fp32, int glu_offset, float glu_alpha,
                        float glu_limit, void* stream);

// The kernel's waits are bounded: a wait that runs out records a code (1xx pipeline, 2xx flag) in
// the status word at the start of the scratch array and the kernel returns normally, so the launch
// itself reports success. This call reads that word for the current device (0 = every launch so
// far completed normally) and, with clear != 0, resets it. It synchronises with the device (a
// four-byte copy to the host), allocates nothing, and must not be made during stream capture.
// While the word is non-zero, later launches give up their waits at once: read and clear it
// before retrying.
int mx_gemm_bf16_static_status(int clear);

// Human-readable text for a return code of mx_gemm_bf16_static.
const char* mx_gemm_bf16_static_error(int code);

#ifdef __cplusplus
}
#endif
