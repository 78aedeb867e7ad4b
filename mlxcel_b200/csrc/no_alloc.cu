// Allocation-free variant of the small-M split-K GEMM (declared in no_alloc.h). The scratch
// (status word, tile counters, fp32 partial tiles) is a file-scope device array. In host code
// the array's name is only a host-side stand-in for the symbol, so its device address is
// resolved once per device with cudaGetSymbolAddress and that pointer is what the kernel gets.
#include <mutex>

#include <cuda_runtime.h>

#include "api.h"
#include "no_alloc.h"

static __device__ __align__(256) unsigned char g_static_scratch[MX_STATIC_SCRATCH_BYTES];

namespace {
struct StaticScratchState {
  void* ptr[64] = {nullptr};
  bool ready[64] = {false};
  std::mutex mu;
};
StaticScratchState& static_scratch_state() {
  static StaticScratchState s;
  return s;
}
}  // namespace

extern "C" const char* mx_gemm_bf16_static_error(int code) {
  switch (code) {
    case 0: return "ok";
    case MX_STATIC_ERR_TOO_LARGE:
      return "mx_gemm_bf16_static: problem exceeds the static scratch limits (M <= 256, N <= 262144, K <= 65536)";
    case MX_STATIC_ERR_SYMBOL:
      return "mx_gemm_bf16_static: could not resolve the device address of the static scratch array";
    case MX_STATIC_ERR_ARGUMENT:
      return "mx_gemm_bf16_static: null pointer, misaligned operand or non-positive size";
    default:
      return code > 0 ? "mx_gemm_bf16_static: CUDA error from the launch (cudaError_t)"
                      : "mx_gemm_bf16_static: argument rejected by the GEMM dispatcher";
  }
}

extern "C" int mx_gemm_bf16_static(const void* x, const void* w, void* out, const void* bias,
                                   const void* residual, int M, int N, int K, int ldx, int ldw,
                                   int ldo, int ldr, int epilogue, int out_fp32, int glu_offset,
                                   float glu_alpha, float glu_limit, void* stream_) {
  if (x == nullptr || w == nullptr || out == nullptr || M <= 0 || N <= 0 || K <= 0)
    return MX_STATIC_ERR_ARGUMENT;
  if (M > MX_STATIC_MAX_M || N > MX_STATIC_MAX_N || K > MX_STATIC_MAX_K)
    return MX_STATIC_ERR_TOO_LARGE;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MX_STATIC_ERR_SYMBOL;
  StaticScratchState& st = static_scratch_state();
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> g(st.mu);
    if (!st.ready[dev]) {
      // Set-up, once per device, with that device current: host code must not pass
      // g_static_scratch itself to a kernel, only the address looked up here.
      void* p = nullptr;
      if (cudaGetSymbolAddress(&p, g_static_scratch) != cudaSuccess || p == nullptr)
        return MX_STATIC_ERR_SYMBOL;
      if (cudaMemset(p, 0, MX_WS_PARTIAL_OFFSET) != cudaSuccess) return MX_STATIC_ERR_SYMBOL;
      st.ptr[dev] = p;
      st.ready[dev] = true;
    }
    scratch = st.ptr[dev];
  }
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  // The array still holds the previous call's words: the tile arrival counters have to start at
  // zero, the partial tiles are fully rewritten before they are read. The status word is left
  // alone: a bounded wait that ran out in an earlier call stays visible until
  // mx_gemm_bf16_static_status reads (and clears) it.
  cudaError_t e = cudaMemsetAsync(static_cast<unsigned char*>(scratch) + MX_WS_COUNTER_OFFSET, 0,
                                  MX_WS_COUNTER_BYTES, stream);
  if (e != cudaSuccess) return static_cast<int>(e);
  // force_mode 2: the weight-rows-on-lanes split-K kernel, the one that needs scratch.
  return mx_gemm_bf16(x, w, out, bias, residual, M, N, K, ldx, ldw, ldo, ldr, epilogue, out_fp32,
                      glu_offset, glu_alpha, glu_limit, scratch, MX_STATIC_SCRATCH_BYTES, 2, 0,
                      stream_, nullptr);
}

extern "C" int mx_gemm_bf16_static_status(int clear) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return MX_STATIC_ERR_SYMBOL;
  StaticScratchState& st = static_scratch_state();
  void* scratch = nullptr;
  {
    std::lock_guard<std::mutex> g(st.mu);
    if (!st.ready[dev]) return 0;   // nothing was ever launched through the static entry point here
    scratch = st.ptr[dev];
  }
  // The status word is the first int of the scratch array. A plain synchronous copy: it waits for
  // the work queued so far on the device, reads four bytes into host memory and allocates nothing.
  int code = 0;
  if (cudaMemcpy(&code, static_cast<unsigned char*>(scratch) + MX_WS_STATUS_OFFSET, sizeof(int),
                 cudaMemcpyDeviceToHost) != cudaSuccess)
    return MX_STATIC_ERR_SYMBOL;
  if (clear && code != 0) {
    const int zero = 0;
    if (cudaMemcpy(static_cast<unsigned char*>(scratch) + MX_WS_STATUS_OFFSET, &zero, sizeof(int),
                   cudaMemcpyHostToDevice) != cudaSuccess)
      return MX_STATIC_ERR_SYMBOL;
  }
  return code;
}
