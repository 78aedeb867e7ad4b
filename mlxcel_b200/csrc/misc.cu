// Host-side helpers of the kernel library: device status word access and build information.
#include "api.h"
#include "common.cuh"

extern "C" int mx_read_status(void* workspace, int clear) {
  int v = 0;
  if (workspace == nullptr) return -1;
  if (cudaMemcpy(&v, static_cast<char*>(workspace) + MX_WS_STATUS_OFFSET, sizeof(int),
                 cudaMemcpyDeviceToHost) != cudaSuccess)
    return -2;
  if (clear && v != 0) {
    // A failed kernel may have left tile counters behind: clear status and counters together.
    cudaMemset(workspace, 0, MX_WS_COUNTER_OFFSET + MX_WS_COUNTER_BYTES);
  }
  return v;
}

extern "C" const char* mx_build_info(void) {
  return "mlxcel_b200 kernels: sm_100a, tcgen05+TMA GEMM, built " __DATE__ " " __TIME__;
}

// Bounded-wait self test: one thread waits until *flag >= target or `limit_ns` passes. On time-out
// it records kErrPeerFlagWait in *status and returns normally (the context stays usable). Used to
// check, without faulting or hanging anything, that a lost peer turns into a readable status.
namespace {
__global__ void wait_probe_kernel(const unsigned int* flag, unsigned int target, int* status,
                                  unsigned long long limit_ns, unsigned long long* waited_ns) {
  const unsigned long long t0 = mx::globaltimer_ns();
  for (;;) {
    unsigned int v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flag) : "memory");
    if (static_cast<int>(v - target) >= 0) break;
    if (mx::globaltimer_ns() - t0 > limit_ns) {
      atomicCAS(status, 0, mx::kErrPeerFlagWait);
      break;
    }
  }
  if (waited_ns != nullptr) *waited_ns = mx::globaltimer_ns() - t0;
}
}  // namespace

extern "C" int mx_wait_probe(const void* flag, unsigned int target, void* status, long long limit_ns,
                             void* waited_ns, void* stream) {
  if (flag == nullptr || status == nullptr || limit_ns <= 0 || limit_ns > 2000000000ll) return -1;
  wait_probe_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const unsigned int*>(flag), target, static_cast<int*>(status),
      static_cast<unsigned long long>(limit_ns), static_cast<unsigned long long*>(waited_ns));
  return static_cast<int>(cudaGetLastError());
}
