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
