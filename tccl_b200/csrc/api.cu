// Library-level entry points that are not kernels.
#include <cuda_runtime.h>

#include "tccl_b200.h"

extern "C" {

int tccl_version(void) { return 100; }

const char* tccl_error_string(int code) {
  if (code >= 0) return cudaGetErrorString((cudaError_t)code);
  switch (-code) {
    case TCCL_EINVAL: return "tccl: invalid launch argument";
    case TCCL_EDTYPE: return "tccl: unsupported dtype";
    case TCCL_EALIGN: return "tccl: pointer or size not aligned as required";
    case TCCL_ESIZE: return "tccl: size outside the supported range";
    default: return "tccl: unknown error";
  }
}

int tccl_num_sms(void) {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return n;
}

}  // extern "C"
