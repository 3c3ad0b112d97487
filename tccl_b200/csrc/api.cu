// Library-level entry points that are not kernels.
#include <cuda_runtime.h>
#include <string.h>

#include "tccl_b200.h"

extern "C" {

int tccl_version(void) { return 100; }

int tccl_debug_checks(void) {
#ifdef TCCL_DEBUG_CHECKS
  return 1;
#else
  return 0;
#endif
}

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

// sizeof of the ABI structs, by name: lets a binding check its own mirror of them
int tccl_sizeof(const char* name) {
#define TCCL_SZ(T) if (!strcmp(name, #T)) return (int)sizeof(T);
  TCCL_SZ(tccl_comm) TCCL_SZ(tccl_coll_args) TCCL_SZ(tccl_launch) TCCL_SZ(tccl_barrier_args) TCCL_SZ(tccl_pads_args)
  TCCL_SZ(tccl_tree_args) TCCL_SZ(tccl_arn_args) TCCL_SZ(tccl_gemm_args) TCCL_SZ(tccl_gemm_rs_args)
  TCCL_SZ(tccl_ag_gemm_args)
#undef TCCL_SZ
  return -1;
}

int tccl_num_sms(void) {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return 0;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
  return n;
}

}  // extern "C"
