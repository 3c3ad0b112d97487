// Host-side helper: build a TMA descriptor for a K-major bf16 matrix
// [rows, k] (k contiguous, `ld` elements between rows) with a box of
// 64 (k) x box_rows and the 128-byte swizzle the UMMA descriptors expect.
// cuTensorMapEncodeTiled is resolved through the runtime so that the library
// does not link against libcuda.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tccl_b200.h"

namespace tccl {
namespace gemm {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

inline int make_tmap_bf16_kmajor(CUtensorMap* map, const void* base, int rows, int k, int ld, int box_rows) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (!fn) return -TCCL_EINVAL;
  cuuint64_t dims[2] = {(cuuint64_t)k, (cuuint64_t)rows};
  cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
  cuuint32_t box[2] = {64u, (cuuint32_t)box_rows};
  cuuint32_t estr[2] = {1u, 1u};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -TCCL_EINVAL;
}

// Emulated ranks of a kernel built on CTA pairs (compile-time cluster dimensions 2 x 1 x 1): one
// launch of `grid` x `world` CTAs.  The ranks' CTAs wait on one another, so all of them must be
// resident together: a cooperative launch guarantees that or fails cleanly; where the runtime does
// not take a cooperative launch of a cluster kernel, the launch goes ahead only if the occupancy
// query says that every cluster fits at once.
inline int launch_pairs_emulated(const void* fn, int grid, int world, size_t smem, cudaStream_t s, const void* arg0,
                                 const void* arg1) {
  void* kargs[2] = {const_cast<void*>(arg0), const_cast<void*>(arg1)};
  cudaError_t e = cudaLaunchCooperativeKernel(fn, dim3(grid, world), dim3(256), kargs, smem, s);
  if (e == cudaSuccess) return 0;
  if (e != cudaErrorInvalidValue && e != cudaErrorNotSupported && e != cudaErrorInvalidConfiguration &&
      e != cudaErrorLaunchFailure)
    return (int)e;
  if (e == cudaErrorLaunchFailure) return (int)e;
  (void)cudaGetLastError();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, world);
  cfg.blockDim = dim3(256);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = s;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int clusters = 0;
  e = cudaOccupancyMaxActiveClusters(&clusters, fn, &cfg);
  if (e != cudaSuccess) return (int)e;
  if (clusters * 2 < grid * world) return (int)cudaErrorCooperativeLaunchTooLarge;
  return (int)cudaLaunchKernelExC(&cfg, fn, kargs);
}

}  // namespace gemm
}  // namespace tccl
