// Stand-alone bf16 GEMM on the tcgen05 mainloop (C = A * Bt^T), plus the
// host-side TMA descriptor helper shared with the fused kernels.  Used to
// validate and time the mainloop by itself; plain library-GEMM work would go to
// cuBLAS, the point of this kernel is to be the body the collectives fuse into.
// The reference has no GEMM (presentation.pdf, slide 4, names the fusion with one as a goal).
#include "gemm_host.cuh"
#include "gemm_tcgen05.cuh"

namespace tccl {
namespace gemm {

struct PlainPolicy {
  const CUtensorMap* map_a;
  __nv_bfloat16* C;
  int M, N, ldc;
  int tiles_n, total;
  __device__ __forceinline__ bool tile(int i, int& mt, int& nt) const {
    const int t = blockIdx.x + i * gridDim.x;
    if (t >= total) return false;
    mt = t / tiles_n;
    nt = t - mt * tiles_n;
    return true;
  }
  __device__ __forceinline__ void epilogue_finish(int, int, const Abort&) const {}
  __device__ __forceinline__ bool before_load(int, int, const Abort&) const { return true; }
  __device__ __forceinline__ void a_tile(int mt, const CUtensorMap*& map, int& y) const {
    map = map_a;
    y = mt * BM;
  }
  __device__ __forceinline__ bool epilogue(int mt, int nt, uint32_t taddr, int quad, int lane, const Abort&, const SmemLayout&) const {
    const int row = mt * BM + quad * 32 + lane;
    __nv_bfloat16* crow = C + (size_t)row * ldc;
#pragma unroll 1
    for (int c = 0; c < BN / 32; ++c) {
      uint32_t r[32];
      tmem_ld_32x32(taddr + c * 32, r);
      tmem_ld_wait();
      const int col0 = nt * BN + c * 32;
      if (row < M) {
#pragma unroll
        for (int v = 0; v < 4; ++v)
          if (col0 + v * 8 < N) st_local(crow + col0 + v * 8, pack8_bf16(r + v * 8));
      }
    }
    return true;
  }
};

__global__ void __launch_bounds__(kThreads, 1)
gemm_plain_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b,
                  const Shape shp, PlainPolicy pol, uint32_t* status) {
  // a private tccl_comm-free run: status words are optional
  tccl_comm fake;
  fake.local = status ? status - TCCL_LOCAL_STATUS : nullptr;
  pol.map_a = &map_a;
  run_mainloop(&map_b, shp, pol, status ? &fake : nullptr, 2000000000ull);
}

}  // namespace gemm
}  // namespace tccl

using namespace tccl::gemm;

extern "C" int tccl_gemm_bf16(const tccl_gemm_args* g, int grid, void* stream) {
  if (!g || g->m <= 0 || g->n <= 0 || g->k <= 0) return -TCCL_EINVAL;
  if ((g->lda % 8) || (g->ldb % 8) || (g->ldc % 8) || (g->n % 8) || (g->k % 8)) return -TCCL_EALIGN;
  if (((uintptr_t)g->a | (uintptr_t)g->bt | (uintptr_t)g->c) & 15) return -TCCL_EALIGN;
  CUtensorMap ma, mb;
  int rc = make_tmap_bf16_kmajor(&ma, g->a, g->m, g->k, g->lda, BM);
  if (rc) return rc;
  rc = make_tmap_bf16_kmajor(&mb, g->bt, g->n, g->k, g->ldb, BN);
  if (rc) return rc;
  PlainPolicy pol;
  pol.map_a = nullptr;
  pol.C = reinterpret_cast<__nv_bfloat16*>(g->c);
  pol.M = g->m;
  pol.N = g->n;
  pol.ldc = g->ldc;
  pol.tiles_n = (g->n + BN - 1) / BN;
  pol.total = ((g->m + BM - 1) / BM) * pol.tiles_n;
  if (grid <= 0) grid = tccl_num_sms();
  if (grid > pol.total) grid = pol.total;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_plain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  Shape shp{g->m, g->n, g->k};
  gemm_plain_kernel<<<grid, kThreads, kSmemBytes, reinterpret_cast<cudaStream_t>(stream)>>>(
      ma, mb, shp, pol, reinterpret_cast<uint32_t*>(g->status));
  return (int)cudaGetLastError();
}
