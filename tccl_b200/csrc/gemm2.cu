// Stand-alone bf16 GEMM on the CTA-pair mainloop (gemm_tcgen05_2cta.cuh):
// C = A * Bt^T with 256 x 256 tiles per pair of SMs, persistent over the tiles.
// The reference has no GEMM (presentation.pdf, slide 4, names the fusion with one as a goal).
#include "gemm_host.cuh"
#include "gemm_tcgen05_2cta.cuh"

namespace tccl {
namespace gemm2 {

// Tile order of a persistent grid of `pairs` CTA pairs over `total` 256 x 256 tiles: the
// whole waves first (tile = pair + i * pairs), then the tiles of the last, partial wave cut
// into left and right halves, so that the tail costs every pair at most half a tile more
// than the pairs that are done.
struct TailSplitSchedule {
  int total, pairs, nfull, rem;
  __host__ __device__ void init(int total_, int pairs_) {
    total = total_;
    pairs = pairs_;
    nfull = (total / pairs) * pairs;
    rem = total - nfull;
  }
  __device__ __forceinline__ bool unit(int pair, int i, int& tile, int& half) const {
    const int u = pair + i * pairs;
    if (u < nfull) {
      tile = u;
      half = 0;
      return true;
    }
    const int h = u - nfull;
    if (h >= 2 * rem) return false;
    tile = nfull + (h >> 1);
    half = 1 + (h & 1);
    return true;
  }
};

// epilogue shared by the plain kernel: tensor memory -> registers -> bf16 rows of C
__device__ __forceinline__ void store_rows(__nv_bfloat16* crow, bool row_ok, int N, int col_base, int ncols, uint32_t taddr) {
#pragma unroll 1
  for (int c = 0; c < ncols / 32; ++c) {
    uint32_t r[32];
    tmem_ld_32x32(taddr + c * 32, r);
    tmem_ld_wait();
    const int col = col_base + c * 32;
    if (row_ok) {
#pragma unroll
      for (int v = 0; v < 4; ++v)
        if (col + v * 8 < N) st_local(crow + col + v * 8, pack8_bf16(r + v * 8));
    }
  }
}

struct PlainPolicy2 {
  const CUtensorMap *map_a, *map_b128, *map_b64;
  __nv_bfloat16* C;
  int M, N, ldc;
  int tiles_n;
  TailSplitSchedule sched;
  __device__ __forceinline__ bool tile(int i, int& mt, int& nt, int& half) const {
    int t;
    if (!sched.unit(blockIdx.x >> 1, i, t, half)) return false;
    const int mt2 = t / tiles_n;
    nt = t - mt2 * tiles_n;
    mt = 2 * mt2;
    return true;
  }
  __device__ __forceinline__ void b_tile(int nt, int half, int cta, const CUtensorMap*& map, int& y) const {
    map = half ? map_b64 : map_b128;
    y = b_rows_default(nt, half, cta);
  }
  __device__ __forceinline__ bool before_load(int, int, const Abort&) const { return true; }
  __device__ __forceinline__ void a_tile(int mt, const CUtensorMap*& map, int& y) const {
    map = map_a;
    y = mt * 128;
  }
  __device__ __forceinline__ void epilogue_finish(int, int, const Abort&) const {}
  __device__ __forceinline__ void between_tiles(int, int, const Abort&) const {}
  __device__ __forceinline__ void epilogue_begin(int, int, const Abort&) const {}
  __device__ __forceinline__ bool epilogue(int mt, int nt, int col0, int ncols, uint32_t taddr, int quad, int lane,
                                           const Abort&, const Smem2&) const {
    const int row = mt * 128 + quad * 32 + lane;
    store_rows(C + (size_t)row * ldc, row < M, N, nt * BN2 + col0, ncols, taddr);
    return true;
  }
};

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b128,
                 const __grid_constant__ CUtensorMap map_b64, const Shape shp, PlainPolicy2 pol, uint32_t* status) {
  tccl_comm fake;
  fake.local = status ? status - TCCL_LOCAL_STATUS : nullptr;
  pol.map_a = &map_a;
  pol.map_b128 = &map_b128;
  pol.map_b64 = &map_b64;
  run_mainloop2(shp, pol, status ? &fake : nullptr, 2000000000ull);
}

}  // namespace gemm2
}  // namespace tccl

using namespace tccl::gemm;
using namespace tccl::gemm2;

extern "C" int tccl_gemm_bf16_pair(const tccl_gemm_args* g, int grid, void* stream) {
  if (!g || g->m <= 0 || g->n <= 0 || g->k <= 0) return -TCCL_EINVAL;
  if ((g->lda % 8) || (g->ldb % 8) || (g->ldc % 8) || (g->n % 8) || (g->k % 8)) return -TCCL_EALIGN;
  if (((uintptr_t)g->a | (uintptr_t)g->bt | (uintptr_t)g->c) & 15) return -TCCL_EALIGN;
  CUtensorMap ma, mb128, mb64;
  int rc = make_tmap_bf16_kmajor(&ma, g->a, g->m, g->k, g->lda, 128);  // each CTA loads 128 rows of A ...
  if (rc) return rc;
  rc = make_tmap_bf16_kmajor(&mb128, g->bt, g->n, g->k, g->ldb, 128);  // ... and 128 rows of Bt (64 for a half tile)
  if (rc) return rc;
  rc = make_tmap_bf16_kmajor(&mb64, g->bt, g->n, g->k, g->ldb, 64);
  if (rc) return rc;
  PlainPolicy2 pol{};
  pol.C = reinterpret_cast<__nv_bfloat16*>(g->c);
  pol.M = g->m;
  pol.N = g->n;
  pol.ldc = g->ldc;
  pol.tiles_n = (g->n + BN2 - 1) / BN2;
  const int total = ((g->m + 255) / 256) * pol.tiles_n;
  if (grid <= 0) grid = tccl_num_sms();
  grid &= ~1;
  if (grid > 2 * total) grid = 2 * total;
  if (grid < 2) return -TCCL_EINVAL;
  pol.sched.init(total, grid / 2);
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem2);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  Shape shp{g->m, g->n, g->k};
  gemm_pair_kernel<<<grid, kThreads, kSmem2, reinterpret_cast<cudaStream_t>(stream)>>>(
      ma, mb128, mb64, shp, pol, reinterpret_cast<uint32_t*>(g->status));
  return (int)cudaGetLastError();
}
