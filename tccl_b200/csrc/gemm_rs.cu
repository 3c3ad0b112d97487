// GEMM -> reduce-scatter in ONE kernel (tensor parallel down-projection):
//   out_r[M/W, N] = rows [r M/W, (r+1) M/W) of  sum_src  A_src[M, K_src] * Bt_src[N, K_src]^T
// Every rank runs the tcgen05 mainloop over all M x N tiles of its partial
// product, ordered by owner: its own rows first, then the next rank's, and so
// on.  The epilogue of every tile converts the accumulator to bf16 into an 8 KB
// shared-memory chunk per 32 columns and hands it to the copy engine: one bulk
// async copy per chunk into slot [src][tile] of the OWNER's staging area — over
// NVLink for a peer, locally for the own rows — and, once a tile's copies are
// complete, a release store raises the tile's flag at the owner.  While tile i
// is on the wire the MMAs of tile i+1 run (second TMEM accumulator).  When a CTA
// has issued its last tile it joins the final phase: all CTAs of the rank share
// out the rank's tiles in 32-row units, wait for the W flags of a unit's tile and
// sum the W staged partials in fp32 (fixed order) into the output rows.  The
// reduction is therefore spread over the whole GPU and overlaps the peers' last
// pushes, instead of sitting in the epilogue of the few CTAs that computed the
// own rows last.
//
// Flags carry the call's epoch (kept in device memory and advanced by the last
// CTA to finish), so nothing has to be reset and a captured graph can replay.
// The entry barrier keeps a fast rank from overwriting a staging slot that a
// slow rank is still reducing from the previous call.
//
// The reference has no kernel of this kind: fusing a matmul with its collective is the goal its
// presentation names (presentation.pdf, slide 4: "fusing (matmul-allreduce) for overlap"); its collectives
// are stand-alone Triton kernels (triton_reduce_scatter.py:59-127, triton_all_gather.py:32-95).
#include "gemm_host.cuh"
#include "gemm_tcgen05.cuh"

namespace tccl {
namespace gemm {

constexpr uint32_t kSlotBytes = BM * BN * 2;  // one bf16 tile

struct alignas(64) GemmRsParams {
  CUtensorMap map_a, map_b;
  Shape shp;
  __nv_bfloat16* out;
  int ldo;
  int tiles_n;
  int tiles_m_per_rank;
  uint64_t* trace;  // optional: 64 words per CTA of %globaltimer stamps (see run_mainloop)
};

__device__ __forceinline__ void epi_bar() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

struct GemmRsPolicy {
  const tccl_comm* c;
  const GemmRsParams* p;
  int bid, nb;
  uint32_t epoch;
  int tpo;  // tiles per owner
  uint32_t* pending_flag;  // epilogue issuer only: flag of the last pushed tile, raised once its copies are done

  __device__ __forceinline__ bool tile(int i, int& mt, int& nt) const {
    const int t = bid + i * nb;
    if (t >= c->world * tpo) return false;
    const int j = t / tpo, local = t - j * tpo;
    int owner = c->rank + j;  // own rows first: they need no link and are reduced last anyway
    if (owner >= c->world) owner -= c->world;
    mt = owner * p->tiles_m_per_rank + local / p->tiles_n;
    nt = local % p->tiles_n;
    return true;
  }
  __device__ __forceinline__ bool before_load(int, int, const Abort&) const { return true; }
  __device__ __forceinline__ void a_tile(int mt, const CUtensorMap*& map, int& y) const {
    map = &p->map_a;
    y = mt * BM;
  }
  // byte offset of (row, 32-column group cg, 16-byte vector v) inside a staging slot:
  // for fixed (cg, v) the 128 rows are contiguous, so a warp's store is one 512-byte run
  static __device__ __forceinline__ uint32_t slot_off(int row, int cg, int v) {
    return (uint32_t)(((cg * 4 + v) * BM + row) * 16);
  }

  // Raise the flag of the previously pushed tile: its bulk copies must be complete (not
  // just read out of shared memory) before the release store.
  __device__ __forceinline__ void flush_pending() {
    if (pending_flag) {
      bulk_wait<0>();
      fence_proxy_async();
      st_release_sys(pending_flag, epoch);
      pending_flag = nullptr;
    }
  }
  __device__ __forceinline__ void epilogue_finish(int quad, int lane, const Abort&) {
    if (quad == 0 && lane == 0) flush_pending();
  }

  __device__ bool epilogue(int mt, int nt, uint32_t taddr, int quad, int lane, const Abort& ab, const SmemLayout& sm) {
    const int me = c->rank;
    const int owner = mt / p->tiles_m_per_rank;
    const int lt = (mt - owner * p->tiles_m_per_rank) * p->tiles_n + nt;
    const int row = quad * 32 + lane;
    const bool issuer = quad == 0 && lane == 0;
    // first of all publish the previous pushed tile: a rank that sat on a pending flag while
    // waiting for its peers' flags would deadlock with peers doing the same
    if (issuer) flush_pending();
    {
      // tensor memory -> registers -> an 8 KB shared-memory chunk per 32 columns
      // (already in the slot's layout) -> ONE bulk async copy to the owner's staging slot.  The
      // copy engine keeps the NVLink writes in flight; the four epilogue warps are free again
      // after ~3 us instead of pacing 64 KB of posted 16-byte stores themselves (measured:
      // 21 us per tile, which made the whole kernel store-issue-bound).
      char* slot = c->stage[owner] + ((size_t)me * tpo + lt) * kSlotBytes;
#pragma unroll 1
      for (int cg = 0; cg < BN / 32; ++cg) {
        uint8_t* buf = sm.epi[cg & 1];
        if (cg >= 2) {
          if (issuer) bulk_wait_read<1>();  // the copy that last used this chunk has read it
          epi_bar();
        }
        uint32_t r[32];
        tmem_ld_32x32(taddr + cg * 32, r);
        tmem_ld_wait();
#pragma unroll
        for (int v = 0; v < 4; ++v) st_shared_v4(buf + (v * BM + row) * 16, pack8_bf16(r + v * 8));
        fence_proxy_async_smem();  // generic-proxy writes -> visible to the bulk copy
        epi_bar();
        if (issuer) {
          bulk_store(slot + (size_t)cg * kEpiChunkBytes, buf, kEpiChunkBytes);
          bulk_commit();
        }
      }
      if (issuer) {
        bulk_wait_read<0>();  // both chunks are free for the next tile
        pending_flag = c->flags[owner] + TCCL_FLAG_TILE + me * TCCL_MAX_TILES + lt;
      }
      epi_bar();
      return !*ab.flag;
    }
  }
};

// Final phase, all threads of all CTAs: unit u = (own tile lt, 32-row quarter).  Thread t of
// the CTA owns (16-byte column group t / 32 [+ 8 per pass], row t % 32): for a fixed column
// group the 32 rows of a quarter are 512 contiguous bytes of every slot.
__device__ void rs_final_reduce(const tccl_comm& c, const GemmRsParams& p, int bid, int nb, uint32_t epoch, int tpo,
                                uint64_t deadline) {
  const int W = c.world, me = c.rank;
  const int t = threadIdx.x;
  for (int u = bid; u < tpo * 4; u += nb) {
    const int lt = u >> 2, qr = u & 3;
    int ok = 1;
    if (t < W)
      ok = wait_reach(c.flags[me] + TCCL_FLAG_TILE + t * TCCL_MAX_TILES + lt, epoch, c, deadline, t, TCCL_W_TILE);
    if (!__syncthreads_and(ok)) return;
    const int mtl = lt / p.tiles_n, nt = lt - mtl * p.tiles_n;
    const int row = qr * 32 + (t & 31);
    const int orow = mtl * BM + row;
    __nv_bfloat16* dst = p.out + (size_t)orow * p.ldo + nt * BN;
    const bool row_ok = me * p.tiles_m_per_rank * BM + orow < p.shp.M;
    const char* slot0 = c.stage[me] + (size_t)lt * kSlotBytes;
    const size_t src_stride = (size_t)tpo * kSlotBytes;
    // two passes (column groups) at a time: 2 W 16-byte loads per thread in flight
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      Vec16 x[2][TCCL_MAX_WORLD];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int cgv = (t >> 5) + 8 * (2 * half + q);  // 0..31 = (32-column group) * 4 + vector
        const uint32_t off = (uint32_t)((cgv * BM + row) * 16);
#pragma unroll
        for (int src = 0; src < TCCL_MAX_WORLD; ++src)
          if (src < W) x[q][src] = ld_peer(slot0 + src * src_stride + off);
      }
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int cgv = (t >> 5) + 8 * (2 * half + q);
        Acc<__nv_bfloat16> acc;
        acc.zero();
#pragma unroll
        for (int src = 0; src < TCCL_MAX_WORLD; ++src)
          if (src < W) acc.add(x[q][src]);
        if (row_ok && nt * BN + cgv * 8 < p.shp.N) st_local(dst + cgv * 8, acc.pack());
      }
    }
  }
}

__device__ __forceinline__ void gemm_rs_body(const tccl_comm& c, const GemmRsParams& p, int bid, int nb) {
  const uint64_t deadline = globaltimer() + c.timeout_ns;
  GemmRsPolicy pol;
  pol.c = &c;
  pol.p = &p;
  pol.bid = bid;
  pol.nb = nb;
  pol.epoch = c.local[TCCL_LOCAL_TILE_EPOCH] + 1u;
  pol.tpo = p.tiles_m_per_rank * p.tiles_n;
  pol.pending_flag = nullptr;
  barrier_p2p(c, bid, deadline);  // the previous call's staging slots are free on every rank
  if (threadIdx.x == 0) tma_prefetch_desc(&p.map_a);
  run_mainloop(&p.map_b, p.shp, pol, &c, c.timeout_ns, p.trace ? p.trace + (size_t)bid * 64 : nullptr);
  rs_final_reduce(c, p, bid, nb, pol.epoch, pol.tpo, deadline);
  if (p.trace && threadIdx.x == 0) p.trace[(size_t)bid * 64 + 62] = globaltimer();
  // the last CTA of this rank to finish publishes the new epoch for the next call
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(c.local + TCCL_LOCAL_SCHED, 1u);
    if (done == (uint32_t)nb - 1u) {
      c.local[TCCL_LOCAL_SCHED] = 0u;
      c.local[TCCL_LOCAL_TILE_EPOCH] = pol.epoch;
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_rs_kernel(const __grid_constant__ tccl_comm comm, const __grid_constant__ GemmRsParams p) {
  gemm_rs_body(comm, p, blockIdx.x, gridDim.x);
}
__global__ void __launch_bounds__(kThreads, 1) gemm_rs_kernel_emu(const tccl_comm* comms, const GemmRsParams* ps) {
  gemm_rs_body(comms[blockIdx.y], ps[blockIdx.y], blockIdx.x, gridDim.x);
}

static int fill_params(GemmRsParams* p, const tccl_gemm_rs_args* g, int world) {
  if (g->m <= 0 || g->n <= 0 || g->k <= 0) return -TCCL_EINVAL;
  if ((g->lda % 8) || (g->ldb % 8) || (g->ldo % 8) || (g->k % 8) || (g->n % BN)) return -TCCL_EALIGN;
  if (g->m % (world * BM)) return -TCCL_ESIZE;  // every rank owns whole 128-row tiles
  if (((uintptr_t)g->a | (uintptr_t)g->bt | (uintptr_t)g->out) & 15) return -TCCL_EALIGN;
  int rc = make_tmap_bf16_kmajor(&p->map_a, g->a, g->m, g->k, g->lda, BM);
  if (rc) return rc;
  rc = make_tmap_bf16_kmajor(&p->map_b, g->bt, g->n, g->k, g->ldb, BN);
  if (rc) return rc;
  p->shp = Shape{g->m, g->n, g->k};
  p->out = reinterpret_cast<__nv_bfloat16*>(g->out);
  p->trace = reinterpret_cast<uint64_t*>(g->trace);
  p->ldo = g->ldo;
  p->tiles_n = g->n / BN;
  p->tiles_m_per_rank = g->m / world / BM;
  if (p->tiles_n * p->tiles_m_per_rank > TCCL_MAX_TILES) return -TCCL_ESIZE;
  return 0;
}

}  // namespace gemm
}  // namespace tccl

using namespace tccl::gemm;

extern "C" uint64_t tccl_gemm_rs_stage_bytes(int m, int n, int world) {
  return (uint64_t)world * (uint64_t)(m / world / BM) * (uint64_t)(n / BN) * kSlotBytes;
}
extern "C" uint64_t tccl_gemm_rs_param_bytes(void) { return sizeof(GemmRsParams); }

// real mode: `comm` and `args` are host structs of the calling rank, `dev_params` unused.
// emulated mode: `comm` is the device array of W communicators, `args` a HOST array of W
// argument structs, `dev_params` device scratch of W * tccl_gemm_rs_param_bytes() bytes
// (64-byte aligned) that receives the kernels' parameter blocks.
extern "C" int tccl_gemm_reduce_scatter(const tccl_comm* comm, const tccl_gemm_rs_args* args, void* dev_params,
                                        uint64_t stage_bytes, const tccl_launch* l) {
  cudaStream_t s = reinterpret_cast<cudaStream_t>(l->stream);
  if (l->grid <= 0) return -TCCL_EINVAL;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_rs_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemm_rs_kernel_emu, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  if (l->n_emu == 0) {
    GemmRsParams p;
    int rc = fill_params(&p, args, comm->world);
    if (rc) return rc;
    if (tccl_gemm_rs_stage_bytes(args->m, args->n, comm->world) > comm->stage_bytes) return -TCCL_ESIZE;
    gemm_rs_kernel<<<l->grid, kThreads, kSmemBytes, s>>>(*comm, p);
    return (int)cudaGetLastError();
  }
  const int W = l->n_emu;
  if (W < 1 || W > TCCL_MAX_WORLD || !dev_params || ((uintptr_t)dev_params & 63)) return -TCCL_EINVAL;
  if (tccl_gemm_rs_stage_bytes(args[0].m, args[0].n, W) > stage_bytes) return -TCCL_ESIZE;
  GemmRsParams ps[TCCL_MAX_WORLD];
  for (int r = 0; r < W; ++r) {
    int rc = fill_params(&ps[r], &args[r], W);
    if (rc) return rc;
  }
  cudaError_t e = cudaMemcpyAsync(dev_params, ps, sizeof(GemmRsParams) * W, cudaMemcpyHostToDevice, s);
  if (e != cudaSuccess) return (int)e;
  const GemmRsParams* dps = reinterpret_cast<const GemmRsParams*>(dev_params);
  void* kargs[2] = {(void*)&comm, (void*)&dps};
  return (int)cudaLaunchCooperativeKernel((const void*)gemm_rs_kernel_emu, dim3(l->grid, W), dim3(kThreads), kargs,
                                          kSmemBytes, s);
}
