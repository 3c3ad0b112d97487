// GEMM -> reduce-scatter in ONE kernel on the CTA-pair mainloop
// (gemm_tcgen05_2cta.cuh):
//   out_r[M/W, N] = rows [r M/W, (r+1) M/W) of  sum_src  A_src[M, K_src] * Bt_src[N, K_src]^T
//
// What differs from the single-CTA form (gemm_rs.cu):
//  * 256 x 256 tiles on pairs of SMs (tcgen05.mma.cta_group::2): each CTA still
//    owns one 128 x 256 partial tile and pushes it, as bf16, with bulk async
//    copies into slot [src][tile] of the OWNER's staging area, then raises the
//    tile's flag there.
//  * Tile order: owner-local tile index outermost, owner innermost (peers first,
//    starting with the next rank, own rows last).  All ranks walk the same local
//    index at about the same time, so tile lt of EVERY owner is complete on all
//    ranks soon after "its" moment — the final reduction of a rank's tiles can
//    start while the mainloop is still running — and every rank always sends to
//    all owners in turn (no hot receiver).
//  * The final reduction is not a phase of its own any more: whenever the
//    epilogue warps of a CTA have handed a tile to the copy engine they look at
//    the rank's reduction cursor, and if the W flags of the next unit (32 rows
//    of one own tile) are up they claim it and sum the W staged partials in fp32
//    into the output rows.  What is left when a CTA runs out of tiles is shared
//    out the same way, now waiting for flags.
//  * No entry barrier: the staging area is used in two halves that alternate
//    from call to call (low bit of a per-communicator call count,
//    TCCL_LOCAL_RS_SEQ).  A rank can reach call n+2 only after its call n+1 got
//    every peer's partials of call n+1, i.e. after every peer has finished call
//    n and with it all reads of the half being reused.  The halves sit at fixed
//    offsets, so this also holds when the shape changes between calls.  A call
//    that follows a different user of the staging area asks for the barrier
//    (TCCL_RS_SYNC_ENTRY).
// Flags carry the epoch shared by the fused GEMM kernels (TCCL_LOCAL_TILE_EPOCH);
// nothing is ever reset.
//
// The reference has no kernel of this kind: fusing a matmul with its collective is the goal its
// presentation names (presentation.pdf, slide 4: "fusing (matmul-allreduce) for overlap"); its collectives
// are stand-alone Triton kernels (triton_reduce_scatter.py:59-127, triton_all_gather.py:32-95).
#include "gemm_host.cuh"
#include "gemm_tcgen05_2cta.cuh"

namespace tccl {
namespace gemm2 {

constexpr uint32_t kSlotBytes2 = 128 * BN2 * 2;  // one CTA's 128 x 256 bf16 partial tile

struct alignas(64) GemmRsPairParams {
  CUtensorMap map_a, map_b;
  Shape shp;
  __nv_bfloat16* out;
  int ldo;
  int tiles_n;
  int tiles_m_per_rank;  // 128-row tiles per owner (even)
  int sync_entry;
  uint64_t half_bytes;   // bytes of one half of the staging area
  uint64_t* trace;       // optional: 64 words per CTA of %globaltimer stamps (see run_mainloop2); [61] kernel end,
                         // [60] mainloop left, [59] first wait of the final reduction over, [58] / [57] units
                         // reduced between tiles / in the final reduction
};

__device__ __forceinline__ void epi_bar2() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

struct GemmRsPairPolicy {
  const tccl_comm* c;
  const GemmRsPairParams* p;
  int pair, npairs;
  uint32_t epoch;
  uint32_t parity;
  int tpo;    // 128-row tiles per owner
  int tpo2;   // pair tiles per owner
  uint32_t* pending_flag;  // epilogue issuer only
  int* s_unit;             // shared: the reduction unit the epilogue warps agreed on (-1 = none)
  uint64_t* trace;         // this CTA's trace words, or null

  __device__ __forceinline__ char* stage_of(int rank) const { return c->stage[rank] + (uint64_t)parity * p->half_bytes; }

  __device__ __forceinline__ bool tile(int i, int& mt, int& nt, int& half) const {
    const int t = pair + i * npairs;
    const int W = c->world;
    if (t >= W * tpo2) return false;
    const int ltp = t / W, j = t - ltp * W;
    int owner = c->rank + 1 + j;  // peers first (the next rank first), own rows last
    if (owner >= W) owner -= W;
    const int mtl2 = ltp / p->tiles_n;
    nt = ltp - mtl2 * p->tiles_n;
    mt = owner * p->tiles_m_per_rank + 2 * mtl2;
    half = 0;
    return true;
  }
  __device__ __forceinline__ void b_tile(int nt, int half, int cta, const CUtensorMap*& map, int& y) const {
    map = &p->map_b;
    y = b_rows_default(nt, half, cta);
  }
  __device__ __forceinline__ bool before_load(int, int, const Abort&) const { return true; }
  __device__ __forceinline__ void a_tile(int mt, const CUtensorMap*& map, int& y) const {
    map = &p->map_a;
    y = mt * 128;
  }

  __device__ __forceinline__ void flush_pending() {
    if (pending_flag) {
      bulk_wait<0>();
      fence_proxy_async();
      st_release_sys(pending_flag, epoch);
      pending_flag = nullptr;
    }
  }

  // Sum the W staged partials of unit u = (own tile lt, 32-row quarter) into the output rows.
  // `nthreads` threads (128: the epilogue warps; 256: the whole CTA), thread `t` of them.
  __device__ __forceinline__ void reduce_unit(int u, int t, int nthreads) const {
    const int W = c->world, me = c->rank;
    const int lt = u >> 2, qr = u & 3;
    const int mtl = lt / p->tiles_n, nt = lt - mtl * p->tiles_n;
    const int row = qr * 32 + (t & 31);
    const int orow = mtl * 128 + row;
    __nv_bfloat16* dst = p->out + (size_t)orow * p->ldo + nt * BN2;
    const bool row_ok = me * p->tiles_m_per_rank * 128 + orow < p->shp.M;
    const char* slot0 = stage_of(me) + (size_t)lt * kSlotBytes2;
    const size_t src_stride = (size_t)tpo * kSlotBytes2;
    const int groups = nthreads >> 5;  // 16-byte column groups handled per pass
    for (int cg0 = (t >> 5); cg0 < 32; cg0 += 2 * groups) {
      Vec16 x[2][TCCL_MAX_WORLD];
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int cgv = cg0 + q * groups;  // 0..31 = (32-column group) * 4 + vector
        const uint32_t off = (uint32_t)((cgv * 128 + row) * 16);
#pragma unroll
        for (int src = 0; src < TCCL_MAX_WORLD; ++src)
          if (src < W) x[q][src] = ld_peer(slot0 + src * src_stride + off);
      }
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int cgv = cg0 + q * groups;
        Acc<__nv_bfloat16> acc;
        acc.zero();
#pragma unroll
        for (int src = 0; src < TCCL_MAX_WORLD; ++src)
          if (src < W) acc.add(x[q][src]);
        if (row_ok && nt * BN2 + cgv * 8 < p->shp.N) st_local(dst + cgv * 8, acc.pack());
      }
    }
  }

  // epilogue warps, between two tiles: claim the next reduction unit if (and only if) its flags are up
  __device__ __forceinline__ void try_reduce(int quad, int lane, int max_units) {
    const int total = tpo * 4;
    for (int k = 0; k < max_units; ++k) {
      if (quad == 0) {
        int unit = -1;
        uint32_t* cursor = c->local + TCCL_LOCAL_RS_NEXT;
        const uint32_t u = *reinterpret_cast<volatile uint32_t*>(cursor);
        if (u < (uint32_t)total) {
          const int lt = (int)(u >> 2);
          bool up = true;
          if (lane < c->world)
            up = (int32_t)(ld_acquire_sys(c->flags[c->rank] + TCCL_FLAG_TILE + lane * TCCL_MAX_TILES + lt) - epoch) >= 0;
          if (__all_sync(0xffffffffu, up)) {
            if (lane == 0 && atomicCAS(cursor, u, u + 1u) == u) unit = (int)u;
          }
        }
        if (lane == 0) *s_unit = unit;
      }
      epi_bar2();
      const int unit = *reinterpret_cast<volatile int*>(s_unit);
      if (unit >= 0) {
        reduce_unit(unit, quad * 32 + lane, 128);
        if (trace && quad == 0 && lane == 0) trace[58] += 1;
      }
      epi_bar2();  // s_unit may be rewritten
      if (unit < 0) break;
    }
  }

  __device__ __forceinline__ void epilogue_finish(int quad, int lane, const Abort&) {
    if (quad == 0 && lane == 0) flush_pending();
  }

  __device__ bool epilogue(int mt, int nt, int, int, uint32_t taddr, int quad, int lane, const Abort& ab, const Smem2& sm) {
    const int me = c->rank;
    const int owner = mt / p->tiles_m_per_rank;
    const int lt = (mt - owner * p->tiles_m_per_rank) * p->tiles_n + nt;
    const int row = quad * 32 + lane;
    const bool issuer = quad == 0 && lane == 0;
    // first of all publish the previously pushed tile
    if (issuer) flush_pending();
    char* slot = stage_of(owner) + ((size_t)me * tpo + lt) * kSlotBytes2;
#pragma unroll 1
    for (int cg = 0; cg < BN2 / 32; ++cg) {
      uint8_t* buf = sm.epi[cg & 1];
      if (cg >= 2) {
        if (issuer) bulk_wait_read<1>();  // the copy that last used this chunk has read it
        epi_bar2();
      }
      uint32_t r[32];
      tmem_ld_32x32(taddr + cg * 32, r);
      tmem_ld_wait();
#pragma unroll
      for (int v = 0; v < 4; ++v) st_shared_v4(buf + (v * 128 + row) * 16, pack8_bf16(r + v * 8));
      fence_proxy_async_smem();
      epi_bar2();
      if (issuer) {
        bulk_store(slot + (size_t)cg * kEpiChunkBytes, buf, kEpiChunkBytes);
        bulk_commit();
      }
    }
    if (issuer) {
      bulk_wait_read<0>();
      pending_flag = c->flags[owner] + TCCL_FLAG_TILE + me * TCCL_MAX_TILES + lt;
    }
    epi_bar2();
    return !*ab.flag;
  }
  // the copy engine has the tile and the accumulator is free again: use the wait for reduction work
  __device__ __forceinline__ void between_tiles(int quad, int lane, const Abort&) { try_reduce(quad, lane, 2); }
  __device__ __forceinline__ void epilogue_begin(int, int, const Abort&) const {}
};

__device__ __forceinline__ void gemm_rs_pair_body(const tccl_comm& c, const GemmRsPairParams& p, int bid, int nb) {
  __shared__ int s_unit;
  const uint64_t deadline = globaltimer() + c.timeout_ns;
  GemmRsPairPolicy pol;
  pol.c = &c;
  pol.p = &p;
  pol.pair = bid >> 1;
  pol.npairs = nb >> 1;
  pol.epoch = c.local[TCCL_LOCAL_TILE_EPOCH] + 1u;
  pol.parity = c.local[TCCL_LOCAL_RS_SEQ] & 1u;
  pol.tpo = p.tiles_m_per_rank * p.tiles_n;
  pol.tpo2 = (p.tiles_m_per_rank / 2) * p.tiles_n;
  pol.pending_flag = nullptr;
  pol.s_unit = &s_unit;
  pol.trace = p.trace ? p.trace + (size_t)bid * 64 : nullptr;
  if (p.sync_entry) barrier_p2p(c, bid, deadline);  // the staging area's previous user is done on every rank
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.map_a);
    tma_prefetch_desc(&p.map_b);
  }
  run_mainloop2(p.shp, pol, &c, c.timeout_ns, p.trace ? p.trace + (size_t)bid * 64 : nullptr);
  // what is left of the reduction, all threads of the CTA, now waiting for flags
  {
    const int total = pol.tpo * 4;
    const int t = threadIdx.x;
    if (pol.trace && t == 0) pol.trace[60] = globaltimer();
    for (;;) {
      if (t == 0) s_unit = (int)atomicAdd(c.local + TCCL_LOCAL_RS_NEXT, 1u);
      __syncthreads();
      const int u = s_unit;
      __syncthreads();
      if (u >= total) break;
      int ok = 1;
      if (t < c.world)
        ok = wait_reach(c.flags[c.rank] + TCCL_FLAG_TILE + t * TCCL_MAX_TILES + (u >> 2), pol.epoch, c, deadline, t,
                        TCCL_W_TILE);
      if (!__syncthreads_and(ok)) break;
      if (pol.trace && t == 0) {
        if (!pol.trace[59]) pol.trace[59] = globaltimer();
        pol.trace[57] += 1;
      }
      pol.reduce_unit(u, t, kThreads);
    }
  }
  // the last CTA of this rank to finish publishes the new epoch and flips the staging half
  __syncthreads();
  if (threadIdx.x == 0) {
    if (p.trace) p.trace[(size_t)bid * 64 + 61] = globaltimer();
    __threadfence();
    const uint32_t done = atomicAdd(c.local + TCCL_LOCAL_SCHED, 1u);
    if (done == (uint32_t)nb - 1u) {
      c.local[TCCL_LOCAL_SCHED] = 0u;
      c.local[TCCL_LOCAL_RS_NEXT] = 0u;
      c.local[TCCL_LOCAL_RS_SEQ] += 1u;
      c.local[TCCL_LOCAL_TILE_EPOCH] = pol.epoch;
    }
  }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_rs_pair_kernel(const __grid_constant__ tccl_comm comm, const __grid_constant__ GemmRsPairParams p) {
  gemm_rs_pair_body(comm, p, blockIdx.x, gridDim.x);
}
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_rs_pair_kernel_emu(const tccl_comm* comms, const GemmRsPairParams* ps) {
  gemm_rs_pair_body(comms[blockIdx.y], ps[blockIdx.y], blockIdx.x, gridDim.x);
}

static int fill_params(GemmRsPairParams* p, const tccl_gemm_rs_args* g, int world, uint64_t stage_bytes, int sync_entry) {
  if (g->m <= 0 || g->n <= 0 || g->k <= 0) return -TCCL_EINVAL;
  if ((g->lda % 8) || (g->ldb % 8) || (g->ldo % 8) || (g->k % 8) || (g->n % BN2)) return -TCCL_EALIGN;
  if (g->m % (world * 256)) return -TCCL_ESIZE;  // every rank owns whole 256-row pair tiles
  if (((uintptr_t)g->a | (uintptr_t)g->bt | (uintptr_t)g->out) & 15) return -TCCL_EALIGN;
  int rc = make_tmap_bf16_kmajor(&p->map_a, g->a, g->m, g->k, g->lda, 128);
  if (rc) return rc;
  rc = make_tmap_bf16_kmajor(&p->map_b, g->bt, g->n, g->k, g->ldb, 128);
  if (rc) return rc;
  p->shp = Shape{g->m, g->n, g->k};
  p->out = reinterpret_cast<__nv_bfloat16*>(g->out);
  p->ldo = g->ldo;
  p->tiles_n = g->n / BN2;
  p->tiles_m_per_rank = g->m / world / 128;
  p->sync_entry = sync_entry;
  p->trace = reinterpret_cast<uint64_t*>(g->trace);
  p->half_bytes = (stage_bytes / 2) & ~(uint64_t)1023;
  if (p->tiles_n * p->tiles_m_per_rank > TCCL_MAX_TILES) return -TCCL_ESIZE;
  if ((uint64_t)world * p->tiles_n * p->tiles_m_per_rank * kSlotBytes2 > p->half_bytes) return -TCCL_ESIZE;
  return 0;
}

}  // namespace gemm2
}  // namespace tccl

using namespace tccl::gemm;
using namespace tccl::gemm2;

// bytes of staging area (per rank) the pair kernel needs for an m x n product: two halves
extern "C" uint64_t tccl_gemm_rs_pair_stage_bytes(int m, int n, int world) {
  return 2ull * (uint64_t)world * (uint64_t)(m / world / 128) * (uint64_t)(n / BN2) * kSlotBytes2 + 2048;
}
extern "C" uint64_t tccl_gemm_rs_pair_param_bytes(void) { return sizeof(GemmRsPairParams); }

// Same calling convention as tccl_gemm_reduce_scatter; l->meta bit 8 (TCCL_RS_SYNC_ENTRY) asks for
// the entry barrier.  l->grid must be even.
extern "C" int tccl_gemm_reduce_scatter_pair(const tccl_comm* comm, const tccl_gemm_rs_args* args, void* dev_params,
                                             uint64_t stage_bytes, const tccl_launch* l) {
  cudaStream_t s = reinterpret_cast<cudaStream_t>(l->stream);
  if (l->grid < 2 || (l->grid & 1)) return -TCCL_EINVAL;
  const int sync_entry = (l->meta & TCCL_RS_SYNC_ENTRY) ? 1 : 0;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(gemm_rs_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem2);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(gemm_rs_pair_kernel_emu, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem2);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  if (l->n_emu == 0) {
    GemmRsPairParams p;
    int rc = fill_params(&p, args, comm->world, comm->stage_bytes, sync_entry);
    if (rc) return rc;
    gemm_rs_pair_kernel<<<l->grid, kThreads, kSmem2, s>>>(*comm, p);
    return (int)cudaGetLastError();
  }
  const int W = l->n_emu;
  if (W < 1 || W > TCCL_MAX_WORLD || !dev_params || ((uintptr_t)dev_params & 63)) return -TCCL_EINVAL;
  GemmRsPairParams ps[TCCL_MAX_WORLD];
  for (int r = 0; r < W; ++r) {
    int rc = fill_params(&ps[r], &args[r], W, stage_bytes, sync_entry);
    if (rc) return rc;
  }
  cudaError_t e = cudaMemcpyAsync(dev_params, ps, sizeof(GemmRsPairParams) * W, cudaMemcpyHostToDevice, s);
  if (e != cudaSuccess) return (int)e;
  const GemmRsPairParams* dps = reinterpret_cast<const GemmRsPairParams*>(dev_params);
  return launch_pairs_emulated((const void*)gemm_rs_pair_kernel_emu, l->grid, W, kSmem2, s, (const void*)&comm,
                               (const void*)&dps);
}
