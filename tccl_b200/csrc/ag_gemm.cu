// All-gather -> GEMM in ONE kernel (tensor parallel up-projection):
//   out_r[M, N_r] = gather_src(A_src[M/W, K]) * Bt_r[N_r, K]^T
// The first `comm_ctas` CTAs move data: they copy this rank's shard, one
// 128-row tile at a time, into slot [rank] of every rank's gathered buffer
// (one multimem.st per vector through the switch when NVLS is there, else one
// posted store per peer); the data mover that finishes a row tile last raises
// the flag [rank][row tile] on every rank to the call's epoch with a release
// store.  The other CTAs run the tcgen05
// mainloop: the M-tiles of the rank's own shard first, straight from the shard,
// then the remote row tiles in the order they arrive; the TMA producer waits for
// a row tile's counter before its first load and reads the rows from LOCAL
// memory (the gathered buffer), never from a peer.  Arrival of row tile i+1
// overlaps the MMAs on row tile i.
//
// Flags carry the call's epoch (the same device-resident epoch the GEMM ->
// reduce-scatter kernel uses; the last CTA to finish advances it), so nothing is
// ever reset and stale flags of earlier calls can never satisfy a wait.
//
// The reference has no kernel of this kind: fusing a matmul with its collective is the goal its
// presentation names (presentation.pdf, slide 4: "fusing (matmul-allreduce) for overlap"); its collectives
// are stand-alone Triton kernels (triton_reduce_scatter.py:59-127, triton_all_gather.py:32-95).
#include "gemm_host.cuh"
#include "gemm_tcgen05.cuh"

namespace tccl {
namespace gemm {

struct alignas(64) AgGemmParams {
  CUtensorMap map_a_shard, map_a_full, map_b;
  Shape shp;
  const char* a_shard;
  char* a_full[TCCL_MAX_WORLD];
  char* mc_a_full;
  __nv_bfloat16* out;
  int lda_shard, lda_full, ldo;
  int tiles_n, tiles_m_per_rank, comm_ctas;
  uint64_t* trace;  // optional: 64 words per CTA of %globaltimer stamps (see run_mainloop)
  int mc_a_full_only;  // 1: force the LSU / multimem.st movers
  int swiglu;  // 1: columns [0,128) of every 256-wide tile are gate, [128,256) up; out = silu(gate) * up
};

struct AgGemmPolicy {
  const tccl_comm* c;
  const AgGemmParams* p;
  int bid, nb;  // among the GEMM CTAs
  uint32_t epoch;

  __device__ __forceinline__ bool tile(int i, int& mt, int& nt) const {
    const int t = bid + i * nb;
    const int tmpr = p->tiles_m_per_rank, tn = p->tiles_n, W = c->world;
    const int own = tmpr * tn;
    if (t >= W * own) return false;
    if (t < own) {  // own rows first: no waiting
      mt = c->rank * tmpr + t / tn;
      nt = t % tn;
      return true;
    }
    // remote rows in arrival order: row tile by row tile, peers from the next rank on
    const int u = t - own;
    const int per_rt = (W - 1) * tn;
    const int rt = u / per_rt, v = u - rt * per_rt;
    int src = c->rank + 1 + v / tn;
    if (src >= W) src -= W;
    mt = src * tmpr + rt;
    nt = v % tn;
    return true;
  }
  __device__ __forceinline__ void epilogue_finish(int, int, const Abort&) const {}
  __device__ __forceinline__ bool before_load(int mt, int, const Abort& ab) const {
    const int src = mt / p->tiles_m_per_rank;
    if (src == c->rank) return true;
    const int rt = mt - src * p->tiles_m_per_rank;
    const bool ok = wait_reach(c->flags[c->rank] + TCCL_FLAG_AG + src * TCCL_MAX_ROW_TILES + rt, epoch, *c,
                               ab.deadline, src, TCCL_W_TILE);
    if (!ok) *ab.flag = 1;
    fence_proxy_async();  // rows written through the generic proxy are read by TMA next
    return ok;
  }
  __device__ __forceinline__ void a_tile(int mt, const CUtensorMap*& map, int& y) const {
    const int src = mt / p->tiles_m_per_rank;
    if (src == c->rank) {
      map = &p->map_a_shard;
      y = (mt - src * p->tiles_m_per_rank) * BM;
    } else {
      map = &p->map_a_full;
      y = mt * BM;
    }
  }
  __device__ __forceinline__ bool epilogue(int mt, int nt, uint32_t taddr, int quad, int lane, const Abort&, const SmemLayout&) const {
    const int row = mt * BM + quad * 32 + lane;
    __nv_bfloat16* crow = p->out + (size_t)row * p->ldo;
    if (p->swiglu) {
      // SwiGLU fused into the epilogue: the weight rows are packed so that each 256-wide
      // tile holds 128 gate columns followed by the 128 matching up columns
#pragma unroll 1
      for (int cg = 0; cg < BN / 64; ++cg) {
        uint32_t g[32], u[32];
        tmem_ld_32x32(taddr + cg * 32, g);
        tmem_ld_32x32(taddr + BN / 2 + cg * 32, u);
        tmem_ld_wait();
        const int col0 = nt * (BN / 2) + cg * 32;
        if (row < p->shp.M) {
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            if (col0 + v * 8 < p->shp.N / 2) {
              uint32_t o[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                const float gv = __uint_as_float(g[v * 8 + e]), uv = __uint_as_float(u[v * 8 + e]);
                o[e] = __float_as_uint(gv / (1.f + __expf(-gv)) * uv);
              }
              st_local(crow + col0 + v * 8, pack8_bf16(o));
            }
          }
        }
      }
      return true;
    }
#pragma unroll 1
    for (int cg = 0; cg < BN / 32; ++cg) {
      uint32_t r[32];
      tmem_ld_32x32(taddr + cg * 32, r);
      tmem_ld_wait();
      const int col0 = nt * BN + cg * 32;
      if (row < p->shp.M) {
#pragma unroll
        for (int v = 0; v < 4; ++v)
          if (col0 + v * 8 < p->shp.N) st_local(crow + col0 + v * 8, pack8_bf16(r + v * 8));
      }
    }
    return true;
  }
};

// Data movers, bulk-copy form: one thread per mover CTA drives the copy engine.  Rows of the
// shard are bulk-loaded into a ring of shared-memory slots and bulk-stored from there to the
// gathered buffer of every rank (plain unicast copies; the peers' memory is only ever written,
// and never through a multicast TMA operation).  An SM's load/store unit sustains only a few
// GB/s of posted remote stores (measured ~3 GB/s per 128 threads), so LSU movers need most of
// the GPU to fill the link; the copy engine lets a handful of CTAs do it and leaves the SMs
// to the GEMM.
constexpr int kMoverSlots = 16;
constexpr uint32_t kMoverSlotBytes = 12 * 1024;  // rows up to 6144 bf16 elements

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ void ag_comm_bulk(const tccl_comm& c, const AgGemmParams& p, int bid, uint32_t epoch) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ int s_abort;
  const uint64_t deadline = globaltimer() + c.timeout_ns;
  barrier_p2p(c, bid, deadline);  // every rank is done reading the buffer from the previous call
  if (threadIdx.x != 0) return;
  uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint64_t* bars = reinterpret_cast<uint64_t*>(base + (size_t)kMoverSlots * kMoverSlotBytes);
  s_abort = 0;
  for (int s = 0; s < kMoverSlots; ++s) mbar_init(bars + s, 1);
  fence_barrier_init();
  Abort ab{&s_abort, &c, c.local + TCCL_LOCAL_STATUS, deadline};
  const int W = c.world, me = c.rank, nc = p.comm_ctas;
  const uint32_t row_bytes = (uint32_t)p.shp.K * 2;
  const int rows_per_rank = p.tiles_m_per_rank * BM;
  uint32_t phases = 0;  // bit s = parity of slot s's mbarrier
  bool ok = true;
  // Batches of kBatch rows alternate between the two halves of the slot ring.  While batch j
  // is being stored, batch j-1 may still be in flight; a row tile is published once the
  // batch that closed it is known complete, i.e. one batch later (every batch is padded to
  // exactly kBatch commit groups so that "at most kBatch groups pending" means "all earlier
  // batches are done").
  constexpr int kBatch = kMoverSlots / 2;
  auto publish = [&](int rt) {
    fence_proxy_async();
    fence_acq_rel_sys();
    const uint32_t done = atomicAdd(c.local + TCCL_LOCAL_AGCNT + rt, 1u);
    if (done == (uint32_t)nc - 1u) {
      c.local[TCCL_LOCAL_AGCNT + rt] = 0u;
      fence_acq_rel_sys();
      for (int q = 0; q < W; ++q) st_release_sys(c.flags[q] + TCCL_FLAG_AG + me * TCCL_MAX_ROW_TILES + rt, epoch);
    }
  };
  int pending_rt = -1;  // row tile closed by the previous batch, not yet published
  uint32_t batch = 0;
  for (int rt = 0; rt < p.tiles_m_per_rank && ok; ++rt) {
    for (int r0 = rt * BM + bid; r0 < (rt + 1) * BM && ok; r0 += nc * kBatch, ++batch) {
      const int set = (batch & 1) * kBatch;
      if (batch >= 2) bulk_wait_read<kBatch>();  // batch - 2 has been read out of this half
      int n = 0;
      for (int row = r0; row < (rt + 1) * BM && n < kBatch; row += nc, ++n) {
        mbar_arrive_expect_tx(bars + set + n, row_bytes);
        bulk_load(base + (size_t)(set + n) * kMoverSlotBytes, p.a_shard + (size_t)row * p.lda_shard * 2, row_bytes,
                  bars + set + n);
      }
      int k = 0;
      for (int row = r0; row < (rt + 1) * BM && k < kBatch; row += nc, ++k) {
        const int sl = set + k;
        ok = mbar_wait(bars + sl, (phases >> sl) & 1u, ab);
        if (!ok) break;
        phases ^= 1u << sl;
        const size_t dst = (size_t)(me * rows_per_rank + row) * p.lda_full * 2;
        for (int q = 0; q < W; ++q) bulk_store(p.a_full[q] + dst, base + (size_t)sl * kMoverSlotBytes, row_bytes);
        bulk_commit();
      }
      for (; k < kBatch; ++k) bulk_commit();  // pad: empty groups
      if (!ok) break;
      if (pending_rt >= 0) {
        bulk_wait<kBatch>();  // everything before this batch is complete
        publish(pending_rt);
        pending_rt = -1;
      }
      if (r0 + nc * kBatch >= (rt + 1) * BM) pending_rt = rt;  // this batch closes the row tile
    }
  }
  bulk_wait<0>();
  if (ok && pending_rt >= 0) publish(pending_rt);
}

// data movers: CTA b of `comm_ctas` copies its share of every row tile of the shard
__device__ void ag_comm_part(const tccl_comm& c, const AgGemmParams& p, int bid, uint32_t epoch) {
  __shared__ int s_last;
  const uint64_t deadline = globaltimer() + c.timeout_ns;
  barrier_p2p(c, bid, deadline);  // every rank is done reading the buffer from the previous call
  const int W = c.world, me = c.rank;
  // Two groups of movers take the row tiles alternately: publishing a row tile needs a
  // system-scope fence that drains the group's stores (a switch round trip), and while one
  // group drains the other keeps the link busy.
  const int groups = p.comm_ctas >= 2 ? 2 : 1;
  const int nc = p.comm_ctas / groups;          // movers per row tile
  const int grp = bid / nc, gb = bid - grp * nc;  // my group, my index inside it
  if (grp >= groups) return;                    // odd mover count: the last CTA sits out
  const int K = p.shp.K;
  const int vec_per_row = K / 8;
  const int rows_per_rank = p.tiles_m_per_rank * BM;
  for (int rt = grp; rt < p.tiles_m_per_rank; rt += groups) {
    const uint32_t nvec = (uint32_t)BM * vec_per_row;
    const uint32_t per = (nvec + nc - 1) / nc;
    const uint32_t lo = min(per * gb, nvec), hi = min(lo + per, nvec);
    // 8 vectors per thread in flight: a mover CTA has to keep ~32 KB on the wire to matter
    constexpr int U = 8;
    for (uint32_t i0 = lo + threadIdx.x; i0 < hi; i0 += U * blockDim.x) {
      Vec16 v[U];
      size_t dst[U];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint32_t i = i0 + u * blockDim.x;
        if (i < hi) {
          const int row = rt * BM + i / vec_per_row, col = (i % vec_per_row) * 8;
          v[u] = ld_peer(p.a_shard + ((size_t)row * p.lda_shard + col) * 2);
          dst[u] = ((size_t)(me * rows_per_rank + row) * p.lda_full + col) * 2;
        }
      }
#pragma unroll
      for (int u = 0; u < U; ++u) {
        if (i0 + u * blockDim.x < hi) {
          if (p.mc_a_full) {
            multimem_st(p.mc_a_full + dst[u], v[u]);
          } else {
            for (int q = 0; q < W; ++q) st_peer(p.a_full[q] + dst[u], v[u]);
          }
        }
      }
    }
    __syncthreads();  // this CTA's share of the row tile is stored
    if (threadIdx.x == 0) {
      // count the movers that are done with this row tile; the last one publishes it
      fence_acq_rel_sys();
      const uint32_t done = atomicAdd(c.local + TCCL_LOCAL_AGCNT + rt, 1u);
      s_last = (done == (uint32_t)nc - 1u);
      if (s_last) {
        c.local[TCCL_LOCAL_AGCNT + rt] = 0u;
        fence_acq_rel_sys();
      }
    }
    __syncthreads();
    if (s_last && (int)threadIdx.x < W)
      st_release_sys(c.flags[threadIdx.x] + TCCL_FLAG_AG + me * TCCL_MAX_ROW_TILES + rt, epoch);
  }
}

__device__ __forceinline__ void ag_gemm_body(const tccl_comm& c, const AgGemmParams& p, int bid, int nb) {
  const uint32_t epoch = c.local[TCCL_LOCAL_TILE_EPOCH] + 1u;
  if (bid < p.comm_ctas) {
    // With NVLS one multimem.st reaches all ranks through the switch (egress = the shard, not
    // W-1 copies of it): the LSU movers win (measured on 8xB200: 117 us against 170-200 us for
    // bulk copies, which must send every copy themselves).  Without NVLS the copy engine moves
    // rows that fit a slot.
    if (!p.mc_a_full && (uint32_t)p.shp.K * 2 <= kMoverSlotBytes && !p.mc_a_full_only)
      ag_comm_bulk(c, p, bid, epoch);
    else
      ag_comm_part(c, p, bid, epoch);
  } else {
    AgGemmPolicy pol;
    pol.c = &c;
    pol.p = &p;
    pol.bid = bid - p.comm_ctas;
    pol.nb = nb - p.comm_ctas;
    pol.epoch = epoch;
    if (threadIdx.x == 0) {
      tma_prefetch_desc(&p.map_a_shard);
      tma_prefetch_desc(&p.map_a_full);
    }
    run_mainloop(&p.map_b, p.shp, pol, &c, c.timeout_ns, p.trace ? p.trace + (size_t)bid * 64 : nullptr);
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const uint32_t done = atomicAdd(c.local + TCCL_LOCAL_SCHED, 1u);
    if (done == (uint32_t)nb - 1u) {
      c.local[TCCL_LOCAL_SCHED] = 0u;
      c.local[TCCL_LOCAL_TILE_EPOCH] = epoch;
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
ag_gemm_kernel(const __grid_constant__ tccl_comm comm, const __grid_constant__ AgGemmParams p) {
  ag_gemm_body(comm, p, blockIdx.x, gridDim.x);
}
__global__ void __launch_bounds__(kThreads, 1) ag_gemm_kernel_emu(const tccl_comm* comms, const AgGemmParams* ps) {
  ag_gemm_body(comms[blockIdx.y], ps[blockIdx.y], blockIdx.x, gridDim.x);
}

static int fill_params(AgGemmParams* p, const tccl_ag_gemm_args* g, int world, int rank, int grid) {
  if (g->m <= 0 || g->n <= 0 || g->k <= 0) return -TCCL_EINVAL;
  if ((g->lda_shard % 8) || (g->lda_full % 8) || (g->ldb % 8) || (g->ldo % 8) || (g->k % 8) || (g->n % 8))
    return -TCCL_EALIGN;
  if (g->m % (world * BM)) return -TCCL_ESIZE;
  if (g->comm_ctas < 1 || g->comm_ctas >= grid) return -TCCL_EINVAL;
  if (((uintptr_t)g->a_shard | (uintptr_t)g->bt | (uintptr_t)g->out | (uintptr_t)g->a_full[rank]) & 15)
    return -TCCL_EALIGN;
  const int rows = g->m / world;
  int rc = make_tmap_bf16_kmajor(&p->map_a_shard, g->a_shard, rows, g->k, g->lda_shard, BM);
  if (rc) return rc;
  rc = make_tmap_bf16_kmajor(&p->map_a_full, g->a_full[rank], g->m, g->k, g->lda_full, BM);
  if (rc) return rc;
  rc = make_tmap_bf16_kmajor(&p->map_b, g->bt, g->n, g->k, g->ldb, BN);
  if (rc) return rc;
  p->shp = Shape{g->m, g->n, g->k};
  p->a_shard = reinterpret_cast<const char*>(g->a_shard);
  for (int q = 0; q < TCCL_MAX_WORLD; ++q) p->a_full[q] = reinterpret_cast<char*>(g->a_full[q]);
  p->mc_a_full = reinterpret_cast<char*>(g->mc_a_full);
  p->out = reinterpret_cast<__nv_bfloat16*>(g->out);
  p->trace = reinterpret_cast<uint64_t*>(g->trace);
  p->lda_shard = g->lda_shard;
  p->lda_full = g->lda_full;
  p->ldo = g->ldo;
  p->tiles_n = (g->n + BN - 1) / BN;
  p->tiles_m_per_rank = rows / BM;
  p->comm_ctas = g->comm_ctas;
  p->swiglu = g->swiglu;
  p->mc_a_full_only = g->lsu_movers;
  if (g->swiglu && (g->n % BN)) return -TCCL_ESIZE;  // whole gate|up tiles only
  if (p->tiles_m_per_rank > TCCL_MAX_ROW_TILES) return -TCCL_ESIZE;
  return 0;
}

}  // namespace gemm
}  // namespace tccl

using namespace tccl::gemm;

extern "C" uint64_t tccl_ag_gemm_param_bytes(void) { return sizeof(AgGemmParams); }

extern "C" int tccl_allgather_gemm(const tccl_comm* comm, const tccl_ag_gemm_args* args, void* dev_params,
                                   const tccl_launch* l) {
  cudaStream_t s = reinterpret_cast<cudaStream_t>(l->stream);
  if (l->grid <= 1) return -TCCL_EINVAL;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(ag_gemm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(ag_gemm_kernel_emu, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmemBytes);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  if (l->n_emu == 0) {
    AgGemmParams p;
    int rc = fill_params(&p, args, comm->world, comm->rank, l->grid);
    if (rc) return rc;
    ag_gemm_kernel<<<l->grid, kThreads, kSmemBytes, s>>>(*comm, p);
    return (int)cudaGetLastError();
  }
  const int W = l->n_emu;
  if (W < 1 || W > TCCL_MAX_WORLD || !dev_params || ((uintptr_t)dev_params & 63)) return -TCCL_EINVAL;
  AgGemmParams ps[TCCL_MAX_WORLD];
  for (int r = 0; r < W; ++r) {
    int rc = fill_params(&ps[r], &args[r], W, r, l->grid);
    if (rc) return rc;
  }
  cudaError_t e = cudaMemcpyAsync(dev_params, ps, sizeof(AgGemmParams) * W, cudaMemcpyHostToDevice, s);
  if (e != cudaSuccess) return (int)e;
  const AgGemmParams* dps = reinterpret_cast<const AgGemmParams*>(dev_params);
  void* kargs[2] = {(void*)&comm, (void*)&dps};
  return (int)cudaLaunchCooperativeKernel((const void*)ag_gemm_kernel_emu, dim3(l->grid, W), dim3(kThreads), kargs,
                                          kSmemBytes, s);
}
