// Blackwell GEMM mainloop on CTA PAIRS: tcgen05.mma.cta_group::2.
//
// Two CTAs of a cluster (two neighbouring SMs) compute one 256 x 256 tile of
// C = A * Bt^T.  Each CTA TMA-loads ITS OWN 128 rows of A and ITS OWN half
// (128 rows) of Bt from this GPU's memory into its own shared memory — plain
// per-CTA loads, nothing is multicast — and one thread of the pair's leader
// (the even CTA) issues the MMAs, which read both CTAs' shared memory: every
// operand byte is fetched from L2 once per pair instead of once per CTA, which
// is what a 128 x 256 single-CTA tile cannot do (it streams 48 KB per k-block
// through each SM against 32 KB here, and the 148 SMs together out-run L2).
// Each CTA ends up with the accumulator rows of its own 128 rows of A in its
// own tensor memory and runs its own epilogue on them.
//
// Synchronisation inside a pair (all mbarriers, all waits bounded):
//   full[s]   (leader's)   the leader's producer arrives with the bytes of BOTH
//                          CTAs' loads; the peer's loads complete on the
//                          leader's barrier (cta_group::2 form of the TMA load).
//   empty[s]  (each CTA's) the MMA thread commits once to its own and once to
//                          the peer's barrier (two plain commits; no multicast).
//   tmem_full[a] (each)    same: two commits when an accumulator is complete.
//   tmem_empty[a] (leader) the 2 x 128 epilogue threads of both CTAs arrive.
// The last partial wave of a shape whose tile count is not a multiple of the
// number of pairs is cut into 256 x 128 half tiles, so the tail costs half a
// tile instead of a whole one.
//
// Policy hooks are the ones of the single-CTA mainloop (gemm_tcgen05.cuh), in
// units of 128-row tiles: tile(i, mt, nt, half) hands out the pair's EVEN m
// tile, CTA c of the pair works on mt + c.
#pragma once
#include "gemm_tcgen05.cuh"

namespace tccl {
namespace gemm2 {

using namespace tccl::gemm;

constexpr int BN2 = 256, BK2 = 64;
constexpr int kStages2 = 6;
constexpr uint32_t kA2 = 128 * BK2 * 2, kB2 = 128 * BK2 * 2;  // per CTA: its 128 A rows, its 128 Bt rows
constexpr uint32_t kStage2 = kA2 + kB2;                       // 32 KB
constexpr size_t kSmem2 = 1024 /*align slack*/ + (size_t)kStages2 * kStage2 + 256 /*barriers*/ + 2 * kEpiChunkBytes;

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// address of the same shared-memory location in CTA `cta` of the cluster
__device__ __forceinline__ uint32_t mapa(uint32_t smem_addr, uint32_t cta) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta));
  return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t cluster_addr) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
// per-CTA TMA load whose completion bytes are counted on a barrier that may live in the peer CTA
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* map, uint32_t bar_cluster_addr,
                                                 int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(bar_cluster_addr), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void tmem_alloc2(uint32_t* dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish2() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc2(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_mma2_bf16(uint32_t d, uint64_t ad, uint64_t bd, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d), "l"(ad), "l"(bd), "r"(idesc), "r"(acc) : "memory");
}
// one arrival on the barrier at `bar_cluster_addr` (this CTA's or the peer's) once every
// MMA this thread has issued so far is complete
__device__ __forceinline__ void tc_commit2(uint32_t bar_cluster_addr) {
  asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar_cluster_addr)
               : "memory");
}

struct Smem2 {
  uint8_t* a[kStages2];
  uint8_t* b[kStages2];
  uint64_t *full, *empty, *tmem_full, *tmem_empty;
  uint32_t* tmem_base;
  int* abort_flag;
  uint8_t* epi[2];
  __device__ explicit Smem2(uint8_t* raw) {
    uint8_t* p = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
    for (int s = 0; s < kStages2; ++s) {
      a[s] = p + (size_t)s * kStage2;
      b[s] = a[s] + kA2;
    }
    uint64_t* bars = reinterpret_cast<uint64_t*>(p + (size_t)kStages2 * kStage2);
    full = bars;
    empty = bars + kStages2;
    tmem_full = bars + 2 * kStages2;
    tmem_empty = bars + 2 * kStages2 + 2;
    tmem_base = reinterpret_cast<uint32_t*>(bars + 2 * kStages2 + 4);
    abort_flag = reinterpret_cast<int*>(tmem_base + 1);
    epi[0] = p + (size_t)kStages2 * kStage2 + 256;
    epi[1] = epi[0] + kEpiChunkBytes;
  }
};

// `half`: 0 = the full 256 columns of n tile nt, 1 / 2 = its left / right 128 columns
// Hooks (Policy):
//   tile(i, mt, nt, half)                  -> false when the PAIR is out of tiles; mt is even
//   a_tile(mt, map, y)                     -> tensor map (box of 128 rows) and row coordinate of m tile mt
//   b_tile(nt, half, cta, map, y)          -> tensor map of Bt (box of 128 rows for half == 0, of 64 rows else) and
//                                             the first Bt row CTA `cta` of the pair loads; b_rows_default() below
//                                             is the plain layout (the pair's rows are consecutive)
//   before_load(mt, nt, ab)                -> producer thread, before the CTA's first load of its m tile
//   epilogue(mt, nt, col0, ncols, taddr, quad, lane, ab, sm)
//                                          -> 4 epilogue warps of each CTA; columns [col0, col0 + ncols) of
//                                             n tile nt start at tensor-memory address taddr
//   epilogue_begin(quad, lane, ab)         -> epilogue warps, once, before they wait for the first accumulator
//   between_tiles(quad, lane, ab)          -> epilogue warps, after a tile's accumulator has been released
//   epilogue_finish(quad, lane, ab)
// `trace` (optional, this CTA's 64 words of %globaltimer stamps): [63] kernel start, [62] side work of
// epilogue_begin done, and for the CTA's i-th tile, i < 14 (words 56..61 belong to the policies): [4i] producer may load, [4i+1] accumulator
// ready, [4i+2] epilogue done.
// first Bt row of CTA `cta` for (n tile, half) when a tile's columns are 256 consecutive rows of Bt
__device__ __forceinline__ int b_rows_default(int nt, int half, int cta) {
  return nt * BN2 + (half == 2 ? 128 : 0) + cta * (half ? 64 : 128);
}

template <class Policy>
__device__ void run_mainloop2(const Shape shp, Policy& pol, const tccl_comm* comm, uint64_t timeout_ns,
                              uint64_t* trace = nullptr) {
  extern __shared__ uint8_t smem_raw[];
  Smem2 sm(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta = cluster_ctarank();  // 0 = leader
  const bool leader = cta == 0;
  const int num_kb = (shp.K + BK2 - 1) / BK2;

  if (threadIdx.x == 0) {
    if (trace) trace[63] = globaltimer();
    *sm.abort_flag = 0;
    for (int s = 0; s < kStages2; ++s) {
      mbar_init(sm.full + s, 1);   // the leader producer's arrive.expect_tx (bytes of both CTAs)
      mbar_init(sm.empty + s, 1);  // one commit from the leader's MMA thread
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(sm.tmem_full + i, 1);
      mbar_init(sm.tmem_empty + i, 2 * 4 * 32);  // the epilogue threads of BOTH CTAs arrive on the leader's barrier
    }
    fence_barrier_init();
  }
  if (warp == 2) {
    tmem_alloc2(sm.tmem_base, kTmemCols);
    tmem_relinquish2();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync();  // both CTAs' barriers are initialised before anyone signals across
  tc_fence_after();
  const uint32_t tmem_base = *sm.tmem_base;
  Abort ab{sm.abort_flag, comm, comm ? comm->local + TCCL_LOCAL_STATUS : nullptr, globaltimer() + timeout_ns};

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (one per CTA)
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      int mt, nt, half;
      for (int i = 0; ok && pol.tile(i, mt, nt, half); ++i) {
        mt += (int)cta;
        ok = pol.before_load(mt, nt, ab);
        if (trace && i < 14) trace[4 * i] = globaltimer();
        const CUtensorMap* map_a;
        int ya;
        pol.a_tile(mt, map_a, ya);
        const int brows = half ? 64 : 128;  // Bt rows this CTA loads per k-block
        const CUtensorMap* map_b;
        int yb;
        pol.b_tile(nt, half, (int)cta, map_b, yb);
        const uint32_t stage_bytes = kA2 + (uint32_t)brows * BK2 * 2;
        for (int kb = 0; ok && kb < num_kb; ++kb, ++it) {
          const int s = it % kStages2;
          ok = mbar_wait(sm.empty + s, ((it / kStages2) & 1) ^ 1, ab);
          if (!ok) break;
          const uint32_t leader_full = mapa(smem_u32(sm.full + s), 0);
          if (leader) mbar_arrive_expect_tx(sm.full + s, 2 * stage_bytes);
          tma_load_2d_pair(sm.a[s], map_a, leader_full, kb * BK2, ya);
          tma_load_2d_pair(sm.b[s], map_b, leader_full, kb * BK2, yb);
        }
      }
    }
  } else if (warp == 1 && leader) {
    // ------------------------------------------------------------ MMA issuer (leader only)
    if (elect_one()) {
      uint32_t it = 0;
      bool ok = true;
      int mt, nt, half;
      const uint32_t peer_empty0 = mapa(smem_u32(sm.empty), 1), peer_tfull0 = mapa(smem_u32(sm.tmem_full), 1);
      for (int i = 0; ok && pol.tile(i, mt, nt, half); ++i) {
        const int acc = i & 1;
        ok = mbar_wait(sm.tmem_empty + acc, ((i >> 1) & 1) ^ 1, ab);  // both epilogues have drained this accumulator
        if (!ok) break;
        tc_fence_after();
        const uint32_t d = tmem_base + acc * BN2;
        const uint32_t idesc = half ? make_idesc_bf16(256, 128) : make_idesc_bf16(256, 256);
        for (int kb = 0; ok && kb < num_kb; ++kb, ++it) {
          const int s = it % kStages2;
          ok = mbar_wait(sm.full + s, (it / kStages2) & 1, ab);
          if (!ok) break;
          tc_fence_after();
          const uint64_t ad = make_desc_sw128(smem_u32(sm.a[s]));
          const uint64_t bd = make_desc_sw128(smem_u32(sm.b[s]));
#pragma unroll
          for (int k = 0; k < BK2 / UMMA_K; ++k)
            tc_mma2_bf16(d, ad + (uint64_t)(k * 2), bd + (uint64_t)(k * 2), idesc, (kb | k) ? 1u : 0u);
          tc_commit2(smem_u32(sm.empty + s));     // frees the stage in this CTA ...
          tc_commit2(peer_empty0 + (uint32_t)s * 8);  // ... and in the peer
        }
        if (ok) {
          tc_commit2(smem_u32(sm.tmem_full + acc));  // accumulator complete: both epilogues may read
          tc_commit2(peer_tfull0 + (uint32_t)acc * 8);
        }
      }
    }
  } else if (warp >= kEpiWarp0) {
    // ------------------------------------------------------------ epilogue (both CTAs, own rows)
    const int quad = warp - kEpiWarp0;
    const uint32_t leader_tempty0 = mapa(smem_u32(sm.tmem_empty), 0);
    bool ok = true;
    int mt, nt, half;
    pol.epilogue_begin(quad, lane, ab);  // the first accumulator is a whole tile away: time for side work
    if (trace && quad == 0 && lane == 0) trace[62] = globaltimer();
    for (int i = 0; ok && pol.tile(i, mt, nt, half); ++i) {
      mt += (int)cta;
      const int acc = i & 1;
      ok = mbar_wait(sm.tmem_full + acc, (i >> 1) & 1, ab);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN2;
      if (trace && i < 14 && quad == 0 && lane == 0) trace[4 * i + 1] = globaltimer();
      ok = pol.epilogue(mt, nt, half == 2 ? 128 : 0, half ? 128 : 256, taddr, quad, lane, ab, sm);
      if (trace && i < 14 && quad == 0 && lane == 0) trace[4 * i + 2] = globaltimer();
      tc_fence_before();
      mbar_arrive_cluster(leader_tempty0 + (uint32_t)acc * 8);  // the leader's tmem_empty[acc], from either CTA
      if (ok) pol.between_tiles(quad, lane, ab);                // the accumulator is released: time for side work
    }
    pol.epilogue_finish(quad, lane, ab);
  }

  // Neither CTA's shared memory or tensor memory may go away while the other can still signal
  // or read it; a CTA that gave up waits here for its partner, which gives up at the same
  // deadline at the latest.  Loads in flight were all counted on `full` barriers that the MMA
  // thread (or nobody, after a failure) consumed; they have landed by the time both CTAs are here
  // unless a wait failed, in which case the deadline (seconds) has long outlasted any copy.
  tc_fence_before();
  __syncthreads();
  cluster_sync();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc2(tmem_base, kTmemCols);
  }
}

}  // namespace gemm2
}  // namespace tccl
