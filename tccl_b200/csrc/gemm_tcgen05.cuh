// Hand-written Blackwell GEMM mainloop: TMA (local, never multicast) -> shared
// memory ring -> tcgen05.mma with the accumulator in tensor memory -> tcgen05.ld
// epilogue.  C[M,N] = A[M,K] * Bt[N,K]^T, bf16 operands, fp32 accumulation.
//
// CTA = 256 threads: warp 0 issues TMA loads, warp 1 issues the MMAs (one
// elected thread each), warp 2 owns the TMEM allocation, warps 4-7 run the
// epilogue (warp q may only touch TMEM lanes 32 (q % 4) .. +31).  The kernel
// is persistent: CTA b walks tiles b, b + gridDim.x, ... of a schedule, and two
// TMEM accumulators (2 x 256 columns) let the MMAs of tile i+1 run under the
// epilogue of tile i.
//
// The reference has no tensor-core code at all; its slide 4 names "matmul +
// allreduce fusion" as the goal.  The fused kernels (gemm_rs.cu, ag_gemm.cu)
// plug their communication into the Prologue / Epilogue hooks of this mainloop.
//
// Every wait (mbarrier or flag) is bounded; after a failed wait the CTA stops
// issuing work, waits (bounded) for its TMA copies in flight, frees its TMEM and
// returns, and the status words say where it gave up.
#pragma once
#include <cuda.h>

#include "common.cuh"

namespace tccl {
namespace gemm {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int kStages = 4;
constexpr int kThreads = 256;
constexpr int kEpiWarp0 = 4;  // first epilogue warp
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kABytes = BM * BK * 2, kBBytes = BN * BK * 2;
constexpr uint32_t kStageBytes = kABytes + kBBytes;
// epilogue staging: two 8 KB chunks (32 columns x 128 rows of bf16) that bulk async copies drain
constexpr uint32_t kEpiChunkBytes = BM * 32 * 2;
constexpr size_t kSmemBytes =
    1024 /*align slack*/ + (size_t)kStages * kStageBytes + 256 /*barriers*/ + 2 * kEpiChunkBytes;

// ------------------------------------------------------------------ PTX
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool elect_one() {
  uint32_t pred;
  asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
  return pred != 0;
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y) : "memory");
}
// bulk async copy shared -> global (the destination may be a peer GPU's memory: plain
// unicast copy, no multicast) and its group bookkeeping
__device__ __forceinline__ void bulk_store(void* gdst, const void* smem_src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;"
               ::"l"(gdst), "r"(smem_u32(smem_src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void bulk_wait_read() {
  asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
template <int N> __device__ __forceinline__ void bulk_wait() {
  asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(void* smem_dst, const Vec16& v) {
  asm volatile("st.shared.v4.b32 [%0], {%1,%2,%3,%4};"
               ::"r"(smem_u32(smem_dst)), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t* smem_dst, uint32_t cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols)
               : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
               : "memory");
}
// D[tmem] (+)= A[smem desc] * B[smem desc]
__device__ __forceinline__ void tc_mma_bf16(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread l of the warp gets lane (base + l)
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes
// with the 128-byte swizzle (what a TMA box of 64 bf16 x R rows with
// CU_TENSOR_MAP_SWIZZLE_128B writes): 8-row groups are 1024 bytes apart.
__device__ __forceinline__ uint64_t make_desc_sw128(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);   // start address, bits [0,14)
  d |= (uint64_t)1 << 16;                        // leading byte offset (unused for swizzled K-major) = 1
  d |= (uint64_t)(1024 >> 4) << 32;              // stride byte offset, bits [32,46)
  d |= (uint64_t)1 << 46;                        // descriptor version (Blackwell)
  d |= (uint64_t)2 << 61;                        // layout: SWIZZLE_128B
  return d;
}
// kind::f16 instruction descriptor: D fp32, A/B bf16, both K-major, M x N
__host__ __device__ constexpr uint32_t make_idesc_bf16(int m, int n) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

// ------------------------------------------------------------- bounded waits
struct Abort {
  volatile int* flag;     // CTA-shared: set once any wait of this CTA has failed
  const tccl_comm* comm;  // may be null (stand-alone GEMM): then only the flag is set
  uint32_t* status;       // global status words (may be null)
  uint64_t deadline;
};

__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const Abort& ab) {
  uint32_t spins = 0;
  while (!mbar_try_wait(bar, parity)) {
    if ((++spins & 255u) == 0u) {
      if (*ab.flag) return false;
      if (globaltimer() > ab.deadline) {
        *ab.flag = 1;
        if (ab.status && atomicCAS(ab.status + TCCL_ST_CODE, 0u, (uint32_t)TCCL_TIMEOUT) == 0u) {
          ab.status[TCCL_ST_BLOCK] = blockIdx.x;
          ab.status[TCCL_ST_PEER] = 0xffffffffu;
          ab.status[TCCL_ST_WHERE] = TCCL_W_MBAR;
          ab.status[TCCL_ST_SEEN] = parity;
          ab.status[TCCL_ST_WANT] = threadIdx.x;
        }
        return false;
      }
    }
  }
  return true;
}

// ------------------------------------------------------------------ mainloop
struct Shape {
  int M, N, K;
};

struct SmemLayout {
  uint8_t* a[kStages];
  uint8_t* b[kStages];
  uint64_t* full;        // [kStages]
  uint64_t* empty;       // [kStages]
  uint64_t* tmem_full;   // [2]
  uint64_t* tmem_empty;  // [2]
  uint32_t* tmem_base;
  int* abort_flag;
  uint8_t* epi[2];       // epilogue staging chunks (kEpiChunkBytes each, 128-byte aligned)
  __device__ explicit SmemLayout(uint8_t* raw) {
    uint8_t* p = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(raw) + 1023) & ~(uintptr_t)1023);
    for (int s = 0; s < kStages; ++s) {
      a[s] = p + (size_t)s * kStageBytes;
      b[s] = a[s] + kABytes;
    }
    uint64_t* bars = reinterpret_cast<uint64_t*>(p + (size_t)kStages * kStageBytes);
    full = bars;
    empty = bars + kStages;
    tmem_full = bars + 2 * kStages;
    tmem_empty = bars + 2 * kStages + 2;
    tmem_base = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 4);
    abort_flag = reinterpret_cast<int*>(tmem_base + 1);
    epi[0] = p + (size_t)kStages * kStageBytes + 256;
    epi[1] = epi[0] + kEpiChunkBytes;
  }
};

// A schedule maps the i-th tile of this CTA to (m_tile, n_tile); hooks:
//   Policy::tile(i, m_tile, n_tile)          -> false when the CTA is out of tiles
//   Policy::a_tile(m_tile, map, y)           -> which tensor map / row coordinate holds the A rows
//   Policy::before_load(m_tile, n_tile, ab)  -> runs in the producer thread before the
//                                               tile's first TMA load (wait for remote rows)
//   Policy::epilogue(m_tile, n_tile, acc_taddr, quad, lane, ab, sm)
//                                            -> runs in the 4 epilogue warps
//   Policy::epilogue_finish(quad, lane, ab)  -> once, in the epilogue warps, after the last tile
template <class Policy>
__device__ void run_mainloop(const CUtensorMap* map_b, const Shape shp, Policy& pol, const tccl_comm* comm,
                             uint64_t timeout_ns, uint64_t* trace = nullptr) {
  // `trace` (optional, this CTA's 64 words): %globaltimer stamps per tile i < 15 —
  // [4i] producer may load, [4i+1] accumulator ready, [4i+2] epilogue done; [63] kernel start
  extern __shared__ uint8_t smem_raw[];
  SmemLayout sm(smem_raw);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int num_kb = (shp.K + BK - 1) / BK;

  if (threadIdx.x == 0) {
    if (trace) trace[63] = globaltimer();
    *sm.abort_flag = 0;
    for (int s = 0; s < kStages; ++s) {
      mbar_init(sm.full + s, 1);
      mbar_init(sm.empty + s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(sm.tmem_full + i, 1);
      mbar_init(sm.tmem_empty + i, 4 * 32);
    }
    fence_barrier_init();
    tma_prefetch_desc(map_b);
  }
  if (warp == 2) {
    tmem_alloc(sm.tmem_base, kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *sm.tmem_base;
  Abort ab{sm.abort_flag, comm, comm ? comm->local + TCCL_LOCAL_STATUS : nullptr, globaltimer() + timeout_ns};

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (elect_one()) {
      uint32_t it = 0;  // k-blocks issued so far
      bool ok = true;
      int mt, nt;
      for (int i = 0; ok && pol.tile(i, mt, nt); ++i) {
        ok = pol.before_load(mt, nt, ab);
        if (trace && i < 15) trace[4 * i] = globaltimer();
        const CUtensorMap* map_a;
        int ya;
        pol.a_tile(mt, map_a, ya);
        for (int kb = 0; ok && kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          const uint32_t ph = (it / kStages) & 1;
          ok = mbar_wait(sm.empty + s, ph ^ 1, ab);
          if (!ok) break;
          mbar_arrive_expect_tx(sm.full + s, kStageBytes);
          tma_load_2d(sm.a[s], map_a, sm.full + s, kb * BK, ya);
          tma_load_2d(sm.b[s], map_b, sm.full + s, kb * BK, nt * BN);
        }
      }
      // copies in flight must land before the CTA may go away: the last kStages
      // loads issued complete their `full` barriers whether or not anyone consumes them
      const uint32_t pending = it < (uint32_t)kStages ? it : (uint32_t)kStages;
      Abort drain = ab;
      int dummy = 0;
      drain.flag = &dummy;
      drain.deadline = globaltimer() + 2000000000ull;
      for (uint32_t j = it - pending; j < it; ++j) mbar_wait(sm.full + (j % kStages), (j / kStages) & 1, drain);
    }
  } else if (warp == 1) {
    // ---------------------------------------------------------------- MMA issuer
    if (elect_one()) {
      constexpr uint32_t idesc = make_idesc_bf16(BM, BN);
      uint32_t it = 0;
      bool ok = true;
      int mt, nt;
      for (int i = 0; ok && pol.tile(i, mt, nt); ++i) {
        const int acc = i & 1;
        const uint32_t acc_ph = (i >> 1) & 1;
        ok = mbar_wait(sm.tmem_empty + acc, acc_ph ^ 1, ab);  // epilogue has drained this accumulator
        if (!ok) break;
        tc_fence_after();
        const uint32_t d = tmem_base + acc * BN;
        for (int kb = 0; ok && kb < num_kb; ++kb, ++it) {
          const int s = it % kStages;
          ok = mbar_wait(sm.full + s, (it / kStages) & 1, ab);
          if (!ok) break;
          tc_fence_after();
          const uint64_t ad = make_desc_sw128(smem_u32(sm.a[s]));
          const uint64_t bd = make_desc_sw128(smem_u32(sm.b[s]));
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            // 16 bf16 = 32 bytes further along K inside the 128-byte swizzle row: +2 in the address field
            tc_mma_bf16(d, ad + (uint64_t)(k * 2), bd + (uint64_t)(k * 2), idesc, (kb | k) ? 1u : 0u);
          }
          tc_commit(sm.empty + s);  // frees the stage when these MMAs have read it
        }
        if (ok) tc_commit(sm.tmem_full + acc);  // accumulator complete
      }
    }
  } else if (warp >= kEpiWarp0) {
    // ---------------------------------------------------------------- epilogue
    const int quad = warp - kEpiWarp0;  // == warp % 4: the TMEM lane quadrant this warp may read
    bool ok = true;
    int mt, nt;
    for (int i = 0; ok && pol.tile(i, mt, nt); ++i) {
      const int acc = i & 1;
      ok = mbar_wait(sm.tmem_full + acc, (i >> 1) & 1, ab);
      if (!ok) break;
      tc_fence_after();
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN;
      if (trace && i < 15 && quad == 0 && lane == 0) trace[4 * i + 1] = globaltimer();
      ok = pol.epilogue(mt, nt, taddr, quad, lane, ab, sm);
      if (trace && i < 15 && quad == 0 && lane == 0) trace[4 * i + 2] = globaltimer();
      tc_fence_before();
      mbar_arrive(sm.tmem_empty + acc);
    }
    pol.epilogue_finish(quad, lane, ab);
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// fp32 x 8 -> one 16-byte vector of bf16
__device__ __forceinline__ Vec16 pack8_bf16(const uint32_t* r) {
  Vec16 v;
  v.x = Acc<__nv_bfloat16>::pk(__uint_as_float(r[0]), __uint_as_float(r[1]));
  v.y = Acc<__nv_bfloat16>::pk(__uint_as_float(r[2]), __uint_as_float(r[3]));
  v.z = Acc<__nv_bfloat16>::pk(__uint_as_float(r[4]), __uint_as_float(r[5]));
  v.w = Acc<__nv_bfloat16>::pk(__uint_as_float(r[6]), __uint_as_float(r[7]));
  return v;
}

}  // namespace gemm
}  // namespace tccl
