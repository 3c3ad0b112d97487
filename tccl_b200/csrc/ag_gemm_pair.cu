// All-gather -> GEMM in ONE kernel on the CTA-pair mainloop
// (gemm_tcgen05_2cta.cuh):
//   out_r[M, N_r] = gather_src(A_src[M/W, K]) * Bt_r[N_r, K]^T
//
// What differs from the single-CTA form (ag_gemm.cu):
//  * No CTA is set aside to move data.  The four epilogue warps of EVERY CTA open
//    as data movers while the producer and MMA warps already compute on the
//    rank's own rows: in a few batches of row tiles each CTA stores its 1/grid
//    share of the shard into the gathered buffer of every rank (one multimem.st
//    per vector through the switch when NVLS is there, else one posted store per
//    peer), and the CTA that completes a batch raises the flags of its row tiles
//    on every rank.  With the whole GPU issuing, the shard is on the wire within
//    microseconds instead of trickling out of 8 CTAs for the length of the kernel,
//    and no SM is lost to the GEMM.
//  * 256 x 256 tiles on pairs of SMs (tcgen05.mma.cta_group::2).  A pair starts
//    on the rank's own rows, straight from the shard, and goes on with the remote
//    row tiles in the order they arrive; each CTA's TMA producer waits for the
//    flag of its own 128 rows and then loads them from LOCAL memory (the gathered
//    buffer) — a tensor map never covers a peer's memory.
//  * No entry barrier when the gathered buffer is the library's own: it has two
//    halves that alternate from call to call (TCCL_LOCAL_AG_SEQ).  A rank reaches
//    call n+2 only after its call n+1 consumed every peer's rows of call n+1,
//    i.e. after every peer has finished call n and stopped reading the half that
//    is being overwritten.  A caller-provided buffer keeps the barrier.
//
// The reference has no kernel of this kind: fusing a matmul with its collective is the goal its
// presentation names (presentation.pdf, slide 4: "fusing (matmul-allreduce) for overlap"); its collectives
// are stand-alone Triton kernels (triton_reduce_scatter.py:59-127, triton_all_gather.py:32-95).
#include "gemm_host.cuh"
#include "gemm_tcgen05_2cta.cuh"

namespace tccl {
namespace gemm2 {

struct alignas(64) AgGemmPairParams {
  CUtensorMap map_a_shard, map_a_full[2], map_b, map_b64;
  Shape shp;
  const char* a_shard;
  char* a_full[TCCL_MAX_WORLD];  // every rank's gathered buffer (half 0)
  char* mc_a_full;               // its multicast alias, or null
  uint64_t half_bytes;           // distance to half 1 (0: one buffer only, entry barrier)
  __nv_bfloat16* out;
  int lda_shard, lda_full, ldo;
  int tiles_n, tiles_m_per_rank;
  int swiglu;
  const int32_t* sched;  // optional: every pair's tiles in running order (see tccl_ag_gemm_args)
  int sched_stride;
  int batches;      // batches the shard's row tiles go out in (each ends in one system-scope fence)
  int ring;         // movers send destination by destination (plain stores) instead of batch by batch to all
  int movers_only;  // diagnostic (timeline tool): move the shard, compute nothing
  uint64_t* trace;  // optional: 64 words per CTA of %globaltimer stamps (see run_mainloop2); [61] kernel end
};

struct AgGemmPairPolicy {
  const tccl_comm* c;
  const AgGemmPairParams* p;
  int pair, npairs;
  uint32_t epoch;
  int parity;
  int* s_last;  // shared: whether this CTA completed a batch of the data-mover phase
  uint64_t* trace;  // this CTA's trace words, or null: [60 - 2 b] batch b stored, [59 - 2 b] batch b fenced

  __device__ __forceinline__ bool tile(int i, int& mt, int& nt, int& half) const {
    if (p->movers_only) return false;
    if (p->sched) {  // the host's plan for this pair
      if (i >= p->sched_stride) return false;
      const int32_t v = __ldg(p->sched + (size_t)pair * p->sched_stride + i);
      if (v < 0) return false;
      mt = v & 0xfff;
      nt = (v >> 12) & 0xffff;
      half = (v >> 28) & 3;
      return true;
    }
    const int t = pair + i * npairs;
    const int tm2 = p->tiles_m_per_rank / 2, tn = p->tiles_n, W = c->world;
    const int own = tm2 * tn;
    half = 0;
    if (t >= W * own) return false;
    if (t < own) {  // own rows first: no waiting
      mt = c->rank * p->tiles_m_per_rank + 2 * (t / tn);
      nt = t % tn;
      return true;
    }
    const int u = t - own;
    if (p->ring) {
      // rows arrive source by source, the previous rank's first (it sends to its next rank first)
      const int j = u / own, v = u - j * own;
      int src = c->rank - 1 - j;
      if (src < 0) src += W;
      mt = src * p->tiles_m_per_rank + 2 * (v / tn);
      nt = v % tn;
      return true;
    }
    // batches to all ranks at once: pair-row by pair-row, peers from the next rank on
    const int per_rt = (W - 1) * tn;
    const int rt2 = u / per_rt, v = u - rt2 * per_rt;
    int src = c->rank + 1 + v / tn;
    if (src >= W) src -= W;
    mt = src * p->tiles_m_per_rank + 2 * rt2;
    nt = v % tn;
    return true;
  }
  __device__ __forceinline__ void b_tile(int nt, int half, int cta, const CUtensorMap*& map, int& y) const {
    map = half ? &p->map_b64 : &p->map_b;
    // gate | up packing: a half tile is 64 gate columns (CTA 0) and the 64 matching up columns (CTA 1)
    y = (p->swiglu && half) ? nt * BN2 + cta * 128 + (half == 2 ? 64 : 0) : b_rows_default(nt, half, cta);
  }
  __device__ __forceinline__ void epilogue_finish(int, int, const Abort&) const {}
  __device__ __forceinline__ void between_tiles(int, int, const Abort&) const {}

  // Ring-ordered form of the data-mover phase: W - 1 rounds, in round j every CTA stores its share of
  // the WHOLE shard into the gathered buffer of rank (me + j) only, with plain stores.  Every round is
  // a permutation (each GPU sends to one peer and receives from one), so a receiver has the previous
  // rank's rows after one round at full link rate, the rows of the rank before that after two, ... —
  // its pairs start on remote tiles after 1 / (W - 1) of the transfer instead of after half of it,
  // and W - 1 copies on the wire cost no more inbound bytes than the switch's multicast (which also
  // returns every row to its sender).  One system-scope fence per round; the CTA that completes a
  // round raises the flags of all the shard's row tiles at that round's destination.  The own rows go
  // into the own gathered buffer last (nobody waits for them: the GEMM reads them from the shard).
  __device__ void ring_movers(int t, uint32_t lo, uint32_t hi, int vec_per_row, int rows_per_rank, uint64_t hoff,
                              int nb) const {
    const int W = c->world, me = c->rank, tm = p->tiles_m_per_rank;
    constexpr int U = 8;
    for (int j = 1; j <= W; ++j) {
      const int dst = (me + j) % W;  // j == W: the own buffer
      char* base = p->a_full[dst] + hoff;
      for (int rt = 0; rt < tm; ++rt) {
        for (uint32_t i0 = lo + t; i0 < hi; i0 += U * 128) {
          Vec16 v[U];
          size_t off[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint32_t i = i0 + u * 128;
            if (i < hi) {
              const int row = rt * 128 + i / vec_per_row, col = (i % vec_per_row) * 8;
              v[u] = ld_peer(p->a_shard + ((size_t)row * p->lda_shard + col) * 2);
              off[u] = ((size_t)(me * rows_per_rank + row) * p->lda_full + col) * 2;
            }
          }
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (i0 + u * 128 < hi) st_peer(base + off[u], v[u]);
        }
      }
      if (j == W) break;  // local copy: no flags
      asm volatile("bar.sync 1, 128;" ::: "memory");  // this CTA's share of the round is stored
      if (t == 0) {
        if (trace && j <= 2) trace[62 - 2 * j] = globaltimer();
        fence_acq_rel_sys();
        if (trace && j <= 2) trace[61 - 2 * j] = globaltimer();
        const uint32_t done = atomicAdd(c->local + TCCL_LOCAL_AGCNT + (j - 1), 1u);
        *s_last = (done == (uint32_t)nb - 1u);
        if (*s_last) {
          c->local[TCCL_LOCAL_AGCNT + (j - 1)] = 0u;
          fence_acq_rel_sys();
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*reinterpret_cast<volatile int*>(s_last)) {
        for (int k = t; k < tm; k += 128)
          st_release_sys(c->flags[dst] + TCCL_FLAG_AG + me * TCCL_MAX_ROW_TILES + k, epoch);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");  // s_last is rewritten by the next round
    }
  }

  // The data-mover phase, run by the four epilogue warps of EVERY CTA while the producer and MMA
  // warps already work on the rank's own rows (the first accumulator is tens of microseconds
  // away).  The shard's row tiles go out in `batches` batches; in each, CTA b stores its 1/grid share of
  // every row tile into the gathered buffer of every rank, and the CTA that completes a batch
  // raises the flags of its row tiles on every rank.  One system-scope fence per batch: a fence
  // per row tile would cost a switch round trip each and hold back the whole kernel.
  __device__ void epilogue_begin(int quad, int lane, const Abort&) const {
    const int W = c->world, me = c->rank, nb = 2 * npairs, bid = blockIdx.x;
    const int t = quad * 32 + lane;
    const int vec_per_row = p->shp.K / 8;
    const int rows_per_rank = p->tiles_m_per_rank * 128;
    const uint64_t hoff = (uint64_t)parity * p->half_bytes;
    const uint32_t nvec = 128u * (uint32_t)vec_per_row;
    const uint32_t per = (nvec + nb - 1) / nb;
    const uint32_t lo = min(per * (uint32_t)bid, nvec), hi = min(lo + per, nvec);
    if (p->ring) {
      ring_movers(t, lo, hi, vec_per_row, rows_per_rank, hoff, nb);
      return;
    }
    const int nbatch = max(1, min(p->batches, p->tiles_m_per_rank));
    for (int b = 0; b < nbatch; ++b) {
      const int rt0 = b * p->tiles_m_per_rank / nbatch, rt1 = (b + 1) * p->tiles_m_per_rank / nbatch;
      for (int rt = rt0; rt < rt1; ++rt) {
        constexpr int U = 8;
        for (uint32_t i0 = lo + t; i0 < hi; i0 += U * 128) {
          Vec16 v[U];
          size_t dst[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint32_t i = i0 + u * 128;
            if (i < hi) {
              const int row = rt * 128 + i / vec_per_row, col = (i % vec_per_row) * 8;
              v[u] = ld_peer(p->a_shard + ((size_t)row * p->lda_shard + col) * 2);
              dst[u] = hoff + ((size_t)(me * rows_per_rank + row) * p->lda_full + col) * 2;
            }
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            if (i0 + u * 128 < hi) {
              if (p->mc_a_full) {
                multimem_st(p->mc_a_full + dst[u], v[u]);
              } else {
                for (int q = 0; q < W; ++q) st_peer(p->a_full[q] + dst[u], v[u]);
              }
            }
          }
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");  // this CTA's share of the batch is stored
      if (t == 0) {
        if (trace && b < 2) trace[60 - 2 * b] = globaltimer();
        fence_acq_rel_sys();
        if (trace && b < 2) trace[59 - 2 * b] = globaltimer();
        const uint32_t done = atomicAdd(c->local + TCCL_LOCAL_AGCNT + b, 1u);
        *s_last = (done == (uint32_t)nb - 1u);
        if (*s_last) {
          c->local[TCCL_LOCAL_AGCNT + b] = 0u;
          fence_acq_rel_sys();
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*reinterpret_cast<volatile int*>(s_last)) {
        for (int k = t; k < W * (rt1 - rt0); k += 128)
          st_release_sys(c->flags[k % W] + TCCL_FLAG_AG + me * TCCL_MAX_ROW_TILES + rt0 + k / W, epoch);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");  // s_last is rewritten by the next batch
    }
  }

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
      y = (mt - src * p->tiles_m_per_rank) * 128;
    } else {
      map = &p->map_a_full[parity];
      y = mt * 128;
    }
  }
  __device__ __forceinline__ bool epilogue(int mt, int nt, int col_lo, int ncols, uint32_t taddr, int quad, int lane,
                                           const Abort&, const Smem2&) const {
    const int row = mt * 128 + quad * 32 + lane;
    __nv_bfloat16* crow = p->out + (size_t)row * p->ldo;
    if (p->swiglu) {
      // every 256-wide tile holds 128 gate columns followed by the 128 matching up columns; a half
      // tile's accumulator holds 64 of each (see b_tile)
      const int hw = ncols / 2;
#pragma unroll 1
      for (int cg = 0; cg < hw / 32; ++cg) {
        uint32_t g[32], u[32];
        tmem_ld_32x32(taddr + cg * 32, g);
        tmem_ld_32x32(taddr + hw + cg * 32, u);
        tmem_ld_wait();
        const int col0 = nt * (BN2 / 2) + col_lo / 2 + cg * 32;
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
    for (int cg = 0; cg < ncols / 32; ++cg) {  // a half tile's 128 columns sit at the start of the accumulator
      uint32_t r[32];
      tmem_ld_32x32(taddr + cg * 32, r);
      tmem_ld_wait();
      const int col0 = nt * BN2 + col_lo + cg * 32;
      if (row < p->shp.M) {
#pragma unroll
        for (int v = 0; v < 4; ++v)
          if (col0 + v * 8 < p->shp.N) st_local(crow + col0 + v * 8, pack8_bf16(r + v * 8));
      }
    }
    return true;
  }
};

__device__ __forceinline__ void ag_gemm_pair_body(const tccl_comm& c, const AgGemmPairParams& p, int bid, int nb) {
  const uint32_t epoch = c.local[TCCL_LOCAL_TILE_EPOCH] + 1u;
  const int parity = p.half_bytes ? (int)(c.local[TCCL_LOCAL_AG_SEQ] & 1u) : 0;
  if (!p.half_bytes) {
    // one buffer only: every rank must be done reading it from the previous call
    barrier_p2p(c, bid, globaltimer() + c.timeout_ns);
  }
  __shared__ int s_last;
  AgGemmPairPolicy pol;
  pol.s_last = &s_last;
  pol.trace = p.trace ? p.trace + (size_t)bid * 64 : nullptr;
  pol.c = &c;
  pol.p = &p;
  pol.pair = bid >> 1;
  pol.npairs = nb >> 1;
  pol.epoch = epoch;
  pol.parity = parity;
  if (threadIdx.x == 0) {
    tma_prefetch_desc(&p.map_a_shard);
    tma_prefetch_desc(&p.map_a_full[parity]);
    tma_prefetch_desc(&p.map_b);
    tma_prefetch_desc(&p.map_b64);
  }
  run_mainloop2(p.shp, pol, &c, c.timeout_ns, p.trace ? p.trace + (size_t)bid * 64 : nullptr);
  __syncthreads();
  if (threadIdx.x == 0) {
    if (p.trace) p.trace[(size_t)bid * 64 + 61] = globaltimer();
    __threadfence();
    const uint32_t done = atomicAdd(c.local + TCCL_LOCAL_SCHED, 1u);
    if (done == (uint32_t)nb - 1u) {
      c.local[TCCL_LOCAL_SCHED] = 0u;
      c.local[TCCL_LOCAL_AG_SEQ] += 1u;
      c.local[TCCL_LOCAL_TILE_EPOCH] = epoch;
    }
  }
}

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
ag_gemm_pair_kernel(const __grid_constant__ tccl_comm comm, const __grid_constant__ AgGemmPairParams p) {
  ag_gemm_pair_body(comm, p, blockIdx.x, gridDim.x);
}
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
ag_gemm_pair_kernel_emu(const tccl_comm* comms, const AgGemmPairParams* ps) {
  ag_gemm_pair_body(comms[blockIdx.y], ps[blockIdx.y], blockIdx.x, gridDim.x);
}

static int fill_params(AgGemmPairParams* p, const tccl_ag_gemm_args* g, int world, int rank, uint64_t half_bytes) {
  if (g->m <= 0 || g->n <= 0 || g->k <= 0) return -TCCL_EINVAL;
  if ((g->lda_shard % 8) || (g->lda_full % 8) || (g->ldb % 8) || (g->ldo % 8) || (g->k % 8) || (g->n % 8))
    return -TCCL_EALIGN;
  if (g->m % (world * 256)) return -TCCL_ESIZE;  // whole 256-row pair tiles per rank
  if (((uintptr_t)g->a_shard | (uintptr_t)g->bt | (uintptr_t)g->out | (uintptr_t)g->a_full[rank] | half_bytes) & 15)
    return -TCCL_EALIGN;
  const int rows = g->m / world;
  int rc = make_tmap_bf16_kmajor(&p->map_a_shard, g->a_shard, rows, g->k, g->lda_shard, 128);
  if (rc) return rc;
  for (int h = 0; h < 2; ++h) {
    const char* base = reinterpret_cast<const char*>(g->a_full[rank]) + (h ? half_bytes : 0);
    rc = make_tmap_bf16_kmajor(&p->map_a_full[h], base, g->m, g->k, g->lda_full, 128);
    if (rc) return rc;
  }
  rc = make_tmap_bf16_kmajor(&p->map_b, g->bt, g->n, g->k, g->ldb, 128);
  if (rc) return rc;
  rc = make_tmap_bf16_kmajor(&p->map_b64, g->bt, g->n, g->k, g->ldb, 64);  // half tiles: 64 rows of Bt per CTA
  if (rc) return rc;
  p->sched = g->sched;
  p->sched_stride = g->sched_stride;
  if (g->sched && g->sched_stride <= 0) return -TCCL_EINVAL;
  p->shp = Shape{g->m, g->n, g->k};
  p->a_shard = reinterpret_cast<const char*>(g->a_shard);
  for (int q = 0; q < TCCL_MAX_WORLD; ++q) p->a_full[q] = reinterpret_cast<char*>(g->a_full[q]);
  p->mc_a_full = reinterpret_cast<char*>(g->mc_a_full);
  p->half_bytes = half_bytes;
  p->out = reinterpret_cast<__nv_bfloat16*>(g->out);
  p->lda_shard = g->lda_shard;
  p->lda_full = g->lda_full;
  p->ldo = g->ldo;
  p->tiles_n = (g->n + BN2 - 1) / BN2;
  p->tiles_m_per_rank = rows / 128;
  p->swiglu = g->swiglu;
  p->batches = g->comm_ctas > 0 ? g->comm_ctas : 2;
  p->movers_only = (g->lsu_movers & 2) != 0;
  p->ring = (g->lsu_movers & 4) != 0;
  p->trace = reinterpret_cast<uint64_t*>(g->trace);
  if (g->swiglu && (g->n % BN2)) return -TCCL_ESIZE;  // whole gate|up tiles only
  if (p->tiles_m_per_rank > TCCL_MAX_ROW_TILES) return -TCCL_ESIZE;
  return 0;
}

}  // namespace gemm2
}  // namespace tccl

using namespace tccl::gemm;
using namespace tccl::gemm2;

extern "C" uint64_t tccl_ag_gemm_pair_param_bytes(void) { return sizeof(AgGemmPairParams); }

// Same calling convention as tccl_allgather_gemm, except that every CTA moves data first: comm_ctas of
// the arguments is the number of batches the shard goes out in (0 = 2); lsu_movers is a set of bits:
// 2 = the diagnostic "move only", 4 = ring-ordered movers (ring_movers above).  `half_bytes`: distance in bytes from a_full[q] to the second
// half of every rank's gathered buffer, or 0 when there is only one buffer (then the kernel opens
// with a barrier).  l->grid must be even.
extern "C" int tccl_allgather_gemm_pair(const tccl_comm* comm, const tccl_ag_gemm_args* args, void* dev_params,
                                        uint64_t half_bytes, const tccl_launch* l) {
  cudaStream_t s = reinterpret_cast<cudaStream_t>(l->stream);
  if (l->grid < 2 || (l->grid & 1)) return -TCCL_EINVAL;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(ag_gemm_pair_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem2);
    if (e == cudaSuccess)
      e = cudaFuncSetAttribute(ag_gemm_pair_kernel_emu, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem2);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  if (l->n_emu == 0) {
    AgGemmPairParams p;
    int rc = fill_params(&p, args, comm->world, comm->rank, half_bytes);
    if (rc) return rc;
    ag_gemm_pair_kernel<<<l->grid, kThreads, kSmem2, s>>>(*comm, p);
    return (int)cudaGetLastError();
  }
  const int W = l->n_emu;
  if (W < 1 || W > TCCL_MAX_WORLD || !dev_params || ((uintptr_t)dev_params & 63)) return -TCCL_EINVAL;
  AgGemmPairParams ps[TCCL_MAX_WORLD];
  for (int r = 0; r < W; ++r) {
    int rc = fill_params(&ps[r], &args[r], W, r, half_bytes);
    if (rc) return rc;
  }
  cudaError_t e = cudaMemcpyAsync(dev_params, ps, sizeof(AgGemmPairParams) * W, cudaMemcpyHostToDevice, s);
  if (e != cudaSuccess) return (int)e;
  const AgGemmPairParams* dps = reinterpret_cast<const AgGemmPairParams*>(dev_params);
  return launch_pairs_emulated((const void*)ag_gemm_pair_kernel_emu, l->grid, W, kSmem2, s, (const void*)&comm,
                               (const void*)&dps);
}
