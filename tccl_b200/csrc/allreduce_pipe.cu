// Two-shot all-reduce with the inbound and the outbound stream decoupled.
//
// In the plain two-shot kernels (collectives.cu) a thread loads (or
// multimem.ld_reduce's) a few vectors of its slice, waits for them, and stores
// (or multimem.st's) the sums to every rank: inside a warp the two directions of
// the link take turns.  Here a CTA is split into REDUCER warps, which only pull
// — they sum slice chunks into a ring of shared-memory stages — and BROADCASTER
// warps, which only push — they store finished stages to all ranks.  The two
// groups meet at mbarriers (full / empty per stage), so the reducers run up to
// `stages` chunks ahead and both directions of NVLink stay busy all the time.
//
// NVLS form: reducers issue multimem.ld_reduce (the switch sums the W copies),
// broadcasters multimem.st (the switch replicates): (1 + 1/W) S bytes per
// direction per GPU.  P2P form: reducers load the W copies and add in fp32,
// broadcasters store to every peer.
//
// As in the other two-shot kernels, slice r is read and written by rank r only,
// and a vector is written after it was read (the value travels through the
// stage), so an in-place reduction needs no barrier between the halves — only
// entry (inputs ready) and exit (results landed everywhere).  The reference has
// one all-reduce, a one-shot that pulls everything into every rank
// (triton_one_shot_all_reduce_no_128.py:35-64).
#include "gemm_tcgen05.cuh"

namespace tccl {

using gemm::Abort;
using gemm::mbar_arrive;
using gemm::mbar_init;
using gemm::mbar_wait;
using gemm::smem_u32;

constexpr int kPipeThreads = 512;
constexpr int kPipeMaxStages = 16;

__device__ __forceinline__ Vec16 ld_shared_v4(const void* p) {
  Vec16 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)) : "memory");
  return v;
}

template <typename T, int W, bool kNvls, int UR>
struct AllReduceTwoShotPipe {
  using Args = tccl_coll_args;
  static constexpr int kMaxThreads = kPipeThreads, kMinBlocks = 1;
  static constexpr int kMaxW = W ? W : TCCL_MAX_WORLD;

  static __device__ void run(const tccl_comm& c, const Args& a, int bid, int nb) {
    extern __shared__ __align__(16) uint8_t pipe_smem[];
    __shared__ uint64_t s_full[kPipeMaxStages], s_empty[kPipeMaxStages];
    __shared__ int s_abort;
    const int world = W ? W : c.world;
    const int nr_warps = (a.flags >> TCCL_F_PIPE_REDUCERS_SHIFT) & 15;  // 1..15 of the 16 warps
    const int stages = ((a.flags >> TCCL_F_PIPE_STAGES_SHIFT) & 15) + 1;
    const int NR = nr_warps * 32, NB = kPipeThreads - NR;
    const int SV = NR * UR;  // vectors per stage
    const int t = threadIdx.x;
    if (t == 0) {
      s_abort = 0;
      for (int s = 0; s < stages; ++s) {
        mbar_init(s_full + s, NR);
        mbar_init(s_empty + s, NB);
      }
      gemm::fence_barrier_init();
    }
    __syncthreads();  // the mbarriers are initialised for everybody
    Entry sync(c, a.flags, bid);
    Abort ab{&s_abort, &c, c.local + TCCL_LOCAL_STATUS, sync.deadline};
    constexpr int VPT = 16 / (int)sizeof(T);
    const uint64_t nvec = a.numel / VPT;
    const uint64_t per = (nvec + world - 1) / world;
    const uint64_t lo = min(per * (uint64_t)c.rank, nvec), n = min(lo + per, nvec) - lo;
    const uint64_t nchunks = (n + SV - 1) / SV;

    if (t < NR) {
      // ------------------------------------------------ reducers: pull and sum
      uint32_t q = 0;
      bool ok = true;
      for (uint64_t ci = bid; ci < nchunks && ok; ci += nb, ++q) {
        const int s = q % stages;
        ok = mbar_wait(s_empty + s, ((q / stages) & 1) ^ 1, ab);
        if (!ok) break;
        const uint64_t base = lo + ci * SV, end = lo + n;
        uint8_t* st = pipe_smem + (size_t)s * SV * 16;
        if (kNvls) {
          Vec16 v[UR];
#pragma unroll
          for (int u = 0; u < UR; ++u) {
            const uint64_t i = base + u * NR + t;
            if (i < end && TCCL_VIN(c, a, i)) v[u] = MultimemOps<T>::ld_reduce(reinterpret_cast<const char*>(a.mc_in) + i * 16);
          }
#pragma unroll
          for (int u = 0; u < UR; ++u) gemm::st_shared_v4(st + (size_t)(u * NR + t) * 16, v[u]);
        } else {
          Vec16 v[kMaxW][UR];
#pragma unroll
          for (int p = 0; p < kMaxW; ++p)
            if (p < world) {
#pragma unroll
              for (int u = 0; u < UR; ++u) {
                const uint64_t i = base + u * NR + t;
                if (i < end && TCCL_VIN(c, a, i)) v[p][u] = ld_peer(reinterpret_cast<const char*>(a.in[p]) + i * 16);
              }
            }
#pragma unroll
          for (int u = 0; u < UR; ++u) {
            Acc<T> acc;
            acc.zero();
            if (base + u * NR + t < end) {
#pragma unroll
              for (int p = 0; p < kMaxW; ++p)
                if (p < world) acc.add(v[p][u]);
            }
            gemm::st_shared_v4(st + (size_t)(u * NR + t) * 16, acc.pack());
          }
        }
        mbar_arrive(s_full + s);  // release: this thread's stage writes are visible to whoever acquires the phase
      }
    } else {
      // --------------------------------------------- broadcasters: push to all
      const int j = t - NR;
      uint32_t q = 0;
      bool ok = true;
      for (uint64_t ci = bid; ci < nchunks && ok; ci += nb, ++q) {
        const int s = q % stages;
        ok = mbar_wait(s_full + s, (q / stages) & 1, ab);
        if (!ok) break;
        const uint64_t base = lo + ci * SV, end = lo + n;
        const uint8_t* st = pipe_smem + (size_t)s * SV * 16;
#pragma unroll 4
        for (int k = j; k < SV; k += NB) {
          const uint64_t i = base + k;
          if (i < end && TCCL_VOUT(c, a, i)) {
            const Vec16 v = ld_shared_v4(st + (size_t)k * 16);
            if (kNvls) {
              multimem_st(reinterpret_cast<char*>(a.mc_out) + i * 16, v);
            } else {
#pragma unroll
              for (int p = 0; p < kMaxW; ++p)
                if (p < world) st_peer(reinterpret_cast<char*>(a.out_peer[p]) + i * 16, v);
            }
          }
        }
        mbar_arrive(s_empty + s);  // the stage has been read: the reducers may refill it
      }
    }
    // ragged tail (numel not a multiple of the vector width): rank 0 sums it for everybody
    const uint64_t tid = (uint64_t)bid * blockDim.x + threadIdx.x;
    if (c.rank == 0 && tid < a.numel - nvec * VPT) {
      const uint64_t e = nvec * VPT + tid;
      float sum = 0.f;
      for (int p = 0; p < world; ++p) sum += to_f32(reinterpret_cast<const volatile T*>(a.in[p])[e]);
      for (int p = 0; p < world; ++p) reinterpret_cast<volatile T*>(a.out_peer[p])[e] = from_f32<T>(sum);
    }
    sync.exit(c, a.flags, bid);
  }
};

template <typename T, int W, bool kNvls>
static int launch_pipe(const tccl_comm* comm, const tccl_coll_args* args, const tccl_launch* l, int flags) {
  const int nr = (flags >> TCCL_F_PIPE_REDUCERS_SHIFT) & 15;
  const int stages = ((flags >> TCCL_F_PIPE_STAGES_SHIFT) & 15) + 1;
  const int ur = (flags >> TCCL_F_PIPE_UNROLL_SHIFT) & 15;
  if (nr < 1 || nr > 15 || stages < 2 || stages > kPipeMaxStages || l->block != kPipeThreads) return -TCCL_EINVAL;
  const size_t smem = (size_t)stages * nr * 32 * ur * 16;
  if (smem > 200 * 1024) return -TCCL_ESIZE;
  switch (ur) {
    case 2: return launch_op<AllReduceTwoShotPipe<T, W, kNvls, 2>>(comm, args, l, smem);
    case 4: return launch_op<AllReduceTwoShotPipe<T, W, kNvls, 4>>(comm, args, l, smem);
    case 8: return launch_op<AllReduceTwoShotPipe<T, W, kNvls, 8>>(comm, args, l, smem);
    default: return -TCCL_EINVAL;
  }
}

template <typename T, bool kNvls>
static int launch_pipe_world(const tccl_comm* comm, const tccl_coll_args* args, const tccl_launch* l, int world,
                             int flags) {
  if (kNvls) return launch_pipe<T, 0, true>(comm, args, l, flags);  // the switch does the summing: W is not unrolled
  switch (world) {
    case 2: return launch_pipe<T, 2, kNvls>(comm, args, l, flags);
    case 4: return launch_pipe<T, 4, kNvls>(comm, args, l, flags);
    case 8: return launch_pipe<T, 8, kNvls>(comm, args, l, flags);
    default: return launch_pipe<T, 0, kNvls>(comm, args, l, flags);
  }
}

}  // namespace tccl

using namespace tccl;

// The pipeline's shape (reducer warps, stages, unroll) sits in bits 8.. of args->flags for the
// kernel and, identically, in bits 8.. of launch->meta for the host (in emulated mode `args`
// is a device pointer the host cannot read).
template <bool kNvls>
static int pipe_entry(const tccl_comm* comm, const tccl_coll_args* args, const tccl_launch* l) {
  const int world = l->n_emu ? l->n_emu : comm->world;
  const int dtype = l->n_emu ? (l->meta & 0xff) : args->dtype;
  const int pipe_flags = l->meta & ~0xff;
  if (l->n_emu == 0 && (args->flags & ~0xff) != pipe_flags) return -TCCL_EINVAL;
  switch (dtype) {
    case TCCL_BF16: return launch_pipe_world<__nv_bfloat16, kNvls>(comm, args, l, world, pipe_flags);
    case TCCL_F32: return launch_pipe_world<float, kNvls>(comm, args, l, world, pipe_flags);
    case TCCL_F16: return launch_pipe_world<__half, kNvls>(comm, args, l, world, pipe_flags);
    default: return -TCCL_EDTYPE;
  }
}

extern "C" int tccl_allreduce_twoshot_pipe_p2p(const tccl_comm* comm, const tccl_coll_args* args, const tccl_launch* l) {
  return pipe_entry<false>(comm, args, l);
}
extern "C" int tccl_allreduce_twoshot_pipe_nvls(const tccl_comm* comm, const tccl_coll_args* args, const tccl_launch* l) {
  return pipe_entry<true>(comm, args, l);
}
