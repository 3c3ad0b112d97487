// Barriers and the flat (NVSwitch-uniform) data collectives: one-shot and
// two-shot all-reduce, all-gather, reduce-scatter, each as a P2P load/store
// kernel and as an NVLS (multimem) kernel.  One kernel launch per collective.
//
// Reference counterparts: barrier_test_kernel (triton_barrier.py:145-151),
// one_shot_all_reduce_kernel (triton_one_shot_all_reduce_no_128.py:35-64),
// one_shot_all_gather_kernel (triton_all_gather.py:32-63),
// one_shot_reduce_scatter_kernel (triton_reduce_scatter.py:59-92).  Differences
// by design: 128-bit accesses everywhere, fp32 accumulation with one rounding,
// a fixed summation order (rank 0..W-1) so that every rank computes the same
// bits, an exit barrier so that a caller may overwrite its input as soon as the
// kernel is done, grids sized for 148 SMs instead of a 24-CTA cap, and bounded
// waits.
#include "common.cuh"

namespace tccl {

template <typename T> struct VecOf { static constexpr int n = 16 / (int)sizeof(T); };

// ------------------------------------------------------------------ barriers
struct BarrierP2POp {
  using Args = tccl_barrier_args;
  static constexpr int kMaxThreads = 1024, kMinBlocks = 1;
  static __device__ void run(const tccl_comm& c, const Args& a, int bid, int) {
    const uint64_t deadline = globaltimer() + c.timeout_ns;
    for (int i = 0; i < a.rounds; ++i) barrier_p2p(c, bid, deadline);
  }
};
struct BarrierNvlsOp {
  using Args = tccl_barrier_args;
  static constexpr int kMaxThreads = 1024, kMinBlocks = 1;
  static __device__ void run(const tccl_comm& c, const Args& a, int bid, int) {
    const uint64_t deadline = globaltimer() + c.timeout_ns;
    for (int i = 0; i < a.rounds; ++i) barrier_nvls(c, bid, deadline);
  }
};

// Self-resetting CAS barrier on externally owned signal pads laid out
// [block][world] — the protocol of the reference's blockwise_barrier
// (triton_barrier.py:89-118): thread t posts 0->1 into rank t's slot
// [block][my rank] (release) and consumes 1->0 from the local slot [block][t]
// (acquire, on the consuming operation itself rather than on trailing loads).
// The pads are all zero again when every rank has returned.
struct BarrierCasOp {
  using Args = tccl_pads_args;
  static constexpr int kMaxThreads = 1024, kMinBlocks = 1;
  static __device__ void run(const tccl_comm& c, const Args& a, int bid, int) {
    const uint64_t deadline = globaltimer() + c.timeout_ns;
    __syncthreads();
    const int t = threadIdx.x;
    if (t < c.world) {
      uint32_t* send = a.pads[t] + bid * c.world + c.rank;
      uint32_t* recv = a.pads[c.rank] + bid * c.world + t;
      uint32_t spins = 0;
      bool ok = true;
      while (cas_release_sys(send, 0u, 1u) != 0u) {
        if ((++spins & 15u) == 0u && (aborted(c) || globaltimer() > deadline)) {
          if (!aborted(c)) record_failure(c, TCCL_TIMEOUT, t, TCCL_W_CAS_SEND, 1u, 0u);
          ok = false;
          break;
        }
      }
      while (ok && cas_acquire_sys(recv, 1u, 0u) != 1u) {
        if ((++spins & 15u) == 0u && (aborted(c) || globaltimer() > deadline)) {
          if (!aborted(c)) record_failure(c, TCCL_TIMEOUT, t, TCCL_W_CAS_WAIT, 0u, 1u);
          break;
        }
      }
    }
    __syncthreads();
  }
};

// Waits on a flag word that nothing ever sets; the wait runs out after
// timeout_ns and the status records it.  Only for testing the failure path.
struct WaitNeverOp {
  using Args = tccl_barrier_args;
  static constexpr int kMaxThreads = 1024, kMinBlocks = 1;
  static __device__ void run(const tccl_comm& c, const Args&, int bid, int) {
    const uint64_t deadline = globaltimer() + c.timeout_ns;
    if (threadIdx.x == 0)
      wait_reach(c.flags[c.rank] + TCCL_FLAG_LL + (bid & 1023), 0x7fffffffu, c, deadline, c.rank, TCCL_W_SIGNAL);
    __syncthreads();
  }
};

// --------------------------------------------------------------- helper pieces
template <int W> struct WorldOf {
  static __device__ __forceinline__ int get(const tccl_comm&) { return W; }
};
template <> struct WorldOf<0> {
  static __device__ __forceinline__ int get(const tccl_comm& c) { return c.world; }
};

template <typename T>
__device__ __forceinline__ const char* vptr(const void* base, uint64_t vec) {
  return reinterpret_cast<const char*>(base) + vec * 16;
}
template <typename T> __device__ __forceinline__ char* vptr(void* base, uint64_t vec) {
  return reinterpret_cast<char*>(base) + vec * 16;
}

// Loop shape shared by the data kernels: in one sweep the grid covers one
// contiguous window of nb * blockDim.x * U vectors (CTA b owns the b-th
// blockDim.x * U slab of it, thread t the vectors t, t + blockDim.x, ... of the
// slab), then the window advances.  All CTAs of all GPUs therefore stream
// through the same few megabytes at a time, which keeps DRAM pages and TLB
// entries hot on the GPUs being read; a plain grid-stride loop scatters each
// thread's U accesses megabytes apart.
#define TCCL_FOR_SLABS(U, n, bid, nb, i0)                                           \
  for (uint64_t i0 = (uint64_t)(bid) * blockDim.x * (U) + threadIdx.x; i0 < (n);    \
       i0 += (uint64_t)(nb) * blockDim.x * (U))

// ---------------------------------------------------- one-shot all-reduce, P2P
// out[i] = sum_r in_r[i]; every rank pulls all W copies (W-1 over NVLink).
template <typename T, int W>
struct AllReduceOneShotP2P {
  using Args = tccl_coll_args;
  // one rank: the reduction is a copy; keep it lean so two CTAs fit an SM
  static constexpr int kMaxThreads = 512, kMinBlocks = W == 1 ? 2 : 1;
  static constexpr int kMaxW = W ? W : TCCL_MAX_WORLD;
  static constexpr int U = W == 1 ? 8 : ((W == 0 || W >= 8) ? 2 : 4);  // vectors per thread per pass
  static __device__ void run(const tccl_comm& c, const Args& a, int bid, int nb) {
    Entry sync(c, a.flags, bid);
    const int world = WorldOf<W>::get(c);
    constexpr int VPT = VecOf<T>::n;
    const uint64_t nvec = a.numel / VPT;
    const uint64_t bs = blockDim.x;
    TCCL_FOR_SLABS(U, nvec, bid, nb, i0) {
      Vec16 v[kMaxW][U];
#pragma unroll
      for (int p = 0; p < kMaxW; ++p)
        if (p < world) {
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (i0 + u * bs < nvec && TCCL_VIN(c, a, i0 + u * bs)) v[p][u] = ld_peer(vptr<T>(a.in[p], i0 + u * bs));
        }
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * bs < nvec && TCCL_VOUT(c, a, i0 + u * bs)) {
          if (W == 1) {  // nothing to add: stream the bits through
            st_local_cs(vptr<T>(a.out, i0 + u * bs), v[0][u]);
            continue;
          }
          Acc<T> acc;
          acc.zero();
#pragma unroll
          for (int p = 0; p < kMaxW; ++p)
            if (p < world) acc.add(v[p][u]);
          st_local(vptr<T>(a.out, i0 + u * bs), acc.pack());
        }
    }
    // ragged tail (numel not a multiple of the vector width)
    const uint64_t tid = (uint64_t)bid * blockDim.x + threadIdx.x;
    if (tid < a.numel - nvec * VPT) {
      const uint64_t e = nvec * VPT + tid;
      float s = 0.f;
      for (int p = 0; p < world; ++p) s += to_f32(reinterpret_cast<const volatile T*>(a.in[p])[e]);
      reinterpret_cast<T*>(a.out)[e] = from_f32<T>(s);
    }
    sync.exit(c, a.flags, bid);
  }
};

// --------------------------------------------------- one-shot all-reduce, NVLS
// out[i] = multimem.ld_reduce(mc_in[i]): the switch sums the W copies.
template <typename T, int W>
struct AllReduceOneShotNvls {
  using Args = tccl_coll_args;
  static constexpr int kMaxThreads = 512, kMinBlocks = 1;
  static constexpr int U = 4;
  static __device__ void run(const tccl_comm& c, const Args& a, int bid, int nb) {
    Entry sync(c, a.flags, bid);
    const int world = WorldOf<W>::get(c);
    constexpr int VPT = VecOf<T>::n;
    const uint64_t nvec = a.numel / VPT;
    const uint64_t bs = blockDim.x;
    TCCL_FOR_SLABS(U, nvec, bid, nb, i0) {
      Vec16 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * bs < nvec && TCCL_VIN(c, a, i0 + u * bs)) v[u] = MultimemOps<T>::ld_reduce(vptr<T>(a.mc_in, i0 + u * bs));
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * bs < nvec && TCCL_VOUT(c, a, i0 + u * bs)) st_local(vptr<T>(a.out, i0 + u * bs), v[u]);
    }
    const uint64_t tid = (uint64_t)bid * blockDim.x + threadIdx.x;
    if (tid < a.numel - nvec * VPT) {
      const uint64_t e = nvec * VPT + tid;
      float s = 0.f;
      for (int p = 0; p < world; ++p) s += to_f32(reinterpret_cast<const volatile T*>(a.in[p])[e]);
      reinterpret_cast<T*>(a.out)[e] = from_f32<T>(s);
    }
    sync.exit(c, a.flags, bid);
  }
};

// --------------------------------------------- one-shot all-reduce, push variant
// Latency path for small messages.  Every rank stores its input into slot
// [half][rank] of every rank's small-message region (posted stores, or one
// multimem.st), then ONE barrier both publishes the data and tells everybody it
// is there, and each rank sums the W slots out of its OWN memory.  Compared with
// the pull variant this drops a barrier round and replaces the peer-load round
// trip by local loads.  The input does not have to live in symmetric memory.
//
// No exit barrier is needed because the two halves of the region alternate from
// call to call.  The half is the low bit of a per-communicator count of completed
// push calls (TCCL_LOCAL_PUSH_SEQ, advanced by the last CTA of each launch), and
// the slot layout is fixed: half h starts at h * ll_bytes / 2 and rank r's slot at
// r * push_slot_bytes, whatever the message size or the grid.  A rank can start
// call n+2 (same half as call n) only after its call n+1 has completed, i.e. after
// a barrier of call n+1 that every peer has reached, and a peer reaches call n+1
// only after its kernel of call n, including the local sum, has finished.  So the
// bytes being overwritten are never still being read, also when consecutive
// calls differ in size or in grid.
__host__ __device__ __forceinline__ uint64_t push_slot_bytes(uint64_t ll_bytes, int world) {
  return (ll_bytes / 2 / (uint64_t)world) & ~(uint64_t)15;
}

template <typename T, int W, bool kNvls>
struct AllReduceOneShotPush {
  using Args = tccl_coll_args;
  static constexpr int kMaxThreads = 512, kMinBlocks = 1;
  static constexpr int kMaxW = W ? W : TCCL_MAX_WORLD;
  static constexpr int U = 2;
  static __device__ void run(const tccl_comm& c, const Args& a, int bid, int nb) {
    const uint64_t deadline = globaltimer() + c.timeout_ns;
    const int world = WorldOf<W>::get(c);
    constexpr int VPT = VecOf<T>::n;
    const uint64_t nvec = a.numel / VPT;  // the host guarantees a whole number of vectors that fits a slot
    const uint64_t slot = push_slot_bytes(c.ll_bytes, world);
    const uint64_t bs = blockDim.x;
    const bool nvls_bar = (a.flags & TCCL_F_NVLS_BARRIER) != 0;
    // stable for the whole launch: only this launch's last CTA advances it, on its way out
    const uint32_t seq = ld_relaxed_sys(c.local + TCCL_LOCAL_PUSH_SEQ);
    const uint64_t base = c.stage_bytes + (uint64_t)(seq & 1u) * (c.ll_bytes / 2);
    const char* src = reinterpret_cast<const char*>(a.in[c.rank]);
    const uint64_t mine = base + (uint64_t)c.rank * slot;
    TCCL_FOR_SLABS(U, nvec, bid, nb, i0) {
#pragma unroll
      for (int u = 0; u < U; ++u) {
        const uint64_t i = i0 + u * bs;
        if (i < nvec && TCCL_VIN(c, a, i) && TCCL_IN_BOUNDS(c, i * 16, 16, slot, TCCL_W_INDEX_OUT)) {
          const Vec16 v = ld_peer(src + i * 16);
          if (kNvls) {
            multimem_st(c.mc_stage + mine + i * 16, v);
          } else {
#pragma unroll
            for (int p = 0; p < kMaxW; ++p)
              if (p < world) st_peer(c.stage[p] + mine + i * 16, v);
          }
        }
      }
    }
    barrier_any(c, bid, deadline, nvls_bar);  // data of all ranks for this CTA's slabs has landed here
    const char* local = c.stage[c.rank] + base;
    TCCL_FOR_SLABS(U, nvec, bid, nb, i0) {
      Vec16 v[kMaxW][U];
#pragma unroll
      for (int p = 0; p < kMaxW; ++p)
        if (p < world) {
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (i0 + u * bs < nvec) v[p][u] = ld_peer(local + (uint64_t)p * slot + (i0 + u * bs) * 16);
        }
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * bs < nvec && TCCL_VOUT(c, a, i0 + u * bs)) {
          Acc<T> acc;
          acc.zero();
#pragma unroll
          for (int p = 0; p < kMaxW; ++p)
            if (p < world) acc.add(v[p][u]);
          st_local(vptr<T>(a.out, i0 + u * bs), acc.pack());
        }
    }
    // the last CTA of this rank to finish flips the half for the next push call
    __syncthreads();
    if (threadIdx.x == 0) {
      __threadfence();
      const uint32_t done = atomicAdd(c.local + TCCL_LOCAL_PUSH_DONE, 1u);
      if (done == (uint32_t)nb - 1u) {
        c.local[TCCL_LOCAL_PUSH_DONE] = 0u;
        st_relaxed_sys(c.local + TCCL_LOCAL_PUSH_SEQ, seq + 1u);
      }
    }
  }
};

// ---------------------------------------------------- two-shot all-reduce, P2P
// Rank r sums vector slice r of all W inputs and writes the result straight
// into slice r of every rank's destination (`out_peer`; the inputs themselves
// when the reduction is in place).  A slice is read and written by its owner
// only, and each vector is written by the thread that read it, so no barrier
// is needed between the two halves — only entry (inputs ready) and exit
// (results landed everywhere).
template <typename T, int W>
struct AllReduceTwoShotP2P {
  using Args = tccl_coll_args;
  static constexpr int kMaxThreads = 512, kMinBlocks = 1;
  static constexpr int kMaxW = W ? W : TCCL_MAX_WORLD;
  static constexpr int U = (W == 0 || W >= 8) ? 2 : 4;
  static __device__ void run(const tccl_comm& c, const Args& a, int bid, int nb) {
    Entry sync(c, a.flags, bid);
    const int world = WorldOf<W>::get(c);
    constexpr int VPT = VecOf<T>::n;
    const uint64_t nvec = a.numel / VPT;
    const uint64_t per = (nvec + world - 1) / world;
    const uint64_t lo = min(per * (uint64_t)c.rank, nvec), n = min(lo + per, nvec) - lo;
    const uint64_t bs = blockDim.x;
    TCCL_FOR_SLABS(U, n, bid, nb, i0) {
      Vec16 v[kMaxW][U];
#pragma unroll
      for (int p = 0; p < kMaxW; ++p)
        if (p < world) {
#pragma unroll
          for (int u = 0; u < U; ++u)
            if (i0 + u * bs < n && TCCL_VIN(c, a, lo + i0 + u * bs)) v[p][u] = ld_peer(vptr<T>(a.in[p], lo + i0 + u * bs));
        }
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * bs < n && TCCL_VOUT(c, a, lo + i0 + u * bs)) {
          Acc<T> acc;
          acc.zero();
#pragma unroll
          for (int p = 0; p < kMaxW; ++p)
            if (p < world) acc.add(v[p][u]);
          const Vec16 r = acc.pack();
#pragma unroll
          for (int p = 0; p < kMaxW; ++p)
            if (p < world) st_peer(vptr<T>(a.out_peer[p], lo + i0 + u * bs), r);
        }
    }
    const uint64_t tid = (uint64_t)bid * blockDim.x + threadIdx.x;
    if (c.rank == 0 && tid < a.numel - nvec * VPT) {
      const uint64_t e = nvec * VPT + tid;
      float s = 0.f;
      for (int p = 0; p < world; ++p) s += to_f32(reinterpret_cast<const volatile T*>(a.in[p])[e]);
      for (int p = 0; p < world; ++p) reinterpret_cast<volatile T*>(a.out_peer[p])[e] = from_f32<T>(s);
    }
    sync.exit(c, a.flags, bid);
  }
};

// --------------------------------------------------- two-shot all-reduce, NVLS
// Rank r ld_reduces slice r through the switch and multimem.st's the sum to
// slice r of every rank's destination.  Per GPU about (1 + 1/W) S bytes in and
// out instead of 2 (W-1)/W S in for the P2P form.
template <typename T, int W>
struct AllReduceTwoShotNvls {
  using Args = tccl_coll_args;
  static constexpr int kMaxThreads = 512, kMinBlocks = 1;
  static constexpr int U = 8;
  static __device__ void run(const tccl_comm& c, const Args& a, int bid, int nb) {
    Entry sync(c, a.flags, bid);
    const int world = WorldOf<W>::get(c);
    constexpr int VPT = VecOf<T>::n;
    const uint64_t nvec = a.numel / VPT;
    const uint64_t per = (nvec + world - 1) / world;
    const uint64_t lo = min(per * (uint64_t)c.rank, nvec), n = min(lo + per, nvec) - lo;
    const uint64_t bs = blockDim.x;
    TCCL_FOR_SLABS(U, n, bid, nb, i0) {
      Vec16 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * bs < n && TCCL_VIN(c, a, lo + i0 + u * bs)) v[u] = MultimemOps<T>::ld_reduce(vptr<T>(a.mc_in, lo + i0 + u * bs));
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * bs < n && TCCL_VOUT(c, a, lo + i0 + u * bs)) multimem_st(vptr<T>(a.mc_out, lo + i0 + u * bs), v[u]);
    }
    const uint64_t tid = (uint64_t)bid * blockDim.x + threadIdx.x;
    if (c.rank == 0 && tid < a.numel - nvec * VPT) {
      const uint64_t e = nvec * VPT + tid;
      float s = 0.f;
      for (int p = 0; p < world; ++p) s += to_f32(reinterpret_cast<const volatile T*>(a.in[p])[e]);
      for (int p = 0; p < world; ++p) reinterpret_cast<volatile T*>(a.out_peer[p])[e] = from_f32<T>(s);
    }
    sync.exit(c, a.flags, bid);
  }
};

// ------------------------------------------------------------ all-gather, pull
// out[p][i] = in_p[i]; the peer order starts at the own rank and every CTA
// walks it from a different offset so that the W-1 streams spread over peers.
template <typename T, int W>
struct AllGatherPullP2P {
  using Args = tccl_coll_args;
  static constexpr int kMaxThreads = 512, kMinBlocks = 1;
  static constexpr int U = 8;
  static __device__ void run(const tccl_comm& c, const Args& a, int bid, int nb) {
    Entry sync(c, a.flags, bid);
    const int world = WorldOf<W>::get(c);
    constexpr int VPT = VecOf<T>::n;
    const uint64_t nvec = a.numel / VPT;
    const uint64_t bs = blockDim.x;
    const uint64_t nthr = (uint64_t)nb * blockDim.x;
    const uint64_t tid = (uint64_t)bid * blockDim.x + threadIdx.x;
    if ((a.numel * sizeof(T)) & 15) {
      // shard size not a multiple of 16 bytes: the output slots of ranks >= 1 are
      // not vector aligned, so copy element by element
      for (int k = 0; k < world; ++k) {
        const int p = (c.rank + k + bid) % world;
        const volatile T* src = reinterpret_cast<const volatile T*>(a.in[p]);
        T* dst = reinterpret_cast<T*>(a.out) + (uint64_t)p * a.numel;
        for (uint64_t e = tid; e < a.numel; e += nthr) dst[e] = src[e];
      }
      sync.exit(c, a.flags, bid);
      return;
    }
    for (int k = 0; k < world; ++k) {
      const int p = (c.rank + k + bid) % world;
      const void* src = a.in[p];
      char* dst = reinterpret_cast<char*>(a.out) + (uint64_t)p * a.numel * sizeof(T);
      TCCL_FOR_SLABS(U, nvec, bid, nb, i0) {
        Vec16 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i0 + u * bs < nvec && TCCL_VIN(c, a, i0 + u * bs)) v[u] = ld_peer(vptr<T>(src, i0 + u * bs));
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i0 + u * bs < nvec && TCCL_VOUT(c, a, (uint64_t)p * nvec + i0 + u * bs)) st_local(dst + (i0 + u * bs) * 16, v[u]);
      }
    }
    sync.exit(c, a.flags, bid);
  }
};

// ------------------------------------------------------------ all-gather, push
// Every rank stores its shard into slot [rank] of every rank's symmetric output
// (posted stores: one NVLink crossing, no load round trip), then the exit
// barrier publishes them.  NVLS form: one multimem.st per vector instead of W.
template <typename T, int W, bool kNvls>
struct AllGatherPush {
  using Args = tccl_coll_args;
  static constexpr int kMaxThreads = 512, kMinBlocks = 1;
  static constexpr int kMaxW = W ? W : TCCL_MAX_WORLD;
  static constexpr int U = 4;
  static __device__ __forceinline__ void put(const tccl_comm& c, const Args& a, int world, uint64_t off,
                                             const Vec16& v) {
    if (kNvls) {
      multimem_st(reinterpret_cast<char*>(a.mc_out) + off, v);
    } else {
#pragma unroll
      for (int p = 0; p < kMaxW; ++p)
        if (p < world) st_peer(reinterpret_cast<char*>(a.out_peer[p]) + off, v);
    }
  }
  static __device__ void run(const tccl_comm& c, const Args& a, int bid, int nb) {
    Entry sync(c, a.flags, bid);
    const int world = WorldOf<W>::get(c);
    constexpr int VPT = VecOf<T>::n;
    const uint64_t nvec = a.numel / VPT;  // the host guarantees a whole number of vectors
    const uint64_t bs = blockDim.x;
    const void* src = a.in[c.rank];
    const uint64_t base = (uint64_t)c.rank * a.numel * sizeof(T);
    TCCL_FOR_SLABS(U, nvec, bid, nb, i0) {
      Vec16 v[U];
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * bs < nvec && TCCL_VIN(c, a, i0 + u * bs)) v[u] = ld_peer(vptr<T>(src, i0 + u * bs));
#pragma unroll
      for (int u = 0; u < U; ++u)
        if (i0 + u * bs < nvec && TCCL_IN_BOUNDS(c, base + (i0 + u * bs) * 16, 16, a.out_bytes, TCCL_W_INDEX_OUT))
          put(c, a, world, base + (i0 + u * bs) * 16, v[u]);
    }
    sync.exit(c, a.flags, bid);
  }
};

// ---------------------------------------------------------------- reduce-scatter
// out[i] = sum_r in_r[rank * per + i], per = numel / W (numel % (W * vector) == 0,
// the reference's contract, triton_reduce_scatter.py:102-104).
template <typename T, int W, bool kNvls>
struct ReduceScatter {
  using Args = tccl_coll_args;
  static constexpr int kMaxThreads = 512, kMinBlocks = 1;
  static constexpr int kMaxW = W ? W : TCCL_MAX_WORLD;
  static constexpr int U = kNvls ? 8 : ((W == 0 || W >= 8) ? 2 : 4);
  static __device__ void run(const tccl_comm& c, const Args& a, int bid, int nb) {
    Entry sync(c, a.flags, bid);
    const int world = WorldOf<W>::get(c);
    constexpr int VPT = VecOf<T>::n;
    const uint64_t per = a.numel / world / VPT;  // vectors per rank
    const uint64_t lo = per * (uint64_t)c.rank;
    const uint64_t bs = blockDim.x;
    if (kNvls) {
      TCCL_FOR_SLABS(U, per, bid, nb, i0) {
        Vec16 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i0 + u * bs < per && TCCL_VIN(c, a, lo + i0 + u * bs)) v[u] = MultimemOps<T>::ld_reduce(vptr<T>(a.mc_in, lo + i0 + u * bs));
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i0 + u * bs < per && TCCL_VOUT(c, a, i0 + u * bs)) st_local(vptr<T>(a.out, i0 + u * bs), v[u]);
      }
    } else {
      TCCL_FOR_SLABS(U, per, bid, nb, i0) {
        Vec16 v[kMaxW][U];
#pragma unroll
        for (int p = 0; p < kMaxW; ++p)
          if (p < world) {
#pragma unroll
            for (int u = 0; u < U; ++u)
              if (i0 + u * bs < per && TCCL_VIN(c, a, lo + i0 + u * bs)) v[p][u] = ld_peer(vptr<T>(a.in[p], lo + i0 + u * bs));
          }
#pragma unroll
        for (int u = 0; u < U; ++u)
          if (i0 + u * bs < per && TCCL_VOUT(c, a, i0 + u * bs)) {
            Acc<T> acc;
            acc.zero();
#pragma unroll
            for (int p = 0; p < kMaxW; ++p)
              if (p < world) acc.add(v[p][u]);
            st_local(vptr<T>(a.out, i0 + u * bs), acc.pack());
          }
      }
    }
    sync.exit(c, a.flags, bid);
  }
};

// ------------------------------------------------------------------ dispatchers
template <template <typename, int> class Op>
static int dispatch(const tccl_comm* comm, const tccl_coll_args* args, const tccl_launch* l, int world, int dtype) {
#define TCCL_W(T)                                                         \
  switch (world) {                                                        \
    case 1: return launch_op<Op<T, 1>>(comm, args, l);                    \
    case 2: return launch_op<Op<T, 2>>(comm, args, l);                    \
    case 4: return launch_op<Op<T, 4>>(comm, args, l);                    \
    case 8: return launch_op<Op<T, 8>>(comm, args, l);                    \
    default: return launch_op<Op<T, 0>>(comm, args, l);                   \
  }
  switch (dtype) {
    case TCCL_BF16: TCCL_W(__nv_bfloat16)
    case TCCL_F32: TCCL_W(float)
    case TCCL_F16: TCCL_W(__half)
    default: return -TCCL_EDTYPE;
  }
#undef TCCL_W
}

template <typename T, int W> using AgPushP2P = AllGatherPush<T, W, false>;
template <typename T, int W> using AgPushNvls = AllGatherPush<T, W, true>;
template <typename T, int W> using RsP2P = ReduceScatter<T, W, false>;
template <typename T, int W> using RsNvls = ReduceScatter<T, W, true>;
template <typename T, int W> using ArPushP2P = AllReduceOneShotPush<T, W, false>;
template <typename T, int W> using ArPushNvls = AllReduceOneShotPush<T, W, true>;

}  // namespace tccl

using namespace tccl;

// The launchers pick a template instance by world size and dtype.  In emulated
// mode `comm`/`args` are device pointers the host cannot read, so the world size
// is n_emu and the dtype comes in the launch struct's `meta` field.
static inline void host_meta(const tccl_comm* comm, const tccl_coll_args* args, const tccl_launch* l, int* world,
                             int* dtype) {
  if (l->n_emu == 0) {
    *world = comm->world;
    *dtype = args ? args->dtype : 0;
  } else {
    *world = l->n_emu;
    *dtype = l->meta & 0xff;
  }
}

extern "C" {

uint64_t tccl_push_slot_bytes(uint64_t ll_bytes, int world) {
  return world >= 1 ? push_slot_bytes(ll_bytes, world) : 0;
}

int tccl_barrier_p2p(const tccl_comm* comm, const tccl_barrier_args* args, const tccl_launch* l) {
  return launch_op<BarrierP2POp>(comm, args, l);
}
int tccl_barrier_nvls(const tccl_comm* comm, const tccl_barrier_args* args, const tccl_launch* l) {
  return launch_op<BarrierNvlsOp>(comm, args, l);
}
int tccl_barrier_cas(const tccl_comm* comm, const tccl_pads_args* args, const tccl_launch* l) {
  return launch_op<BarrierCasOp>(comm, args, l);
}
int tccl_wait_never(const tccl_comm* comm, const tccl_barrier_args* args, const tccl_launch* l) {
  return launch_op<WaitNeverOp>(comm, args, l);
}

#define TCCL_COLL(name, Op)                                                                   \
  int name(const tccl_comm* comm, const tccl_coll_args* args, const tccl_launch* l) {         \
    int world, dtype;                                                                         \
    host_meta(comm, args, l, &world, &dtype);                                                 \
    return dispatch<Op>(comm, args, l, world, dtype);                                         \
  }
TCCL_COLL(tccl_allreduce_oneshot_p2p, AllReduceOneShotP2P)
TCCL_COLL(tccl_allreduce_oneshot_nvls, AllReduceOneShotNvls)
TCCL_COLL(tccl_allreduce_push_p2p, ArPushP2P)
TCCL_COLL(tccl_allreduce_push_nvls, ArPushNvls)
TCCL_COLL(tccl_allreduce_twoshot_p2p, AllReduceTwoShotP2P)
TCCL_COLL(tccl_allreduce_twoshot_nvls, AllReduceTwoShotNvls)
TCCL_COLL(tccl_allgather_pull_p2p, AllGatherPullP2P)
TCCL_COLL(tccl_allgather_push_p2p, AgPushP2P)
TCCL_COLL(tccl_allgather_push_nvls, AgPushNvls)
TCCL_COLL(tccl_reducescatter_p2p, RsP2P)
TCCL_COLL(tccl_reducescatter_nvls, RsNvls)
#undef TCCL_COLL

}  // extern "C"
