// Device-side building blocks: PTX wrappers (system-scope release/acquire,
// 128-bit peer loads, NVLS multimem), bounded waits with status reporting, and
// the real/emulated kernel entry scaffolding.  sm_100a only.
//
// These replace the reference's inline-PTX helpers (`load_128`,
// triton_all_gather.py:14-29; `add_v8_bf16`, triton_reduce_scatter.py:32-56;
// `add_v4_bf16`, triton_one_shot_all_reduce_no_128.py:13-32; the CAS spins of
// triton_barrier.py:108-118) with fp32 accumulation and waits that give up.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "tccl_b200.h"

namespace tccl {

// ---------------------------------------------------------------- PTX: sync
__device__ __forceinline__ uint64_t globaltimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint32_t ld_relaxed_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_release_sys_add(uint32_t* p, uint32_t v) {
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void multimem_red_release_add(uint32_t* mc, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t cas_release_sys(uint32_t* p, uint32_t cmp, uint32_t val) {
  uint32_t old;
  asm volatile("atom.release.sys.global.cas.b32 %0, [%1], %2, %3;"
               : "=r"(old) : "l"(p), "r"(cmp), "r"(val) : "memory");
  return old;
}
__device__ __forceinline__ uint32_t cas_acquire_sys(uint32_t* p, uint32_t cmp, uint32_t val) {
  uint32_t old;
  asm volatile("atom.acquire.sys.global.cas.b32 %0, [%1], %2, %3;"
               : "=r"(old) : "l"(p), "r"(cmp), "r"(val) : "memory");
  return old;
}
__device__ __forceinline__ void fence_acq_rel_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }

// ---------------------------------------------------------------- PTX: data
struct alignas(16) Vec16 {
  uint32_t x, y, z, w;
};

// Peer data is read after a system-scope acquire; the relaxed.sys load keeps
// the access out of the (non-coherent) L1 for lines a peer may rewrite later.
__device__ __forceinline__ Vec16 ld_peer(const void* p) {
  Vec16 v;
  asm volatile("ld.relaxed.sys.global.L1::no_allocate.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ void st_peer(void* p, const Vec16& v) {
  asm volatile("st.relaxed.sys.global.v4.b32 [%0], {%1,%2,%3,%4};"
               ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
__device__ __forceinline__ void st_local(void* p, const Vec16& v) {
  asm volatile("st.global.v4.b32 [%0], {%1,%2,%3,%4};"
               ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}
// streaming store: the output of a large collective is not re-read by this kernel
__device__ __forceinline__ void st_local_cs(void* p, const Vec16& v) {
  asm volatile("st.global.cs.v4.b32 [%0], {%1,%2,%3,%4};"
               ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

template <typename T> struct MultimemOps;
template <> struct MultimemOps<__nv_bfloat16> {
  static __device__ __forceinline__ Vec16 ld_reduce(const void* mc) {
    Vec16 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
template <> struct MultimemOps<__half> {
  static __device__ __forceinline__ Vec16 ld_reduce(const void* mc) {
    Vec16 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
template <> struct MultimemOps<float> {
  static __device__ __forceinline__ Vec16 ld_reduce(const void* mc) {
    Vec16 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(mc) : "memory");
    return v;
  }
};
__device__ __forceinline__ void multimem_st(void* mc, const Vec16& v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};"
               ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

// ------------------------------------------------- fp32 accumulation of a Vec16
template <typename T> struct Acc;  // fp32 accumulator for one 16-byte vector of T

template <> struct Acc<float> {
  float a[4];
  __device__ __forceinline__ void zero() { a[0] = a[1] = a[2] = a[3] = 0.f; }
  __device__ __forceinline__ void add(const Vec16& v) {
    a[0] += __uint_as_float(v.x); a[1] += __uint_as_float(v.y);
    a[2] += __uint_as_float(v.z); a[3] += __uint_as_float(v.w);
  }
  __device__ __forceinline__ Vec16 pack() const {
    return Vec16{__float_as_uint(a[0]), __float_as_uint(a[1]), __float_as_uint(a[2]), __float_as_uint(a[3])};
  }
};
template <> struct Acc<__nv_bfloat16> {
  float a[8];
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = 0.f;
  }
  static __device__ __forceinline__ float lo(uint32_t u) { return __uint_as_float(u << 16); }
  static __device__ __forceinline__ float hi(uint32_t u) { return __uint_as_float(u & 0xffff0000u); }
  __device__ __forceinline__ void add(const Vec16& v) {
    a[0] += lo(v.x); a[1] += hi(v.x); a[2] += lo(v.y); a[3] += hi(v.y);
    a[4] += lo(v.z); a[5] += hi(v.z); a[6] += lo(v.w); a[7] += hi(v.w);
  }
  static __device__ __forceinline__ uint32_t pk(float l, float h) {
    uint32_t r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(h), "f"(l));
    return r;
  }
  __device__ __forceinline__ Vec16 pack() const {
    return Vec16{pk(a[0], a[1]), pk(a[2], a[3]), pk(a[4], a[5]), pk(a[6], a[7])};
  }
};
template <> struct Acc<__half> {
  float a[8];
  __device__ __forceinline__ void zero() {
#pragma unroll
    for (int i = 0; i < 8; ++i) a[i] = 0.f;
  }
  __device__ __forceinline__ void add(const Vec16& v) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(*reinterpret_cast<const __half2*>(&u[i]));
      a[2 * i] += f.x; a[2 * i + 1] += f.y;
    }
  }
  __device__ __forceinline__ Vec16 pack() const {
    uint32_t u[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      __half2 h = __floats2half2_rn(a[2 * i], a[2 * i + 1]);
      u[i] = *reinterpret_cast<uint32_t*>(&h);
    }
    return Vec16{u[0], u[1], u[2], u[3]};
  }
};

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f32<__half>(float v) { return __float2half_rn(v); }

// --------------------------------------------------------- status / bounded wait
__device__ __forceinline__ uint32_t* status_of(const tccl_comm& c) { return c.local + TCCL_LOCAL_STATUS; }

static __device__ __noinline__ void record_failure(const tccl_comm& c, int code, int peer, int where,
                                            uint32_t seen, uint32_t want) {
  uint32_t* st = status_of(c);
  if (atomicCAS(st + TCCL_ST_CODE, 0u, (uint32_t)code) == 0u) {
    st[TCCL_ST_BLOCK] = blockIdx.x;
    st[TCCL_ST_PEER] = (uint32_t)peer;
    st[TCCL_ST_WHERE] = (uint32_t)where;
    st[TCCL_ST_SEEN] = seen;
    st[TCCL_ST_WANT] = want;
  }
  __threadfence();
  atomicExch(st + TCCL_ST_ABORT, 1u);
}

// Bounds checks of the TCCL_DEBUG_CHECKS build: `bytes` at offset `off` of a buffer whose usable
// extent the host has passed along.  A miss records TCCL_BAD_INDEX with the offending offset and
// the extent (low 32 bits each) and the caller SKIPS the access; nothing traps.  In the regular
// build the macro is the constant true and the extents are not looked at.
#ifdef TCCL_DEBUG_CHECKS
static __device__ __noinline__ bool bad_index(const tccl_comm& c, uint64_t off, uint64_t extent, int where) {
  record_failure(c, TCCL_BAD_INDEX, c.rank, where, (uint32_t)off, (uint32_t)extent);
  return false;
}
#define TCCL_IN_BOUNDS(c, off, bytes, extent, where) \
  (((uint64_t)(off) + (uint64_t)(bytes) <= (uint64_t)(extent)) ? true : bad_index((c), (uint64_t)(off), (uint64_t)(extent), (where)))
#else
#define TCCL_IN_BOUNDS(c, off, bytes, extent, where) true
#endif
// vector `vec` (16 bytes) of an input / output of the flat collectives
#define TCCL_VIN(c, a, vec) TCCL_IN_BOUNDS(c, (uint64_t)(vec) * 16, 16, (a).in_bytes, TCCL_W_INDEX_IN)
#define TCCL_VOUT(c, a, vec) TCCL_IN_BOUNDS(c, (uint64_t)(vec) * 16, 16, (a).out_bytes, TCCL_W_INDEX_OUT)

__device__ __forceinline__ bool aborted(const tccl_comm& c) {
  return *reinterpret_cast<volatile uint32_t*>(status_of(c) + TCCL_ST_ABORT) != 0u;
}

// Polls `flag` (acquire, system scope) until it reaches `want` in wrap-around
// order.  Gives up after `timeout_ns` or as soon as another waiter of this rank
// gave up; then records where and returns false.  Never traps, never loops on.
__device__ __forceinline__ bool wait_reach(const uint32_t* flag, uint32_t want, const tccl_comm& c,
                                           uint64_t deadline, int peer, int where) {
  uint32_t spins = 0;
  for (;;) {
    uint32_t v = ld_acquire_sys(flag);
    if ((int32_t)(v - want) >= 0) return true;
    if ((++spins & 63u) == 0u) {
      if (aborted(c)) return false;
      if (globaltimer() > deadline) {
        record_failure(c, TCCL_TIMEOUT, peer, where, v, want);
        return false;
      }
    }
  }
}

// ------------------------------------------------------------- epoch barriers
// All-to-all barrier between the CTAs with the same block index on all ranks,
// on the library's own flag region.  Row `bid` of every rank's flag region has
// one word per source rank; a barrier round is "store my new epoch into my
// word of every peer's row (release), poll my own row until every word reached
// the epoch (acquire)".  The epoch lives in local device memory and is advanced
// by the kernel itself, so there is no host-side state and a captured graph can
// replay it.  Stores are posted: one NVLink crossing per round instead of the
// reference's two CAS round trips (triton_barrier.py:108-118).
//
// Must be called by all threads of the CTA.  Writes made by any thread of the
// CTA before the call are visible to every peer thread after its call returns.
__device__ __forceinline__ void barrier_p2p(const tccl_comm& c, int bid, uint64_t deadline) {
  __syncthreads();
  const int t = threadIdx.x;
  if (t < c.world) {
    const uint32_t e = c.local[TCCL_LOCAL_EPOCH + bid] + 1u;
    st_release_sys(c.flags[t] + TCCL_FLAG_BAR + bid * TCCL_MAX_WORLD + c.rank, e);
    wait_reach(c.flags[c.rank] + TCCL_FLAG_BAR + bid * TCCL_MAX_WORLD + t, e, c, deadline, t, TCCL_W_BARRIER);
  }
  __syncthreads();
  if (t == 0) c.local[TCCL_LOCAL_EPOCH + bid] += 1u;
}

// NVLS flavour: one multimem.red adds 1 to word `bid` on every rank at once;
// a round is complete when the local word reached world * epoch.
__device__ __forceinline__ void barrier_nvls(const tccl_comm& c, int bid, uint64_t deadline) {
  __syncthreads();
  if (threadIdx.x == 0) {
    const uint32_t e = c.local[TCCL_LOCAL_MCEPOCH + bid] + 1u;
    multimem_red_release_add(c.mc_flags + TCCL_FLAG_MCBAR + bid, 1u);
    wait_reach(c.flags[c.rank] + TCCL_FLAG_MCBAR + bid, e * (uint32_t)c.world, c, deadline, -1, TCCL_W_MCBARRIER);
    c.local[TCCL_LOCAL_MCEPOCH + bid] = e;
  }
  __syncthreads();
}

__device__ __forceinline__ void barrier_any(const tccl_comm& c, int bid, uint64_t deadline, bool nvls) {
  if (nvls) barrier_nvls(c, bid, deadline);
  else barrier_p2p(c, bid, deadline);
}

// entry / exit synchronisation shared by the data kernels
struct Entry {
  uint64_t deadline;
  bool nvls_bar;
  __device__ __forceinline__ Entry(const tccl_comm& c, int flags, int bid)
      : deadline(globaltimer() + c.timeout_ns), nvls_bar((flags & TCCL_F_NVLS_BARRIER) != 0) {
    if (!(flags & TCCL_F_NO_ENTRY_BARRIER)) barrier_any(c, bid, deadline, nvls_bar);
  }
  __device__ __forceinline__ void exit(const tccl_comm& c, int flags, int bid) {
    if (!(flags & TCCL_F_NO_EXIT_BARRIER)) barrier_any(c, bid, deadline, nvls_bar);
  }
};

// ---------------------------------------------------------- kernel scaffolding
// Every collective is a struct `Op` with `using Args = ...` and
// `static __device__ void run(const tccl_comm&, const Args&, int bid, int nblocks)`.
template <class Op>
__global__ void __launch_bounds__(Op::kMaxThreads, Op::kMinBlocks)
kernel_real(const __grid_constant__ tccl_comm comm, const __grid_constant__ typename Op::Args args) {
  Op::run(comm, args, blockIdx.x, gridDim.x);
}
template <class Op>
__global__ void __launch_bounds__(Op::kMaxThreads, Op::kMinBlocks)
kernel_emu(const tccl_comm* comms, const typename Op::Args* args) {
  Op::run(comms[blockIdx.y], args[blockIdx.y], blockIdx.x, gridDim.x);
}

template <class Op>
inline int launch_op(const tccl_comm* comm, const typename Op::Args* args, const tccl_launch* l,
                     size_t smem = 0) {
  cudaStream_t s = reinterpret_cast<cudaStream_t>(l->stream);
  if (l->grid <= 0 || l->block <= 0 || l->block > Op::kMaxThreads) return -TCCL_EINVAL;
  if (l->n_emu == 0) {
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(kernel_real<Op>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kernel_real<Op><<<l->grid, l->block, smem, s>>>(*comm, *args);
    return (int)cudaGetLastError();
  }
  if (l->n_emu < 0 || l->n_emu > TCCL_MAX_WORLD) return -TCCL_EINVAL;
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(kernel_emu<Op>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  void* kargs[2] = {(void*)&comm, (void*)&args};
  // cooperative: all emulated ranks' CTAs must be resident at once, or the launch fails cleanly
  return (int)cudaLaunchCooperativeKernel((const void*)kernel_emu<Op>, dim3(l->grid, l->n_emu), dim3(l->block),
                                          kargs, smem, s);
}

}  // namespace tccl
