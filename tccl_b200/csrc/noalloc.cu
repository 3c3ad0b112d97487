// The allocation-free entry point declared in tccl_noalloc.h: a one-shot
// all-reduce over buffers of the current device whose barrier scratch is a
// static device array instead of memory the caller (or anyone) allocates.
#include <cooperative_groups.h>

#include <mutex>

#include "common.cuh"
#include "tccl_noalloc.h"

namespace cg = cooperative_groups;
using namespace tccl;

// The scratch.  In host code this name is only a handle for the runtime's symbol
// table, not a device address; the host obtains the address once per device with
// cudaGetSymbolAddress (below) and hands it to the kernel.
static __device__ __align__(256) uint32_t g_noalloc_scratch[TCCL_NOALLOC_SCRATCH_BYTES / 4];

struct NoAllocParams {
  const void* in[TCCL_NOALLOC_MAX_RANKS];
  void* out[TCCL_NOALLOC_MAX_RANKS];
  uint64_t numel;
  uint64_t timeout_ns;
  uint32_t* scratch;
  int32_t world;
};

__device__ __forceinline__ uint32_t* na_flags(uint32_t* scratch, int rank) {
  return scratch + rank * TCCL_NOALLOC_FLAG_WORDS;
}
__device__ __forceinline__ uint32_t* na_local(uint32_t* scratch, int rank) {
  return scratch + TCCL_NOALLOC_MAX_RANKS * TCCL_NOALLOC_FLAG_WORDS + rank * TCCL_NOALLOC_LOCAL_WORDS;
}

template <typename T>
__global__ void __launch_bounds__(512, 1) noalloc_allreduce_kernel(const __grid_constant__ NoAllocParams p) {
  const int rank = blockIdx.y, bid = blockIdx.x, nb = gridDim.x;
  const int world = p.world;
  // The scratch still holds the previous call's flags, epochs and status: bring
  // the words this launch depends on back to zero, then let nobody pass before
  // every block has done so.
  {
    uint32_t* f = na_flags(p.scratch, rank);
    uint32_t* l = na_local(p.scratch, rank);
    for (int i = bid * blockDim.x + threadIdx.x; i < TCCL_NOALLOC_FLAG_WORDS; i += nb * blockDim.x) f[i] = 0u;
    if (bid == 0) {
      for (int i = threadIdx.x; i < TCCL_NOALLOC_MAX_CTAS; i += blockDim.x) l[TCCL_LOCAL_EPOCH + i] = 0u;
      for (int i = threadIdx.x; i < TCCL_ST_WORDS; i += blockDim.x) l[TCCL_LOCAL_STATUS + i] = 0u;
    }
    __threadfence();
    cg::this_grid().sync();
  }

  __shared__ tccl_comm c;
  if (threadIdx.x == 0) {
    c.world = world;
    c.rank = rank;
    for (int q = 0; q < TCCL_MAX_WORLD; ++q) {
      c.flags[q] = q < world ? na_flags(p.scratch, q) : nullptr;
      c.stage[q] = nullptr;
    }
    c.mc_flags = nullptr;
    c.mc_stage = nullptr;
    c.local = na_local(p.scratch, rank);
    c.stage_bytes = 0;
    c.timeout_ns = p.timeout_ns;
  }
  __syncthreads();

  const uint64_t deadline = globaltimer() + p.timeout_ns;
  barrier_p2p(c, bid, deadline);  // all emulated ranks are inside the kernel
  constexpr int VPT = 16 / (int)sizeof(T);
  const uint64_t nvec = p.numel / VPT;
  const uint64_t nthr = (uint64_t)nb * blockDim.x;
  const uint64_t tid = (uint64_t)bid * blockDim.x + threadIdx.x;
  char* out = reinterpret_cast<char*>(p.out[rank]);
  for (uint64_t i = tid; i < nvec; i += nthr) {
    Acc<T> acc;
    acc.zero();
    for (int q = 0; q < world; ++q) acc.add(ld_peer(reinterpret_cast<const char*>(p.in[q]) + i * 16));
    st_local(out + i * 16, acc.pack());
  }
  if (tid < p.numel - nvec * VPT) {
    const uint64_t e = nvec * VPT + tid;
    float s = 0.f;
    for (int q = 0; q < world; ++q) s += to_f32(reinterpret_cast<const volatile T*>(p.in[q])[e]);
    reinterpret_cast<T*>(out)[e] = from_f32<T>(s);
  }
  barrier_p2p(c, bid, deadline);  // nobody leaves while a peer may still read its input
}

// ---------------------------------------------------------------- host side
namespace {
constexpr int kMaxDevices = 64;
std::mutex g_scratch_mutex;             // first calls from several host threads may coincide
uint32_t* g_scratch_addr[kMaxDevices];  // device address of g_noalloc_scratch, per device
bool g_scratch_ready[kMaxDevices];

// First use on a device: resolve the device address of the static array while
// that device is current.  (Passing `g_noalloc_scratch` itself to a kernel from
// host code would pass the host-side shadow of the symbol.)
int scratch_for_current_device(uint32_t** ptr) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return (int)e;
  if (dev < 0 || dev >= kMaxDevices) return -TCCL_EINVAL;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (!g_scratch_ready[dev]) {
    void* addr = nullptr;
    e = cudaGetSymbolAddress(&addr, g_noalloc_scratch);
    if (e != cudaSuccess) return (int)e;
    g_scratch_addr[dev] = reinterpret_cast<uint32_t*>(addr);
    g_scratch_ready[dev] = true;
  }
  *ptr = g_scratch_addr[dev];
  return 0;
}
}  // namespace

extern "C" int tccl_allreduce_local_noalloc(const void* const* in, void* const* out, int n_ranks, uint64_t numel,
                                            int dtype, int ctas, void* stream) {
  if (!in || !out || n_ranks < 1 || ctas < 1) return -TCCL_EINVAL;
  if (n_ranks > TCCL_NOALLOC_MAX_RANKS || ctas > TCCL_NOALLOC_MAX_CTAS) return -TCCL_ESIZE;
  NoAllocParams p{};
  for (int r = 0; r < n_ranks; ++r) {
    if (!in[r] || !out[r]) return -TCCL_EINVAL;
    if ((reinterpret_cast<uintptr_t>(in[r]) | reinterpret_cast<uintptr_t>(out[r])) & 15) return -TCCL_EALIGN;
    p.in[r] = in[r];
    p.out[r] = out[r];
  }
  // an output may not be one of the inputs: a rank stores its sums while the others still read
  for (int r = 0; r < n_ranks; ++r)
    for (int q = 0; q < n_ranks; ++q)
      if (out[r] == in[q]) return -TCCL_EINVAL;
  p.numel = numel;
  p.timeout_ns = 2000000000ull;
  p.world = n_ranks;
  int rc = scratch_for_current_device(&p.scratch);
  if (rc) return rc;
  const void* fn = nullptr;
  switch (dtype) {
    case TCCL_BF16: fn = (const void*)noalloc_allreduce_kernel<__nv_bfloat16>; break;
    case TCCL_F32: fn = (const void*)noalloc_allreduce_kernel<float>; break;
    case TCCL_F16: fn = (const void*)noalloc_allreduce_kernel<__half>; break;
    default: return -TCCL_EDTYPE;
  }
  void* kargs[1] = {(void*)&p};
  // cooperative: the emulated ranks' blocks wait on one another and the launch
  // opens with a grid-wide sync, so all of them must be resident together
  return (int)cudaLaunchCooperativeKernel(fn, dim3(ctas, n_ranks), dim3(512), kargs, 0,
                                          reinterpret_cast<cudaStream_t>(stream));
}

extern "C" int tccl_noalloc_last_status(int rank, uint32_t* words, void* stream) {
  if (!words || rank < 0 || rank >= TCCL_NOALLOC_MAX_RANKS) return -TCCL_EINVAL;
  uint32_t* scratch = nullptr;
  int rc = scratch_for_current_device(&scratch);
  if (rc) return rc;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  cudaError_t e = cudaStreamSynchronize(s);
  if (e != cudaSuccess) return (int)e;
  const uint32_t* src = scratch + TCCL_NOALLOC_MAX_RANKS * TCCL_NOALLOC_FLAG_WORDS + rank * TCCL_NOALLOC_LOCAL_WORDS +
                        TCCL_LOCAL_STATUS;
  return (int)cudaMemcpy(words, src, TCCL_ST_WORDS * sizeof(uint32_t), cudaMemcpyDeviceToHost);
}
