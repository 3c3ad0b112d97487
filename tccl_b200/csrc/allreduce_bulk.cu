// Two-shot all-reduce whose data crosses NVLink as BULK async copies.
//
// The plain two-shot kernel (collectives.cu) moves every vector with a 16-byte
// load or store issued by a thread; on this link that tops out near 655 GB/s per
// direction, while the copy path moves the same bytes in larger packets.  Here
// no thread touches remote memory:
//   loader  (one thread): cp.async.bulk global -> shared of the next chunk of
//           this rank's slice from EVERY rank's input (its own included), all
//           completing on one mbarrier per stage;
//   reducers (six warps): sum the W chunks out of shared memory in fp32 and
//           write the result into an output stage in shared memory;
//   storer  (one thread): cp.async.bulk shared -> global of that stage into
//           EVERY rank's destination, one bulk group per chunk.
// The three meet at mbarriers (full / empty per input stage and per output
// stage), so loads, sums and stores of different chunks overlap and both
// directions of the link stay busy.  No load here is a multicast: every copy
// names one source and one destination.
//
// As in the other two-shot kernels, slice r is read and written by rank r only
// and a chunk is stored after it was loaded, so an in-place reduction needs only
// the entry barrier (inputs ready) and the exit barrier (after
// cp.async.bulk.wait_group 0: results landed everywhere).  The reference has one
// all-reduce, a one-shot that pulls everything into every rank
// (triton_one_shot_all_reduce_no_128.py:35-64).
#include "gemm_tcgen05.cuh"

namespace tccl {

using gemm::Abort;
using gemm::mbar_arrive;
using gemm::mbar_arrive_expect_tx;
using gemm::mbar_init;
using gemm::mbar_wait;
using gemm::smem_u32;

constexpr int kBulkThreads = 256;          // warp 0: loader, warps 1..6: reducers, warp 7: storer
constexpr int kBulkReducers = 6 * 32;
constexpr int kBulkInStages = 3, kBulkOutStages = 2;
constexpr uint32_t kBulkSmemBudget = 192 * 1024;

// bytes per rank and stage: 3 input stages of W chunks + 2 output stages must fit the budget
__host__ __device__ __forceinline__ uint32_t bulk_chunk_bytes(int world) {
  uint32_t c = kBulkSmemBudget / (uint32_t)(kBulkInStages * world + kBulkOutStages);
  c = c > 16384u ? 16384u : c;
  return c & ~1023u;
}

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               :: "r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ Vec16 ld_shared_vec(const void* p) {
  Vec16 v;
  asm volatile("ld.shared.v4.b32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_u32(p)) : "memory");
  return v;
}

template <typename T>
struct AllReduceTwoShotBulk {
  using Args = tccl_coll_args;
  static constexpr int kMaxThreads = kBulkThreads, kMinBlocks = 1;

  static __device__ void run(const tccl_comm& c, const Args& a, int bid, int nb) {
    extern __shared__ __align__(128) uint8_t bulk_smem[];
    __shared__ uint64_t s_full_in[kBulkInStages], s_empty_in[kBulkInStages];
    __shared__ uint64_t s_full_out[kBulkOutStages], s_empty_out[kBulkOutStages];
    __shared__ int s_abort;
    const int world = c.world;
    const uint32_t CB = bulk_chunk_bytes(world);
    const int t = threadIdx.x;
    if (t == 0) {
      s_abort = 0;
      for (int s = 0; s < kBulkInStages; ++s) {
        mbar_init(s_full_in + s, 1);               // the loader's arrive + the bytes of W copies
        mbar_init(s_empty_in + s, kBulkReducers);  // every reducer thread has read the stage
      }
      for (int s = 0; s < kBulkOutStages; ++s) {
        mbar_init(s_full_out + s, kBulkReducers);  // every reducer thread has written its part
        mbar_init(s_empty_out + s, 1);             // the storer's copies have read the stage
      }
      gemm::fence_barrier_init();
    }
    __syncthreads();
    Entry sync(c, a.flags, bid);
    Abort ab{&s_abort, &c, c.local + TCCL_LOCAL_STATUS, sync.deadline};
    constexpr int VPT = 16 / (int)sizeof(T);
    const uint64_t nvec = a.numel / VPT;
    const uint64_t per = (nvec + world - 1) / world;
    const uint64_t lo = min(per * (uint64_t)c.rank, nvec), n = min(lo + per, nvec) - lo;  // this rank's slice
    const uint64_t CV = CB / 16;
    const uint64_t nchunks = (n + CV - 1) / CV;
    uint8_t* in_st = bulk_smem;                                              // [stage][rank][CB]
    uint8_t* out_st = bulk_smem + (size_t)kBulkInStages * world * CB;        // [stage][CB]

    if (t == 0) {
      // ------------------------------------------------------------ loader
      uint32_t q = 0;
      bool ok = true;
      for (uint64_t ci = bid; ci < nchunks && ok; ci += nb, ++q) {
        const int s = q % kBulkInStages;
        ok = mbar_wait(s_empty_in + s, ((q / kBulkInStages) & 1) ^ 1, ab);
        if (!ok) break;
        const uint64_t v0 = lo + ci * CV;
        const uint32_t bytes = (uint32_t)(min(CV, lo + n - v0) * 16);
        mbar_arrive_expect_tx(s_full_in + s, bytes * (uint32_t)world);
        for (int p = 0; p < world; ++p)
          bulk_load(in_st + ((size_t)s * world + p) * CB, reinterpret_cast<const char*>(a.in[p]) + v0 * 16, bytes,
                    s_full_in + s);
      }
    } else if (t >= 32 && t < 32 + kBulkReducers) {
      // ------------------------------------------------------------ reducers
      const int j = t - 32;
      uint32_t q = 0;
      bool ok = true;
      for (uint64_t ci = bid; ci < nchunks && ok; ci += nb, ++q) {
        const int s = q % kBulkInStages, so = q % kBulkOutStages;
        ok = mbar_wait(s_full_in + s, (q / kBulkInStages) & 1, ab);
        if (!ok) break;
        ok = mbar_wait(s_empty_out + so, ((q / kBulkOutStages) & 1) ^ 1, ab);
        if (!ok) break;
        const uint64_t v0 = lo + ci * CV;
        const uint32_t cnt = (uint32_t)min(CV, lo + n - v0);
        const uint8_t* src = in_st + (size_t)s * world * CB;
        uint8_t* dst = out_st + (size_t)so * CB;
        for (uint32_t k = j; k < cnt; k += kBulkReducers) {
          Acc<T> acc;
          acc.zero();
          for (int p = 0; p < world; ++p) acc.add(ld_shared_vec(src + (size_t)p * CB + (size_t)k * 16));
          gemm::st_shared_v4(dst + (size_t)k * 16, acc.pack());
        }
        gemm::fence_proxy_async_smem();  // the copy engine reads what this thread wrote
        mbar_arrive(s_full_out + so);
        mbar_arrive(s_empty_in + s);
      }
    } else if (t == kBulkThreads - 32) {
      // ------------------------------------------------------------ storer
      uint32_t q = 0;
      bool ok = true;
      for (uint64_t ci = bid; ci < nchunks && ok; ci += nb, ++q) {
        const int so = q % kBulkOutStages;
        ok = mbar_wait(s_full_out + so, (q / kBulkOutStages) & 1, ab);
        if (!ok) break;
        const uint64_t v0 = lo + ci * CV;
        const uint32_t bytes = (uint32_t)(min(CV, lo + n - v0) * 16);
        for (int p = 0; p < world; ++p)
          gemm::bulk_store(reinterpret_cast<char*>(a.out_peer[p]) + v0 * 16, out_st + (size_t)so * CB, bytes);
        gemm::bulk_commit();
        if (q >= 1) {
          gemm::bulk_wait_read<1>();  // the previous chunk's copies have read their stage
          mbar_arrive(s_empty_out + ((q - 1) % kBulkOutStages));
        }
      }
      gemm::bulk_wait<0>();  // every copy of this CTA has landed (also after a wait that gave up)
      gemm::fence_proxy_async();
    }
    // ragged tail (numel not a multiple of the vector width): rank 0 sums it for everybody
    const uint64_t tid = (uint64_t)bid * blockDim.x + threadIdx.x;
    if (c.rank == 0 && tid < a.numel - nvec * VPT) {
      const uint64_t e = nvec * VPT + tid;
      float sum = 0.f;
      for (int p = 0; p < world; ++p) sum += to_f32(reinterpret_cast<const volatile T*>(a.in[p])[e]);
      for (int p = 0; p < world; ++p) reinterpret_cast<volatile T*>(a.out_peer[p])[e] = from_f32<T>(sum);
    }
    sync.exit(c, a.flags, bid);  // opens with a CTA barrier: the storer's wait_group is behind it
  }
};

}  // namespace tccl

using namespace tccl;

extern "C" uint32_t tccl_allreduce_bulk_chunk_bytes(int world) { return bulk_chunk_bytes(world); }

// Inputs and destinations must be 16-byte aligned symmetric buffers; l->block must be 256.
extern "C" int tccl_allreduce_twoshot_bulk(const tccl_comm* comm, const tccl_coll_args* args, const tccl_launch* l) {
  const int world = l->n_emu ? l->n_emu : comm->world;
  const int dtype = l->n_emu ? (l->meta & 0xff) : args->dtype;
  if (l->block != kBulkThreads) return -TCCL_EINVAL;
  const size_t smem = (size_t)(kBulkInStages * world + kBulkOutStages) * bulk_chunk_bytes(world);
  if (l->n_emu == 0) {
    for (int p = 0; p < world; ++p)
      if (((uintptr_t)args->in[p] | (uintptr_t)args->out_peer[p]) & 15) return -TCCL_EALIGN;
  }
  switch (dtype) {
    case TCCL_BF16: return launch_op<AllReduceTwoShotBulk<__nv_bfloat16>>(comm, args, l, smem);
    case TCCL_F32: return launch_op<AllReduceTwoShotBulk<float>>(comm, args, l, smem);
    case TCCL_F16: return launch_op<AllReduceTwoShotBulk<__half>>(comm, args, l, smem);
    default: return -TCCL_EDTYPE;
  }
}
