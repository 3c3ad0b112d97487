// Double-binary-tree all-reduce for SMALL messages: the flag travels with the data.
//
// In the chunked kernel (tree_allreduce.cu) a hop is "store the slice, make the
// stores visible (a release: wait for every store to be acknowledged over
// NVLink), store a counter, the receiver polls the counter, then reads".  For a
// few kilobytes that is two fabric round trips of pure protocol per tree level,
// six levels up and down at 8 ranks.  Here every 16-byte line that crosses the
// link is {payload, flag, payload, flag}: 8 bytes of data and the call's sequence
// number twice.  The receiver polls the LINE; once both flags show the number
// it waits for, the two payload words next to them are valid (8-byte halves of
// an aligned vector store arrive whole).  No release, no counter, no barrier
// inside the CTA: every thread follows its own lines up and down the trees, and
// a hop costs one posted store plus the polling loop.
//
// Layout: each (tree, k) pipeline owns, in every rank's LL region (a part of the
// tree ring of its own, so that it only ever holds lines of this format), the
// slots [tree][left | right | down][k][seq % depth]; a slot holds 4096 lines =
// 32 KiB of payload.  One slot per pipeline and call (the host picks K so that
// the message fits), numbered by the pipeline's own count of calls of this
// kernel (TCCL_LOCAL_TREE_LL_SEQ).  A slot is reused
// TCCL_TREE_RING_DEPTH calls later; a rank can run at most one call ahead of a
// neighbour (it needs the neighbour's contribution to finish), so the old
// lines have long been consumed, and their flags differ from the new number.
//
// The sums reach every rank through the down slots, so no user tensor has to be
// symmetric here: the input is read and the result written by their owner only.
//
// Same trees and the same "two sends and two receives per GPU" as the algorithm the reference intends
// (triton_double_tree_allreduce.py:227-335, tree.py:36-51); its own kernel never completes a reduction.
#include "common.cuh"

namespace tccl {

constexpr int kLLDepth = TCCL_TREE_RING_DEPTH;
constexpr uint64_t kLLSlot = TCCL_TREE_LL_SLOT_BYTES;      // bytes per slot
constexpr uint32_t kLLLines = TCCL_TREE_LL_SLOT_BYTES / 16;  // lines per slot, 8 payload bytes each

template <typename T>
struct TreeAllReduceLL {
  using Args = tccl_tree_args;
  static constexpr int kMaxThreads = 512, kMinBlocks = 1;

  // slot `which` (0 = from the left child, 1 = from the right child, 2 = from the parent) of pipeline (tree, k)
  static __device__ __forceinline__ char* slot(const tccl_comm& c, int rank, int tree, int which, int k, uint32_t seq) {
    const uint64_t idx = ((uint64_t)((tree * 3 + which) * TCCL_TREE_LL_MAX_CTAS + k)) * kLLDepth + (seq % kLLDepth);
    return c.stage[rank] + c.stage_bytes + c.ll_bytes + idx * kLLSlot;
  }
  static __device__ __forceinline__ void put(char* line, uint32_t d0, uint32_t d1, uint32_t flag) {
    st_peer(line, Vec16{d0, flag, d1, flag});
  }
  // polls until both flags of the line show `flag`; false after the deadline (or once this rank has aborted)
  static __device__ __forceinline__ bool get(const char* line, uint32_t flag, uint32_t& d0, uint32_t& d1,
                                             const tccl_comm& c, uint64_t deadline, int peer, int where) {
    uint32_t spins = 0;
    for (;;) {
      const Vec16 v = ld_peer(line);
      if (v.y == flag && v.w == flag) {
        d0 = v.x;
        d1 = v.z;
        return true;
      }
      if ((++spins & 63u) == 0u) {
        if (aborted(c)) return false;
        if (globaltimer() > deadline) {
          record_failure(c, TCCL_TIMEOUT, peer, where, v.y, flag);
          return false;
        }
      }
    }
  }
  // 8 payload bytes as fp32 accumulators and back
  static constexpr int E = 8 / (int)sizeof(T);
  static __device__ __forceinline__ void unpack(uint32_t d0, uint32_t d1, float* f) {
    Acc<T> a;
    a.zero();
    a.add(Vec16{d0, d1, 0u, 0u});
#pragma unroll
    for (int e = 0; e < E; ++e) f[e] = a.a[e];
  }
  static __device__ __forceinline__ void pack(const float* f, uint32_t& d0, uint32_t& d1) {
    Acc<T> a;
    a.zero();
#pragma unroll
    for (int e = 0; e < E; ++e) a.a[e] = f[e];
    const Vec16 v = a.pack();
    d0 = v.x;
    d1 = v.y;
  }

  static __device__ void run(const tccl_comm& c, const Args& a, int bid, int nb) {
    const uint64_t deadline = globaltimer() + c.timeout_ns;
    const int K = a.ctas_per_role;
    const int role = bid / K, k = bid - role * K;
    const int tree = role & 1;
    const bool is_up = role < 2;
    const int parent = a.parent[tree], left = a.left[tree], right = a.right[tree];
    const int me = c.rank;
    const int cslot = a.child_slot[tree];
    // the message in 8-byte lines; tree 0 takes the first half, tree 1 the rest; pipeline k a contiguous share
    const uint64_t nlines = a.numel * sizeof(T) / 8;
    const uint64_t half0 = (nlines + 1) / 2;
    const uint64_t tlo = tree ? half0 : 0, tn = tree ? nlines - half0 : half0;
    const uint64_t per = (tn + K - 1) / K;
    const uint64_t lo = tlo + min(per * (uint64_t)k, tn), n = min(per, tn - min(per * (uint64_t)k, tn));
    // this kernel's own call count per pipeline: the chunked kernel's counters also pace its
    // acknowledgements and must advance with its chunks only
    uint32_t* seq_word = c.local + TCCL_LOCAL_TREE_LL_SEQ + role * TCCL_TREE_LL_MAX_CTAS + k;
    const uint32_t g = *seq_word;
    const uint32_t flag = g + 1u;
    const char* in = reinterpret_cast<const char*>(a.in);
    char* res = reinterpret_cast<char*>(a.buf[me]);  // this rank's own result buffer (may be null)
    char* out = reinterpret_cast<char*>(a.out);
    const int t = threadIdx.x, nt = blockDim.x;
    bool ok = true;

    if (is_up) {
      const char* lslot = left >= 0 ? slot(c, me, tree, 0, k, g) : nullptr;
      const char* rslot = right >= 0 ? slot(c, me, tree, 1, k, g) : nullptr;
      char* pslot = parent >= 0 ? slot(c, parent, tree, cslot, k, g) : nullptr;
      char* ldown = left >= 0 ? slot(c, left, tree, 2, k, g) : nullptr;
      char* rdown = right >= 0 ? slot(c, right, tree, 2, k, g) : nullptr;
      for (uint64_t i = t; i < n && ok; i += nt) {
        uint32_t d0, d1;
        asm volatile("ld.relaxed.sys.global.L1::no_allocate.v2.b32 {%0,%1}, [%2];"
                     : "=r"(d0), "=r"(d1) : "l"(in + (lo + i) * 8) : "memory");
        if (lslot) {
          float s[E], v[E];
          unpack(d0, d1, s);
          uint32_t x0, x1;
          ok = get(lslot + i * 16, flag, x0, x1, c, deadline, left, TCCL_W_TREE_UP);
          unpack(x0, x1, v);
#pragma unroll
          for (int e = 0; e < E; ++e) s[e] += v[e];
          if (ok && rslot) {
            ok = get(rslot + i * 16, flag, x0, x1, c, deadline, right, TCCL_W_TREE_UP);
            unpack(x0, x1, v);
#pragma unroll
            for (int e = 0; e < E; ++e) s[e] += v[e];
          }
          pack(s, d0, d1);
        }
        if (!ok) break;
        if (pslot) {
          put(pslot + i * 16, d0, d1, flag);
        } else {  // the root: d0, d1 are final
          if (ldown) put(ldown + i * 16, d0, d1, flag);
          if (rdown) put(rdown + i * 16, d0, d1, flag);
          if (res) *reinterpret_cast<uint2*>(res + (lo + i) * 8) = make_uint2(d0, d1);
          if (out) *reinterpret_cast<uint2*>(out + (lo + i) * 8) = make_uint2(d0, d1);
        }
      }
    } else if (parent >= 0) {
      const char* dslot = slot(c, me, tree, 2, k, g);
      char* ldown = left >= 0 ? slot(c, left, tree, 2, k, g) : nullptr;
      char* rdown = right >= 0 ? slot(c, right, tree, 2, k, g) : nullptr;
      for (uint64_t i = t; i < n && ok; i += nt) {
        uint32_t d0, d1;
        ok = get(dslot + i * 16, flag, d0, d1, c, deadline, parent, TCCL_W_TREE_DOWN);
        if (!ok) break;
        if (ldown) put(ldown + i * 16, d0, d1, flag);
        if (rdown) put(rdown + i * 16, d0, d1, flag);
        if (res) *reinterpret_cast<uint2*>(res + (lo + i) * 8) = make_uint2(d0, d1);
        if (out) *reinterpret_cast<uint2*>(out + (lo + i) * 8) = make_uint2(d0, d1);
      }
    }
    ok = __syncthreads_and(ok);
    if (ok && t == 0) *seq_word = g + 1u;
  }
};

}  // namespace tccl

using namespace tccl;

// One slot per pipeline: numel * sizeof(T) <= 2 trees * ctas_per_role * 32 KiB, ctas_per_role <=
// TCCL_TREE_LL_MAX_CTAS.  args->buf[rank] (this rank's own result buffer, for the in-place form) and
// args->out may each be null; the other entries of buf are not used.
extern "C" int tccl_allreduce_tree_ll(const tccl_comm* comm, const tccl_tree_args* args, const tccl_launch* l) {
  const int dtype = l->n_emu ? (l->meta & 0xff) : args->dtype;
  if (l->n_emu == 0) {
    const int K = args->ctas_per_role;
    const uint64_t esz = args->dtype == TCCL_F32 ? 4 : 2;
    if (K < 1 || K > TCCL_TREE_LL_MAX_CTAS || l->grid != 4 * K) return -TCCL_ESIZE;
    if (comm->tree_bytes < TCCL_TREE_LL_BYTES) return -TCCL_ESIZE;
    if (args->numel * esz > 2ull * K * (TCCL_TREE_LL_SLOT_BYTES / 2) || (args->numel * esz) % 16) return -TCCL_ESIZE;
  }
  switch (dtype) {
    case TCCL_BF16: return launch_op<TreeAllReduceLL<__nv_bfloat16>>(comm, args, l);
    case TCCL_F32: return launch_op<TreeAllReduceLL<float>>(comm, args, l);
    case TCCL_F16: return launch_op<TreeAllReduceLL<__half>>(comm, args, l);
    default: return -TCCL_EDTYPE;
  }
}
