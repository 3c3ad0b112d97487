// Pipelined double-binary-tree all-reduce, push form.
//
// The message is cut into chunks; chunk c travels over tree c % 2 (the two
// complementary trees of parallel/tree.py).  The grid is 4 K CTAs:
//   role 0/1 = "up" worker of tree 0/1, role 2/3 = "down" worker of tree 0/1,
// and CTA k of a role owns the k-th slice of every chunk of its tree, so each
// (tree, k) pair is an independent pipeline.
//
// Data only ever moves by posted STORES into the receiver's memory, followed by
// one release store of a counter — one NVLink crossing per tree level, where a
// pull design pays a flag crossing plus a load round trip:
//   up, chunk n:   a child stores its partial (own input + what its children
//                  stored into ITS ring) into slot [tree][child slot][k][n % D]
//                  of the PARENT's ring and bumps the parent's UP counter; the
//                  parent sums out of its own memory.  The root stores the final
//                  slice into its own result buffer and into its children's and
//                  bumps their DOWN counter.
//   down, chunk n: wait DOWN; the final slice is already in the own result
//                  buffer; store it on into the children's and bump their DOWN.
//   ring reuse:    after a parent has read slot n % D it bumps the child's ACK
//                  counter; a child stores chunk n only once ACK >= n + 1 - D.
// Each rank sends and receives what the reference's design intends — "two sends
// and two receives per GPU" — but for real: the reference's kernel
// (triton_double_tree_allreduce.py:227-335) never adds the children, never
// broadcasts down and cannot terminate.
//
// No entry and no exit barrier.  All counters count chunks since the
// communicator was created (each pipeline keeps its running total in local
// memory, TCCL_LOCAL_TREE_SEQ), so nothing is reset between calls; the ring is a
// region of its own with a layout that does not depend on the message
// ([tree][child slot][cta][n % D], fixed slice size), so a rank that is a call
// ahead can only touch a slot after the ACK that frees it; the input is read by
// its owner only; and a result buffer is written by the parent only after the
// owner has contributed the same chunk of the same call.
//
// Two forms of the way down.  Push (`kPullDown` false, the default): a parent
// stores the sum into its children's result buffers, as described above: one
// crossing per level.  Pull (`kPullDown` true): a parent only bumps its
// children's DOWN counter and each child LOADS the slice from the parent's
// result buffer, which moves the down traffic's issue from the parent's SMs
// (two children to serve) to the children's.  A parent whose buffer is pulled
// from must not return while a child may still be reading (its caller may
// overwrite the buffer next): each child acknowledges every slice it has pulled
// (DACK counter at the parent) and the parent's down worker waits for the last
// acknowledgement before it leaves.  Measured, pushing wins (512 MiB: 859 vs
// 963 us at 2 ranks, 1765 vs 1921 us at 8): the link is what both forms fill, and
// the pull adds a load round trip per slice.
//
// What a slice costs is protocol, not data: a flag crossing, and a release that
// waits until every store of the CTA has been acknowledged.  Hence large ring
// slices (TCCL_TREE_SLICE_BYTES) and ONE fence.acq_rel.sys per slice followed by
// relaxed stores of all the counters, instead of a st.release per counter.
//
// The element count must be a whole number of 16-byte vectors (the reference
// asks the same: triton_double_tree_allreduce.py:346-348).
#include "common.cuh"

namespace tccl {

constexpr int kTreeDepth = TCCL_TREE_RING_DEPTH;
constexpr uint64_t kTreeSlice = TCCL_TREE_SLICE_BYTES;

__host__ __device__ __forceinline__ int tree_max_ctas(uint64_t tree_bytes) {
  if (tree_bytes < TCCL_TREE_LL_BYTES) return 0;  // the small-message part comes first
  const uint64_t k = (tree_bytes - TCCL_TREE_LL_BYTES) / (4ull * kTreeDepth * kTreeSlice);
  return (int)(k < TCCL_TREE_MAX_CTAS ? k : TCCL_TREE_MAX_CTAS);
}

template <typename T, bool kPullDown>
struct TreeAllReduce {
  using Args = tccl_tree_args;
  static constexpr int kMaxThreads = 512, kMinBlocks = 1;
  static constexpr int U = 4;  // vectors in flight per thread and source

  static __device__ __forceinline__ uint32_t* up_flag(const tccl_comm& c, int rank, int tree, int k, int slot) {
    return c.flags[rank] + TCCL_FLAG_TREE_UP + ((tree * TCCL_TREE_MAX_CTAS + k) * 2 + slot);
  }
  static __device__ __forceinline__ uint32_t* down_flag(const tccl_comm& c, int rank, int tree, int k) {
    return c.flags[rank] + TCCL_FLAG_TREE_DOWN + (tree * TCCL_TREE_MAX_CTAS + k);
  }
  static __device__ __forceinline__ uint32_t* ack_flag(const tccl_comm& c, int rank, int tree, int k) {
    return c.flags[rank] + TCCL_FLAG_TREE_ACK + (tree * TCCL_TREE_MAX_CTAS + k);
  }
  // at the parent, written by the child in `slot`: slices of the way down that the child has pulled
  static __device__ __forceinline__ uint32_t* dack_flag(const tccl_comm& c, int rank, int tree, int k, int slot) {
    return c.flags[rank] + TCCL_FLAG_TREE_DACK + ((tree * TCCL_TREE_MAX_CTAS + k) * 2 + slot);
  }
  // ring slot of (tree, child slot, cta, chunk sequence number) in `rank`'s memory
  static __device__ __forceinline__ char* ring(const tccl_comm& c, int rank, int tree, int cslot, int k, uint32_t seq) {
    const int kmax = tree_max_ctas(c.tree_bytes);
    const uint64_t idx = ((uint64_t)((tree * 2 + cslot) * kmax + k)) * kTreeDepth + (seq % kTreeDepth);
    return c.stage[rank] + c.stage_bytes + c.ll_bytes + TCCL_TREE_LL_BYTES + idx * kTreeSlice;
  }

  static __device__ void run(const tccl_comm& c, const Args& a, int bid, int nb) {
    const uint64_t deadline = globaltimer() + c.timeout_ns;
    const int K = a.ctas_per_role;
    const int role = bid / K, k = bid - role * K;
    const int tree = role & 1;
    const bool is_up = role < 2;
    const int parent = a.parent[tree], left = a.left[tree], right = a.right[tree];
    const int me = c.rank;
    constexpr int VPT = 16 / (int)sizeof(T);
    const uint64_t nvec = a.numel / VPT;
    const uint64_t cv = a.chunk_vecs;
    const uint64_t nchunks = (nvec + cv - 1) / cv;                                  // all chunks
    const uint64_t mine = nchunks > (uint64_t)tree ? (nchunks - tree + 1) / 2 : 0;  // chunks of my tree
    const char* in = reinterpret_cast<const char*>(a.in);
    char* res = reinterpret_cast<char*>(a.buf[me]);
    char* lres = left >= 0 ? reinterpret_cast<char*>(a.buf[left]) : nullptr;
    char* rres = right >= 0 ? reinterpret_cast<char*>(a.buf[right]) : nullptr;
    char* out = reinterpret_cast<char*>(a.out);
    const int t = threadIdx.x, nt = blockDim.x;
    uint32_t* seq_word = c.local + TCCL_LOCAL_TREE_SEQ + role * TCCL_TREE_MAX_CTAS + k;
    const uint32_t base = *seq_word;  // chunks this pipeline has moved in earlier calls
    const int cslot = a.child_slot[tree];

    bool ok = true;
    if (is_up) {
      for (uint64_t n = 0; n < mine && ok; ++n) {
        const uint32_t g = base + (uint32_t)n;  // running chunk number of this pipeline
        // the children's partials are in my ring; the slot I am about to fill at the parent is free
        if (t < 2) {
          const int kid = t == 0 ? left : right;
          if (kid >= 0) ok = wait_reach(up_flag(c, me, tree, k, t), g + 1u, c, deadline, kid, TCCL_W_TREE_UP);
        } else if (t == 2 && parent >= 0) {
          ok = wait_reach(ack_flag(c, me, tree, k), g + 1u - (uint32_t)kTreeDepth, c, deadline, parent, TCCL_W_TREE_UP);
        }
        ok = __syncthreads_and(ok);
        if (!ok) break;
        const uint64_t clo = (2 * n + tree) * cv, chi = min(clo + cv, nvec);
        const uint64_t per = (chi - clo + K - 1) / K, lo = min(clo + per * k, chi), hi = min(lo + per, chi);
        const char* lring = left >= 0 ? ring(c, me, tree, 0, k, g) : nullptr;
        const char* rring = right >= 0 ? ring(c, me, tree, 1, k, g) : nullptr;
        char* pring = parent >= 0 ? ring(c, parent, tree, cslot, k, g) : nullptr;
        for (uint64_t i0 = lo + t; i0 < hi; i0 += (uint64_t)U * nt) {
          Vec16 vo[U], vl[U], vr[U];
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint64_t i = i0 + (uint64_t)u * nt;
            if (i < hi) {
              vo[u] = ld_peer(in + i * 16);
              if (lring) vl[u] = ld_peer(lring + (i - lo) * 16);
              if (rring) vr[u] = ld_peer(rring + (i - lo) * 16);
            }
          }
#pragma unroll
          for (int u = 0; u < U; ++u) {
            const uint64_t i = i0 + (uint64_t)u * nt;
            if (i < hi) {
              Vec16 r = vo[u];
              if (lring) {
                Acc<T> acc;
                acc.zero();
                acc.add(vo[u]);
                acc.add(vl[u]);
                if (rring) acc.add(vr[u]);
                r = acc.pack();
              }
              if (pring) {
                st_peer(pring + (i - lo) * 16, r);
              } else {  // the root: this is the final value
                st_peer(res + i * 16, r);
                if (!kPullDown) {
                  if (lres) st_peer(lres + i * 16, r);
                  if (rres) st_peer(rres + i * 16, r);
                }
                if (out) st_local(out + i * 16, r);
              }
            }
          }
        }
        __syncthreads();  // every thread has used what it loaded and issued its stores
        if (t == 0) {
          // ONE release fence (it waits until the CTA's stores have been performed; a per-flag
          // st.release would pay that once per flag), then the counters as relaxed stores
          fence_acq_rel_sys();
          if (parent >= 0) {
            st_relaxed_sys(up_flag(c, parent, tree, k, cslot), g + 1u);
          } else {
            if (left >= 0) st_relaxed_sys(down_flag(c, left, tree, k), g + 1u);
            if (right >= 0) st_relaxed_sys(down_flag(c, right, tree, k), g + 1u);
          }
          if (left >= 0) st_relaxed_sys(ack_flag(c, left, tree, k), g + 1u);
          if (right >= 0) st_relaxed_sys(ack_flag(c, right, tree, k), g + 1u);
        }
      }
    } else {
      const char* pres = parent >= 0 ? reinterpret_cast<const char*>(a.buf[parent]) : nullptr;
      for (uint64_t n = 0; parent >= 0 && n < mine && ok; ++n) {
        const uint32_t g = base + (uint32_t)n;
        if (t == 0) ok = wait_reach(down_flag(c, me, tree, k), g + 1u, c, deadline, parent, TCCL_W_TREE_DOWN);
        ok = __syncthreads_and(ok);
        if (!ok) break;
        if (kPullDown || lres || out) {
          const uint64_t clo = (2 * n + tree) * cv, chi = min(clo + cv, nvec);
          const uint64_t per = (chi - clo + K - 1) / K, lo = min(clo + per * k, chi), hi = min(lo + per, chi);
          constexpr int UD = 8;
          // pull: the slice is in the PARENT's result buffer; push: it is already in the own one
          const char* src = kPullDown ? pres : res;
          for (uint64_t i0 = lo + t; i0 < hi; i0 += (uint64_t)UD * nt) {
            Vec16 v[UD];
#pragma unroll
            for (int u = 0; u < UD; ++u) {
              const uint64_t i = i0 + (uint64_t)u * nt;
              if (i < hi) v[u] = ld_peer(src + i * 16);
            }
#pragma unroll
            for (int u = 0; u < UD; ++u) {
              const uint64_t i = i0 + (uint64_t)u * nt;
              if (i < hi) {
                if (kPullDown) {
                  st_peer(res + i * 16, v[u]);  // own buffer: the children pull it from here
                } else {
                  if (lres) st_peer(lres + i * 16, v[u]);
                  if (rres) st_peer(rres + i * 16, v[u]);
                }
                if (out) st_local(out + i * 16, v[u]);
              }
            }
          }
          __syncthreads();  // every thread's loads are complete (their values were stored) and its stores issued
          if (t == 0) {
            fence_acq_rel_sys();
            if (left >= 0) st_relaxed_sys(down_flag(c, left, tree, k), g + 1u);
            if (right >= 0) st_relaxed_sys(down_flag(c, right, tree, k), g + 1u);
            // pull: this slice of the parent's buffer is no longer needed
            if (kPullDown) st_relaxed_sys(dack_flag(c, parent, tree, k, cslot), g + 1u);
          }
        }
      }
      if (kPullDown && ok && mine) {
        // nobody may still be loading from this rank's result buffer when the kernel returns
        if (t < 2) {
          const int kid = t == 0 ? left : right;
          if (kid >= 0)
            ok = wait_reach(dack_flag(c, me, tree, k, t), base + (uint32_t)mine, c, deadline, kid, TCCL_W_TREE_DOWN);
        }
        ok = __syncthreads_and(ok);
      }
    }
    if (ok && t == 0) *seq_word = base + (uint32_t)mine;
  }
};

}  // namespace tccl

using namespace tccl;

extern "C" int tccl_tree_max_ctas(uint64_t tree_bytes) { return tree_max_ctas(tree_bytes); }

extern "C" int tccl_allreduce_tree(const tccl_comm* comm, const tccl_tree_args* args, const tccl_launch* l) {
  const int dtype = l->n_emu ? (l->meta & 0xff) : args->dtype;
  if (l->n_emu == 0) {
    const int K = args->ctas_per_role;
    if (K < 1 || K > tree_max_ctas(comm->tree_bytes) || l->grid != 4 * K) return -TCCL_ESIZE;
    if (args->chunk_vecs < 1 || args->chunk_vecs > (uint64_t)K * (TCCL_TREE_SLICE_BYTES / 16)) return -TCCL_ESIZE;
  }
  if (l->meta & TCCL_TREE_PULL_DOWN) {  // on request: children load the sum from their parent
    switch (dtype) {
      case TCCL_BF16: return launch_op<TreeAllReduce<__nv_bfloat16, true>>(comm, args, l);
      case TCCL_F32: return launch_op<TreeAllReduce<float, true>>(comm, args, l);
      case TCCL_F16: return launch_op<TreeAllReduce<__half, true>>(comm, args, l);
      default: return -TCCL_EDTYPE;
    }
  }
  switch (dtype) {
    case TCCL_BF16: return launch_op<TreeAllReduce<__nv_bfloat16, false>>(comm, args, l);
    case TCCL_F32: return launch_op<TreeAllReduce<float, false>>(comm, args, l);
    case TCCL_F16: return launch_op<TreeAllReduce<__half, false>>(comm, args, l);
    default: return -TCCL_EDTYPE;
  }
}
