// Pipelined double-binary-tree all-reduce, in place in the symmetric buffers.
//
// The message is cut into chunks; chunk c travels over tree c % 2 (the two
// complementary trees of parallel/tree.py).  The grid is 4 K CTAs:
//   role 0/1 = "up" worker of tree 0/1, role 2/3 = "down" worker of tree 0/1,
// and CTA k of a role owns the k-th slice of every chunk of its tree, so each
// (tree, k) pair is an independent pipeline with its own counters:
//   UP[tree][k][slot]  written by the child in `slot`: chunks whose partial is in place
//   DOWN[tree][k]      written by the parent: chunks whose final value is in place
// Up worker, chunk n:   wait UP >= n+1 for each child; partial = own + children
//                       (pulled from the children's buffers); store in place;
//                       bump the parent's UP — the root bumps its child's DOWN.
// Down worker, chunk n: wait DOWN >= n+1; pull the final slice from the
//                       parent's buffer into the own buffer (and `out`); bump
//                       the children's DOWN.
// Up workers never wait for down workers, so the two phases of different chunks
// overlap and the pipeline depth is bounded only by the message.  Each rank
// sends and receives what the reference's design intends — "two sends and two
// receives per GPU" — but for real: the reference's kernel
// (triton_double_tree_allreduce.py:227-335) never adds the children, never
// broadcasts down and cannot terminate.
//
// The element count must be a whole number of 16-byte vectors (the reference
// asks the same: triton_double_tree_allreduce.py:346-348).
//
// All counters live in the waiter's flag region, are written with release
// stores by a single producer, polled with acquire loads, and are zeroed by
// their owner before the exit barrier, so a launch always starts from zero.
#include "common.cuh"

namespace tccl {

template <typename T>
struct TreeAllReduce {
  using Args = tccl_tree_args;
  static constexpr int kMaxThreads = 512, kMinBlocks = 1;
  static constexpr int U = 4;   // vectors in flight per thread and source, up phase
  static constexpr int UD = 8;  // down phase (one source)

  static __device__ __forceinline__ uint32_t* up_flag(const tccl_comm& c, int rank, int tree, int k, int slot) {
    return c.flags[rank] + TCCL_FLAG_TREE_UP + ((tree * TCCL_TREE_MAX_CTAS + k) * 2 + slot);
  }
  static __device__ __forceinline__ uint32_t* down_flag(const tccl_comm& c, int rank, int tree, int k) {
    return c.flags[rank] + TCCL_FLAG_TREE_DOWN + (tree * TCCL_TREE_MAX_CTAS + k);
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
    const uint64_t nchunks = (nvec + cv - 1) / cv;                    // all chunks
    const uint64_t mine = nchunks > (uint64_t)tree ? (nchunks - tree + 1) / 2 : 0;  // chunks of my tree
    char* own = reinterpret_cast<char*>(a.buf[me]);
    const char* lbuf = left >= 0 ? reinterpret_cast<const char*>(a.buf[left]) : nullptr;
    const char* rbuf = right >= 0 ? reinterpret_cast<const char*>(a.buf[right]) : nullptr;
    const char* pbuf = parent >= 0 ? reinterpret_cast<const char*>(a.buf[parent]) : nullptr;
    char* out = reinterpret_cast<char*>(a.out);
    const int t = threadIdx.x, nt = blockDim.x;

    barrier_p2p(c, bid, deadline);  // every rank's buffer is ready, every counter is zero

    bool ok = true;
    if (is_up) {
      const bool leaf = left < 0 && right < 0;
      if (leaf) {
        // nothing to add: every chunk of a leaf is "published" from the start
        if (t == 0 && parent >= 0 && mine) st_release_sys(up_flag(c, parent, tree, k, a.child_slot[tree]), (uint32_t)mine);
        if (parent < 0 && out) {  // world of one rank: the result is the input
          for (uint64_t n = 0; n < mine; ++n) {
            const uint64_t clo = (2 * n + tree) * cv, chi = min(clo + cv, nvec);
            const uint64_t per = (chi - clo + K - 1) / K, lo = min(clo + per * k, chi), hi = min(lo + per, chi);
            for (uint64_t i = lo + t; i < hi; i += nt) st_local(out + i * 16, ld_peer(own + i * 16));
          }
        }
      } else {
        for (uint64_t n = 0; n < mine && ok; ++n) {
          if (t < 2) {
            const int kid = t == 0 ? left : right;
            if (kid >= 0) ok = wait_reach(up_flag(c, me, tree, k, t), (uint32_t)(n + 1), c, deadline, kid, TCCL_W_TREE_UP);
          }
          ok = __syncthreads_and(ok);
          if (!ok) break;
          const uint64_t clo = (2 * n + tree) * cv, chi = min(clo + cv, nvec);
          const uint64_t per = (chi - clo + K - 1) / K, lo = min(clo + per * k, chi), hi = min(lo + per, chi);
          uint64_t i = lo + t;
          for (; i + (U - 1) * (uint64_t)nt < hi; i += (uint64_t)U * nt) {
            Vec16 vo[U], vl[U], vr[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const uint64_t off = (i + (uint64_t)u * nt) * 16;
              vo[u] = ld_peer(own + off);
              vl[u] = ld_peer(lbuf + off);
              if (rbuf) vr[u] = ld_peer(rbuf + off);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
              const uint64_t off = (i + (uint64_t)u * nt) * 16;
              Acc<T> acc;
              acc.zero();
              acc.add(vo[u]);
              acc.add(vl[u]);
              if (rbuf) acc.add(vr[u]);
              const Vec16 r = acc.pack();
              st_peer(own + off, r);
              if (parent < 0 && out) st_local(out + off, r);
            }
          }
          for (; i < hi; i += nt) {
            Acc<T> acc;
            acc.zero();
            acc.add(ld_peer(own + i * 16));
            acc.add(ld_peer(lbuf + i * 16));
            if (rbuf) acc.add(ld_peer(rbuf + i * 16));
            const Vec16 r = acc.pack();
            st_peer(own + i * 16, r);
            if (parent < 0 && out) st_local(out + i * 16, r);
          }
          __syncthreads();  // the whole slice is stored before the release below
          if (t == 0) {
            if (parent >= 0) {
              st_release_sys(up_flag(c, parent, tree, k, a.child_slot[tree]), (uint32_t)(n + 1));
            } else {
              st_release_sys(down_flag(c, left, tree, k), (uint32_t)(n + 1));
              if (right >= 0) st_release_sys(down_flag(c, right, tree, k), (uint32_t)(n + 1));
            }
          }
        }
      }
    } else if (parent >= 0) {
      for (uint64_t n = 0; n < mine && ok; ++n) {
        if (t == 0) ok = wait_reach(down_flag(c, me, tree, k), (uint32_t)(n + 1), c, deadline, parent, TCCL_W_TREE_DOWN);
        ok = __syncthreads_and(ok);
        if (!ok) break;
        const uint64_t clo = (2 * n + tree) * cv, chi = min(clo + cv, nvec);
        const uint64_t per = (chi - clo + K - 1) / K, lo = min(clo + per * k, chi), hi = min(lo + per, chi);
        uint64_t i = lo + t;
        for (; i + (UD - 1) * (uint64_t)nt < hi; i += (uint64_t)UD * nt) {
          Vec16 v[UD];
#pragma unroll
          for (int u = 0; u < UD; ++u) v[u] = ld_peer(pbuf + (i + (uint64_t)u * nt) * 16);
#pragma unroll
          for (int u = 0; u < UD; ++u) {
            const uint64_t off = (i + (uint64_t)u * nt) * 16;
            st_peer(own + off, v[u]);
            if (out) st_local(out + off, v[u]);
          }
        }
        for (; i < hi; i += nt) {
          const Vec16 v = ld_peer(pbuf + i * 16);
          st_peer(own + i * 16, v);
          if (out) st_local(out + i * 16, v);
        }
        __syncthreads();
        if (t == 0) {
          if (left >= 0) st_release_sys(down_flag(c, left, tree, k), (uint32_t)(n + 1));
          if (right >= 0) st_release_sys(down_flag(c, right, tree, k), (uint32_t)(n + 1));
        }
      }
    }

    // zero the counters this CTA consumed, then leave together
    __syncthreads();
    if (t == 0) {
      if (is_up) {
        st_relaxed_sys(up_flag(c, me, tree, k, 0), 0u);
        st_relaxed_sys(up_flag(c, me, tree, k, 1), 0u);
      } else {
        st_relaxed_sys(down_flag(c, me, tree, k), 0u);
      }
    }
    barrier_p2p(c, bid, deadline);
  }
};

}  // namespace tccl

using namespace tccl;

extern "C" int tccl_allreduce_tree(const tccl_comm* comm, const tccl_tree_args* args, const tccl_launch* l) {
  const int dtype = l->n_emu ? (l->meta & 0xff) : args->dtype;
  switch (dtype) {
    case TCCL_BF16: return launch_op<TreeAllReduce<__nv_bfloat16>>(comm, args, l);
    case TCCL_F32: return launch_op<TreeAllReduce<float>>(comm, args, l);
    case TCCL_F16: return launch_op<TreeAllReduce<__half>>(comm, args, l);
    default: return -TCCL_EDTYPE;
  }
}
