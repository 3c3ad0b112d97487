// all-reduce + bias + residual add + RMSNorm in ONE kernel (two-shot over token
// rows): rank r owns rows [r T/W, (r+1) T/W).  For each owned row a CTA sums the
// W partial rows (multimem.ld_reduce through the switch, or W peer loads with
// fp32 accumulation), adds bias and residual, reduces sum(v^2) over the row in
// the CTA, scales by rsqrt(mean + eps) * weight and stores the normalised row to
// EVERY rank's output (one multimem.st, or W posted stores); the pre-norm sum can
// be broadcast the same way as the next layer's residual.  The row lives in
// registers between the reduction and the normalisation, so the all-reduced
// activations never make an extra trip through HBM, and the unfused sequence
// (all-reduce kernel, then an elementwise kernel, then a norm kernel) collapses
// into one launch with one entry and one exit barrier.
//
// The reference's all-reduce is a stand-alone one-shot kernel (triton_one_shot_all_reduce_no_128.py:35-96);
// fusing collectives with the compute around them is the goal its presentation names (presentation.pdf, slide 4).
#include "common.cuh"

namespace tccl {

template <typename T, bool kNvls, int MV>
struct AllReduceRmsNorm {
  using Args = tccl_arn_args;
  // MV = 16-byte vectors per thread (hidden <= 512 * MV * (16 / sizeof(T))).  With one
  // vector per thread the kernel is small enough for two CTAs per SM: twice the rows in
  // flight, which is what hides the peer-load and barrier latency of a row.
  static constexpr int kMaxThreads = 512, kMinBlocks = MV == 1 ? 2 : 1;
  static constexpr int kMaxVec = MV;
  // rows handled together by a CTA: all their loads are issued before the first
  // reduction, so a CTA pays the peer-load / switch latency once per R rows
  // (measured on 8xB200, 4096 x 4096 bf16: R = 1 with two CTAs per SM beats R = 4 with fewer CTAs)
  static constexpr int R = 1;
  static constexpr int VPT = 16 / (int)sizeof(T);

  static __device__ __forceinline__ void unpack(const Vec16& v, float* f) {
    Acc<T> a;
    a.zero();
    a.add(v);
#pragma unroll
    for (int i = 0; i < VPT; ++i) f[i] = a.a[i];
  }
  static __device__ __forceinline__ Vec16 pack(const float* f) {
    Acc<T> a;
#pragma unroll
    for (int i = 0; i < VPT; ++i) a.a[i] = f[i];
    return a.pack();
  }

  static __device__ void run(const tccl_comm& c, const Args& a, int bid, int nb) {
    __shared__ float s_part[R][16];
    __shared__ float s_scale[R];
    const uint64_t deadline = globaltimer() + c.timeout_ns;
    const bool nvls_bar = (a.flags & TCCL_F_NVLS_BARRIER) != 0;
    barrier_any(c, bid, deadline, nvls_bar);
    const int W = c.world, me = c.rank;
    const int H = a.hidden, nvec = H / VPT;
    const int per = (a.tokens + W - 1) / W;
    const int row_lo = min(per * me, a.tokens), row_hi = min(row_lo + per, a.tokens);
    const int t = threadIdx.x, nt = blockDim.x;
    const int warp = t >> 5, lane = t & 31, nwarps = nt >> 5;
    for (int row0 = row_lo + bid * R; row0 < row_hi; row0 += nb * R) {
      float v[R][kMaxVec][VPT];
      float ss[R];
      // phase 1: fetch and sum the partial rows (all R rows in flight at once)
#pragma unroll
      for (int q = 0; q < R; ++q) {
        const int row = row0 + q;
        ss[q] = 0.f;
        if (row < row_hi) {
          const size_t rbase = (size_t)row * H * sizeof(T);
#pragma unroll
          for (int j = 0; j < kMaxVec; ++j) {
            const int i = t + j * nt;
            if (i < nvec) {
              const size_t off = rbase + (size_t)i * 16;
              if (kNvls) {
                unpack(MultimemOps<T>::ld_reduce(reinterpret_cast<const char*>(a.mc_x) + off), v[q][j]);
              } else {
                Acc<T> acc;
                acc.zero();
                for (int p = 0; p < W; ++p) acc.add(ld_peer(reinterpret_cast<const char*>(a.x[p]) + off));
#pragma unroll
                for (int e = 0; e < VPT; ++e) v[q][j][e] = acc.a[e];
              }
            }
          }
        }
      }
      // phase 2: bias, residual, optional pre-norm output, sum of squares
#pragma unroll
      for (int q = 0; q < R; ++q) {
        const int row = row0 + q;
        if (row < row_hi) {
          const size_t rbase = (size_t)row * H * sizeof(T);
#pragma unroll
          for (int j = 0; j < kMaxVec; ++j) {
            const int i = t + j * nt;
            if (i < nvec) {
              const size_t off = rbase + (size_t)i * 16;
              float b[VPT], r[VPT];
              if (a.bias) {
                unpack(ld_peer(reinterpret_cast<const char*>(a.bias) + (size_t)i * 16), b);
#pragma unroll
                for (int e = 0; e < VPT; ++e) v[q][j][e] += b[e];
              }
              if (a.residual) {
                unpack(ld_peer(reinterpret_cast<const char*>(a.residual) + off), r);
#pragma unroll
                for (int e = 0; e < VPT; ++e) v[q][j][e] += r[e];
              }
              if (a.res_out[0]) {
                // the next layer's residual is the sum rounded to T; normalise what was stored
                const Vec16 pk = pack(v[q][j]);
                if (kNvls) {
                  multimem_st(reinterpret_cast<char*>(a.mc_res_out) + off, pk);
                } else {
                  for (int p = 0; p < W; ++p) st_peer(reinterpret_cast<char*>(a.res_out[p]) + off, pk);
                }
                unpack(pk, v[q][j]);
              }
#pragma unroll
              for (int e = 0; e < VPT; ++e) ss[q] += v[q][j][e] * v[q][j][e];
            }
          }
        }
        // sum of squares over the row: warp shuffle, then across warps through shared memory
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss[q] += __shfl_xor_sync(0xffffffffu, ss[q], o);
        if (lane == 0) s_part[q][warp] = ss[q];
      }
      __syncthreads();
      if (warp < R) {
        float tot = lane < nwarps ? s_part[warp][lane] : 0.f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) tot += __shfl_xor_sync(0xffffffffu, tot, o);
        if (lane == 0) s_scale[warp] = rsqrtf(tot / (float)H + a.eps);
      }
      __syncthreads();
      // phase 3: normalise and store to every rank
#pragma unroll
      for (int q = 0; q < R; ++q) {
        const int row = row0 + q;
        if (row < row_hi) {
          const size_t rbase = (size_t)row * H * sizeof(T);
          const float scale = s_scale[q];
#pragma unroll
          for (int j = 0; j < kMaxVec; ++j) {
            const int i = t + j * nt;
            if (i < nvec) {
              float wv[VPT], o[VPT];
              unpack(ld_peer(reinterpret_cast<const char*>(a.weight) + (size_t)i * 16), wv);
#pragma unroll
              for (int e = 0; e < VPT; ++e) o[e] = v[q][j][e] * scale * wv[e];
              const Vec16 pk = pack(o);
              const size_t off = rbase + (size_t)i * 16;
              if (kNvls) {
                multimem_st(reinterpret_cast<char*>(a.mc_out) + off, pk);
              } else {
                for (int p = 0; p < W; ++p) st_peer(reinterpret_cast<char*>(a.out[p]) + off, pk);
              }
            }
          }
        }
      }
      __syncthreads();  // s_part / s_scale are reused by the next batch of rows
    }
    barrier_any(c, bid, deadline, nvls_bar);  // every rank's rows have landed everywhere
  }
};

}  // namespace tccl

using namespace tccl;

template <typename T, bool kNvls>
static int launch_by_width(const tccl_comm* comm, const tccl_arn_args* args, const tccl_launch* l, int hidden) {
  const int nvec = hidden / (16 / (int)sizeof(T));
  if (nvec <= 512) return launch_op<AllReduceRmsNorm<T, kNvls, 1>>(comm, args, l);
  if (nvec <= 1024) return launch_op<AllReduceRmsNorm<T, kNvls, 2>>(comm, args, l);
  if (nvec <= 2048) return launch_op<AllReduceRmsNorm<T, kNvls, 4>>(comm, args, l);
  return -TCCL_ESIZE;
}

// `hidden` is passed separately because in emulated mode `args` is a device pointer.
extern "C" int tccl_allreduce_bias_residual_rmsnorm(const tccl_comm* comm, const tccl_arn_args* args, int nvls,
                                                    int hidden, const tccl_launch* l) {
  const int dtype = l->n_emu ? (l->meta & 0xff) : args->dtype;
  if (nvls) {
    switch (dtype) {
      case TCCL_BF16: return launch_by_width<__nv_bfloat16, true>(comm, args, l, hidden);
      case TCCL_F16: return launch_by_width<__half, true>(comm, args, l, hidden);
      case TCCL_F32: return launch_by_width<float, true>(comm, args, l, hidden);
      default: return -TCCL_EDTYPE;
    }
  }
  switch (dtype) {
    case TCCL_BF16: return launch_by_width<__nv_bfloat16, false>(comm, args, l, hidden);
    case TCCL_F16: return launch_by_width<__half, false>(comm, args, l, hidden);
    case TCCL_F32: return launch_by_width<float, false>(comm, args, l, hidden);
    default: return -TCCL_EDTYPE;
  }
}
