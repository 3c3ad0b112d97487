// Host build of the synchronisation protocols (CPU ranks over POSIX shared
// memory, C++ acquire/release atomics in place of the PTX ones): the epoch
// barrier and the pipelined double-tree all-reduce, with the same flag layout
// (tccl_b200.h), the same bounded waits and the same status words as the
// device kernels, plus switches that inject faults — a rank that never sends
// one signal, a rank that stalls, a rank that stops half way.  Failure handling
// is tested here, on the host, because a GPU must never be hung or faulted on
// purpose.  The reference has neither timeouts nor fault tests: all its spins
// are unbounded (triton_barrier.py:108-118).
#include <atomic>
#include <chrono>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

#include "../tccl_b200.h"

namespace {

using clk = std::chrono::steady_clock;

struct HostComm {
  int world, rank;
  uint32_t* flags[TCCL_MAX_WORLD];  // every rank's flag region (shared memory)
  uint32_t* local;                  // this rank's private words
  uint64_t timeout_ns;
};

inline std::atomic<uint32_t>& A(uint32_t* p) { return *reinterpret_cast<std::atomic<uint32_t>*>(p); }

void record_failure(const HostComm& c, int code, int block, int peer, int where, uint32_t seen, uint32_t want) {
  uint32_t* st = c.local + TCCL_LOCAL_STATUS;
  uint32_t expected = 0;
  if (A(st + TCCL_ST_CODE).compare_exchange_strong(expected, (uint32_t)code)) {
    st[TCCL_ST_BLOCK] = (uint32_t)block;
    st[TCCL_ST_PEER] = (uint32_t)peer;
    st[TCCL_ST_WHERE] = (uint32_t)where;
    st[TCCL_ST_SEEN] = seen;
    st[TCCL_ST_WANT] = want;
  }
  A(st + TCCL_ST_ABORT).store(1u, std::memory_order_release);
}
inline bool aborted(const HostComm& c) {
  return A(c.local + TCCL_LOCAL_STATUS + TCCL_ST_ABORT).load(std::memory_order_relaxed) != 0;
}

// same contract as the device wait_reach(): acquire-poll until the flag reaches `want`
// (wrap-around order), give up at the deadline or as soon as this rank has aborted
bool wait_reach(uint32_t* flag, uint32_t want, const HostComm& c, clk::time_point deadline, int block, int peer,
                int where) {
  uint32_t spins = 0;
  for (;;) {
    const uint32_t v = A(flag).load(std::memory_order_acquire);
    if ((int32_t)(v - want) >= 0) return true;
    if ((++spins & 63u) == 0u) {
      if (aborted(c)) return false;
      if (clk::now() > deadline) {
        record_failure(c, TCCL_TIMEOUT, block, peer, where, v, want);
        return false;
      }
      std::this_thread::yield();
    }
  }
}

struct Faults {
  int drop_signal_to;   // barrier: never signal this peer (-1 = none)
  int stall_ms;         // sleep this long before signalling
  int stop_after_chunk; // tree: stop taking part after this many chunks (-1 = never)
};

bool barrier(const HostComm& c, int bid, clk::time_point deadline, const Faults& f) {
  const uint32_t e = c.local[TCCL_LOCAL_EPOCH + bid] + 1u;
  if (f.stall_ms > 0) std::this_thread::sleep_for(std::chrono::milliseconds(f.stall_ms));
  for (int p = 0; p < c.world; ++p) {
    if (p == f.drop_signal_to) continue;  // injected fault: the signal is lost
    A(c.flags[p] + TCCL_FLAG_BAR + bid * TCCL_MAX_WORLD + c.rank).store(e, std::memory_order_release);
  }
  bool ok = true;
  for (int p = 0; p < c.world && ok; ++p)
    ok = wait_reach(c.flags[c.rank] + TCCL_FLAG_BAR + bid * TCCL_MAX_WORLD + p, e, c, deadline, bid, p, TCCL_W_BARRIER);
  c.local[TCCL_LOCAL_EPOCH + bid] = e;
  return ok;
}

uint32_t* up_flag(const HostComm& c, int rank, int tree, int k, int slot) {
  return c.flags[rank] + TCCL_FLAG_TREE_UP + ((tree * TCCL_TREE_MAX_CTAS + k) * 2 + slot);
}
uint32_t* down_flag(const HostComm& c, int rank, int tree, int k) {
  return c.flags[rank] + TCCL_FLAG_TREE_DOWN + (tree * TCCL_TREE_MAX_CTAS + k);
}

struct TreeJob {
  float* buf[TCCL_MAX_WORLD];
  uint64_t numel, chunk;
  int parent[2], left[2], right[2], child_slot[2];
};

// one (tree, direction) worker = what one CTA does on the device (K = 1 slice)
void tree_worker(const HostComm& c, const TreeJob& j, int tree, bool is_up, clk::time_point deadline, const Faults& f) {
  const int me = c.rank, parent = j.parent[tree], left = j.left[tree], right = j.right[tree];
  const uint64_t nchunks = (j.numel + j.chunk - 1) / j.chunk;
  const uint64_t mine = nchunks > (uint64_t)tree ? (nchunks - tree + 1) / 2 : 0;
  float* own = j.buf[me];
  if (is_up) {
    const bool leaf = left < 0 && right < 0;
    if (leaf) {
      if (parent >= 0 && mine && f.stop_after_chunk != 0)
        A(up_flag(c, parent, tree, 0, j.child_slot[tree])).store(
            (uint32_t)(f.stop_after_chunk > 0 && (uint64_t)f.stop_after_chunk < mine ? f.stop_after_chunk : mine),
            std::memory_order_release);
      return;
    }
    for (uint64_t n = 0; n < mine; ++n) {
      if (f.stop_after_chunk >= 0 && n >= (uint64_t)f.stop_after_chunk) return;  // injected: this rank stops here
      if (!wait_reach(up_flag(c, me, tree, 0, 0), (uint32_t)(n + 1), c, deadline, tree, left, TCCL_W_TREE_UP)) return;
      if (right >= 0 &&
          !wait_reach(up_flag(c, me, tree, 0, 1), (uint32_t)(n + 1), c, deadline, tree, right, TCCL_W_TREE_UP))
        return;
      const uint64_t lo = (2 * n + tree) * j.chunk, hi = std::min(lo + j.chunk, j.numel);
      for (uint64_t i = lo; i < hi; ++i) own[i] += j.buf[left][i] + (right >= 0 ? j.buf[right][i] : 0.f);
      if (parent >= 0) {
        A(up_flag(c, parent, tree, 0, j.child_slot[tree])).store((uint32_t)(n + 1), std::memory_order_release);
      } else {
        A(down_flag(c, left, tree, 0)).store((uint32_t)(n + 1), std::memory_order_release);
        if (right >= 0) A(down_flag(c, right, tree, 0)).store((uint32_t)(n + 1), std::memory_order_release);
      }
    }
  } else if (parent >= 0) {
    for (uint64_t n = 0; n < mine; ++n) {
      if (f.stop_after_chunk >= 0 && n >= (uint64_t)f.stop_after_chunk) return;
      if (!wait_reach(down_flag(c, me, tree, 0), (uint32_t)(n + 1), c, deadline, 2 + tree, parent, TCCL_W_TREE_DOWN))
        return;
      const uint64_t lo = (2 * n + tree) * j.chunk, hi = std::min(lo + j.chunk, j.numel);
      std::memcpy(own + lo, j.buf[parent] + lo, (hi - lo) * sizeof(float));
      if (left >= 0) A(down_flag(c, left, tree, 0)).store((uint32_t)(n + 1), std::memory_order_release);
      if (right >= 0) A(down_flag(c, right, tree, 0)).store((uint32_t)(n + 1), std::memory_order_release);
    }
  }
}

}  // namespace

extern "C" {

struct hp_comm {
  int32_t world, rank;
  uint64_t flags[TCCL_MAX_WORLD];
  uint64_t local;
  uint64_t timeout_ns;
};
struct hp_faults {
  int32_t drop_signal_to, stall_ms, stop_after_chunk;
};
struct hp_tree {
  uint64_t buf[TCCL_MAX_WORLD];
  uint64_t numel, chunk;
  int32_t parent[2], left[2], right[2], child_slot[2];
};

static HostComm to_comm(const hp_comm* h) {
  HostComm c;
  c.world = h->world;
  c.rank = h->rank;
  for (int p = 0; p < TCCL_MAX_WORLD; ++p) c.flags[p] = reinterpret_cast<uint32_t*>(h->flags[p]);
  c.local = reinterpret_cast<uint32_t*>(h->local);
  c.timeout_ns = h->timeout_ns;
  return c;
}

// returns 1 on success, 0 if a wait gave up (see the status words)
int hp_barrier(const hp_comm* h, int bid, int rounds, const hp_faults* f) {
  HostComm c = to_comm(h);
  Faults ft{f ? f->drop_signal_to : -1, f ? f->stall_ms : 0, -1};
  const auto deadline = clk::now() + std::chrono::nanoseconds(c.timeout_ns);
  for (int i = 0; i < rounds; ++i)
    if (!barrier(c, bid, deadline, ft)) return 0;
  return 1;
}

// pipelined double-tree all-reduce in place over float buffers in shared memory
int hp_tree_allreduce(const hp_comm* h, const hp_tree* t, const hp_faults* f) {
  HostComm c = to_comm(h);
  Faults ft{-1, f ? f->stall_ms : 0, f ? f->stop_after_chunk : -1};
  Faults none{-1, 0, -1};
  TreeJob j;
  for (int p = 0; p < TCCL_MAX_WORLD; ++p) j.buf[p] = reinterpret_cast<float*>(t->buf[p]);
  j.numel = t->numel;
  j.chunk = t->chunk;
  for (int i = 0; i < 2; ++i) {
    j.parent[i] = t->parent[i];
    j.left[i] = t->left[i];
    j.right[i] = t->right[i];
    j.child_slot[i] = t->child_slot[i];
  }
  const auto deadline = clk::now() + std::chrono::nanoseconds(c.timeout_ns);
  if (!barrier(c, 0, deadline, none)) return 0;  // buffers ready, counters zero
  std::vector<std::thread> th;
  for (int tree = 0; tree < 2; ++tree)
    for (int up = 0; up < 2; ++up) th.emplace_back([&, tree, up] { tree_worker(c, j, tree, up != 0, deadline, ft); });
  for (auto& x : th) x.join();
  // the owner zeroes the counters it consumed, then everybody leaves together
  for (int tree = 0; tree < 2; ++tree) {
    A(up_flag(c, c.rank, tree, 0, 0)).store(0u, std::memory_order_relaxed);
    A(up_flag(c, c.rank, tree, 0, 1)).store(0u, std::memory_order_relaxed);
    A(down_flag(c, c.rank, tree, 0)).store(0u, std::memory_order_relaxed);
  }
  const bool ok = barrier(c, 0, deadline, none);
  return ok && !aborted(c) ? 1 : 0;
}

}  // extern "C"

// ---------------------------------------------------------------------------
// In-process self-test: `world` ranks as threads of one process.  Built with
// -fsanitize=thread this checks that every plain (non-atomic) access of the data
// buffers is ordered by the release/acquire flag protocol — the race detector the
// GPU side cannot have.  Returns 0 on success, a positive code otherwise.
extern "C" int hp_selftest_threads(int world, int numel, int chunk, int rounds) {
  if (world < 1 || world > TCCL_MAX_WORLD) return 100;
  std::vector<std::vector<uint32_t>> flags(world, std::vector<uint32_t>(TCCL_FLAG_WORDS, 0u));
  std::vector<std::vector<uint32_t>> local(world, std::vector<uint32_t>(TCCL_LOCAL_WORDS, 0u));
  std::vector<std::vector<float>> data(world, std::vector<float>(numel));
  for (int r = 0; r < world; ++r)
    for (int i = 0; i < numel; ++i) data[r][i] = (float)((r + 1) * ((i % 7) + 1));
  // neighbours: the same low-bit rule as parallel/tree.py
  auto nbr_a = [&](int N, int r, int* parent, int* left, int* right) {
    *parent = *left = *right = -1;
    if (N == 1) return;
    if (r == 0) {
      int top = 1;
      while (top * 2 <= N - 1) top *= 2;
      *left = top;
      return;
    }
    const int s = r & -r;
    int up = (r ^ s) | (s << 1);
    if (up >= N) up = r ^ s;
    *parent = up;
    if (s == 1) return;
    *left = r - (s >> 1);
    int step = s >> 1, rt = r + step;
    while (rt >= N && step > 1) {
      step >>= 1;
      rt = r + step;
    }
    *right = rt >= N ? -1 : rt;
  };
  auto nbr = [&](int N, int r, int tree, int* parent, int* left, int* right) {
    if (tree == 0) return nbr_a(N, r, parent, left, right);
    nbr_a(N, (r + 1) % N, parent, left, right);
    auto back = [&](int x) { return x < 0 ? -1 : (x - 1 + N) % N; };
    *parent = back(*parent);
    *left = back(*left);
    *right = back(*right);
  };
  std::vector<int> results(world, 0);
  std::vector<std::thread> ranks;
  for (int r = 0; r < world; ++r) {
    ranks.emplace_back([&, r] {
      hp_comm h{};
      h.world = world;
      h.rank = r;
      for (int p = 0; p < world; ++p) h.flags[p] = reinterpret_cast<uint64_t>(flags[p].data());
      h.local = reinterpret_cast<uint64_t>(local[r].data());
      h.timeout_ns = 20ull * 1000 * 1000 * 1000;
      hp_faults none{-1, 0, -1};
      int ok = hp_barrier(&h, 1, rounds, &none);
      hp_tree t{};
      for (int p = 0; p < world; ++p) t.buf[p] = reinterpret_cast<uint64_t>(data[p].data());
      t.numel = (uint64_t)numel;
      t.chunk = (uint64_t)chunk;
      for (int tr = 0; tr < 2; ++tr) {
        int parent, left, right;
        nbr(world, r, tr, &parent, &left, &right);
        t.parent[tr] = parent;
        t.left[tr] = left;
        t.right[tr] = right;
        t.child_slot[tr] = 0;
        if (parent >= 0) {
          int pp, pl, pr;
          nbr(world, parent, tr, &pp, &pl, &pr);
          t.child_slot[tr] = pl == r ? 0 : 1;
        }
      }
      ok = ok && hp_tree_allreduce(&h, &t, &none);
      results[r] = ok;
    });
  }
  for (auto& th : ranks) th.join();
  for (int r = 0; r < world; ++r)
    if (!results[r]) return 1;
  const float tot = (float)(world * (world + 1) / 2);
  for (int r = 0; r < world; ++r)
    for (int i = 0; i < numel; ++i)
      if (data[r][i] != tot * (float)((i % 7) + 1)) return 2;
  return 0;
}
