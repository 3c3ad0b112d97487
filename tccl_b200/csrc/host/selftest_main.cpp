// Stand-alone driver of the in-process protocol self-test (see host_protocol.cpp);
// meant to be built with -fsanitize=thread.
#include <cstdio>
#include <cstdlib>
#include <cstring>

extern "C" int hp_selftest_threads(int world, int numel, int chunk, int rounds);
extern "C" int hp_selftest_gemm_rs(int world, int ctas, int tiles_per_owner, int calls);
extern "C" int hp_selftest_ag(int world, int movers, int consumers, int row_tiles, int calls);
extern "C" int hp_selftest_push(int world, int calls, int scheme);
extern "C" int hp_selftest_ag_pair(int world, int ctas, int row_tiles, int calls, int mode);
extern "C" int hp_selftest_rs_pair(int world, int ctas, int tiles_per_owner, int calls, int mode);
extern "C" int hp_selftest_tree_ll(int world, int numel, int calls, int depth);
extern "C" int hp_selftest_bulk(int world, int ctas, int chunk, int chunks_per_cta, int calls, int early_release);

int main(int argc, char** argv) {
  if (argc > 2 && std::strcmp(argv[1], "push-broken-variant") == 0) {
    // the size-dependent layout with a per-CTA epoch parity: expected to be reported as a race
    const int rc = hp_selftest_push(std::atoi(argv[2]), 300, 1);
    std::printf("hp_selftest_push(broken variant) -> %d\n", rc);
    return rc;
  }
  if (argc > 2 && std::strcmp(argv[1], "ag-pair-broken-variant") == 0) {
    // one gathered buffer, no halves, no barrier: a rank one call ahead overwrites rows a peer still reads
    const int rc = hp_selftest_ag_pair(std::atoi(argv[2]), 3, 4, 200, 2);
    std::printf("hp_selftest_ag_pair(broken variant) -> %d\n", rc);
    return rc;
  }
  if (argc > 2 && std::strcmp(argv[1], "rs-pair-broken-variant") == 0) {
    // one staging half, no barrier: a rank one call ahead overwrites partials a peer is still summing
    const int rc = hp_selftest_rs_pair(std::atoi(argv[2]), 3, 5, 200, 2);
    std::printf("hp_selftest_rs_pair(broken variant) -> %d\n", rc);
    return rc;
  }
  if (argc > 2 && std::strcmp(argv[1], "bulk-broken-variant") == 0) {
    // output stages freed when their copies are issued, not when they have been read: expected to be reported
    const int rc = hp_selftest_bulk(std::atoi(argv[2]), 2, 4096, 12, 2, 1);
    std::printf("hp_selftest_bulk(broken variant) -> %d\n", rc);
    return rc;
  }
  const int world = argc > 1 ? std::atoi(argv[1]) : 4;
  const int numel = argc > 2 ? std::atoi(argv[2]) : 1 << 14;
  const int chunk = argc > 3 ? std::atoi(argv[3]) : 1 << 9;
  int rc = hp_selftest_threads(world, numel, chunk, 50);
  std::printf("hp_selftest_threads(world=%d) -> %d\n", world, rc);
  if (rc) return rc;
  rc = hp_selftest_gemm_rs(world, 5, 7, 3);
  std::printf("hp_selftest_gemm_rs(world=%d) -> %d\n", world, rc);
  if (rc) return rc;
  rc = hp_selftest_ag(world, 3, 4, 4, 3);
  std::printf("hp_selftest_ag(world=%d) -> %d\n", world, rc);
  if (rc) return rc;
  rc = hp_selftest_push(world, 300, 0);
  std::printf("hp_selftest_push(world=%d) -> %d\n", world, rc);
  if (rc) return rc;
  for (int ring = 0; ring < 2; ++ring) {
    rc = hp_selftest_ag_pair(world, 3, 4, 40, ring);
    std::printf("hp_selftest_ag_pair(world=%d, ring=%d) -> %d\n", world, ring, rc);
    if (rc) return rc;
  }
  for (int depth = 1; depth <= 4; depth += 3) {
    rc = hp_selftest_tree_ll(world, 194, 60, depth);
    std::printf("hp_selftest_tree_ll(world=%d, depth=%d) -> %d\n", world, depth, rc);
    if (rc) return rc;
  }
  rc = hp_selftest_rs_pair(world, 3, 5, 40, 0);
  std::printf("hp_selftest_rs_pair(world=%d) -> %d\n", world, rc);
  if (rc) return rc;
  rc = hp_selftest_bulk(world, 2, 48, 7, 2, 0);
  std::printf("hp_selftest_bulk(world=%d) -> %d\n", world, rc);
  return rc;
}
