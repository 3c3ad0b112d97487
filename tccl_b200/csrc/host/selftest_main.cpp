// Stand-alone driver of the in-process protocol self-test (see host_protocol.cpp);
// meant to be built with -fsanitize=thread.
#include <cstdio>
#include <cstdlib>

extern "C" int hp_selftest_threads(int world, int numel, int chunk, int rounds);
extern "C" int hp_selftest_gemm_rs(int world, int ctas, int tiles_per_owner, int calls);
extern "C" int hp_selftest_ag(int world, int movers, int consumers, int row_tiles, int calls);
extern "C" int hp_selftest_push(int world, int calls);

int main(int argc, char** argv) {
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
  rc = hp_selftest_push(world, 200);
  std::printf("hp_selftest_push(world=%d) -> %d\n", world, rc);
  return rc;
}
