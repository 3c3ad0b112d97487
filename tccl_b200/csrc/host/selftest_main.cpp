// Stand-alone driver of the in-process protocol self-test (see host_protocol.cpp);
// meant to be built with -fsanitize=thread.
#include <cstdio>
#include <cstdlib>

extern "C" int hp_selftest_threads(int world, int numel, int chunk, int rounds);

int main(int argc, char** argv) {
  const int world = argc > 1 ? std::atoi(argv[1]) : 4;
  const int numel = argc > 2 ? std::atoi(argv[2]) : 1 << 14;
  const int chunk = argc > 3 ? std::atoi(argv[3]) : 1 << 9;
  const int rc = hp_selftest_threads(world, numel, chunk, 50);
  std::printf("hp_selftest_threads(world=%d) -> %d\n", world, rc);
  return rc;
}
