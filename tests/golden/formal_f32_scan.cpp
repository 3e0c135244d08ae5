// Host tool for the golden vectors of the correctly rounded binary32 / TF32 function family. It compiles the library's
// own evaluator (vibe_compiler_b200/csrc/formal_functions_f32.cuh builds for the host too) and
//   scan <function>          writes every binary32 operand encoding whose evaluation takes the double-double step
//                            (the operands whose value lies within 2^-46 of a rounding boundary) to stdout, 4 bytes each;
//   eval <function> <tf32>   reads operand encodings from stdin and writes (result bits, flags) pairs to stdout.
// Build: g++ -O2 -std=c++17 -pthread -o formal_f32_scan formal_f32_scan.cpp   (make_formal_function_f32_expected.py does it)
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <vector>

#include "../../vibe_compiler_b200/csrc/formal_functions_f32.cuh"

using namespace wb200::ff32;

int main(int argc, char **argv) {
  if (argc < 3) return 2;
  const int function = atoi(argv[2]);
  if (!strcmp(argv[1], "scan")) {
    const int threads = static_cast<int>(std::thread::hardware_concurrency());
    std::vector<std::vector<uint32_t>> found(threads);
    std::vector<std::thread> pool;
    for (int t = 0; t < threads; ++t)
      pool.emplace_back([&, t]() {
        const uint64_t chunk = ((1ull << 32) + threads - 1) / threads;
        const uint64_t end = (t + 1) * chunk < (1ull << 32) ? (t + 1) * chunk : (1ull << 32);
        for (uint64_t a = t * chunk; a < end; ++a) {
          uint32_t flags;
          bool second;
          correctly_rounded(function, false, static_cast<uint32_t>(a), &flags, &second);
          if (second) found[t].push_back(static_cast<uint32_t>(a));
        }
      });
    for (auto &thread : pool) thread.join();
    for (auto &list : found) fwrite(list.data(), 4, list.size(), stdout);
    return 0;
  }
  if (!strcmp(argv[1], "eval") && argc >= 4) {
    const bool tf32 = atoi(argv[3]) != 0;
    uint32_t operand;
    while (fread(&operand, 4, 1, stdin) == 1) {
      uint32_t out[2];
      bool second;
      out[0] = correctly_rounded(function, tf32, operand, &out[1], &second);
      fwrite(out, 4, 2, stdout);
    }
    return 0;
  }
  return 2;
}
