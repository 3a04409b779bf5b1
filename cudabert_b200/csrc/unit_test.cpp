// Stand-alone driver of the library's built-in latency / throughput loop, the counterpart of
// the reference's unit_test program (cuda_bert/test/test.cpp:4-46): it calls test(batch, seq,
// iterations, large, gpu) for a grid of shapes and prints what test() prints.
//   unit_test [large(0|1)] [gpu] [iterations]
// Expects the weights in model_npy/base_uncased or model_npy/large_uncased under the CWD.
#include <cstdio>
#include <cstdlib>

#include "../../include/cudabert.h"

int main(int argc, char** argv) {
  const bool large = argc > 1 ? std::atoi(argv[1]) != 0 : false;
  const int gpu = argc > 2 ? std::atoi(argv[2]) : 0;
  const int iters = argc > 3 ? std::atoi(argv[3]) : 100;
  const int batches[] = {1, 8, 32, 128};
  const int seqs[] = {32, 128, 200};
  for (int s : seqs)
    for (int b : batches) test(b, s, iters, large, gpu);
  return 0;
}
