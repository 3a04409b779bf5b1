// Stand-in for the CUDA-samples header of the same name (see helper_cuda.h beside this file).
// The reference relies on it only for declarations it pulls in indirectly.
#pragma once
#include <algorithm>
#include <cassert>
#include <cmath>
#include <cstring>
using std::max;
using std::min;
