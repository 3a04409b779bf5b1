// Minimal reader for the weight files of the reference's model directory: NumPy .npy,
// format version 1.x-3.x, little-endian float32, C order.  The reference reads them with the
// vendored cnpy (cnpy/cnpy.cpp:108-201) and aborts on anything but 4-byte words
// (utils/load_model.cc:93); this reader reports an error string instead of aborting.
#pragma once
#include <cstddef>
#include <string>
#include <vector>

namespace cb {

struct NpyArray {
  std::vector<size_t> shape;
  std::vector<float> data;
  size_t numel() const {
    size_t n = 1;
    for (size_t d : shape) n *= d;
    return n;
  }
};

// Returns true on success; on failure `err` says why (missing file, bad magic, dtype other
// than '<f4', Fortran order, truncated payload).
bool load_npy_f32(const std::string& path, NpyArray* out, std::string* err);

// Regular files of `dir` whose name ends in ".npy", sorted by name.
bool list_npy_files(const std::string& dir, std::vector<std::string>* names, std::string* err);

}  // namespace cb
