#include "npy.h"

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <dirent.h>
#include <sys/stat.h>

namespace cb {

namespace {

bool find_value(const std::string& hdr, const std::string& key, size_t* pos) {
  const size_t k = hdr.find("'" + key + "'");
  if (k == std::string::npos) return false;
  const size_t c = hdr.find(':', k);
  if (c == std::string::npos) return false;
  *pos = c + 1;
  return true;
}

}  // namespace

bool load_npy_f32(const std::string& path, NpyArray* out, std::string* err) {
  FILE* f = std::fopen(path.c_str(), "rb");
  if (!f) {
    *err = "cannot open " + path;
    return false;
  }
  auto fail = [&](const std::string& why) {
    *err = path + ": " + why;
    std::fclose(f);
    return false;
  };
  unsigned char pre[12];
  if (std::fread(pre, 1, 10, f) != 10) return fail("truncated header");
  if (std::memcmp(pre, "\x93NUMPY", 6) != 0) return fail("not an .npy file (bad magic)");
  const int major = pre[6];
  size_t hlen = 0;
  if (major == 1) {
    hlen = pre[8] | (static_cast<size_t>(pre[9]) << 8);
  } else if (major == 2 || major == 3) {
    if (std::fread(pre + 10, 1, 2, f) != 2) return fail("truncated header");
    hlen = pre[8] | (static_cast<size_t>(pre[9]) << 8) | (static_cast<size_t>(pre[10]) << 16) |
           (static_cast<size_t>(pre[11]) << 24);
  } else {
    return fail("unsupported .npy version");
  }
  if (hlen == 0 || hlen > (1u << 20)) return fail("implausible header length");
  std::string hdr(hlen, '\0');
  if (std::fread(&hdr[0], 1, hlen, f) != hlen) return fail("truncated header");

  size_t p;
  if (!find_value(hdr, "descr", &p)) return fail("header has no 'descr'");
  const size_t q0 = hdr.find('\'', p);
  const size_t q1 = (q0 == std::string::npos) ? q0 : hdr.find('\'', q0 + 1);
  if (q1 == std::string::npos) return fail("malformed 'descr'");
  const std::string descr = hdr.substr(q0 + 1, q1 - q0 - 1);
  if (descr != "<f4" && descr != "=f4" && descr != "|f4")
    return fail("dtype is " + descr + ", only little-endian float32 ('<f4') weights are accepted");

  if (!find_value(hdr, "fortran_order", &p)) return fail("header has no 'fortran_order'");
  const size_t t = hdr.find_first_not_of(" ", p);
  if (t != std::string::npos && hdr.compare(t, 4, "True") == 0) return fail("Fortran-order arrays are not accepted");

  if (!find_value(hdr, "shape", &p)) return fail("header has no 'shape'");
  const size_t l = hdr.find('(', p), r = hdr.find(')', p);
  if (l == std::string::npos || r == std::string::npos || r < l) return fail("malformed 'shape'");
  out->shape.clear();
  size_t i = l + 1;
  while (i < r) {
    while (i < r && (hdr[i] == ' ' || hdr[i] == ',')) ++i;
    if (i >= r) break;
    size_t v = 0;
    bool any = false;
    while (i < r && hdr[i] >= '0' && hdr[i] <= '9') {
      v = v * 10 + static_cast<size_t>(hdr[i] - '0');
      ++i;
      any = true;
    }
    if (!any) return fail("malformed 'shape'");
    out->shape.push_back(v);
  }
  const size_t n = out->numel();
  out->data.resize(n);
  if (n && std::fread(out->data.data(), sizeof(float), n, f) != n) return fail("payload shorter than the shape says");
  std::fclose(f);
  return true;
}

bool list_npy_files(const std::string& dir, std::vector<std::string>* names, std::string* err) {
  DIR* d = opendir(dir.c_str());
  if (!d) {
    *err = "cannot open model directory " + dir;
    return false;
  }
  names->clear();
  while (dirent* e = readdir(d)) {
    const std::string n = e->d_name;
    if (n.size() > 4 && n.compare(n.size() - 4, 4, ".npy") == 0) names->push_back(n);
  }
  closedir(d);
  std::sort(names->begin(), names->end());
  return true;
}

}  // namespace cb
