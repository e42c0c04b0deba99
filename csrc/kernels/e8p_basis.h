// Host construction of the 256x8 E8P basis (even integers from {2, 6, 10}, 227
// inner-shell rows in lexicographic order, 29 outer rows with five sixes spread
// evenly over the 56 five-coordinate subsets, last coordinate sign-fixed by the
// parity of sum/4).  Must equal orinfer_b200.quant.e8p.basis(); tests compare them.
#pragma once
#include <stdint.h>
#include <vector>

namespace orinfer {

inline void build_e8p_basis(int8_t out[256][8]) {
  int rows = 0;
  int v[8];
  for (int code = 0; code < 6561; ++code) {          // base-3 digits, first coordinate major
    int c = code, norm = 0;
    for (int d = 7; d >= 0; --d) {
      v[d] = 4 * (c % 3) + 2;
      c /= 3;
      norm += v[d] * v[d];
    }
    if (norm <= 160) {
      for (int d = 0; d < 8; ++d) out[rows][d] = static_cast<int8_t>(v[d]);
      ++rows;
    }
  }
  std::vector<std::vector<int>> subsets;
  for (int a = 0; a < 8; ++a)
    for (int b = a + 1; b < 8; ++b)
      for (int c = b + 1; c < 8; ++c)
        for (int d = c + 1; d < 8; ++d)
          for (int e = d + 1; e < 8; ++e) subsets.push_back({a, b, c, d, e});
  for (int i = 0; i < 29; ++i) {
    for (int d = 0; d < 8; ++d) out[rows][d] = 2;
    for (int idx : subsets[i * static_cast<int>(subsets.size()) / 29]) out[rows][idx] = 6;
    ++rows;
  }
  for (int r = 0; r < 256; ++r) {
    int sum = 0;
    for (int d = 0; d < 8; ++d) sum += out[r][d];
    if ((sum / 4) % 2) out[r][7] = static_cast<int8_t>(-out[r][7]);
  }
}

}  // namespace orinfer
