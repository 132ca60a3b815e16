// Decoder of the six (F,H,W) axis orders: maps a position in a head's reordered token
// sequence to the token it came from.  Order ids follow paroattention/cogvideox.py:38-45.
#pragma once
#include <cstdint>

namespace paro {

struct PermDecoder {
  int size[3];   // extents of the reordered axes, slowest first
  int axis[3];   // which of (f, y, x) each reordered axis is
  int Hh, W;

  __host__ __device__ PermDecoder(int order_id, int F, int Hh_, int W_) : Hh(Hh_), W(W_) {
    // 0 FHW, 1 FWH, 2 HWF, 3 HFW, 4 WHF, 5 WFH
    const int tab[6][3] = {{0, 1, 2}, {0, 2, 1}, {1, 2, 0}, {1, 0, 2}, {2, 1, 0}, {2, 0, 1}};
    const int ext[3] = {F, Hh_, W_};
    const int o = (order_id >= 0 && order_id < 6) ? order_id : 0;
    for (int i = 0; i < 3; ++i) {
      axis[i] = tab[o][i];
      size[i] = ext[tab[o][i]];
    }
  }

  // j: position among the reordered video tokens; returns the source token index and its
  // (f, y, x) grid coordinate.
  __host__ __device__ __forceinline__ int source(int j, int& f, int& y, int& x) const {
    int c[3];
    c[2] = j % size[2];
    const int t = j / size[2];
    c[1] = t % size[1];
    c[0] = t / size[1];
    int fyx[3];
    fyx[axis[0]] = c[0];
    fyx[axis[1]] = c[1];
    fyx[axis[2]] = c[2];
    f = fyx[0];
    y = fyx[1];
    x = fyx[2];
    return (f * Hh + y) * W + x;
  }
};

}  // namespace paro
