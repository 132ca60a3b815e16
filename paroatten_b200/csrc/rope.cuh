// 3D-RoPE helpers shared by the reorder kernel and the fused reorder+quantise kernels.
#pragma once
#include <type_traits>

#include "common.cuh"

namespace paro {

struct RopeArgs {
  int mode;            // PARO_ROPE_*
  const void* cos_tab; // [F+Hh+W, D/2]; or, when sin_tab is NULL, [F+Hh+W, D/2, 2] holding (cos, sin) side by side
  const void* sin_tab; // [F+Hh+W, D/2] or NULL (one 8- or 16-byte load then fetches both values of a pair)
  int pairs_f, pairs_h;
};

// Angles of the thread's four channel pairs, kept from one row to the next: consecutive rows of the
// reordered sequence differ in the fastest grid coordinate only, so the pairs driven by the other two
// coordinates find their (cos, sin) already in registers and skip the table load.
template <int MODE> struct RotCache {
  using F = typename std::conditional<MODE == PARO_ROPE_REAL_F32, float, double>::type;
  F c[4], s[4];
  int row[4];
  __device__ __forceinline__ RotCache() {
#pragma unroll
    for (int p = 0; p < 4; ++p) row[p] = -1;
  }
};

// Rotates the four channel pairs held in `x` (channels c8..c8+7 of a token at grid
// coordinate f,y,x).  Products and sums are rounded separately (no fused multiply-add) so that
// results equal a plain elementwise evaluation.
// MODE: PARO_ROPE_REAL_F32 or PARO_ROPE_COMPLEX_F64 (compile time, so that a kernel only carries the
// registers of the arithmetic it uses).
template <typename T, int MODE>
__device__ __forceinline__ void rotate8(Pack8<T>& x, int c8, int D, int f, int y, int xw,
                                        int F, int Hh, const RopeArgs& r, RotCache<MODE>& cache) {
  using FT = typename RotCache<MODE>::F;
  using FT2 = typename std::conditional<MODE == PARO_ROPE_REAL_F32, float2, double2>::type;
  const int half = D >> 1;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int pair = (c8 >> 1) + p;
    const int row = pair < r.pairs_f ? f : (pair < r.pairs_f + r.pairs_h ? F + y : F + Hh + xw);
    if (row != cache.row[p]) {
      const size_t t = (size_t)row * half + pair;
      if (r.sin_tab == nullptr) {
        const FT2 cs = static_cast<const FT2*>(r.cos_tab)[t];
        cache.c[p] = cs.x; cache.s[p] = cs.y;
      } else {
        cache.c[p] = static_cast<const FT*>(r.cos_tab)[t];
        cache.s[p] = static_cast<const FT*>(r.sin_tab)[t];
      }
      cache.row[p] = row;
    }
    const FT c = cache.c[p], s = cache.s[p];
    if constexpr (MODE == PARO_ROPE_REAL_F32) {
      const float x0 = F16Traits<T>::to_float(x.e[2 * p]);
      const float x1 = F16Traits<T>::to_float(x.e[2 * p + 1]);
      const float o0 = __fadd_rn(__fmul_rn(x0, c), __fmul_rn(-x1, s));
      const float o1 = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s));
      x.e[2 * p] = F16Traits<T>::from_float(o0);
      x.e[2 * p + 1] = F16Traits<T>::from_float(o1);
    } else {
      const double x0 = (double)F16Traits<T>::to_float(x.e[2 * p]);
      const double x1 = (double)F16Traits<T>::to_float(x.e[2 * p + 1]);
      const double re = __dsub_rn(__dmul_rn(x0, c), __dmul_rn(x1, s));
      const double im = __dadd_rn(__dmul_rn(x0, s), __dmul_rn(x1, c));
      x.e[2 * p] = F16Traits<T>::from_float(__double2float_rn(re));
      x.e[2 * p + 1] = F16Traits<T>::from_float(__double2float_rn(im));
    }
  }
}

// Without a cache: straight-line code, every pair's angles are loaded (what the quantiser front ends use;
// there the compare-and-skip of the cached form costs more than the loads it saves).
template <typename T, int MODE>
__device__ __forceinline__ void rotate8(Pack8<T>& x, int c8, int D, int f, int y, int xw,
                                        int F, int Hh, const RopeArgs& r) {
  using FT = typename RotCache<MODE>::F;
  using FT2 = typename std::conditional<MODE == PARO_ROPE_REAL_F32, float2, double2>::type;
  const int half = D >> 1;
#pragma unroll
  for (int p = 0; p < 4; ++p) {
    const int pair = (c8 >> 1) + p;
    const int row = pair < r.pairs_f ? f : (pair < r.pairs_f + r.pairs_h ? F + y : F + Hh + xw);
    const size_t t = (size_t)row * half + pair;
    FT c, s;
    if (r.sin_tab == nullptr) {
      const FT2 cs = static_cast<const FT2*>(r.cos_tab)[t];
      c = cs.x; s = cs.y;
    } else {
      c = static_cast<const FT*>(r.cos_tab)[t];
      s = static_cast<const FT*>(r.sin_tab)[t];
    }
    if constexpr (MODE == PARO_ROPE_REAL_F32) {
      const float x0 = F16Traits<T>::to_float(x.e[2 * p]);
      const float x1 = F16Traits<T>::to_float(x.e[2 * p + 1]);
      const float o0 = __fadd_rn(__fmul_rn(x0, c), __fmul_rn(-x1, s));
      const float o1 = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s));
      x.e[2 * p] = F16Traits<T>::from_float(o0);
      x.e[2 * p + 1] = F16Traits<T>::from_float(o1);
    } else {
      const double x0 = (double)F16Traits<T>::to_float(x.e[2 * p]);
      const double x1 = (double)F16Traits<T>::to_float(x.e[2 * p + 1]);
      const double re = __dsub_rn(__dmul_rn(x0, c), __dmul_rn(x1, s));
      const double im = __dadd_rn(__dmul_rn(x0, s), __dmul_rn(x1, c));
      x.e[2 * p] = F16Traits<T>::from_float(__double2float_rn(re));
      x.e[2 * p + 1] = F16Traits<T>::from_float(__double2float_rn(im));
    }
  }
}

}  // namespace paro
