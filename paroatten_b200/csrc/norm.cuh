// Q/K normalisation folded into the pre-attention passes (the processors call norm_q / norm_k between
// the projection and RoPE: cogvideox.py:161-164, wan.py:150-153).  Two forms:
//   PARO_NORM_LAYER_HEAD  LayerNorm over the D channels of one (token, head), affine weight/bias [D]
//   PARO_NORM_RMS_ALL     RMSNorm over all H*D channels of a token (statistic precomputed per token
//                         by paro_row_inv_rms), weight [H*D]
// Sums are taken in fp64 (exact for 16-bit inputs in practice, hence independent of their order);
// every other operation is a separately rounded fp32 operation; results are rounded to the input
// dtype, as a module call on a 16-bit tensor would.
#pragma once
#include "common.cuh"

namespace paro {

struct NormArgs {
  int mode;              // PARO_NORM_*
  const void* weight;    // input dtype
  const void* bias;      // input dtype or nullptr (layer norm only)
  const float* inv_rms;  // [B, N] fp32 (RMS only)
  float eps;
};

// Normalises the 8 channels c8..c8+7 of one token row held by this thread.  The row is spread over
// TPR consecutive lanes (TPR = D/8); every lane of the warp must call this (full-mask shuffles).
template <typename T, int NM, int TPR>
__device__ __forceinline__ void normalize8(Pack8<T>& x, int c8, int D, int b, int h, int N, int tok,
                                           const NormArgs& a) {
  if constexpr (NM == PARO_NORM_LAYER_HEAD) {
    float f[8];
    double s = 0.0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      f[j] = F16Traits<T>::to_float(x.e[j]);
      s += (double)f[j];
    }
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mean = __double2float_rn(s / (double)D);
    double q = 0.0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const double d = (double)f[j] - (double)mean;
      q += d * d;
    }
#pragma unroll
    for (int o = TPR / 2; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    const float var = __double2float_rn(q / (double)D);
    const float rstd = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(var, a.eps)));
    Pack8<T> w, bb;
    w.v = *reinterpret_cast<const uint4*>(static_cast<const T*>(a.weight) + c8);
    if (a.bias) bb.v = *reinterpret_cast<const uint4*>(static_cast<const T*>(a.bias) + c8);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float y = __fmul_rn(__fmul_rn(__fsub_rn(f[j], mean), rstd), F16Traits<T>::to_float(w.e[j]));
      if (a.bias) y = __fadd_rn(y, F16Traits<T>::to_float(bb.e[j]));
      x.e[j] = F16Traits<T>::from_float(y);
    }
  } else if constexpr (NM == PARO_NORM_RMS_ALL) {
    const float inv = a.inv_rms[(size_t)b * N + tok];
    Pack8<T> w;
    w.v = *reinterpret_cast<const uint4*>(static_cast<const T*>(a.weight) + (size_t)h * D + c8);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const T y1 = F16Traits<T>::from_float(__fmul_rn(F16Traits<T>::to_float(x.e[j]), inv));
      x.e[j] = F16Traits<T>::from_float(__fmul_rn(F16Traits<T>::to_float(y1), F16Traits<T>::to_float(w.e[j])));
    }
  }
}

// Host-side check shared by the entry points that take a norm.
inline int check_norm(const char* who, int mode, const void* weight, const void* bias, const float* inv_rms, float eps) {
  PARO_REQUIRE(mode >= PARO_NORM_NONE && mode <= PARO_NORM_RMS_ALL, PARO_EINVAL, "%s: unknown norm_mode %d", who, mode);
  if (mode == PARO_NORM_NONE) return PARO_OK;
  PARO_REQUIRE(weight && aligned16(weight), PARO_EINVAL, "%s: norm weight null or not 16-byte aligned", who);
  PARO_REQUIRE(!bias || aligned16(bias), PARO_EALIGN, "%s: norm bias not 16-byte aligned", who);
  PARO_REQUIRE(mode != PARO_NORM_RMS_ALL || inv_rms, PARO_EINVAL, "%s: RMS norm needs the per-token inv_rms table", who);
  PARO_REQUIRE(mode != PARO_NORM_RMS_ALL || !bias, PARO_EINVAL, "%s: RMS norm takes no bias", who);
  PARO_REQUIRE(eps >= 0.f, PARO_EINVAL, "%s: negative eps", who);
  return PARO_OK;
}

}  // namespace paro
