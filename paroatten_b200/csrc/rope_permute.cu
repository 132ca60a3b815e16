// Fused 3D-RoPE + per-head token permutation (gather on read, coalesced 16-byte stores on
// write).  HBM-bound: each element is read once and written once; the per-axis angle tables
// are a few KB and stay in L1/L2.
#include "common.cuh"
#include "perm.cuh"
#include "norm.cuh"
#include "rope.cuh"

namespace paro {

// Block = 256 threads; a thread owns one 16-byte slice of PASSES consecutive rows (consecutive rows share
// the slow grid coordinates, so most of their rotation angles are reused from registers).
// blockIdx.x: group of rows, blockIdx.y: b*H + h.
template <typename T, int D, int MODE, int NM>
__global__ void __launch_bounds__(256)
rope_permute_kernel(const T* __restrict__ in, T* __restrict__ out, int H, int N,
                    int64_t sb, int64_t sh, int64_t sn, int n_text, int F, int Hh, int W,
                    const int32_t* __restrict__ order_ids, int inverse, RopeArgs rope, NormArgs norm) {
  constexpr int TPR = D / 8;            // threads per row
  constexpr int ROWS = 256 / TPR;       // rows per pass
  constexpr int PASSES = 4;
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  const int c8 = (threadIdx.x % TPR) * 8;
  const int r0 = blockIdx.x * (ROWS * PASSES) + (threadIdx.x / TPR) * PASSES;
  const PermDecoder dec(order_ids ? order_ids[h] : 0, F, Hh, W);
  const T* src_base = in + b * sb + h * sh;
  T* dst_base = out + (size_t)bh * N * D;

  Pack8<T> val[PASSES];
  int dst_row[PASSES], src_row[PASSES], fy[PASSES], yy[PASSES], xx[PASSES];
#pragma unroll
  for (int i = 0; i < PASSES; ++i) {
    const int row = r0 + i;
    dst_row[i] = -1;
    src_row[i] = 0;
    val[i].v = make_uint4(0, 0, 0, 0);
    if (row >= N) continue;
    int src = row, dst = row;
    fy[i] = yy[i] = xx[i] = -1;
    if (row >= n_text) {
      const int j = row - n_text;
      int f, y, x;
      const int other = n_text + dec.source(j, f, y, x);
      if (order_ids == nullptr) {
        // natural order: the coordinate of j itself
        const PermDecoder ident(0, F, Hh, W);
        ident.source(j, f, y, x);
      } else if (inverse) {
        dst = other;
      } else {
        src = other;
      }
      fy[i] = f; yy[i] = y; xx[i] = x;
    }
    dst_row[i] = dst;
    src_row[i] = src;
    val[i].v = *reinterpret_cast<const uint4*>(src_base + (size_t)src * sn + c8);
  }
  [[maybe_unused]] RotCache<MODE == PARO_ROPE_REAL_F32 ? PARO_ROPE_REAL_F32 : PARO_ROPE_COMPLEX_F64> rot;
#pragma unroll
  for (int i = 0; i < PASSES; ++i) {
    // every lane takes part in the normalisation's shuffles, also those whose row is past the end
    if constexpr (NM != PARO_NORM_NONE) normalize8<T, NM, TPR>(val[i], c8, D, b, h, N, src_row[i], norm);
    if (dst_row[i] < 0) continue;
    if constexpr (MODE != PARO_ROPE_NONE) {
      if (fy[i] >= 0) rotate8<T, MODE>(val[i], c8, D, fy[i], yy[i], xx[i], F, Hh, rope, rot);
    }
    *reinterpret_cast<uint4*>(dst_base + (size_t)dst_row[i] * D + c8) = val[i].v;
  }
}

template <typename T, int MODE, int NM>
int launch_rope_mode(const void* in, void* out, int B, int H, int N, int D, int64_t sb, int64_t sh, int64_t sn,
                     int n_text, int F, int Hh, int W, const int32_t* order_ids, int inverse,
                     const RopeArgs& rope, const NormArgs& norm, cudaStream_t s) {
  if (D == 128) {
    dim3 grid((N + 63) / 64, B * H);
    rope_permute_kernel<T, 128, MODE, NM><<<grid, 256, 0, s>>>((const T*)in, (T*)out, H, N, sb, sh, sn, n_text, F, Hh,
                                                               W, order_ids, inverse, rope, norm);
  } else {
    dim3 grid((N + 127) / 128, B * H);
    rope_permute_kernel<T, 64, MODE, NM><<<grid, 256, 0, s>>>((const T*)in, (T*)out, H, N, sb, sh, sn, n_text, F, Hh,
                                                              W, order_ids, inverse, rope, norm);
  }
  return check_launch("rope_permute_kernel");
}

template <typename T>
int launch_rope(const void* in, void* out, int B, int H, int N, int D, int64_t sb, int64_t sh, int64_t sn,
                int n_text, int F, int Hh, int W, const int32_t* order_ids, int inverse,
                const RopeArgs& rope, const NormArgs& norm, cudaStream_t s) {
#define PARO_ROPE_CASE(M, NMODE) \
  return launch_rope_mode<T, M, NMODE>(in, out, B, H, N, D, sb, sh, sn, n_text, F, Hh, W, order_ids, inverse, rope, norm, s)
#define PARO_ROPE_NORMS(M)                                                   \
  if (norm.mode == PARO_NORM_LAYER_HEAD) PARO_ROPE_CASE(M, PARO_NORM_LAYER_HEAD); \
  if (norm.mode == PARO_NORM_RMS_ALL) PARO_ROPE_CASE(M, PARO_NORM_RMS_ALL);      \
  PARO_ROPE_CASE(M, PARO_NORM_NONE)
  if (rope.mode == PARO_ROPE_REAL_F32) { PARO_ROPE_NORMS(PARO_ROPE_REAL_F32); }
  if (rope.mode == PARO_ROPE_COMPLEX_F64) { PARO_ROPE_NORMS(PARO_ROPE_COMPLEX_F64); }
  PARO_ROPE_NORMS(PARO_ROPE_NONE);
#undef PARO_ROPE_NORMS
#undef PARO_ROPE_CASE
}

// One warp per token: sum of squares over all H*D channels in fp64.
template <typename T>
__global__ void __launch_bounds__(256)
row_inv_rms_kernel(const T* __restrict__ x, int H, int N, int D, int64_t sb, int64_t sh, int64_t sn, float eps,
                   float* __restrict__ inv_rms, int rows) {
  const int row = blockIdx.x * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  const int b = row / N, n = row % N;
  const T* base = x + b * sb + (size_t)n * sn;
  const int per_head = D / 8;   // 16-byte pieces per head
  double s = 0.0;
  for (int i = lane; i < H * per_head; i += 32) {
    Pack8<T> v;
    v.v = *reinterpret_cast<const uint4*>(base + (size_t)(i / per_head) * sh + (i % per_head) * 8);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float f = F16Traits<T>::to_float(v.e[j]);
      s += (double)__fmul_rn(f, f);   // exact: 16 significant bits
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
  if (lane == 0) {
    const float ms = __double2float_rn(s / (double)((size_t)H * D));
    inv_rms[row] = __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(ms, eps)));
  }
}

}  // namespace paro

using namespace paro;

extern "C" int paro_rope_permute(const void* in, void* out, int dtype, int B, int H, int N, int D,
                                 int64_t stride_b, int64_t stride_h, int64_t stride_n,
                                 int n_text, int F, int Hh, int W, const int32_t* order_ids, int inverse,
                                 int rope_mode, const void* cos_tab, const void* sin_tab,
                                 int pairs_f, int pairs_h, paro_stream_t stream) {
  if (int rc = check_tensor("paro_rope_permute(in)", in, dtype, B, H, N, D, stride_b, stride_h, stride_n)) return rc;
  PARO_REQUIRE(out && aligned16(out), PARO_EALIGN, "paro_rope_permute: out null or not 16-byte aligned");
  PARO_REQUIRE(in != out, PARO_EINVAL, "paro_rope_permute: in-place operation is not supported");
  PARO_REQUIRE(F > 0 && Hh > 0 && W > 0 && n_text >= 0 && (int64_t)n_text + (int64_t)F * Hh * W == N, PARO_ESHAPE,
               "paro_rope_permute: n_text + F*H*W = %lld != N = %d", (long long)n_text + (long long)F * Hh * W, N);
  PARO_REQUIRE(rope_mode >= PARO_ROPE_NONE && rope_mode <= PARO_ROPE_COMPLEX_F64, PARO_EINVAL,
               "paro_rope_permute: unknown rope_mode %d", rope_mode);
  PARO_REQUIRE(!(inverse && rope_mode != PARO_ROPE_NONE), PARO_EINVAL,
               "paro_rope_permute: the inverse permutation does not rotate");
  if (rope_mode != PARO_ROPE_NONE) {
    PARO_REQUIRE(cos_tab, PARO_EINVAL, "paro_rope_permute: rope tables missing");   // sin_tab NULL = interleaved (cos, sin) table
    PARO_REQUIRE(pairs_f >= 0 && pairs_h >= 0 && pairs_f + pairs_h <= D / 2, PARO_ESHAPE,
                 "paro_rope_permute: pairs_f + pairs_h exceeds D/2");
  }
  RopeArgs r{rope_mode, cos_tab, sin_tab, pairs_f, pairs_h};
  NormArgs nm{};
  cudaStream_t s = (cudaStream_t)stream;
  return dtype == PARO_F16
             ? launch_rope<__half>(in, out, B, H, N, D, stride_b, stride_h, stride_n, n_text, F, Hh, W, order_ids, inverse, r, nm, s)
             : launch_rope<__nv_bfloat16>(in, out, B, H, N, D, stride_b, stride_h, stride_n, n_text, F, Hh, W, order_ids, inverse, r, nm, s);
}

extern "C" int paro_rope_permute_norm(const void* in, void* out, int dtype, int B, int H, int N, int D,
                                      int64_t stride_b, int64_t stride_h, int64_t stride_n,
                                      int n_text, int F, int Hh, int W, const int32_t* order_ids,
                                      int rope_mode, const void* cos_tab, const void* sin_tab,
                                      int pairs_f, int pairs_h,
                                      int norm_mode, const void* norm_weight, const void* norm_bias,
                                      const float* inv_rms, float eps, paro_stream_t stream) {
  if (int rc = check_tensor("paro_rope_permute_norm(in)", in, dtype, B, H, N, D, stride_b, stride_h, stride_n)) return rc;
  PARO_REQUIRE(out && aligned16(out), PARO_EALIGN, "paro_rope_permute_norm: out null or not 16-byte aligned");
  PARO_REQUIRE(in != out, PARO_EINVAL, "paro_rope_permute_norm: in-place operation is not supported");
  PARO_REQUIRE(F > 0 && Hh > 0 && W > 0 && n_text >= 0 && (int64_t)n_text + (int64_t)F * Hh * W == N, PARO_ESHAPE,
               "paro_rope_permute_norm: n_text + F*H*W = %lld != N = %d", (long long)n_text + (long long)F * Hh * W, N);
  PARO_REQUIRE(rope_mode >= PARO_ROPE_NONE && rope_mode <= PARO_ROPE_COMPLEX_F64, PARO_EINVAL,
               "paro_rope_permute_norm: unknown rope_mode %d", rope_mode);
  if (rope_mode != PARO_ROPE_NONE) {
    PARO_REQUIRE(cos_tab, PARO_EINVAL, "paro_rope_permute_norm: rope tables missing");
    PARO_REQUIRE(pairs_f >= 0 && pairs_h >= 0 && pairs_f + pairs_h <= D / 2, PARO_ESHAPE,
                 "paro_rope_permute_norm: pairs_f + pairs_h exceeds D/2");
  }
  if (int rc = check_norm("paro_rope_permute_norm", norm_mode, norm_weight, norm_bias, inv_rms, eps)) return rc;
  RopeArgs r{rope_mode, cos_tab, sin_tab, pairs_f, pairs_h};
  NormArgs nm{norm_mode, norm_weight, norm_bias, inv_rms, eps};
  cudaStream_t s = (cudaStream_t)stream;
  return dtype == PARO_F16
             ? launch_rope<__half>(in, out, B, H, N, D, stride_b, stride_h, stride_n, n_text, F, Hh, W, order_ids, 0, r, nm, s)
             : launch_rope<__nv_bfloat16>(in, out, B, H, N, D, stride_b, stride_h, stride_n, n_text, F, Hh, W, order_ids, 0, r, nm, s);
}

extern "C" int paro_row_inv_rms(const void* x, int dtype, int B, int H, int N, int D,
                                int64_t stride_b, int64_t stride_h, int64_t stride_n,
                                float eps, float* inv_rms, paro_stream_t stream) {
  if (int rc = check_tensor("paro_row_inv_rms(x)", x, dtype, B, H, N, D, stride_b, stride_h, stride_n)) return rc;
  PARO_REQUIRE(inv_rms, PARO_EINVAL, "paro_row_inv_rms: null output");
  PARO_REQUIRE(eps >= 0.f, PARO_EINVAL, "paro_row_inv_rms: negative eps");
  const long long rows = (long long)B * N;
  PARO_REQUIRE(rows <= 0x7fffffffLL, PARO_ESHAPE, "paro_row_inv_rms: too many rows");
  cudaStream_t s = (cudaStream_t)stream;
  const unsigned grid = (unsigned)((rows + 7) / 8);
  if (dtype == PARO_F16)
    row_inv_rms_kernel<__half><<<grid, 256, 0, s>>>((const __half*)x, H, N, D, stride_b, stride_h, stride_n, eps, inv_rms,
                                                    (int)rows);
  else
    row_inv_rms_kernel<__nv_bfloat16><<<grid, 256, 0, s>>>((const __nv_bfloat16*)x, H, N, D, stride_b, stride_h, stride_n,
                                                           eps, inv_rms, (int)rows);
  return check_launch("row_inv_rms_kernel");
}
