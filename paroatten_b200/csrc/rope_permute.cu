// Fused 3D-RoPE + per-head token permutation (gather on read, coalesced 16-byte stores on
// write).  HBM-bound: each element is read once and written once; the per-axis angle tables
// are a few KB and stay in L1/L2.
#include "common.cuh"
#include "perm.cuh"
#include "rope.cuh"

namespace paro {

// Block = 256 threads; a thread owns one 16-byte slice of a row and walks ROWS_PER_THREAD rows.
// blockIdx.x: group of rows, blockIdx.y: b*H + h.
template <typename T, int D, int MODE>
__global__ void __launch_bounds__(256)
rope_permute_kernel(const T* __restrict__ in, T* __restrict__ out, int H, int N,
                    int64_t sb, int64_t sh, int64_t sn, int n_text, int F, int Hh, int W,
                    const int32_t* __restrict__ order_ids, int inverse, RopeArgs rope) {
  constexpr int TPR = D / 8;            // threads per row
  constexpr int ROWS = 256 / TPR;       // rows per pass
  constexpr int PASSES = 4;
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  const int c8 = (threadIdx.x % TPR) * 8;
  const int r0 = blockIdx.x * (ROWS * PASSES) + threadIdx.x / TPR;
  const PermDecoder dec(order_ids ? order_ids[h] : 0, F, Hh, W);
  const T* src_base = in + b * sb + h * sh;
  T* dst_base = out + (size_t)bh * N * D;

  Pack8<T> val[PASSES];
  int dst_row[PASSES], fy[PASSES], yy[PASSES], xx[PASSES];
#pragma unroll
  for (int i = 0; i < PASSES; ++i) {
    const int row = r0 + i * ROWS;
    dst_row[i] = -1;
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
    val[i].v = *reinterpret_cast<const uint4*>(src_base + (size_t)src * sn + c8);
  }
#pragma unroll
  for (int i = 0; i < PASSES; ++i) {
    if (dst_row[i] < 0) continue;
    if constexpr (MODE != PARO_ROPE_NONE) {
      if (fy[i] >= 0) rotate8<T, MODE>(val[i], c8, D, fy[i], yy[i], xx[i], F, Hh, rope);
    }
    *reinterpret_cast<uint4*>(dst_base + (size_t)dst_row[i] * D + c8) = val[i].v;
  }
}

template <typename T, int MODE>
int launch_rope_mode(const void* in, void* out, int B, int H, int N, int D, int64_t sb, int64_t sh, int64_t sn,
                     int n_text, int F, int Hh, int W, const int32_t* order_ids, int inverse,
                     const RopeArgs& rope, cudaStream_t s) {
  if (D == 128) {
    dim3 grid((N + 63) / 64, B * H);
    rope_permute_kernel<T, 128, MODE><<<grid, 256, 0, s>>>((const T*)in, (T*)out, H, N, sb, sh, sn, n_text, F, Hh, W,
                                                           order_ids, inverse, rope);
  } else {
    dim3 grid((N + 127) / 128, B * H);
    rope_permute_kernel<T, 64, MODE><<<grid, 256, 0, s>>>((const T*)in, (T*)out, H, N, sb, sh, sn, n_text, F, Hh, W,
                                                          order_ids, inverse, rope);
  }
  return check_launch("rope_permute_kernel");
}

template <typename T>
int launch_rope(const void* in, void* out, int B, int H, int N, int D, int64_t sb, int64_t sh, int64_t sn,
                int n_text, int F, int Hh, int W, const int32_t* order_ids, int inverse,
                const RopeArgs& rope, cudaStream_t s) {
#define PARO_ROPE_CASE(M) \
  return launch_rope_mode<T, M>(in, out, B, H, N, D, sb, sh, sn, n_text, F, Hh, W, order_ids, inverse, rope, s)
  if (rope.mode == PARO_ROPE_REAL_F32) PARO_ROPE_CASE(PARO_ROPE_REAL_F32);
  if (rope.mode == PARO_ROPE_COMPLEX_F64) PARO_ROPE_CASE(PARO_ROPE_COMPLEX_F64);
  PARO_ROPE_CASE(PARO_ROPE_NONE);
#undef PARO_ROPE_CASE
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
    PARO_REQUIRE(cos_tab && sin_tab, PARO_EINVAL, "paro_rope_permute: rope tables missing");
    PARO_REQUIRE(pairs_f >= 0 && pairs_h >= 0 && pairs_f + pairs_h <= D / 2, PARO_ESHAPE,
                 "paro_rope_permute: pairs_f + pairs_h exceeds D/2");
  }
  RopeArgs r{rope_mode, cos_tab, sin_tab, pairs_f, pairs_h};
  cudaStream_t s = (cudaStream_t)stream;
  return dtype == PARO_F16
             ? launch_rope<__half>(in, out, B, H, N, D, stride_b, stride_h, stride_n, n_text, F, Hh, W, order_ids, inverse, r, s)
             : launch_rope<__nv_bfloat16>(in, out, B, H, N, D, stride_b, stride_h, stride_n, n_text, F, Hh, W, order_ids, inverse, r, s);
}
