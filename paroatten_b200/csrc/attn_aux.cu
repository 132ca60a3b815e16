// Two small companions of the attention kernel:
//   paro_plan_validate      checks walk lists that were not built by this library (loaded from a file,
//                           handed over the C ABI) before the attention kernel follows them;
//   paro_merge_attn_states  combines two partial attention results (O, LSE) computed over disjoint sets
//                           of key blocks into the result over their union -- what the LSE output is for
//                           (sequence-parallel / ring composition, reference core.py:55-57).
#include "common.cuh"

namespace paro {

enum PlanFault : int32_t {
  PLAN_OK = 0,
  PLAN_BAD_OFFSETS = 1,     // pair_ptr not starting at 0, not monotone, or beyond the schedule's length
  PLAN_BAD_COUNT = 2,       // more steps than slots, a negative count, or steps for a q-block that does not exist
  PLAN_BAD_BLOCK = 3,       // a k-block id >= nbk inside a q-block's steps
  PLAN_BAD_FILLER = 4,      // an entry past a q-block's steps that is not the 0xFFFF filler
  PLAN_BAD_ORDER = 5,       // k-blocks of a section (shared / own) not strictly ascending
};

// One warp per pair of q-blocks.  report[0] = fault, [1] = pair row, [2] = step, [3] = offending value;
// the first fault found wins.
__global__ void plan_validate_kernel(const int32_t* __restrict__ pair_ptr, const uint32_t* __restrict__ sched,
                                     const int32_t* __restrict__ cnt, int prows, int npairs, int nbq, int nbk,
                                     long long sched_len, int32_t* __restrict__ report) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  auto fault = [&](int code, int row, int step, int value) {
    if (atomicCAS(report, 0, code) == 0) {
      report[1] = row;
      report[2] = step;
      report[3] = value;
    }
  };
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < prows; r += warps) {
    const long long e0 = pair_ptr[r], e1 = pair_ptr[r + 1];
    if ((r == 0 && e0 != 0) || e0 < 0 || e1 < e0 || e1 > sched_len) {
      if (lane == 0) fault(PLAN_BAD_OFFSETS, r, 0, (int)e1);
      continue;
    }
    const int slots = (int)(e1 - e0);
    const int na = cnt[2 * r] & 0xFFFF, nb = cnt[2 * r + 1] & 0xFFFF;   // (high halves: optional q-block ids)
    const bool has_second = 2 * (r % npairs) + 1 < nbq;
    const int qa = (int)((uint32_t)cnt[2 * r] >> 16), qb = (int)((uint32_t)cnt[2 * r + 1] >> 16);
    if (qa > nbq || qb > nbq) {   // q-block id + 1 of a half, 0 = none given
      if (lane == 0) fault(PLAN_BAD_BLOCK, r, -1, qa > nbq ? qa - 1 : qb - 1);
      continue;
    }
    if (na < 0 || nb < 0 || na > slots || nb > slots || (!has_second && nb != 0)) {
      if (lane == 0) fault(PLAN_BAD_COUNT, r, 0, na > slots || na < 0 ? na : nb);
      continue;
    }
    for (int i = lane; i < slots; i += 32) {
      const uint32_t e = sched[e0 + i];
      const int ka = (int)(e & 0xFFFFu), kb = (int)(e >> 16);
      if (i < na ? ka >= nbk : ka != 0xFFFF) fault(i < na ? PLAN_BAD_BLOCK : PLAN_BAD_FILLER, r, i, ka);
      if (i < nb ? kb >= nbk : kb != 0xFFFF) fault(i < nb ? PLAN_BAD_BLOCK : PLAN_BAD_FILLER, r, i, kb);
      if (i > 0 && i < max(na, nb)) {
        // sections: shared steps (ka == kb) first, then each q-block's own steps; ascending inside a section
        const uint32_t ep = sched[e0 + i - 1];
        const int pa = (int)(ep & 0xFFFFu), pb = (int)(ep >> 16);
        const bool sh = i < na && i < nb && ka == kb, psh = (i - 1) < na && (i - 1) < nb && pa == pb;
        if (sh && !psh) fault(PLAN_BAD_ORDER, r, i, ka);                 // a shared step after an own step
        if (sh == psh) {
          if (i < na && ka <= pa) fault(PLAN_BAD_ORDER, r, i, ka);
          if (i < nb && kb <= pb) fault(PLAN_BAD_ORDER, r, i, kb);
        }
      }
    }
  }
}

// out = (o_a * w_a + o_b * w_b), w_x = exp(lse_x - lse), lse = log(exp(lse_a) + exp(lse_b)); a side whose
// LSE is -inf (no kept block for that row) contributes nothing.  One thread per 8 channels of a row.
template <typename T>
__global__ void merge_states_kernel(const T* __restrict__ oa, const float* __restrict__ la, const T* __restrict__ ob,
                                    const float* __restrict__ lb, T* __restrict__ out, float* __restrict__ lo, int H,
                                    int N, int D, int64_t sb, int64_t sh, int64_t sn, long long rows) {
  const int tpr = D / 8;
  const long long t = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  const long long row = t / tpr;
  if (row >= rows) return;
  const int c8 = (int)(t % tpr) * 8;
  const int n = (int)(row % N);
  const long long bh = row / N;
  const int h = (int)(bh % H);
  const long long b = bh / H;
  const float a = la[row], c = lb[row];
  const float m = fmaxf(a, c);
  float wa = 0.f, wb = 0.f, l = -INFINITY;
  if (m > -INFINITY) {
    const float ea = expf(a - m), eb = expf(c - m);   // exp(-inf) = 0
    const float s = ea + eb;
    wa = ea / s;
    wb = eb / s;
    l = m + logf(s);
  }
  const int64_t off = b * sb + h * sh + (int64_t)n * sn + c8;
  Pack8<T> pa, pb, po;
  pa.v = *reinterpret_cast<const uint4*>(oa + off);
  pb.v = *reinterpret_cast<const uint4*>(ob + off);
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    // a weight of exactly 0 drops that side even when it holds Inf or NaN (unwritten rows)
    const float va = wa != 0.f ? wa * F16Traits<T>::to_float(pa.e[j]) : 0.f;
    const float vb = wb != 0.f ? wb * F16Traits<T>::to_float(pb.e[j]) : 0.f;
    po.e[j] = F16Traits<T>::from_float(va + vb);
  }
  *reinterpret_cast<uint4*>(out + off) = po.v;
  if (lo && c8 == 0) lo[row] = l;
}

}  // namespace paro

using namespace paro;

extern "C" int paro_plan_validate(const int32_t* pair_ptr, const uint32_t* sched, const int32_t* sched_cnt, int slices,
                                  int nbq, int nbk, int64_t sched_len, int32_t* report, paro_stream_t stream) {
  PARO_REQUIRE(pair_ptr && sched && sched_cnt && report, PARO_EINVAL, "paro_plan_validate: null pointer");
  PARO_REQUIRE(slices > 0 && nbq > 0 && nbk > 0 && nbk < 0xFFFF && sched_len >= 0, PARO_ESHAPE,
               "paro_plan_validate: bad sizes (slices %d, nbq %d, nbk %d)", slices, nbq, nbk);
  cudaStream_t s = (cudaStream_t)stream;
  const int npairs = (nbq + 1) / 2;
  const long long prows = (long long)slices * npairs;
  PARO_REQUIRE(prows < (1ll << 31), PARO_ESHAPE, "paro_plan_validate: too many pairs");
  PARO_CUDA_OK(cudaMemsetAsync(report, 0, 4 * sizeof(int32_t), s));
  plan_validate_kernel<<<(unsigned)min(4096ll, (prows + 7) / 8), 256, 0, s>>>(pair_ptr, sched, sched_cnt, (int)prows,
                                                                              npairs, nbq, nbk, sched_len, report);
  if (int rc = check_launch("plan_validate_kernel")) return rc;
  int32_t w[4] = {0, 0, 0, 0};
  PARO_CUDA_OK(cudaMemcpyAsync(w, report, sizeof(w), cudaMemcpyDeviceToHost, s));
  PARO_CUDA_OK(cudaStreamSynchronize(s));
  static const char* const what[] = {"", "offsets not monotone from 0 or beyond the schedule", "step count out of range",
                                     "k-block id out of range", "entry past a q-block's steps is not the filler",
                                     "k-blocks of a section not strictly ascending"};
  if (w[0] != 0)
    return fail(PARO_EINVAL, "sparse plan rejected: %s (pair row %d, step %d, value %d)",
                what[w[0] >= 1 && w[0] <= 5 ? w[0] : 0], w[1], w[2], w[3]);
  return PARO_OK;
}

extern "C" int paro_merge_attn_states(const void* o_a, const float* lse_a, const void* o_b, const float* lse_b, void* out,
                                      float* lse_out, int dtype, int B, int H, int N, int D, int64_t stride_b,
                                      int64_t stride_h, int64_t stride_n, paro_stream_t stream) {
  PARO_REQUIRE(lse_a && lse_b, PARO_EINVAL, "paro_merge_attn_states: null pointer");
  if (int rc = check_tensor("paro_merge_attn_states(o_a)", o_a, dtype, B, H, N, D, stride_b, stride_h, stride_n)) return rc;
  if (int rc = check_tensor("paro_merge_attn_states(o_b)", o_b, dtype, B, H, N, D, stride_b, stride_h, stride_n)) return rc;
  if (int rc = check_tensor("paro_merge_attn_states(out)", out, dtype, B, H, N, D, stride_b, stride_h, stride_n)) return rc;
  const long long rows = (long long)B * H * N;
  const long long threads = rows * (D / 8);
  const unsigned blocks = (unsigned)((threads + 255) / 256);
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PARO_F16)
    merge_states_kernel<__half><<<blocks, 256, 0, s>>>((const __half*)o_a, lse_a, (const __half*)o_b, lse_b, (__half*)out,
                                                       lse_out, H, N, D, stride_b, stride_h, stride_n, rows);
  else
    merge_states_kernel<__nv_bfloat16><<<blocks, 256, 0, s>>>((const __nv_bfloat16*)o_a, lse_a, (const __nv_bfloat16*)o_b,
                                                              lse_b, (__nv_bfloat16*)out, lse_out, H, N, D, stride_b,
                                                              stride_h, stride_n, rows);
  return check_launch("merge_states_kernel");
}
