// Token-permutation index tables and compaction of the boolean block mask into walk lists.
// Integer work only; every result is compared bit-for-bit with the CPU oracle.
#include "common.cuh"
#include "perm.cuh"

namespace paro {

__global__ void perm_index_kernel(const int32_t* __restrict__ order_ids, int F, int Hh, int W,
                                  int32_t* __restrict__ idx) {
  const int h = blockIdx.y;
  const int n_img = F * Hh * W;
  const PermDecoder dec(order_ids[h], F, Hh, W);
  for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < n_img; j += gridDim.x * blockDim.x) {
    int f, y, x;
    idx[(size_t)h * n_img + j] = dec.source(j, f, y, x);
  }
}

// One warp per row: kept blocks of a q-block (pair == 0) or of the union of q-blocks 2p, 2p+1
// (pair == 1).  counts go to out[row + 1]; the scan turns them into exclusive offsets.
template <bool PAIR>
__device__ __forceinline__ uint32_t row_flags(const uint8_t* __restrict__ mask, int slice, int row,
                                              int nbq, int nbk, int kb) {
  if (kb >= nbk) return 0;
  if (!PAIR) return mask[((size_t)slice * nbq + row) * nbk + kb] != 0;
  const int q0 = 2 * row, q1 = 2 * row + 1;
  uint32_t f = mask[((size_t)slice * nbq + q0) * nbk + kb] != 0;
  if (q1 < nbq) f |= (mask[((size_t)slice * nbq + q1) * nbk + kb] != 0) << 1;
  return f;
}

template <bool PAIR>
__global__ void plan_count_kernel(const uint8_t* __restrict__ mask, int slices, int nbq, int nbk,
                                  int rows_per_slice, int32_t* __restrict__ out) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int total = slices * rows_per_slice;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < total; r += warps) {
    const int slice = r / rows_per_slice, row = r % rows_per_slice;
    int cnt = 0;
    for (int k0 = 0; k0 < nbk; k0 += 32)
      cnt += __popc(__ballot_sync(0xffffffffu, row_flags<PAIR>(mask, slice, row, nbq, nbk, k0 + lane) != 0));
    if (lane == 0) out[r + 1] = cnt;
  }
  if (blockIdx.x == 0 && threadIdx.x == 0) out[0] = 0;
}

// In-place inclusive scan of a[1..n] by a single block (a[0] stays 0): each thread owns a
// contiguous segment.  n is at most a few hundred thousand rows.
__global__ void scan_kernel(int32_t* __restrict__ a, int n) {
  __shared__ int32_t part[1024];
  const int t = threadIdx.x;
  const int seg = (n + blockDim.x - 1) / blockDim.x;
  const int lo = 1 + t * seg, hi = min(n + 1, lo + seg);
  int32_t s = 0;
  for (int i = lo; i < hi; ++i) s += a[i];
  part[t] = s;
  __syncthreads();
  for (int off = 1; off < (int)blockDim.x; off <<= 1) {
    int32_t v = (t >= off) ? part[t - off] : 0;
    __syncthreads();
    part[t] += v;
    __syncthreads();
  }
  int32_t run = (t == 0) ? 0 : part[t - 1];
  for (int i = lo; i < hi; ++i) {
    run += a[i];
    a[i] = run;
  }
}

template <bool PAIR>
__global__ void plan_fill_kernel(const uint8_t* __restrict__ mask, int slices, int nbq, int nbk,
                                 int rows_per_slice, const int32_t* __restrict__ ptr,
                                 int32_t* __restrict__ out, int64_t cap) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  const int total = slices * rows_per_slice;
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < total; r += warps) {
    const int slice = r / rows_per_slice, row = r % rows_per_slice;
    int64_t base = ptr[r];
    for (int k0 = 0; k0 < nbk; k0 += 32) {
      const uint32_t f = row_flags<PAIR>(mask, slice, row, nbq, nbk, k0 + lane);
      const uint32_t b = __ballot_sync(0xffffffffu, f != 0);
      if (f) {
        const int64_t pos = base + __popc(b & ((1u << lane) - 1u));
        if (pos < cap) out[pos] = PAIR ? ((k0 + lane) * 4 + (int)f) : (k0 + lane);
      }
      base += __popc(b);
    }
  }
}

// Schedule of one pair of adjacent q-blocks, built from its merged list (ascending kb*4 + flags):
// first the k-blocks BOTH q-blocks keep, in ascending order -- one tile then serves all 128 rows --
// then the r-th block only q-block 2p keeps side by side with the r-th block only q-block 2p+1
// keeps.  Entry i = kbA | kbB << 16 (0xFFFF = this q-block has no tile in step i); both q-blocks'
// steps are contiguous from 0.  One warp per pair; the pair's entries live at the offsets of its
// merged list (a schedule is never longer than the merged list), unused slots keep 0xFFFFFFFF.
__global__ void plan_schedule_kernel(const int32_t* __restrict__ pair_ptr, const int32_t* __restrict__ pair_ent,
                                     int prows, uint32_t* __restrict__ sched, int32_t* __restrict__ cnt) {
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  uint16_t* sched16 = reinterpret_cast<uint16_t*>(sched);
  for (int r = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; r < prows; r += warps) {
    const int e0 = pair_ptr[r], e1 = pair_ptr[r + 1];
    for (int e = e0 + lane; e < e1; e += 32) sched[e] = 0xFFFFFFFFu;
    __syncwarp();
    int ns = 0;
    for (int e = e0; e < e1; e += 32) {
      const int v = e + lane < e1 ? pair_ent[e + lane] : 0;
      ns += __popc(__ballot_sync(0xffffffffu, (v & 3) == 3));
    }
    int c3 = 0, c1 = 0, c2 = 0;
    for (int e = e0; e < e1; e += 32) {
      const int v = e + lane < e1 ? pair_ent[e + lane] : 0;
      const int f = v & 3, kb = v >> 2;
      const uint32_t m3 = __ballot_sync(0xffffffffu, f == 3), m1 = __ballot_sync(0xffffffffu, f == 1),
                     m2 = __ballot_sync(0xffffffffu, f == 2);
      const uint32_t below = (1u << lane) - 1u;
      if (f == 3) {
        const int slot = c3 + __popc(m3 & below);
        sched[e0 + slot] = (uint32_t)kb | ((uint32_t)kb << 16);
      } else if (f == 1) {
        sched16[2 * (size_t)(e0 + ns + c1 + __popc(m1 & below))] = (uint16_t)kb;
      } else if (f == 2) {
        sched16[2 * (size_t)(e0 + ns + c2 + __popc(m2 & below)) + 1] = (uint16_t)kb;
      }
      c3 += __popc(m3); c1 += __popc(m1); c2 += __popc(m2);
    }
    if (lane == 0) {
      cnt[2 * r] = ns + c1;
      cnt[2 * r + 1] = ns + c2;
    }
  }
}


}  // namespace paro

using namespace paro;

extern "C" int paro_build_perm_index(const int32_t* order_ids, int H, int F, int Hh, int W,
                                     int32_t* idx, paro_stream_t stream) {
  PARO_REQUIRE(order_ids && idx, PARO_EINVAL, "paro_build_perm_index: null pointer");
  PARO_REQUIRE(H > 0 && F > 0 && Hh > 0 && W > 0, PARO_ESHAPE, "paro_build_perm_index: empty grid");
  PARO_REQUIRE((int64_t)F * Hh * W < (1ll << 31), PARO_ESHAPE, "paro_build_perm_index: grid too large");
  const int n_img = F * Hh * W;
  dim3 grid((unsigned)min(1024, (n_img + 255) / 256), (unsigned)H);
  perm_index_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(order_ids, F, Hh, W, idx);
  return check_launch("perm_index_kernel");
}

extern "C" int paro_plan_count(const uint8_t* mask, int slices, int nbq, int nbk,
                               int32_t* row_ptr, int32_t* pair_ptr, paro_stream_t stream) {
  PARO_REQUIRE(mask && row_ptr && pair_ptr, PARO_EINVAL, "paro_plan_count: null pointer");
  PARO_REQUIRE(slices > 0 && nbq > 0 && nbk > 0, PARO_ESHAPE, "paro_plan_count: empty mask");
  PARO_REQUIRE((int64_t)slices * nbq * nbk < (1ll << 31), PARO_ESHAPE, "paro_plan_count: mask too large");
  cudaStream_t s = (cudaStream_t)stream;
  const int npairs = (nbq + 1) / 2;
  const int rows = slices * nbq, prow = slices * npairs;
  plan_count_kernel<false><<<min(4096, (rows + 7) / 8), 256, 0, s>>>(mask, slices, nbq, nbk, nbq, row_ptr);
  plan_count_kernel<true><<<min(4096, (prow + 7) / 8), 256, 0, s>>>(mask, slices, nbq, nbk, npairs, pair_ptr);
  scan_kernel<<<1, 1024, 0, s>>>(row_ptr, rows);
  scan_kernel<<<1, 1024, 0, s>>>(pair_ptr, prow);
  return check_launch("plan_count", 4);
}

extern "C" int paro_plan_fill(const uint8_t* mask, int slices, int nbq, int nbk,
                              const int32_t* row_ptr, int32_t* cols, int64_t cols_cap,
                              const int32_t* pair_ptr, int32_t* pair_ent, int64_t pair_cap,
                              paro_stream_t stream) {
  PARO_REQUIRE(mask && row_ptr && pair_ptr, PARO_EINVAL, "paro_plan_fill: null pointer");
  PARO_REQUIRE(slices > 0 && nbq > 0 && nbk > 0, PARO_ESHAPE, "paro_plan_fill: empty mask");
  PARO_REQUIRE((cols || cols_cap == 0) && (pair_ent || pair_cap == 0), PARO_EINVAL,
               "paro_plan_fill: null output with non-zero capacity");
  cudaStream_t s = (cudaStream_t)stream;
  const int npairs = (nbq + 1) / 2;
  const int rows = slices * nbq, prow = slices * npairs;
  if (cols_cap > 0)
    plan_fill_kernel<false><<<min(4096, (rows + 7) / 8), 256, 0, s>>>(mask, slices, nbq, nbk, nbq, row_ptr,
                                                                      cols, cols_cap);
  if (pair_cap > 0)
    plan_fill_kernel<true><<<min(4096, (prow + 7) / 8), 256, 0, s>>>(mask, slices, nbq, nbk, npairs, pair_ptr,
                                                                     pair_ent, pair_cap);
  return check_launch("plan_fill", (cols_cap > 0) + (pair_cap > 0));
}

extern "C" int paro_plan_schedule(const int32_t* pair_ptr, const int32_t* pair_ent, int slices, int nbq, int nbk,
                                  uint32_t* sched, int32_t* sched_cnt, paro_stream_t stream) {
  PARO_REQUIRE(pair_ptr && sched_cnt, PARO_EINVAL, "paro_plan_schedule: null pointer");
  PARO_REQUIRE(slices > 0 && nbq > 0, PARO_ESHAPE, "paro_plan_schedule: empty plan");
  PARO_REQUIRE(nbk > 0 && nbk < 0xFFFF, PARO_ESHAPE, "paro_plan_schedule: nbk = %d does not fit 16 bits", nbk);
  const int prow = slices * ((nbq + 1) / 2);
  plan_schedule_kernel<<<min(4096, (prow + 7) / 8), 256, 0, (cudaStream_t)stream>>>(pair_ptr, pair_ent, prow, sched,
                                                                                    sched_cnt);
  return check_launch("plan_schedule_kernel");
}
