// Types and small device helpers of the block-sparse attention kernel (sparse_attn.cu).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "common.cuh"
#include "umma.cuh"

namespace paro {

constexpr int ATT_THREADS = 384;
constexpr int ATT_SOFTMAX_THREADS = 256;
constexpr int TMEM_COLS = 256;
constexpr long long WAIT_LIMIT = 400000000;  // SM cycles (~0.2 s) before a wait gives up
constexpr float SCORE_BIAS = 12582912.0f;    // 1.5 * 2^23, bit pattern 0x4B400000

// Words of the redo work space handed to paro_sparse_attn: [0] number of work items the fixed-reference walk
// gave back, [1..] the items (block indices of the fast launch).
constexpr int REDO_HEADER = 1;

struct AttnParams {
  const int8_t* q8;
  const float* q_scale;
  const float* k_scale;
  const float* v_scale;
  const float* vm;
  const int32_t* pair_ptr;
  const uint32_t* sched;
  const int32_t* sched_cnt;
  const int32_t* inv_idx;
  void* out;
  float* lse;
  int32_t* status;
  int32_t* redo;        // work space described above
  int64_t osb, osh, osn;
  int plan_slices, q_group, n_text;
  int B, H, N, npairs, nb;
  int from_list;        // 1: work items are read from the redo list (second launch)
  float scale_log2;     // sm_scale * log2(e)
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Packed pairs of fp32 (sm_100a has 2-wide fp32 FMA / ADD).
__device__ __forceinline__ uint64_t pack2(float a, float b) {
  uint64_t r;
  asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(a), "f"(b));
  return r;
}
__device__ __forceinline__ void unpack2(uint64_t r, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(r));
}
__device__ __forceinline__ uint64_t fma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t r;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
  return r;
}
__device__ __forceinline__ uint64_t add2(uint64_t a, uint64_t b) {
  uint64_t r;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
  return r;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float r;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
  return r;
}
// Two fp32 -> one 32-bit word of two bf16 (first argument in the low half).
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  uint32_t r;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
  return r;
}
// Global load that stays where it is written (the compiler may not sink it towards its use).
__device__ __forceinline__ uint32_t ld_pinned_u32(const uint32_t* ptr) {
  uint32_t v;
  asm volatile("ld.global.nc.u32 %0, [%1];" : "=r"(v) : "l"(ptr));
  return v;
}
__device__ __forceinline__ void named_barrier(int id, int threads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ void report_timeout(const AttnParams& p, volatile int* abort_flag, int where, int iter) {
  if (atomicCAS(p.status, 0, PARO_ETIMEOUT) == 0) {
    p.status[1] = where;
    p.status[2] = (int)blockIdx.x;
    p.status[3] = iter;
  }
  *abort_flag = 1;
}

// Hand-off of a value between two warps through shared memory (release/acquire at CTA scope).
__device__ __forceinline__ int ld_acquire_shared(const volatile int* ptr) {
  int v;
  asm volatile("ld.acquire.cta.shared.b32 %0, [%1];"
               : "=r"(v)
               : "r"(umma::smem_u32(const_cast<const int*>(ptr)))
               : "memory");
  return v;
}
__device__ __forceinline__ void st_release_shared(volatile int* ptr, int v) {
  asm volatile("st.release.cta.shared.b32 [%0], %1;" ::"r"(umma::smem_u32(const_cast<int*>(ptr))), "r"(v) : "memory");
}
// The same by the lanes for which `pred` holds, as one predicated instruction (no divergent branch: see
// umma::mbar_arrive_if).
__device__ __forceinline__ void st_release_shared_if(volatile int* ptr, int v, bool pred) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %2, 0;\n\t"
      "@p st.release.cta.shared.b32 [%0], %1;\n\t}"
      ::"r"(umma::smem_u32(const_cast<int*>(ptr))), "r"(v), "r"((uint32_t)pred)
      : "memory");
}

// What a ring producer remembers about the last S tiles it loaded, oldest first: the commit barrier that
// tells when the MMAs reading the tile have finished (shared-memory address | phase parity << 31).
// Before it reuses a stage, the producer waits on the oldest entry -- the tile that holds that stage.
template <int S> struct ReleaseFifo {
  uint32_t tok[S];
  __device__ __forceinline__ uint32_t oldest() const { return tok[0]; }
  __device__ __forceinline__ void push(uint32_t v) {
#pragma unroll
    for (int k = 0; k + 1 < S; ++k) tok[k] = tok[k + 1];
    tok[S - 1] = v;
  }
};
__device__ __forceinline__ uint32_t commit_token(uint32_t bars_saddr, int half, int step) {
  return (bars_saddr + 32u * (uint32_t)half + 8u * ((uint32_t)step & 3u)) | ((((uint32_t)step >> 2) & 1u) << 31);
}

}  // namespace paro
