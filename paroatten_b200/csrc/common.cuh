// Shared host/device helpers of libparo_b200: error reporting and 16-bit float conversion.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/paro_b200.h"

namespace paro {

// Thread-local message returned by paro_last_error().
char* error_buffer();
int fail(int code, const char* fmt, ...);

#define PARO_CUDA_OK(expr)                                                              \
  do {                                                                                  \
    cudaError_t e__ = (expr);                                                           \
    if (e__ != cudaSuccess)                                                             \
      return ::paro::fail(PARO_ECUDA, "%s: %s", #expr, cudaGetErrorString(e__));        \
  } while (0)

#define PARO_REQUIRE(cond, code, ...) \
  do {                                \
    if (!(cond)) return ::paro::fail(code, __VA_ARGS__); \
  } while (0)

// Process-wide count of kernels this library has launched (read by paro_launch_count()).
void count_launches(int n);
long long launches();

inline int check_launch(const char* what, int n_kernels = 1) {
  count_launches(n_kernels);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(PARO_ECUDA, "%s launch: %s", what, cudaGetErrorString(e));
  return PARO_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Common argument checks for a [B,H,N,D] tensor addressed through element strides.
int check_tensor(const char* name, const void* p, int dtype, int B, int H, int N, int D,
                 int64_t sb, int64_t sh, int64_t sn);

template <typename T> struct F16Traits;
template <> struct F16Traits<__half> {
  static __device__ __forceinline__ float to_float(__half v) { return __half2float(v); }
  static __device__ __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
};
template <> struct F16Traits<__nv_bfloat16> {
  static __device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
  static __device__ __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
};

// Eight 16-bit values moved as one 16-byte vector.
template <typename T> union Pack8 {
  uint4 v;
  T e[8];
};

}  // namespace paro
