// INT8 quantisation of Q / mean-smoothed K and FP8-e4m3 quantisation of V.
// All three are HBM-bound streaming kernels: 16-byte loads, every input element read once per
// pass, results compared bit-for-bit with the CPU oracle (IEEE divide/multiply, no fast-math).
#include <cuda_fp8.h>

#include <mutex>
#include <type_traits>

#include "common.cuh"
#include "norm.cuh"
#include "perm.cuh"
#include "rope.cuh"

namespace paro {

// Optional front end of the fused kernels: row `tok` of the (reordered) sequence is read from
// token source(tok) of the input and rotated by that token's grid position, i.e. the quantisers
// consume RoPE + per-head reordering on the fly instead of a materialised bf16 copy.
struct Gather {
  int enabled;        // 0: plain input, tok -> tok, no RoPE
  int n_text, F, Hh, W;
  const int32_t* order_ids;   // [H] or nullptr (natural order)
  RopeArgs rope;
};

// GM (compile time): 0 plain input; 1 reordering only; 2 reordering + fp32 rotation; 3 reordering +
// fp64 rotation.  A kernel instance only carries the code and registers of its own mode.
enum { GM_PLAIN = 0, GM_REORDER = 1, GM_ROPE_F32 = 2, GM_ROPE_F64 = 3 };

inline int gather_mode(const Gather& g) {
  if (!g.enabled) return GM_PLAIN;
  if (g.rope.mode == PARO_ROPE_REAL_F32) return GM_ROPE_F32;
  if (g.rope.mode == PARO_ROPE_COMPLEX_F64) return GM_ROPE_F64;
  return GM_REORDER;
}

template <int GM>
struct GatherCtx {
  const Gather& g;
  PermDecoder dec;
  __device__ GatherCtx(const Gather& g_, int h)
      : g(g_), dec(GM != GM_PLAIN && g_.order_ids ? g_.order_ids[h] : 0, g_.F, g_.Hh, g_.W) {}
  // source token of row `tok`; f < 0 for rows that are not rotated (text tokens, or no gather)
  __device__ __forceinline__ int source(int tok, int& f, int& y, int& x) const {
    f = y = x = -1;
    if constexpr (GM == GM_PLAIN) return tok;
    if (tok < g.n_text) return tok;
    const int src = g.n_text + dec.source(tok - g.n_text, f, y, x);
    return src;
  }
  template <typename T> __device__ __forceinline__ void rotate(Pack8<T>& v, int c8, int D, int f, int y, int x) const {
    if constexpr (GM == GM_ROPE_F32) {
      if (f >= 0) rotate8<T, PARO_ROPE_REAL_F32>(v, c8, D, f, y, x, g.F, g.Hh, g.rope);
    } else if constexpr (GM == GM_ROPE_F64) {
      if (f >= 0) rotate8<T, PARO_ROPE_COMPLEX_F64>(v, c8, D, f, y, x, g.F, g.Hh, g.rope);
    }
  }
};

// Calls `fn(std::integral_constant<int, GM>)` for the mode of `g`.
template <typename Fn> void dispatch_gather(const Gather& g, Fn&& fn) {
  switch (gather_mode(g)) {
    case GM_REORDER: fn(std::integral_constant<int, GM_REORDER>{}); break;
    case GM_ROPE_F32: fn(std::integral_constant<int, GM_ROPE_F32>{}); break;
    case GM_ROPE_F64: fn(std::integral_constant<int, GM_ROPE_F64>{}); break;
    default: fn(std::integral_constant<int, GM_PLAIN>{}); break;
  }
}

constexpr int STATS_CHUNK = 512;  // tokens reduced by one CTA of the channel-statistics pass

struct ChannelPartial {
  double sum;
  float mx, mn;
};

// ---------------------------------------------------------------------------------------------
// Pass 1 of the per-channel reductions: per (b,h, chunk of tokens) the fp64 sum, max and min of
// every channel.  Thread = one 8-channel slice of a token row; rows of the chunk are walked in a
// fixed order and the cross-thread reduction is sequential, so results do not depend on timing.
template <typename T, int D, int GM>
__global__ void __launch_bounds__(256)
channel_stats_kernel(const T* __restrict__ x, int H, int N, int64_t sb, int64_t sh, int64_t sn,
                     ChannelPartial* __restrict__ part, int chunks, const Gather gather) {
  constexpr int TPR = D / 8;
  constexpr int ROWS = 256 / TPR;
  __shared__ double s_sum[ROWS][D + 1];
  __shared__ float s_mx[ROWS][D + 1];
  __shared__ float s_mn[ROWS][D + 1];
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  const int c8 = (threadIdx.x % TPR) * 8, r = threadIdx.x / TPR;
  const int t0 = blockIdx.x * STATS_CHUNK, t1 = min(N, t0 + STATS_CHUNK);
  const T* base = x + b * sb + h * sh;
  const GatherCtx<GM> gc(gather, h);
  double sum[8];
  float mx[8], mn[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) { sum[j] = 0.0; mx[j] = -INFINITY; mn[j] = INFINITY; }
  // four rows are in flight per thread; they are accumulated in the order of a plain loop
  for (int t = t0 + r; t < t1; t += 4 * ROWS) {
    Pack8<T> v[4];
    int gf[4], gy[4], gx[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int tu = t + u * ROWS;
      gf[u] = gy[u] = gx[u] = -1;
      if (tu < t1) v[u].v = *reinterpret_cast<const uint4*>(base + (size_t)gc.source(tu, gf[u], gy[u], gx[u]) * sn + c8);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      if (t + u * ROWS >= t1) break;
      gc.rotate(v[u], c8, D, gf[u], gy[u], gx[u]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const float f = F16Traits<T>::to_float(v[u].e[j]);
        sum[j] += (double)f;
        mx[j] = fmaxf(mx[j], f);
        mn[j] = fminf(mn[j], f);
      }
    }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) { s_sum[r][c8 + j] = sum[j]; s_mx[r][c8 + j] = mx[j]; s_mn[r][c8 + j] = mn[j]; }
  __syncthreads();
  if (threadIdx.x < D) {
    double s = 0.0;
    float a = -INFINITY, i = INFINITY;
    for (int k = 0; k < ROWS; ++k) {
      s += s_sum[k][threadIdx.x];
      a = fmaxf(a, s_mx[k][threadIdx.x]);
      i = fminf(i, s_mn[k][threadIdx.x]);
    }
    ChannelPartial p{s, a, i};
    part[((size_t)bh * chunks + blockIdx.x) * D + threadIdx.x] = p;
  }
}

// Pass 2: fold the chunk partials of one (b,h) in chunk order.
// mean = fp32(sum/N); amax = max(1e-7, max(|max-mean|, |min-mean|)) (equal to max|x-mean|, the
// form of fused.cu:385-389); scale = amax/scale_max.
template <typename T>
__global__ void channel_finalize_kernel(const ChannelPartial* __restrict__ part, int chunks, int D, int N,
                                        int smooth, float scale_max, T* __restrict__ mean_t,
                                        float* __restrict__ mean_f32, float* __restrict__ scale,
                                        float* __restrict__ inv_out, float* __restrict__ mean_used) {
  const int bh = blockIdx.x, d = threadIdx.x;
  double s = 0.0;
  float a = -INFINITY, i = INFINITY;
  for (int c = 0; c < chunks; ++c) {
    const ChannelPartial p = part[((size_t)bh * chunks + c) * D + d];
    s += p.sum;
    a = fmaxf(a, p.mx);
    i = fminf(i, p.mn);
  }
  const float mean = smooth ? __double2float_rn(s / (double)N) : 0.0f;
  if (mean_t) mean_t[(size_t)bh * D + d] = F16Traits<T>::from_float(__double2float_rn(s / (double)N));
  if (mean_f32) mean_f32[(size_t)bh * D + d] = __double2float_rn(s / (double)N);
  if (scale) {
    const float amax = fmaxf(1e-7f, fmaxf(fabsf(__fsub_rn(a, mean)), fabsf(__fsub_rn(i, mean))));
    scale[(size_t)bh * D + d] = __fdiv_rn(amax, scale_max);
    inv_out[(size_t)bh * D + d] = __fdiv_rn(scale_max, amax);
    mean_used[(size_t)bh * D + d] = mean;
  }
}

// ---------------------------------------------------------------------------------------------
// INT8: CTA = 128 threads = one 64-token block; warp w owns tokens 16w..16w+15.
template <typename T, int D, int GROUP, int GM, int NM>
__global__ void __launch_bounds__(128, GM == GM_ROPE_F64 ? 4 : (GM == GM_ROPE_F32 || NM != PARO_NORM_NONE ? 5 : 6))
quant_int8_kernel(const T* __restrict__ x, const T* __restrict__ km, int8_t* __restrict__ out,
                  float* __restrict__ scale, int H, int N, int64_t sb, int64_t sh, int64_t sn,
                  float fold, int n_scale_per_bh, const Gather gather, const NormArgs norm) {
  constexpr int TPR = D / 8;          // threads per token row
  constexpr int RPL = 32 / TPR;       // rows covered by one warp-wide load
  constexpr int LOADS = 16 / RPL;     // loads per thread
  __shared__ float s_amax[4];
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c8 = (lane % TPR) * 8;
  const int tok0 = blockIdx.x * 64 + warp * 16 + lane / TPR;
  const T* base = x + b * sb + h * sh;
  const GatherCtx<GM> gc(gather, h);

  float mean[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) mean[j] = 0.f;
  if (km) {
    Pack8<T> m;
    m.v = *reinterpret_cast<const uint4*>(km + (size_t)bh * D + c8);
#pragma unroll
    for (int j = 0; j < 8; ++j) mean[j] = F16Traits<T>::to_float(m.e[j]);
  }

  // the (rotated) rows stay packed in registers; they are widened once for the maximum and once more
  // for the rounding, which costs a shift per element and halves the registers held across the barrier
  Pack8<T> row[LOADS];
  float amax = 0.f;
  auto widen = [&](const Pack8<T>& p, int j) {
    float f = F16Traits<T>::to_float(p.e[j]);
    if (km) f = __fsub_rn(f, mean[j]);
    if (fold != 0.f) f = __fmul_rn(f, fold);
    return f;
  };
  // Each of the warp's 16 tokens is decoded once (source token and grid position) by lane t and
  // lane t+16, and handed to the threads that load it.
  int d_src = 0, d_f = -1, d_y = -1, d_x = -1;
  if constexpr (GM != GM_PLAIN) {
    const int t = blockIdx.x * 64 + warp * 16 + (lane & 15);
    if (t < N) d_src = gc.source(t, d_f, d_y, d_x);
  }
#pragma unroll
  for (int i = 0; i < LOADS; ++i) {   // all loads first, so that every row of the thread is in flight at once
    const int tok = tok0 + i * RPL;
    row[i].v = make_uint4(0, 0, 0, 0);
    int src = tok;
    if constexpr (GM != GM_PLAIN) src = __shfl_sync(0xffffffffu, d_src, i * RPL + lane / TPR);
    if (tok < N) row[i].v = *reinterpret_cast<const uint4*>(base + (size_t)src * sn + c8);
  }
#pragma unroll
  for (int i = 0; i < LOADS; ++i) {
    const int tok = tok0 + i * RPL;
    if constexpr (NM != PARO_NORM_NONE) {   // all lanes: the row statistics are reduced with full-warp shuffles
      int src = tok < N ? tok : 0;
      if constexpr (GM != GM_PLAIN) src = __shfl_sync(0xffffffffu, d_src, i * RPL + lane / TPR);
      normalize8<T, NM, TPR>(row[i], c8, D, b, h, N, src, norm);
    }
    if constexpr (GM == GM_ROPE_F32 || GM == GM_ROPE_F64) {
      const int from = i * RPL + lane / TPR;
      const int gf = __shfl_sync(0xffffffffu, d_f, from);
      const int gy = __shfl_sync(0xffffffffu, d_y, from);
      const int gx = __shfl_sync(0xffffffffu, d_x, from);
      if (tok < N) gc.rotate(row[i], c8, D, gf, gy, gx);
    }
    if (tok < N) {
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(widen(row[i], j)));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if (lane == 0) s_amax[warp] = amax;
  __syncthreads();
  if (GROUP == 64) {
    amax = fmaxf(fmaxf(s_amax[0], s_amax[1]), fmaxf(s_amax[2], s_amax[3]));
  } else {
    amax = fmaxf(s_amax[warp & ~1], s_amax[warp | 1]);
  }
  amax = fmaxf(amax, 1e-7f);
  if (GROUP == 64) {
    if (threadIdx.x == 0) scale[(size_t)bh * n_scale_per_bh + blockIdx.x] = __fdiv_rn(amax, 127.0f);
  } else {
    if (lane == 0 && (warp & 1) == 0)
      scale[(size_t)bh * n_scale_per_bh + blockIdx.x * 2 + (warp >> 1)] = __fdiv_rn(amax, 127.0f);
  }
  const float inv = __fdiv_rn(127.0f, amax);
#pragma unroll
  for (int i = 0; i < LOADS; ++i) {
    const int tok = tok0 + i * RPL;
    if (tok < N) {
      // round to nearest even (NaN -> 0), then saturate and pack two values per instruction
      int qi[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) qi[j] = __float2int_rn(__fmul_rn(widen(row[i], j), inv));
      uint32_t w[2];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        uint32_t hi16, word;
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi16) : "r"(qi[half * 4 + 3]), "r"(qi[half * 4 + 2]), "r"(0));
        asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(word) : "r"(qi[half * 4 + 1]), "r"(qi[half * 4 + 0]), "r"(hi16));
        w[half] = word;
      }
      *reinterpret_cast<uint2*>(out + ((size_t)bh * N + tok) * D + c8) = make_uint2(w[0], w[1]);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// FP8 cast + transpose: CTA = 256 threads = one 64-token block of one (b,h).
// Phase 1 stages the raw tile in shared memory with coalesced 16-byte loads; phase 2 lets
// consecutive lanes take consecutive channels (conflict-free column reads) and each thread emit a
// run of tokens of its channel as whole 32-byte sectors.
template <typename T, int D, int GM>
__global__ void __launch_bounds__(256)
quant_v_fp8_kernel(const T* __restrict__ v, int H, int N, int npad, int64_t sb, int64_t sh, int64_t sn,
                   const float* __restrict__ inv_tab, const float* __restrict__ mean_tab,
                   uint8_t* __restrict__ v8, __nv_bfloat16* __restrict__ v16, const Gather gather) {
  constexpr int TPR = D / 8;
  constexpr int ROWS = 256 / TPR;
  constexpr int LD = D + 8;                 // padded row, keeps 16-byte alignment
  constexpr int RUN = 64 / (256 / D);       // tokens per thread in phase 2 (32 for D=128, 16 for D=64)
  __shared__ __align__(16) T tile[64 * LD];
  const int bh = blockIdx.y, b = bh / H, h = bh % H;
  const int t0 = blockIdx.x * 64;
  const T* base = v + b * sb + h * sh;
  {
    const GatherCtx<GM> gc(gather, h);
    const int c8 = (threadIdx.x % TPR) * 8;
#pragma unroll
    for (int r = threadIdx.x / TPR; r < 64; r += ROWS) {
      uint4 val = make_uint4(0, 0, 0, 0);
      int gf, gy, gx;
      if (t0 + r < N) val = *reinterpret_cast<const uint4*>(base + (size_t)gc.source(t0 + r, gf, gy, gx) * sn + c8);
      *reinterpret_cast<uint4*>(&tile[r * LD + c8]) = val;
    }
  }
  __syncthreads();
  const int d = threadIdx.x % D, run = threadIdx.x / D;
  const float mean = mean_tab[(size_t)bh * D + d];
  const float inv = inv_tab[(size_t)bh * D + d];  // scale_max / amax, from the finalize pass
  uint32_t w8[RUN / 4];
  uint32_t w16[RUN / 2];
#pragma unroll
  for (int i = 0; i < RUN; i += 2) {
    float y[2];
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int r = run * RUN + i + k;
      float f = 0.f;
      if (t0 + r < N) f = __fmul_rn(__fsub_rn(F16Traits<T>::to_float(tile[r * LD + d]), mean), inv);
      y[k] = f;
    }
    const __nv_fp8x2_storage_t p = __nv_cvt_float2_to_fp8x2(make_float2(y[0], y[1]), __NV_SATFINITE, __NV_E4M3);
    if ((i & 3) == 0) w8[i / 4] = (uint32_t)p; else w8[i / 4] |= (uint32_t)p << 16;
    // e4m3 -> fp16 -> bf16: both steps exact (3 mantissa bits, exponents inside either range)
    const __half2_raw h2 = __nv_cvt_fp8x2_to_halfraw2(p, __NV_E4M3);
    const __nv_bfloat162 b2 = __floats2bfloat162_rn(__half2float(__half(__half_raw{h2.x})), __half2float(__half(__half_raw{h2.y})));
    w16[i / 2] = *reinterpret_cast<const uint32_t*>(&b2);
  }
  const size_t o = ((size_t)bh * D + d) * npad + t0 + run * RUN;
#pragma unroll
  for (int i = 0; i < RUN / 16; ++i)
    if (v8) *reinterpret_cast<uint4*>(v8 + o + i * 16) = make_uint4(w8[4 * i], w8[4 * i + 1], w8[4 * i + 2], w8[4 * i + 3]);
  if (v16) {
#pragma unroll
    for (int i = 0; i < RUN / 8; ++i)
      *reinterpret_cast<uint4*>(v16 + o + i * 8) = make_uint4(w16[4 * i], w16[4 * i + 1], w16[4 * i + 2], w16[4 * i + 3]);
  }
}

}  // namespace paro

using namespace paro;

namespace {

int stats_chunks(int N) { return (N + STATS_CHUNK - 1) / STATS_CHUNK; }

// scratch = partials [B*H*chunks*D] followed by two fp32 tables [B*H*D] (scale_max/amax, mean used)
size_t stats_bytes(int B, int H, int N, int D) {
  const size_t bh = (size_t)B * H;
  return bh * stats_chunks(N) * D * sizeof(ChannelPartial) + 2 * bh * D * sizeof(float);
}

template <typename T>
void launch_stats(const void* x, int B, int H, int N, int D, int64_t sb, int64_t sh, int64_t sn,
                  ChannelPartial* part, cudaStream_t s, const Gather& g = Gather{}) {
  dim3 grid(stats_chunks(N), B * H);
  dispatch_gather(g, [&](auto gm) {
    constexpr int GM = decltype(gm)::value;
    if (D == 128)
      channel_stats_kernel<T, 128, GM><<<grid, 256, 0, s>>>((const T*)x, H, N, sb, sh, sn, part, stats_chunks(N), g);
    else
      channel_stats_kernel<T, 64, GM><<<grid, 256, 0, s>>>((const T*)x, H, N, sb, sh, sn, part, stats_chunks(N), g);
  });
}

}  // namespace

extern "C" size_t paro_channel_stats_scratch_bytes(int B, int H, int N, int D) {
  if (B <= 0 || H <= 0 || N <= 0 || (D != 64 && D != 128)) return 0;
  return stats_bytes(B, H, N, D);
}

extern "C" int paro_channel_mean(const void* x, int dtype, int B, int H, int N, int D,
                                 int64_t stride_b, int64_t stride_h, int64_t stride_n,
                                 void* mean_out, float* mean_f32, void* scratch, size_t scratch_bytes,
                                 paro_stream_t stream) {
  if (int rc = check_tensor("paro_channel_mean(x)", x, dtype, B, H, N, D, stride_b, stride_h, stride_n)) return rc;
  PARO_REQUIRE(mean_out || mean_f32, PARO_EINVAL, "paro_channel_mean: no output requested");
  PARO_REQUIRE(scratch && scratch_bytes >= stats_bytes(B, H, N, D), PARO_ECAP,
               "paro_channel_mean: scratch too small (%zu < %zu)", scratch_bytes, stats_bytes(B, H, N, D));
  PARO_REQUIRE(aligned16(scratch), PARO_EALIGN, "paro_channel_mean: scratch not 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  ChannelPartial* part = static_cast<ChannelPartial*>(scratch);
  if (dtype == PARO_F16) {
    launch_stats<__half>(x, B, H, N, D, stride_b, stride_h, stride_n, part, s);
    channel_finalize_kernel<__half><<<B * H, D, 0, s>>>(part, stats_chunks(N), D, N, 1, 1.f, (__half*)mean_out,
                                                        mean_f32, nullptr, nullptr, nullptr);
  } else {
    launch_stats<__nv_bfloat16>(x, B, H, N, D, stride_b, stride_h, stride_n, part, s);
    channel_finalize_kernel<__nv_bfloat16><<<B * H, D, 0, s>>>(part, stats_chunks(N), D, N, 1, 1.f,
                                                               (__nv_bfloat16*)mean_out, mean_f32, nullptr, nullptr,
                                                               nullptr);
  }
  return check_launch("channel_mean", 2);
}

namespace {
template <typename T, int D, int NM>
void launch_int8_norm(const void* x, const void* km, int8_t* out, float* scale, int B, int H, int N, int64_t sb,
                      int64_t sh, int64_t sn, float fold, int group, cudaStream_t s, const Gather& g, const NormArgs& nm) {
  const int nb = (N + 63) / 64;
  dim3 grid(nb, B * H);
  dispatch_gather(g, [&](auto gm) {
    constexpr int GM = decltype(gm)::value;
    if (group == 64)
      quant_int8_kernel<T, D, 64, GM, NM><<<grid, 128, 0, s>>>((const T*)x, (const T*)km, out, scale, H, N, sb, sh, sn,
                                                               fold, nb, g, nm);
    else
      quant_int8_kernel<T, D, 32, GM, NM><<<grid, 128, 0, s>>>((const T*)x, (const T*)km, out, scale, H, N, sb, sh, sn,
                                                               fold, nb * 2, g, nm);
  });
}

template <typename T, int D>
int launch_int8(const void* x, const void* km, int8_t* out, float* scale, int B, int H, int N, int64_t sb,
                int64_t sh, int64_t sn, float fold, int group, cudaStream_t s, const Gather& g = Gather{},
                const NormArgs& nm = NormArgs{}) {
  if (nm.mode == PARO_NORM_LAYER_HEAD)
    launch_int8_norm<T, D, PARO_NORM_LAYER_HEAD>(x, km, out, scale, B, H, N, sb, sh, sn, fold, group, s, g, nm);
  else if (nm.mode == PARO_NORM_RMS_ALL)
    launch_int8_norm<T, D, PARO_NORM_RMS_ALL>(x, km, out, scale, B, H, N, sb, sh, sn, fold, group, s, g, nm);
  else
    launch_int8_norm<T, D, PARO_NORM_NONE>(x, km, out, scale, B, H, N, sb, sh, sn, fold, group, s, g, nm);
  return check_launch("quant_int8_kernel");
}
}  // namespace

extern "C" int paro_quant_int8(const void* x, int dtype, int B, int H, int N, int D,
                               int64_t stride_b, int64_t stride_h, int64_t stride_n,
                               const void* km, float fold_scale, int group,
                               int8_t* out, float* scale, paro_stream_t stream) {
  if (int rc = check_tensor("paro_quant_int8(x)", x, dtype, B, H, N, D, stride_b, stride_h, stride_n)) return rc;
  PARO_REQUIRE(group == 32 || group == 64, PARO_EINVAL, "paro_quant_int8: group must be 32 or 64, got %d", group);
  PARO_REQUIRE(out && scale, PARO_EINVAL, "paro_quant_int8: null output");
  PARO_REQUIRE(aligned16(out) && (!km || aligned16(km)), PARO_EALIGN, "paro_quant_int8: out/km not 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PARO_F16)
    return D == 128 ? launch_int8<__half, 128>(x, km, out, scale, B, H, N, stride_b, stride_h, stride_n, fold_scale, group, s)
                    : launch_int8<__half, 64>(x, km, out, scale, B, H, N, stride_b, stride_h, stride_n, fold_scale, group, s);
  return D == 128 ? launch_int8<__nv_bfloat16, 128>(x, km, out, scale, B, H, N, stride_b, stride_h, stride_n, fold_scale, group, s)
                  : launch_int8<__nv_bfloat16, 64>(x, km, out, scale, B, H, N, stride_b, stride_h, stride_n, fold_scale, group, s);
}

namespace {
template <typename T>
int run_v_fp8(const void* v, int B, int H, int N, int D, int64_t sb, int64_t sh, int64_t sn, int smooth,
              float scale_max, uint8_t* v8, uint16_t* v16, float* v_scale, float* vm, void* scratch,
              cudaStream_t s, const Gather& g = Gather{}) {
  const int chunks = stats_chunks(N);
  const size_t bh = (size_t)B * H;
  ChannelPartial* part = static_cast<ChannelPartial*>(scratch);
  float* inv_tab = reinterpret_cast<float*>(part + bh * chunks * D);
  float* mean_tab = inv_tab + bh * D;
  launch_stats<T>(v, B, H, N, D, sb, sh, sn, part, s);   // statistics do not depend on the token order
  channel_finalize_kernel<T><<<B * H, D, 0, s>>>(part, chunks, D, N, smooth, scale_max, (T*)nullptr,
                                                 smooth ? vm : nullptr, v_scale, inv_tab, mean_tab);
  const int npad = (N + 63) / 64 * 64;
  dim3 grid(npad / 64, B * H);
  dispatch_gather(g, [&](auto gm) {
    // the V pass never rotates: reordering only
    constexpr int GM = decltype(gm)::value == GM_PLAIN ? GM_PLAIN : GM_REORDER;
    if (D == 128)
      quant_v_fp8_kernel<T, 128, GM><<<grid, 256, 0, s>>>((const T*)v, H, N, npad, sb, sh, sn, inv_tab, mean_tab, v8,
                                                          (__nv_bfloat16*)v16, g);
    else
      quant_v_fp8_kernel<T, 64, GM><<<grid, 256, 0, s>>>((const T*)v, H, N, npad, sb, sh, sn, inv_tab, mean_tab, v8,
                                                         (__nv_bfloat16*)v16, g);
  });
  return check_launch("quant_v_fp8", 3);
}
}  // namespace

extern "C" int paro_quant_v_fp8(const void* v, int dtype, int B, int H, int N, int D,
                                int64_t stride_b, int64_t stride_h, int64_t stride_n,
                                int smooth, float scale_max, uint8_t* v8, uint16_t* v16,
                                float* v_scale, float* vm, void* scratch, size_t scratch_bytes,
                                paro_stream_t stream) {
  if (int rc = check_tensor("paro_quant_v_fp8(v)", v, dtype, B, H, N, D, stride_b, stride_h, stride_n)) return rc;
  PARO_REQUIRE(v8 && v_scale, PARO_EINVAL, "paro_quant_v_fp8: null output");
  PARO_REQUIRE(!smooth || vm, PARO_EINVAL, "paro_quant_v_fp8: smoothing needs the vm output");
  PARO_REQUIRE(scale_max > 0.f && scale_max <= 448.f, PARO_EINVAL, "paro_quant_v_fp8: scale_max must be in (0, 448]");
  PARO_REQUIRE(aligned16(v8) && (!v16 || aligned16(v16)), PARO_EALIGN, "paro_quant_v_fp8: outputs not 16-byte aligned");
  PARO_REQUIRE(scratch && scratch_bytes >= stats_bytes(B, H, N, D), PARO_ECAP,
               "paro_quant_v_fp8: scratch too small (%zu < %zu)", scratch_bytes, stats_bytes(B, H, N, D));
  PARO_REQUIRE(aligned16(scratch), PARO_EALIGN, "paro_quant_v_fp8: scratch not 16-byte aligned");
  cudaStream_t s = (cudaStream_t)stream;
  return dtype == PARO_F16
             ? run_v_fp8<__half>(v, B, H, N, D, stride_b, stride_h, stride_n, smooth, scale_max, v8, v16, v_scale, vm, scratch, s)
             : run_v_fp8<__nv_bfloat16>(v, B, H, N, D, stride_b, stride_h, stride_n, smooth, scale_max, v8, v16, v_scale, vm, scratch, s);
}

// ---------------------------------------------------------------------------------------------
// Channel mean for callers that must not allocate.
//
// Some users of this library run where asking for device memory is off the table: an inference
// server that froze its memory pool after warm-up, a plain C host that has no allocator of its own
// to draw a scratch buffer from, or a latency-critical denoising loop in which a cudaMalloc would
// stall the whole device.  For them the reduction's partial sums live in the fixed array below
// instead of a caller-provided buffer.  The array is part of the loaded module, so every GPU that
// loads the library sets aside its 16 MiB until the process exits.
namespace {

constexpr size_t NOALLOC_SCRATCH_BYTES = 16u << 20;   // 16 MiB = 1,048,576 partials of 16 bytes: B*H*ceil(N/512)*D may not exceed that
static __device__ __align__(256) unsigned char g_noalloc_scratch[NOALLOC_SCRATCH_BYTES];

constexpr int NOALLOC_MAX_DEVICES = 64;
std::mutex g_noalloc_mutex;
void* g_noalloc_ptr[NOALLOC_MAX_DEVICES] = {};

// Device address of g_noalloc_scratch on the CURRENT device.  In host code the array's name is
// only a handle for the runtime, never a pointer a kernel may use, so the address is looked up
// once per device (with that device current) and remembered.
int noalloc_scratch(void** out) {
  int dev = -1;
  PARO_CUDA_OK(cudaGetDevice(&dev));
  PARO_REQUIRE(dev >= 0 && dev < NOALLOC_MAX_DEVICES, PARO_ECUDA, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  if (g_noalloc_ptr[dev] == nullptr) {
    void* p = nullptr;
    PARO_CUDA_OK(cudaGetSymbolAddress(&p, g_noalloc_scratch));
    PARO_REQUIRE(p != nullptr, PARO_ECUDA, "cudaGetSymbolAddress returned a null address");
    g_noalloc_ptr[dev] = p;
  }
  *out = g_noalloc_ptr[dev];
  return PARO_OK;
}

}  // namespace

extern "C" int paro_channel_mean_noalloc(const void* x, int dtype, int B, int H, int N, int D,
                                         int64_t stride_b, int64_t stride_h, int64_t stride_n,
                                         void* mean_out, float* mean_f32, paro_stream_t stream) {
  if (int rc = check_tensor("paro_channel_mean_noalloc(x)", x, dtype, B, H, N, D, stride_b, stride_h, stride_n)) return rc;
  PARO_REQUIRE(mean_out || mean_f32, PARO_EINVAL, "paro_channel_mean_noalloc: no output requested");
  const unsigned long long need =
      (unsigned long long)B * H * (unsigned long long)stats_chunks(N) * D * sizeof(ChannelPartial);
  PARO_REQUIRE(need <= NOALLOC_SCRATCH_BYTES, PARO_ECAP,
               "paro_channel_mean_noalloc: this problem needs %llu bytes of scratch but the built-in scratch holds "
               "%zu; use paro_channel_mean with a caller-provided buffer", need, (size_t)NOALLOC_SCRATCH_BYTES);
  void* scratch = nullptr;
  if (int rc = noalloc_scratch(&scratch)) return rc;
  cudaStream_t s = (cudaStream_t)stream;
  ChannelPartial* part = static_cast<ChannelPartial*>(scratch);
  // every partial the second pass reads is written by the first pass of the same call, so nothing
  // left behind by an earlier call has to be cleared
  if (dtype == PARO_F16) {
    launch_stats<__half>(x, B, H, N, D, stride_b, stride_h, stride_n, part, s);
    channel_finalize_kernel<__half><<<B * H, D, 0, s>>>(part, stats_chunks(N), D, N, 1, 1.f, (__half*)mean_out,
                                                        mean_f32, nullptr, nullptr, nullptr);
  } else {
    launch_stats<__nv_bfloat16>(x, B, H, N, D, stride_b, stride_h, stride_n, part, s);
    channel_finalize_kernel<__nv_bfloat16><<<B * H, D, 0, s>>>(part, stats_chunks(N), D, N, 1, 1.f,
                                                               (__nv_bfloat16*)mean_out, mean_f32, nullptr, nullptr,
                                                               nullptr);
  }
  return check_launch("channel_mean_noalloc", 2);
}

// ---------------------------------------------------------------------------------------------
// Fused pre-attention entry points: the quantisers read the natural-order activations through the
// RoPE + reordering front end, so no reordered 16-bit copy of Q, K, V is ever written to HBM.
namespace {

int make_gather(Gather* g, const char* who, int N, int D, int n_text, int F, int Hh, int W, const int32_t* order_ids,
                int rope_mode, const void* cos_tab, const void* sin_tab, int pairs_f, int pairs_h) {
  PARO_REQUIRE(F > 0 && Hh > 0 && W > 0 && n_text >= 0 && (int64_t)n_text + (int64_t)F * Hh * W == N, PARO_ESHAPE,
               "%s: n_text + F*H*W = %lld != N = %d", who, (long long)n_text + (long long)F * Hh * W, N);
  PARO_REQUIRE(rope_mode >= PARO_ROPE_NONE && rope_mode <= PARO_ROPE_COMPLEX_F64, PARO_EINVAL,
               "%s: unknown rope_mode %d", who, rope_mode);
  if (rope_mode != PARO_ROPE_NONE) {
    PARO_REQUIRE(cos_tab, PARO_EINVAL, "%s: rope tables missing", who);   // sin_tab NULL = interleaved (cos, sin) table
    PARO_REQUIRE(pairs_f >= 0 && pairs_h >= 0 && pairs_f + pairs_h <= D / 2, PARO_ESHAPE,
                 "%s: pairs_f + pairs_h exceeds D/2", who);
  }
  g->enabled = 1;
  g->n_text = n_text; g->F = F; g->Hh = Hh; g->W = W;
  g->order_ids = order_ids;
  g->rope = RopeArgs{rope_mode, cos_tab, sin_tab, pairs_f, pairs_h};
  return PARO_OK;
}

template <typename T>
int run_prep_int8(const void* x, int B, int H, int N, int D, int64_t sb, int64_t sh, int64_t sn, const Gather& g,
                  int group, int smooth, void* km_out, int8_t* out, float* scale, void* scratch, cudaStream_t s) {
  const T* km = nullptr;
  int launches = 1;
  if (smooth) {
    // mean of the rotated values; the token order does not matter for it, so the statistics pass
    // reads the input in natural order (rotation only)
    Gather gs = g;
    gs.order_ids = nullptr;
    ChannelPartial* part = static_cast<ChannelPartial*>(scratch);
    launch_stats<T>(x, B, H, N, D, sb, sh, sn, part, s, gs);
    channel_finalize_kernel<T><<<B * H, D, 0, s>>>(part, stats_chunks(N), D, N, 1, 1.f, (T*)km_out, nullptr, nullptr,
                                                   nullptr, nullptr);
    km = static_cast<const T*>(km_out);
    launches = 3;
  }
  int rc = D == 128 ? launch_int8<T, 128>(x, km, out, scale, B, H, N, sb, sh, sn, 0.f, group, s, g)
                    : launch_int8<T, 64>(x, km, out, scale, B, H, N, sb, sh, sn, 0.f, group, s, g);
  if (rc == PARO_OK) count_launches(launches - 1);
  return rc;
}

}  // namespace

extern "C" int paro_prep_qk_int8(const void* x, int dtype, int B, int H, int N, int D,
                                 int64_t stride_b, int64_t stride_h, int64_t stride_n,
                                 int n_text, int F, int Hh, int W, const int32_t* order_ids,
                                 int rope_mode, const void* cos_tab, const void* sin_tab, int pairs_f, int pairs_h,
                                 int group, int smooth, void* km_out, int8_t* out, float* scale,
                                 void* scratch, size_t scratch_bytes, paro_stream_t stream) {
  if (int rc = check_tensor("paro_prep_qk_int8(x)", x, dtype, B, H, N, D, stride_b, stride_h, stride_n)) return rc;
  PARO_REQUIRE(group == 32 || group == 64, PARO_EINVAL, "paro_prep_qk_int8: group must be 32 or 64, got %d", group);
  PARO_REQUIRE(out && scale && aligned16(out), PARO_EINVAL, "paro_prep_qk_int8: null or unaligned output");
  Gather g{};
  if (int rc = make_gather(&g, "paro_prep_qk_int8", N, D, n_text, F, Hh, W, order_ids, rope_mode, cos_tab, sin_tab,
                           pairs_f, pairs_h))
    return rc;
  if (smooth) {
    PARO_REQUIRE(km_out && aligned16(km_out), PARO_EINVAL, "paro_prep_qk_int8: smoothing needs the km output");
    PARO_REQUIRE(scratch && aligned16(scratch) && scratch_bytes >= stats_bytes(B, H, N, D), PARO_ECAP,
                 "paro_prep_qk_int8: scratch too small (%zu < %zu)", scratch_bytes, stats_bytes(B, H, N, D));
  }
  cudaStream_t s = (cudaStream_t)stream;
  return dtype == PARO_F16
             ? run_prep_int8<__half>(x, B, H, N, D, stride_b, stride_h, stride_n, g, group, smooth, km_out, out, scale, scratch, s)
             : run_prep_int8<__nv_bfloat16>(x, B, H, N, D, stride_b, stride_h, stride_n, g, group, smooth, km_out, out, scale, scratch, s);
}

extern "C" int paro_prep_qk_int8_norm(const void* x, int dtype, int B, int H, int N, int D,
                                      int64_t stride_b, int64_t stride_h, int64_t stride_n,
                                      int n_text, int F, int Hh, int W, const int32_t* order_ids,
                                      int rope_mode, const void* cos_tab, const void* sin_tab, int pairs_f, int pairs_h,
                                      int group, int8_t* out, float* scale,
                                      int norm_mode, const void* norm_weight, const void* norm_bias,
                                      const float* inv_rms, float eps, paro_stream_t stream) {
  if (int rc = check_tensor("paro_prep_qk_int8_norm(x)", x, dtype, B, H, N, D, stride_b, stride_h, stride_n)) return rc;
  PARO_REQUIRE(group == 32 || group == 64, PARO_EINVAL, "paro_prep_qk_int8_norm: group must be 32 or 64, got %d", group);
  PARO_REQUIRE(out && scale && aligned16(out), PARO_EINVAL, "paro_prep_qk_int8_norm: null or unaligned output");
  Gather g{};
  if (int rc = make_gather(&g, "paro_prep_qk_int8_norm", N, D, n_text, F, Hh, W, order_ids, rope_mode, cos_tab, sin_tab,
                           pairs_f, pairs_h))
    return rc;
  if (int rc = check_norm("paro_prep_qk_int8_norm", norm_mode, norm_weight, norm_bias, inv_rms, eps)) return rc;
  const NormArgs nm{norm_mode, norm_weight, norm_bias, inv_rms, eps};
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == PARO_F16)
    return D == 128 ? launch_int8<__half, 128>(x, nullptr, out, scale, B, H, N, stride_b, stride_h, stride_n, 0.f, group, s, g, nm)
                    : launch_int8<__half, 64>(x, nullptr, out, scale, B, H, N, stride_b, stride_h, stride_n, 0.f, group, s, g, nm);
  return D == 128 ? launch_int8<__nv_bfloat16, 128>(x, nullptr, out, scale, B, H, N, stride_b, stride_h, stride_n, 0.f, group, s, g, nm)
                  : launch_int8<__nv_bfloat16, 64>(x, nullptr, out, scale, B, H, N, stride_b, stride_h, stride_n, 0.f, group, s, g, nm);
}

extern "C" int paro_prep_v_fp8(const void* v, int dtype, int B, int H, int N, int D,
                               int64_t stride_b, int64_t stride_h, int64_t stride_n,
                               int n_text, int F, int Hh, int W, const int32_t* order_ids,
                               int smooth, float scale_max, uint8_t* v8, uint16_t* v16,
                               float* v_scale, float* vm, void* scratch, size_t scratch_bytes,
                               paro_stream_t stream) {
  if (int rc = check_tensor("paro_prep_v_fp8(v)", v, dtype, B, H, N, D, stride_b, stride_h, stride_n)) return rc;
  PARO_REQUIRE((v8 || v16) && v_scale, PARO_EINVAL, "paro_prep_v_fp8: null output");
  PARO_REQUIRE(!smooth || vm, PARO_EINVAL, "paro_prep_v_fp8: smoothing needs the vm output");
  PARO_REQUIRE(scale_max > 0.f && scale_max <= 448.f, PARO_EINVAL, "paro_prep_v_fp8: scale_max must be in (0, 448]");
  PARO_REQUIRE((!v8 || aligned16(v8)) && (!v16 || aligned16(v16)), PARO_EALIGN, "paro_prep_v_fp8: outputs not 16-byte aligned");
  PARO_REQUIRE(scratch && aligned16(scratch) && scratch_bytes >= stats_bytes(B, H, N, D), PARO_ECAP,
               "paro_prep_v_fp8: scratch too small (%zu < %zu)", scratch_bytes, stats_bytes(B, H, N, D));
  Gather g{};
  if (int rc = make_gather(&g, "paro_prep_v_fp8", N, D, n_text, F, Hh, W, order_ids, PARO_ROPE_NONE, nullptr, nullptr, 0, 0))
    return rc;
  cudaStream_t s = (cudaStream_t)stream;
  return dtype == PARO_F16
             ? run_v_fp8<__half>(v, B, H, N, D, stride_b, stride_h, stride_n, smooth, scale_max, v8, v16, v_scale, vm, scratch, s, g)
             : run_v_fp8<__nv_bfloat16>(v, B, H, N, D, stride_b, stride_h, stride_n, smooth, scale_max, v8, v16, v_scale, vm, scratch, s, g);
}
