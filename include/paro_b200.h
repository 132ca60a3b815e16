/*
 * paro_b200.h -- C ABI of libparo_b200.so: PAROAttention's quantized, reordered,
 * block-sparse attention path for NVIDIA B200 (sm_100a).
 *
 * Conventions (they replace the torch-extension conventions of the reference,
 * csrc/qattn/pybind_sm80.cpp:23-26, csrc/fused/pybind.cpp:23-32, csrc/rope/pybind.cpp:7):
 *   - every pointer is a DEVICE pointer on the current device unless said otherwise;
 *   - the caller owns every buffer, scratch included (sizes from the *_scratch_bytes calls);
 *   - every call is asynchronous on `stream` (a cudaStream_t) and returns 0 or a negative
 *     PARO_E* code; paro_last_error() gives the message of the calling thread's last failure;
 *   - tensors are [B,H,N,D] addressed through element strides (stride_d == 1), so both the
 *     reference's "HND" and "NHD" layouts are accepted (core.py:176, fused.cu:452-470);
 *   - D is 64 or 128 (core.py:181-192), dtype is PARO_F16 or PARO_BF16 (core.py:163).
 * There is no CPU fallback: a call made without a usable CUDA device fails with PARO_ECUDA.
 */
#ifndef PARO_B200_H
#define PARO_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* paro_stream_t; /* cudaStream_t */

enum {
  PARO_OK = 0,
  PARO_EINVAL = -1,   /* bad flag, null pointer, unsupported dtype */
  PARO_ESHAPE = -2,   /* unsupported or inconsistent sizes */
  PARO_EALIGN = -3,   /* pointer or stride not aligned as required */
  PARO_ETIMEOUT = -4, /* a bounded device-side wait expired (reported through the status word) */
  PARO_ECUDA = -5,    /* CUDA runtime / driver error */
  PARO_ECAP = -6      /* caller-provided capacity too small */
};

enum { PARO_F16 = 0, PARO_BF16 = 1 };
enum { PARO_ROPE_NONE = 0, PARO_ROPE_REAL_F32 = 1, PARO_ROPE_COMPLEX_F64 = 2 };
enum { PARO_NORM_NONE = 0, PARO_NORM_LAYER_HEAD = 1, PARO_NORM_RMS_ALL = 2 };
enum { PARO_ATTN_FAST = 0, PARO_ATTN_EXACT = 1 };

int paro_version(void);
const char* paro_last_error(void);
/* Number of kernels this library has launched in this process so far. */
long long paro_launch_count(void);

/* ---- token permutation --------------------------------------------------------------- */

/* idx[h][j] = index (within the F*Hh*W video tokens) of the token that lands at position j
 * after head h's axis reordering; order ids 0..5 = FHW,FWH,HWF,HFW,WHF,WFH.
 * Replaces the per-head reshape/permute of paroattention/cogvideox.py:38-56 (wan.py:40-56). */
int paro_build_perm_index(const int32_t* order_ids, int H, int F, int Hh, int W,
                          int32_t* idx, paro_stream_t stream);

/* Fused 3D-RoPE + per-head token permutation of ONE tensor, out-of-place.
 *   forward (inverse=0): out[b,h,n_text+j,:] = rope(in[b,h,n_text+idx_h[j],:]); text rows copied;
 *   inverse (inverse=1): out[b,h,n_text+idx_h[j],:] = in[b,h,n_text+j,:] (rope_mode must be NONE).
 * order_ids == NULL means no permutation (RoPE only).  `out` is contiguous [B,H,N,D].
 * cos_tab/sin_tab: [F+Hh+W, D/2] per-axis tables (row = axis base + coordinate), fp32 for
 * PARO_ROPE_REAL_F32 (pairs (2i,2i+1): o0=x0*c-x1*s, o1=x1*c+x0*s, as diffusers'
 * apply_rotary_emb at cogvideox.py:167-172), fp64 for PARO_ROPE_COMPLEX_F64 (wan.py:161-164).
 * pairs_f/pairs_h: how many leading channel pairs follow the f / h coordinate (rest: w).
 * sin_tab == NULL (all entry points that take the two tables): cos_tab is then ONE table
 * [F+Hh+W, D/2, 2] with cos and sin of a pair side by side, fetched by a single load.
 * Replaces csrc/rope/rope.cu:14-48 (rope_permutation) and permute_qk / permute_attn_out
 * (cogvideox.py:22-110). */
int paro_rope_permute(const void* in, void* out, int dtype, int B, int H, int N, int D,
                      int64_t stride_b, int64_t stride_h, int64_t stride_n,
                      int n_text, int F, int Hh, int W, const int32_t* order_ids, int inverse,
                      int rope_mode, const void* cos_tab, const void* sin_tab,
                      int pairs_f, int pairs_h, paro_stream_t stream);

/* ---- quantisers ------------------------------------------------------------------------ */

/* Mean over tokens, [B,H,N,D] -> mean_out [B,H,D] in the input dtype (the `km` the reference
 * expects from its caller, quant.py:46-48) and/or mean_f32 [B,H,D]; either may be NULL.
 * Deterministic: fp64 partial sums in a fixed order.  scratch: paro_channel_stats_scratch_bytes. */
size_t paro_channel_stats_scratch_bytes(int B, int H, int N, int D);
int paro_channel_mean(const void* x, int dtype, int B, int H, int N, int D,
                      int64_t stride_b, int64_t stride_h, int64_t stride_n,
                      void* mean_out, float* mean_f32, void* scratch, size_t scratch_bytes,
                      paro_stream_t stream);

/* paro_channel_mean for callers that cannot allocate device memory -- for example a server whose
 * memory pool is frozen after warm-up, a C host with no allocator to take scratch from, or a
 * latency-critical loop where a cudaMalloc would stall the device.  No counterpart in the
 * reference.  Same inputs, outputs and results as paro_channel_mean; the partial sums live in a
 * 16 MiB array built into the library (held on every GPU that loads it, until the process exits)
 * instead of caller scratch.  Limits and rules:
 *   - B*H*ceil(N/512)*D*16 bytes must fit in 16 MiB, otherwise PARO_ECAP (nothing is launched);
 *   - the call allocates nothing (no cudaMalloc/cudaFree, no allocating library routine);
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress),
 *     so make that first call before starting any stream capture -- and during warm-up: with
 *     CUDA's lazy module loading it is also the moment the driver places the 16 MiB array in that
 *     GPU's memory, so on a GPU with no room left this first call can fail with PARO_ECUDA;
 *   - all calls on a device share the one array: calls that may overlap on the GPU (different
 *     streams without ordering) race and must be serialised by the caller.  The array keeps the
 *     previous call's contents; every value a call reads is written by that call first. */
int paro_channel_mean_noalloc(const void* x, int dtype, int B, int H, int N, int D,
                              int64_t stride_b, int64_t stride_h, int64_t stride_n,
                              void* mean_out, float* mean_f32, paro_stream_t stream);

/* Per-group symmetric INT8: group = 32 (the reference's per-warp Q, quant.py:105-180 ->
 * fused.cu:685-768) or 64 (per-block Q/K, fused.cu:429-682).  km (nullable, [B,H,D], input
 * dtype) is subtracted first (fused.cu:594-682); fold_scale != 0 multiplies x before
 * quantising (quant.py:91-96).  out: contiguous int8 [B,H,N,D]; scale: fp32
 * [B,H,ceil(N/64)*(64/group)].  amax=max(1e-7,max|x|), scale=amax/127,
 * q=sat(rint(x*(127/amax))) in IEEE fp32 (fused.cu:95-197, without its fast-math divide). */
int paro_quant_int8(const void* x, int dtype, int B, int H, int N, int D,
                    int64_t stride_b, int64_t stride_h, int64_t stride_n,
                    const void* km, float fold_scale, int group,
                    int8_t* out, float* scale, paro_stream_t stream);

/* Per-channel FP8-e4m3 of V written token-contiguous: v8 [B,H,D,ceil64(N)] zero padded,
 * v_scale [B,H,D] = amax/scale_max, vm [B,H,D] (mean, when smooth != 0).  v16 (nullable)
 * receives the same e4m3 values widened (exactly) to bf16, the operand format of paro_sparse_attn.
 * Replaces per_channel_fp8 (quant.py:224-293 -> fused.cu:262-427); the 16-token shuffle of
 * fused.cu:287-291 is an mma.sync artefact and is not applied. */
int paro_quant_v_fp8(const void* v, int dtype, int B, int H, int N, int D,
                     int64_t stride_b, int64_t stride_h, int64_t stride_n,
                     int smooth, float scale_max, uint8_t* v8, uint16_t* v16,
                     float* v_scale, float* vm, void* scratch, size_t scratch_bytes,
                     paro_stream_t stream);

/* Fused pre-attention passes: the same quantisers reading the NATURAL-order activations through
 * the RoPE + per-head reordering front end of paro_rope_permute, so that the reordered 16-bit copy
 * is never written (the processors' sequence apply_rotary_emb -> permute_qk -> per_warp_int8,
 * cogvideox.py:167-186, in one or two passes per tensor).  Arguments as in paro_rope_permute and
 * paro_quant_int8 / paro_quant_v_fp8.  paro_prep_qk_int8: smooth != 0 first reduces the mean of
 * the rotated values into km_out ([B,H,D], input dtype; needs scratch of
 * paro_channel_stats_scratch_bytes) and subtracts it.  paro_prep_v_fp8: V is reordered only (never
 * rotated); v8 or v16 may be NULL. */
int paro_prep_qk_int8(const void* x, int dtype, int B, int H, int N, int D,
                      int64_t stride_b, int64_t stride_h, int64_t stride_n,
                      int n_text, int F, int Hh, int W, const int32_t* order_ids,
                      int rope_mode, const void* cos_tab, const void* sin_tab, int pairs_f, int pairs_h,
                      int group, int smooth, void* km_out, int8_t* out, float* scale,
                      void* scratch, size_t scratch_bytes, paro_stream_t stream);
int paro_prep_v_fp8(const void* v, int dtype, int B, int H, int N, int D,
                    int64_t stride_b, int64_t stride_h, int64_t stride_n,
                    int n_text, int F, int Hh, int W, const int32_t* order_ids,
                    int smooth, float scale_max, uint8_t* v8, uint16_t* v16,
                    float* v_scale, float* vm, void* scratch, size_t scratch_bytes,
                    paro_stream_t stream);

/* ---- Q/K normalisation folded into the passes above ----------------------------------------
 * The processors call attn.norm_q / attn.norm_k between the projection and RoPE
 * (cogvideox.py:161-164, wan.py:150-153; modules of the un-vendored diffusers package).  The
 * *_norm entry points apply that normalisation to each row as it is read, before the rotation:
 *   PARO_NORM_LAYER_HEAD  y = (x - mean) / sqrt(var + eps) * weight + bias over the D channels of one
 *                         (token, head); weight, bias (nullable): [D] in the input dtype
 *   PARO_NORM_RMS_ALL     y = dtype(dtype(x * inv_rms[b, token]) * weight[h*D + c]) with the statistic
 *                         over all H*D channels of the token ("rms_norm_across_heads", wan.py:531);
 *                         weight [H*D] in the input dtype, inv_rms [B,N] fp32 from paro_row_inv_rms
 * Sums in fp64, all other operations separately rounded fp32, result rounded to the input dtype.
 * All tokens are normalised (text tokens too).  The remaining arguments are those of
 * paro_rope_permute / paro_prep_qk_int8; paro_prep_qk_int8_norm does not support smooth != 0. */
int paro_row_inv_rms(const void* x, int dtype, int B, int H, int N, int D,
                     int64_t stride_b, int64_t stride_h, int64_t stride_n,
                     float eps, float* inv_rms, paro_stream_t stream);
int paro_rope_permute_norm(const void* in, void* out, int dtype, int B, int H, int N, int D,
                           int64_t stride_b, int64_t stride_h, int64_t stride_n,
                           int n_text, int F, int Hh, int W, const int32_t* order_ids,
                           int rope_mode, const void* cos_tab, const void* sin_tab,
                           int pairs_f, int pairs_h,
                           int norm_mode, const void* norm_weight, const void* norm_bias,
                           const float* inv_rms, float eps, paro_stream_t stream);
int paro_prep_qk_int8_norm(const void* x, int dtype, int B, int H, int N, int D,
                           int64_t stride_b, int64_t stride_h, int64_t stride_n,
                           int n_text, int F, int Hh, int W, const int32_t* order_ids,
                           int rope_mode, const void* cos_tab, const void* sin_tab, int pairs_f, int pairs_h,
                           int group, int8_t* out, float* scale,
                           int norm_mode, const void* norm_weight, const void* norm_bias,
                           const float* inv_rms, float eps, paro_stream_t stream);

/* ---- sparse plan ----------------------------------------------------------------------- */

/* mask: bytes [slices, nbq, nbk], non-zero = keep (the `sparse` argument of
 * csrc/qattn/qk_int_sv_f16_cuda_sm80.cu:53,222,268).  Step 1 writes the exclusive prefix
 * sums row_ptr [slices*nbq+1] (kept blocks per q-block) and pair_ptr [slices*ceil(nbq/2)+1]
 * (union of kept blocks per pair of adjacent q-blocks).  The caller reads the last element of
 * each to size cols / pair_ent, then step 2 fills them: cols ascending kb per row; pair_ent
 * ascending kb*4 + (keep(2p) | keep(2p+1)<<1). */
int paro_plan_count(const uint8_t* mask, int slices, int nbq, int nbk,
                    int32_t* row_ptr, int32_t* pair_ptr, paro_stream_t stream);
int paro_plan_fill(const uint8_t* mask, int slices, int nbq, int nbk,
                   const int32_t* row_ptr, int32_t* cols, int64_t cols_cap,
                   const int32_t* pair_ptr, int32_t* pair_ent, int64_t pair_cap,
                   paro_stream_t stream);

/* Walk order of the attention kernel, one schedule per pair of adjacent q-blocks (2p, 2p+1), built
 * from the merged lists of paro_plan_fill: first the k-blocks both q-blocks keep (ascending; one
 * K/V tile and one full-height MMA serve both), then the r-th block only 2p keeps beside the r-th
 * block only 2p+1 keeps.  sched [size of pair_ent], entries of pair r from offset pair_ptr[r]:
 * kbA | kbB << 16, 0xFFFF = no tile for that q-block in this step (needs nbk < 65535);
 * sched_cnt [2 * slices*ceil(nbq/2)]: steps of q-block 2p, steps of q-block 2p+1 (each contiguous
 * from step 0), in the low 16 bits of each word.  A caller that pairs q-blocks differently (the walk
 * costs the UNION of a pair's two lists, so q-blocks that share many k-blocks make cheap pairs) builds
 * the lists from the mask with its rows in pair order and, before handing sched_cnt to paro_sparse_attn,
 * ORs (q-block id + 1) << 16 into each word: the half then stands for that q-block (rows, scales, output
 * rows); high half 0 = the adjacent pairing.  No counterpart in the reference (it tests one mask byte per block in the loop,
 * qk_int_sv_f16_cuda_sm80.cu:268). */
int paro_plan_schedule(const int32_t* pair_ptr, const int32_t* pair_ent, int slices, int nbq, int nbk,
                       uint32_t* sched, int32_t* sched_cnt, paro_stream_t stream);

/* Checks walk lists that did not come from paro_plan_schedule in this process (read from a file, built
 * by other code) before paro_sparse_attn follows them: pair_ptr starts at 0, is monotone and stays within
 * sched_len entries; each q-block's step count fits its pair's slots (and is 0 for a q-block past the end);
 * every k-block id inside a q-block's steps is < nbk and every entry past them is the 0xFFFF filler;
 * shared steps come first and the k-blocks of each section ascend strictly (so none repeats); a q-block id
 * carried in the high half of a step count is < nbq.
 * report: 4 device words of scratch.  Synchronises `stream`; returns PARO_OK or PARO_EINVAL with the first
 * fault in paro_last_error().  The reference shape-checks its mask argument in the same spirit
 * (csrc/qattn/qk_int_sv_f16_cuda_sm80.cu:1034-1038). */
int paro_plan_validate(const int32_t* pair_ptr, const uint32_t* sched, const int32_t* sched_cnt,
                       int slices, int nbq, int nbk, int64_t sched_len, int32_t* report,
                       paro_stream_t stream);

/* ---- attention ------------------------------------------------------------------------- */

/* Block-sparse attention over the kept 64x64 blocks with the inverse permutation fused
 * into the output store.  Replaces qk_int8_sv_f16_accum_f16_attn
 * (csrc/qattn/attn_cuda_sm80.h:19-30, qk_int_sv_f16_cuda_sm80.cu:905-1080) followed by
 * permute_attn_out (cogvideox.py:64-110).
 *   q8,k8: contiguous int8 [B,H,N,D]; q_scale [B,H,ceil(N/64)*(64/q_group)], k_scale
 *   [B,H,ceil(N/64)]; v16: bf16 [B,H,D,ceil64(N)] (e4m3 values), v_scale/vm [B,H,D] (vm may
 *   be NULL); pair_ptr from paro_plan_count, sched/sched_cnt from paro_plan_schedule (the walk
 *   order per pair of q-blocks; paro_plan_validate checks lists that were not built here),
 *   plan_slices = H (shared by the batch) or B*H;
 *   inv_idx (nullable): table of paro_build_perm_index -- output row n_text+j of head h is
 *   stored at token n_text+inv_idx[h][j]; out: [B,H,N,D] through element strides; lse
 *   (nullable) fp32 [B,H,N] in output token order, natural log; status: int32[4] device
 *   words, zero before the first call; a non-zero word 0 makes later launches return at once.
 * S = (q8.k8^T) * q_scale * k_scale * sm_scale * log2(e); P = 2^(S - m) over kept blocks and
 * columns < N, rounded to bf16; O = (P.v16) / sum(P) * v_scale + vm with fp32 accumulation.
 * mode PARO_ATTN_EXACT: m is the running row maximum (online softmax, one launch).
 * mode PARO_ATTN_FAST (what the Python layer uses): m is fixed per row from its first kept
 * block, which lets every step run independently of the one before; two launches: the fast
 * walk, then the exact walk over the work items the fast one gave back because a row's
 * scores rose more than 2^120 above its first block (usually none).  It needs the work
 * space `redo` of paro_sparse_attn_redo_bytes(B,H,N) bytes (device memory, contents
 * irrelevant on entry; afterwards word 0 holds the number of work items given back);
 * calls that share a work space must be on one stream. */
size_t paro_sparse_attn_redo_bytes(int B, int H, int N);
int paro_sparse_attn(const int8_t* q8, const int8_t* k8, const uint16_t* v16,
                     const float* q_scale, int q_group, const float* k_scale,
                     const float* v_scale, const float* vm,
                     const int32_t* pair_ptr, const uint32_t* sched, const int32_t* sched_cnt,
                     int plan_slices,
                     const int32_t* inv_idx, int n_text,
                     void* out, int out_dtype,
                     int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_n,
                     float* lse, int B, int H, int N, int D, float sm_scale, int mode,
                     int32_t* redo, size_t redo_bytes,
                     int32_t* status, paro_stream_t stream);

/* Merges two partial results of paro_sparse_attn computed over DISJOINT sets of key blocks (for
 * instance the two halves of a sequence held by two ranks) into the result over their union:
 * lse = log(exp(lse_a) + exp(lse_b)), out = o_a * exp(lse_a - lse) + o_b * exp(lse_b - lse), fp32 math,
 * out in the tensors' dtype.  A row whose LSE is -inf on one side (no kept block there) takes the other
 * side unchanged.  o_a, o_b, out: [B,H,N,D] through the same element strides (out may alias o_a or o_b);
 * lse_*: fp32 [B,H,N] contiguous, natural log; lse_out may be NULL.  This is the consumer of the LSE
 * output that the reference returns "for cases like Ring Attention" (paroattention/core.py:55-57,
 * kernel qk_int_sv_f16_cuda_sm80.cu:711-723) and leaves to the caller. */
int paro_merge_attn_states(const void* o_a, const float* lse_a, const void* o_b, const float* lse_b,
                           void* out, float* lse_out, int dtype, int B, int H, int N, int D,
                           int64_t stride_b, int64_t stride_h, int64_t stride_n, paro_stream_t stream);

/* Synchronises `stream`, copies the 4 status words to host_out (host pointer, may be NULL)
 * and returns PARO_OK, PARO_ETIMEOUT (word 0 non-zero) or PARO_ECUDA.  After a timeout word 1 names
 * the waiter that gave up (1 K loader, 9 V loader, 2/3 score issuer, 5 P.V issuer, 6 softmax
 * waiting for scores, 7/8 softmax waiting for P.V, 10 softmax waiting for the running maximum),
 * word 2 the work item (block index) and word 3 its step. */
int paro_status_poll(const int32_t* status, int32_t* host_out, paro_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* PARO_B200_H */
