// Block-sparse attention over kept 64x64 blocks for sm_100a: the fast walk.
//
// Work item (one CTA): a PAIR of adjacent 64-row q-blocks of one (batch, head), walking the pair's
// schedule (shared k-blocks first, then the halves' own blocks side by side; see paro_plan_schedule).
//
// What makes this walk fast is that no step depends on the step before it:
//   * Fixed reference exponent.  P = 2^(s - m_ref) where m_ref is fixed per row when the row's FIRST
//     kept block has been seen (its maximum + REF_OFFSET), instead of a running maximum.  P is kept
//     in bf16 (8 exponent bits) and accumulated in fp32, so any score up to 2^120 above the first
//     block's maximum is representable and nothing ever has to be rescaled: no maximum is handed
//     from step to step, the two warp sets of a half never wait for each other, and the accumulator
//     is only touched by the tensor core.  A row sum that leaves the safe range (a score more than
//     ~2^120 above the row's first block, or a non-finite value) makes the CTA give its work item
//     back through the redo list; the exact-maximum kernel (sparse_attn.cu) then computes that pair.
//   * P travels through shared memory (one 8 KB buffer per half and warp set), which leaves tensor
//     memory for TWO score buffers (one per warp set): Q.K^T of step i+2 is issued as soon as the
//     scores of step i are in registers.
//   * P.V is computed transposed, O^T[D x 64] += V^T[D x 64 tokens] . P^T, so every accumulator lane
//     (a channel of the head dimension) does useful work for either half; the epilogue transposes
//     back through shared memory and stores rows at their un-permuted token.
//
//   warps 0-7   softmax + epilogue.  Row r of the 128-row tile belongs to two threads, one per WARP
//               SET: warp w (< 4, set 0) takes the even steps of its half, warp w+4 the odd steps.
//   warp 8      TMA producer: the query tile (once), then the K ring (int8 tiles)
//   warp 9      TMA producer for the V^T ring (bf16 tiles, D rows x 64 tokens)
//   warp 10     owns TMEM; one lane issues S = Q.K^T (kind::i8, both operands in shared memory,
//               lane-masked so that a tile only writes the rows of the half it belongs to)
//   warp 11     one lane issues O^T += V^T.P^T (kind::f16 on bf16, fp32 accumulators)
//
// TMEM (256 columns per CTA, two CTAs per SM): S of even steps [0,64), S of odd steps [64,128),
// O^T [128,256) (columns = the 128 query rows of the pair; lanes = channels, for D = 64 the M=64
// layout: channel 16j+i on lane 32j+i).  Every wait is bounded; on expiry the CTA records a code
// in the status words, raises a shared abort flag, waits (bounded) for its own copies and MMAs in
// flight, frees TMEM and returns.
#include "attn_common.cuh"

namespace paro {

using namespace umma;

constexpr float REF_OFFSET = 20.f;            // the first block's maximum maps to P = 2^-20
constexpr float ROWSUM_LIMIT = 1.2676506e30f; // 2^100: a step's row sum beyond it gives the pair back
namespace { }

template <int D> struct FastCfg {
  static constexpr int K_STAGES = (D == 128) ? 3 : 6;
  static constexpr int V_STAGES = (D == 128) ? 2 : 4;
  static constexpr int Q_BYTES = 128 * D;
  static constexpr int K_BYTES = 64 * D;
  static constexpr int V_BYTES = D * 128;    // D rows of 64 bf16
  static constexpr int P_BYTES = 64 * 128;   // 64 rows of 64 bf16
  static constexpr int TILE_BYTES = Q_BYTES + K_STAGES * K_BYTES + V_STAGES * V_BYTES + 4 * P_BYTES;
  static constexpr int AUX_BYTES = 4096;     // barriers, TMEM pointer, flags, v_scale, vm, row exchange
  static constexpr int SMEM_BYTES = TILE_BYTES + AUX_BYTES + 1024 /* alignment slack */;
  static_assert(4 * P_BYTES >= 128 * D * 2, "the P buffers double as the output staging area");
};

template <int D, typename OutT>
__global__ void __launch_bounds__(ATT_THREADS, 2)
sparse_attn_fast_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                        const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  using Cfg = FastCfg<D>;
  constexpr int KST = Cfg::K_STAGES, VST = Cfg::V_STAGES;
  constexpr bool SHARE_TILES = (D == 128);

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sQ = smem;
  uint8_t* sK = sQ + Cfg::Q_BYTES;
  uint8_t* sV = sK + KST * Cfg::K_BYTES;
  uint8_t* sP = sV + VST * Cfg::V_BYTES;   // [set][half][64 rows][128 B], 128-byte swizzle
  uint8_t* aux = smem + Cfg::TILE_BYTES;
  // mbarriers.  [h][set]: one per half of the pair and per warp set (= parity of the step index), so
  // that each barrier is arrived on and waited for by the same parties in every phase.
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(aux);   // [1]     Q tile landed
  uint64_t* bar_kfull = bar_q + 1;                      // [KST]   K tile landed
  uint64_t* bar_kfree = bar_kfull + KST;                // [KST]   the Q.K^T that read the K stage finished
  uint64_t* bar_vfull = bar_kfree + KST;                // [VST]   V tile landed
  uint64_t* bar_vfree = bar_vfull + VST;                // [VST]   the P.V that read the V stage finished
  uint64_t* bar_sready = bar_vfree + VST;               // [2][2]  scores of (half, set) in TMEM
  uint64_t* bar_sfree = bar_sready + 4;                 // [2][2]  ... copied to registers
  uint64_t* bar_pready = bar_sfree + 4;                 // [2][2]  P of (half, set) in shared memory
  uint64_t* bar_pfree = bar_pready + 4;                 // [2][2]  the P.V that read it finished
  uint64_t* bar_done = bar_pfree + 4;                   // [2]     every P.V of the half finished (one phase)
  uint64_t* bar_drain = bar_done + 2;                   // [2]     issuers' MMAs retired (abort path only)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_drain + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* s_drain = abort_flag + 1;                  // 1: an earlier launch or CTA failed, leave at once
  volatile int* s_redo = s_drain + 1;                      // 1: a row sum left the safe range
  volatile int* s_mflag = s_redo + 1;                      // [4]  reference exponents of the quadrant published
  float* s_vscale = reinterpret_cast<float*>(aux + 512);   // [D]
  float* s_vm = s_vscale + D;                              // [D]
  volatile float* s_mref = reinterpret_cast<volatile float*>(aux + 1536);   // [128] reference exponent of each row
  float* s_xl = reinterpret_cast<float*>(aux + 2048);                       // [2][128] row-sum exchange
  float* s_inv = reinterpret_cast<float*>(aux + 3072);                      // [128] 1 / row sum
  static_assert(512 + 2 * D * 4 <= 1536 && 3072 + 128 * 4 <= Cfg::AUX_BYTES, "aux area too small");
  static_assert((21 + 2 * KST + 2 * VST) * 8 + 4 + 28 <= 512, "barrier area too small");

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // one thread decides for the whole CTA whether an earlier failure makes this launch drain
  if (threadIdx.x == 0) *s_drain = *reinterpret_cast<volatile int32_t*>(p.status) != 0;
  __syncthreads();
  if (*s_drain) return;

  const int bh = blockIdx.x / p.npairs, pair = blockIdx.x % p.npairs;
  const int slice = bh % p.plan_slices;
  const int prow = slice * p.npairs + pair;
  const uint32_t* sched = p.sched + p.pair_ptr[prow];
  const int n_a = p.sched_cnt[2 * prow], n_b = p.sched_cnt[2 * prow + 1];
  const int n_steps = max(n_a, n_b);

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 1);
    for (int i = 0; i < KST; ++i) {
      mbar_init(bar_kfull + i, 1);
      mbar_init(bar_kfree + i, 1);
    }
    for (int i = 0; i < VST; ++i) {
      mbar_init(bar_vfull + i, 1);
      mbar_init(bar_vfree + i, 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(bar_sready + i, 1);
      mbar_init(bar_sfree + i, 2);    // the two warps (lane quadrants) of a half in one warp set
      mbar_init(bar_pready + i, 2);
      mbar_init(bar_pfree + i, 1);
      s_mflag[i] = 0;
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(bar_done + i, 1);
      mbar_init(bar_drain + i, 1);
    }
    *abort_flag = 0;
    *s_redo = 0;
    fence_barrier_init();
  }
  if (warp == 10) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tO = tmem_base + 128u;

  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 32;");
    if (warp == 8 && lane == 0) {
      // ---------------------------------------------------------------- TMA producer: Q tile, K ring
      tma_prefetch_desc(&tm_q);
      tma_prefetch_desc(&tm_k);
      if (n_steps > 0) {
        mbar_arrive_expect_tx(bar_q, Cfg::Q_BYTES);
        tma_load_3d(sQ, &tm_q, 0, pair * 128, bh, bar_q);   // rows past the end of the sequence arrive as zeros
      }
      bool ok = true;
      int t = 0;   // tiles so far = position in the ring
      uint32_t e_cur = n_steps > 0 ? sched[0] : 0u, e_nxt = n_steps > 1 ? sched[1] : 0u;
      for (int i = 0; i < n_steps && ok; ++i) {
        const StepGroups g(e_cur, SHARE_TILES);
        e_cur = e_nxt;
        if (i + 2 < n_steps) e_nxt = ld_pinned_u32(sched + i + 2);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          if (!g.act[j]) continue;
          const int st = t % KST, use = t / KST;
          if (use > 0 && !mbar_wait_bounded(bar_kfree + st, (use - 1) & 1, abort_flag, WAIT_LIMIT)) {
            report_timeout(p, abort_flag, 1, i);
            ok = false;
            break;
          }
          ++t;
          mbar_arrive_expect_tx(bar_kfull + st, Cfg::K_BYTES);
          tma_load_3d(sK + st * Cfg::K_BYTES, &tm_k, 0, g.kblk[j] * 64, bh, bar_kfull + st);
        }
      }
      if (*abort_flag) {   // leaving early: the copies this thread started must have landed first
        if (n_steps > 0) mbar_wait_plain_bounded(bar_q, 0, WAIT_LIMIT);
        for (int u = max(0, t - KST); u < t; ++u) mbar_wait_plain_bounded(bar_kfull + u % KST, (u / KST) & 1, WAIT_LIMIT);
      }
    } else if (warp == 9 && lane == 0) {
      // ---------------------------------------------------------------- TMA producer: V ring
      tma_prefetch_desc(&tm_v);
      bool ok = true;
      int t = 0;
      uint32_t e_cur = n_steps > 0 ? sched[0] : 0u, e_nxt = n_steps > 1 ? sched[1] : 0u;
      for (int i = 0; i < n_steps && ok; ++i) {
        const StepGroups g(e_cur, SHARE_TILES);
        e_cur = e_nxt;
        if (i + 2 < n_steps) e_nxt = ld_pinned_u32(sched + i + 2);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          if (!g.act[j]) continue;
          const int st = t % VST, use = t / VST;
          if (use > 0 && !mbar_wait_bounded(bar_vfree + st, (use - 1) & 1, abort_flag, WAIT_LIMIT)) {
            report_timeout(p, abort_flag, 9, i);
            ok = false;
            break;
          }
          ++t;
          mbar_arrive_expect_tx(bar_vfull + st, Cfg::V_BYTES);
          tma_load_3d(sV + st * Cfg::V_BYTES, &tm_v, g.kblk[j] * 64, 0, bh, bar_vfull + st);
        }
      }
      if (*abort_flag)
        for (int u = max(0, t - VST); u < t; ++u) mbar_wait_plain_bounded(bar_vfull + u % VST, (u / VST) & 1, WAIT_LIMIT);
    } else if (warp == 10 && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer: S = Q.K^T
      constexpr uint32_t IDESC_QK = instr_desc(2, 1, 1, 128, 64);  // s32 += s8 * s8
      bool ok = n_steps == 0 || mbar_wait_bounded(bar_q, 0, abort_flag, WAIT_LIMIT);
      if (!ok) report_timeout(p, abort_flag, 2, -1);
      const uint64_t dQ = smem_desc(smem_u32(sQ), D);
      int t = 0;
      uint32_t e_cur = n_steps > 0 ? sched[0] : 0u, e_nxt = n_steps > 1 ? sched[1] : 0u;
      for (int i = 0; i < n_steps && ok; ++i) {
        const StepGroups g(e_cur, SHARE_TILES);
        e_cur = e_nxt;
        if (i + 2 < n_steps) e_nxt = ld_pinned_u32(sched + i + 2);
        const int set = i & 1;
#pragma unroll
        for (int j = 0; j < 2; ++j) {   // one MMA group per tile; lane-masked unless it serves both halves
          if (!g.act[j]) continue;
          const int w = g.which[j], st = t % KST, use = t / KST;
          ++t;
          // the scores of step i-2 (same warp set) of the halves served are in registers
          bool good = true;
          if (i >= 2) {
            const int ph = ((i - 2) >> 1) & 1;
            if (w != 1) good = good && mbar_wait_bounded(bar_sfree + set, ph, abort_flag, WAIT_LIMIT);
            if (w != 0) good = good && mbar_wait_bounded(bar_sfree + 2 + set, ph, abort_flag, WAIT_LIMIT);
          }
          good = good && mbar_wait_bounded(bar_kfull + st, use & 1, abort_flag, WAIT_LIMIT);
          if (!good) {
            report_timeout(p, abort_flag, 3, i);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t dK = smem_desc(smem_u32(sK + st * Cfg::K_BYTES), D);
          // lanes NOT written: the rows of a half the tile does not serve
          const uint32_t lo = w == 1 ? 0xffffffffu : 0u, hi = w == 0 ? 0xffffffffu : 0u;
#pragma unroll
          for (int k = 0; k < D / 32; ++k)
            mma_i8_ss_masked(tmem_base + 64u * set, desc_advance(dQ, 32 * k), desc_advance(dK, 32 * k), IDESC_QK, k > 0, lo,
                             lo, hi, hi);
          mma_commit(bar_kfree + st);
          if (w != 1) mma_commit(bar_sready + set);
          if (w != 0) mma_commit(bar_sready + 2 + set);
        }
      }
      if (*abort_flag) {
        mma_commit(bar_drain);
        mbar_wait_plain_bounded(bar_drain, 0, WAIT_LIMIT);
      }
    } else if (warp == 11 && lane == 0) {
      // ---------------------------------------------------------------- MMA issuer: O^T += V^T.P^T
      constexpr uint32_t IDESC_PV1 = instr_desc(1, 1, 1, D, 64);    // f32 += bf16 * bf16, one half's 64 columns
      constexpr uint32_t IDESC_PV2 = instr_desc(1, 1, 1, D, 128);   // a shared tile: both halves' columns
      bool ok = true;
      int t = 0;
      uint32_t e_cur = n_steps > 0 ? sched[0] : 0u, e_nxt = n_steps > 1 ? sched[1] : 0u;
      for (int i = 0; i < n_steps && ok; ++i) {
        const StepGroups g(e_cur, SHARE_TILES);
        e_cur = e_nxt;
        if (i + 2 < n_steps) e_nxt = ld_pinned_u32(sched + i + 2);
        const int set = i & 1, ph = (i >> 1) & 1;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          if (!g.act[j]) continue;
          const int w = g.which[j], st = t % VST, use = t / VST;
          ++t;
          bool good = true;
          if (w != 1) good = good && mbar_wait_bounded(bar_pready + set, ph, abort_flag, WAIT_LIMIT);
          if (w != 0) good = good && mbar_wait_bounded(bar_pready + 2 + set, ph, abort_flag, WAIT_LIMIT);
          good = good && mbar_wait_bounded(bar_vfull + st, use & 1, abort_flag, WAIT_LIMIT);
          if (!good) {
            report_timeout(p, abort_flag, 5, i);
            ok = false;
            break;
          }
          tc_fence_after();
          const uint64_t dV = smem_desc(smem_u32(sV + st * Cfg::V_BYTES), 128);
          const int h0 = w == 1 ? 1 : 0;   // first half served
          const uint64_t dP = smem_desc(smem_u32(sP + (set * 2 + h0) * Cfg::P_BYTES), 128);
          // both halves start at step 0, so a tile that serves both never mixes a first with a later step
#pragma unroll
          for (int k = 0; k < 4; ++k)
            mma_f16_ss(tO + 64u * h0, desc_advance(dV, 32 * k), desc_advance(dP, 32 * k), w == 2 ? IDESC_PV2 : IDESC_PV1,
                       (i > 0 || k > 0) ? 1u : 0u);
          mma_commit(bar_vfree + st);
          if (w != 1) {
            mma_commit(bar_pfree + set);
            if (i == n_a - 1) mma_commit(bar_done);
          }
          if (w != 0) {
            mma_commit(bar_pfree + 2 + set);
            if (i == n_b - 1) mma_commit(bar_done + 1);
          }
        }
      }
      if (*abort_flag) {
        mma_commit(bar_drain + 1);
        mbar_wait_plain_bounded(bar_drain + 1, 0, WAIT_LIMIT);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    const int qd = warp & 3;                 // TMEM lane quadrant this warp may touch
    const int set = warp >> 2;               // warp set: steps of this parity; in the epilogue, the half whose columns it reads
    const int r = qd * 32 + lane;            // row inside the 128-row tile
    const int half = qd >> 1;                // which q-block of the pair
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    const int n_mine = half ? n_b : n_a;
    auto my_kb = [&](int i) { return (int)((sched[i] >> (16 * half)) & 0xFFFFu); };   // this half's k-block of step i
    if (threadIdx.x < D) {
      s_vscale[threadIdx.x] = p.v_scale[(size_t)bh * D + threadIdx.x];
      s_vm[threadIdx.x] = p.vm ? p.vm[(size_t)bh * D + threadIdx.x] : 0.f;
    }

    const int tok = pair * 128 + r;
    const int per_bh = p.nb * (64 / p.q_group);
    // rows past the end of the sequence get a tiny positive scale (not 0: the -inf of masked columns
    // times 0 would be NaN and read as a row sum out of range); they are never stored
    const float rowscale = tok < p.N ? p.q_scale[(size_t)bh * per_bh + tok / p.q_group] * p.scale_log2 : 1e-30f;
    float m_ref = 0.f, l = 0.f;   // l: this thread's share of the row sum (the steps of its parity)
    bool ok = true, redo = false;
    auto wait_bar = [&](uint64_t* bar, int phase, int code, int i) {
      const bool good = __all_sync(0xffffffffu, mbar_wait_bounded(bar, phase & 1, abort_flag, WAIT_LIMIT));
      if (!good) report_timeout(p, abort_flag, code, i);
      tc_fence_after();
      return good;
    };
    uint64_t* const my_sready = bar_sready + 2 * half + set;
    uint64_t* const my_sfree = bar_sfree + 2 * half + set;
    uint64_t* const my_pready = bar_pready + 2 * half + set;
    uint64_t* const my_pfree = bar_pfree + 2 * half + set;
    const uint32_t tS = tmem_base + 64u * set + lane_off;
    // this thread's row of its P buffer; 16-byte chunk c of the row sits at chunk position c ^ (row % 8)
    const uint32_t p_row = smem_u32(sP + (set * 2 + half) * Cfg::P_BYTES) + (uint32_t)(r & 63) * 128u;
    const uint32_t p_xor = (uint32_t)(r & 7);
    const float* kscale_bh = p.k_scale + (size_t)bh * p.nb;
    int kb_next = set < n_mine ? min(my_kb(set), p.nb - 1) : 0;
    float ks_next = set < n_mine ? kscale_bh[kb_next] : 0.f;
    for (int i = set; i < n_mine; i += 2) {
      const int kb = kb_next;
      const float kscale = ks_next;
      if (i + 2 < n_mine) {   // fetched one step ahead so that the loads are off the critical path
        kb_next = min(my_kb(i + 2), p.nb - 1);
        ks_next = kscale_bh[kb_next];
      }
      ok = wait_bar(my_sready, i >> 1, 6, i);
      if (!ok) break;
      float f[64];
      {
        uint32_t s[64];
        tmem_ld32(tS, s);
        tmem_ld32(tS + 32u, s + 32);
        tmem_wait_ld();
        // the scores are in registers: let the issuer overwrite this buffer with step i+2
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(my_sfree);
        // int32 scores -> fp32 by an integer addition: the bit pattern 0x4B400000 + s is the float
        // SCORE_BIAS + s exactly (|s| <= 127 * 127 * D < 2^22); the bias is folded into the constant of
        // the multiply-add that forms the exponent.
#pragma unroll
        for (int j = 0; j < 64; ++j) f[j] = __int_as_float((int)s[j] + 0x4B400000);
      }
      const int valid = min(64, p.N - kb * 64);   // columns inside the sequence
      if (valid < 64) {
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (j >= valid) f[j] = -INFINITY;
      }
      const float sc = rowscale * kscale;
      if (i == 0) {
        // the row's reference exponent: the maximum of its first kept block, lifted by REF_OFFSET
        float mx4[4] = {f[0], f[1], f[2], f[3]};
#pragma unroll
        for (int j = 4; j < 64; j += 8) {
          mx4[0] = max3(mx4[0], f[j], f[j + 1]);
          mx4[1] = max3(mx4[1], f[j + 2], f[j + 3]);
          if (j + 4 < 64) {
            mx4[2] = max3(mx4[2], f[j + 4], f[j + 5]);
            mx4[3] = max3(mx4[3], f[j + 6], f[j + 7]);
          }
        }
        m_ref = (fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) - SCORE_BIAS) * sc + REF_OFFSET;
        s_mref[r] = m_ref;
        __syncwarp();
        if (lane == 0) st_release_shared(s_mflag + qd, 1);
      } else if (i == 1) {
        bool seen = ld_acquire_shared(s_mflag + qd) != 0;
        if (!seen) {
          const long long t0 = clock64();
          while (!(seen = ld_acquire_shared(s_mflag + qd) != 0)) {
            if (*abort_flag || clock64() - t0 > WAIT_LIMIT) break;
          }
        }
        if (!__all_sync(0xffffffffu, seen)) {
          report_timeout(p, abort_flag, 10, i);
          ok = false;
          break;
        }
        m_ref = s_mref[r];
      }
      const float xoff = fmaf(-SCORE_BIAS, sc, -m_ref);   // (bias + s) * sc + xoff = s * sc - m_ref
      const uint64_t sc2 = pack2(sc, sc), xoff2 = pack2(xoff, xoff);
      uint64_t sum2[2] = {0ull, 0ull};
      uint32_t pk[32];
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float x0, x1;
        unpack2(fma2(pack2(f[2 * j], f[2 * j + 1]), sc2, xoff2), x0, x1);
        const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);   // 2^-inf = 0 for masked columns
        sum2[j & 1] = add2(sum2[j & 1], pack2(p0, p1));
        pk[j] = pack_bf16x2(p0, p1);
      }
      float sa, sb;
      unpack2(add2(sum2[0], sum2[1]), sa, sb);
      const float step_sum = sa + sb;
      redo = redo || !(step_sum < ROWSUM_LIMIT);   // also catches NaN
      l += step_sum;
      // this buffer is rewritten only after the P.V that read its previous contents (step i-2) has finished
      if (i >= 2) {
        ok = wait_bar(my_pfree, (i - 2) >> 1, 7, i);
        if (!ok) break;
      }
#pragma unroll
      for (int c = 0; c < 8; ++c)
        asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(p_row + ((((uint32_t)c) ^ p_xor) << 4)),
                     "r"(pk[4 * c]), "r"(pk[4 * c + 1]), "r"(pk[4 * c + 2]), "r"(pk[4 * c + 3])
                     : "memory");
      fence_proxy_async();   // generic-proxy stores -> visible to the tensor core's reads
      __syncwarp();
      if (lane == 0) mbar_arrive(my_pready);   // one arrival per warp
    }
    if (redo) *s_redo = 1;

    // ---- epilogue.  Row sums: both threads' shares, same reference exponent.
    named_barrier(1, ATT_SOFTMAX_THREADS);
    s_xl[set * 128 + r] = l;
    named_barrier(1, ATT_SOFTMAX_THREADS);
    if (set == 0) {
      l += s_xl[128 + r];
      s_inv[r] = l > 0.f ? 1.f / l : 0.f;
    }
    const bool give_back = *s_redo != 0;
    // every P.V of both halves has retired: O^T is complete and the P buffers are free for staging
    if (ok && n_a > 0) ok = wait_bar(bar_done, 0, 8, n_a);
    if (ok && n_b > 0) ok = wait_bar(bar_done + 1, 0, 8, n_b);
    named_barrier(1, ATT_SOFTMAX_THREADS);
    ok = ok && !*abort_flag;
    const int b = bh / p.H, h = bh % p.H;
    if (ok && !give_back) {
      // This thread: channel d of O^T (TMEM lane), the 64 query rows of half `set` (columns).
      const int n_e = set ? n_b : n_a;
      const bool lane_live = D == 128 || lane < 16;
      const int d = D == 128 ? r : 16 * qd + (lane & 15);
      const float vs = s_vscale[d], vmean = s_vm[d];
      OutT* stage = reinterpret_cast<OutT*>(sP);   // [128 rows][D]
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t o[32];
        if (n_e > 0) {
          tmem_ld32(tO + lane_off + (uint32_t)(64 * set + 32 * c), o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = 0u;
        }
        if (lane_live) {
#pragma unroll
          for (int j = 0; j < 32; ++j) {
            const int row = 64 * set + 32 * c + j;
            const float inv_l = s_inv[row];
            const float val = inv_l > 0.f ? fmaf(__uint_as_float(o[j]) * inv_l, vs, vmean) : 0.f;
            stage[row * D + d] = F16Traits<OutT>::from_float(val);
          }
        }
      }
    }
    named_barrier(1, ATT_SOFTMAX_THREADS);
    if (ok && !give_back) {
      // rows of the staging tile -> their un-permuted tokens, 16 bytes per lane
      constexpr int LPR = D / 8;            // lanes per row
      constexpr int RPI = 32 / LPR;         // rows per warp instruction
      const uint8_t* stage = sP;
#pragma unroll 1
      for (int it = 0; it < 16 / RPI; ++it) {
        const int row = warp * 16 + it * RPI + lane / LPR;
        const int tk = pair * 128 + row;
        if (tk < p.N) {
          int dst = tk;
          if (p.inv_idx && tk >= p.n_text) dst = p.n_text + p.inv_idx[(size_t)h * (p.N - p.n_text) + (tk - p.n_text)];
          OutT* orow = static_cast<OutT*>(p.out) + b * p.osb + h * p.osh + (int64_t)dst * p.osn;
          *reinterpret_cast<uint4*>(orow + 8 * (lane % LPR)) =
              *reinterpret_cast<const uint4*>(stage + (size_t)row * D * 2 + 16 * (lane % LPR));
        }
      }
      if (set == 0 && tok < p.N && p.lse) {
        int dst = tok;
        if (p.inv_idx && tok >= p.n_text) dst = p.n_text + p.inv_idx[(size_t)h * (p.N - p.n_text) + (tok - p.n_text)];
        // m_ref of set 0 is the row's reference when the half has steps at all
        p.lse[(size_t)bh * p.N + dst] = l > 0.f ? (log2f(l) + m_ref) * 0.6931471805599453f : -INFINITY;
      }
    }
    if (ok && give_back && threadIdx.x == 0) {
      const int slot = atomicAdd(p.redo, 1);
      p.redo[REDO_HEADER + slot] = (int)blockIdx.x;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 10) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int D, typename OutT>
static int launch_fast(const int8_t* k8, const uint16_t* v16, const AttnParams& p, unsigned ctas, cudaStream_t s) {
  using Cfg = FastCfg<D>;
  const uint64_t BH = (uint64_t)p.B * p.H;
  const uint64_t npad = (uint64_t)p.nb * 64;
  const CUtensorMapSwizzle swz_qk = D == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  CUtensorMap tq, tk, tv;
  if (int rc = make_tensor_map(&tq, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, p.q8, D, p.N, BH, D, 128, swz_qk)) return rc;
  if (int rc = make_tensor_map(&tk, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k8, D, p.N, BH, D, 64, swz_qk)) return rc;
  if (int rc = make_tensor_map(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, v16, npad, D, BH, 64, D, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  auto kern = sparse_attn_fast_kernel<D, OutT>;
  PARO_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
  constexpr int carveout_pct = (2 * (Cfg::SMEM_BYTES + 1024) * 100 + 228 * 1024 - 1) / (228 * 1024);
  PARO_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, carveout_pct < 100 ? carveout_pct : 100));
  kern<<<ctas, ATT_THREADS, Cfg::SMEM_BYTES, s>>>(tq, tk, tv, p);
  return check_launch("sparse_attn_fast_kernel");
}

int launch_attn_fast(const int8_t* k8, const uint16_t* v16, const AttnParams& p, int D, int out_dtype, unsigned ctas,
                     cudaStream_t s) {
  if (D == 128)
    return out_dtype == PARO_F16 ? launch_fast<128, __half>(k8, v16, p, ctas, s)
                                 : launch_fast<128, __nv_bfloat16>(k8, v16, p, ctas, s);
  return out_dtype == PARO_F16 ? launch_fast<64, __half>(k8, v16, p, ctas, s)
                               : launch_fast<64, __nv_bfloat16>(k8, v16, p, ctas, s);
}

}  // namespace paro
