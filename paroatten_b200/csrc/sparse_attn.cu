// Block-sparse attention over kept 64x64 blocks for sm_100a.  One kernel, two walks (template flag):
// the FIXED-REFERENCE walk, which paro_sparse_attn runs on every work item, and the EXACT walk
// (running row maximum, online softmax with rescaling), which then computes the few work items the
// first one gave back (rows whose scores span more than its exponent range), read from the redo list.
//
// Work item (one CTA): a PAIR of adjacent 64-row q-blocks of one (batch, head), i.e. a 128-row
// tile -- the native tcgen05.mma M.  The pair walks a schedule built with the plan: first the
// k-blocks BOTH q-blocks keep (one K/V tile and one full-height MMA group serve all 128 rows), then
// the remaining blocks of the upper half side by side with the remaining blocks of the lower half.
// In a side-by-side step each MMA is issued with the query tile of all 128 rows but with a lane mask
// that keeps it from writing the other half's accumulator rows, so both halves always have work (all
// four SM sub-partitions run exponentials) and nothing is computed for blocks that are not kept.
//
//   warps 0-7   softmax + epilogue.  Row r of the tile belongs to two threads, one in each WARP SET:
//               warp w (< 4, set 0) handles the even steps of its half, warp w+4 (set 1) the odd
//               steps (both may touch TMEM lane quadrant w).  A thread handles the whole row (64
//               scores) of its steps, so two consecutive steps of a half are in flight at once.
//               Base-2 softmax in fp32; each thread keeps its own share of the row sum (and, in the
//               exact walk, the running row maximum passes from step to step through shared memory).
//               P is written to TMEM as bf16; the epilogue stores O/l * v_scale + vm at the row's
//               un-permuted position.  These warps take the registers the others give up.
//   warp 8      one lane: TMA producer for the K ring (int8 tiles)
//   warp 9      one lane: TMA producer for the V^T ring (bf16 tiles)
//   warp 10     owns TMEM; issues S = Q.K^T (kind::i8, A = Q from TMEM, int32 accumulators)
//   warp 11     issues O += P.V (kind::f16 on bf16, A = P from TMEM, fp32 accumulators in TMEM)
//               The two issuer warps run their loops with all 32 lanes converged, so that descriptors
//               and addresses are formed in uniform registers; the tcgen05 instructions themselves
//               are guarded by the elected lane's predicate.
//
// Hand-offs.  An issuer commits ONCE per tile, to the barrier of (half, step mod 4): "scores ready"
// for Q.K^T, "P.V done" for P.V.  The softmax warps wait on it, and so does the ring's producer when it
// wants that tile's stage back.  The softmax warps release S the moment the scores are in registers
// and write P after all of a step's arithmetic.
//
// TMEM (256 columns per CTA): S [0,64) int32 scores, P [64,96) bf16 probabilities, Q [96,128) the
// int8 query tile (A operand of Q.K^T read from TMEM, so it is not re-read from shared memory for
// every k-block), O [128,128+D) fp32.  Q.K^T of step i+1 overlaps the exponentials of step i (and the
// other warp set starts on step i+1 while step i is still being exponentiated), and P.V of step i
// overlaps the softmax of step i+1; two CTAs share an SM so that one CTA's softmax overlaps the
// other's MMAs.  Every wait is bounded: on expiry the CTA records a code in the status words, raises
// a shared abort flag and unwinds (copies landed, MMAs retired, TMEM freed).
#include <mutex>
#include <type_traits>

#include "attn_common.cuh"

namespace paro {

using namespace umma;

// Developer aid, compiled out unless PARO_TRACE=<block index> is defined: that CTA of the fixed-reference
// launch stamps clock64() at the hand-off points of its first 160 steps (roles: 0/1 K/V producer, 2/3
// Q.K^T / P.V issuer, 4.. softmax warps; paro_debug_trace copies the table to the host).  This is how the
// per-role time budget of a step was measured.
#ifdef PARO_TRACE
__device__ long long g_trace[16][160][8];
#define TR(role, step, ev) do { if (FIXED && blockIdx.x == PARO_TRACE && (step) < 160) g_trace[role][step][ev] = clock64(); } while (0)
#define TRL(role, step, ev) do { if (lead) TR(role, step, ev); } while (0)   // in a role whose whole warp runs: one lane stamps
#else
#define TR(role, step, ev)
#define TRL(role, step, ev)
#endif
constexpr float RESCALE_TAU = 8.0f;            // exact walk: rescale O only when the row max grows by > 2^8
constexpr float REF_OFFSET = 20.f;             // fixed reference: the first block's maximum maps to P = 2^-20
constexpr float ROWSUM_LIMIT = 1.2676506e30f;  // 2^100: a step's row sum beyond it gives the pair back

template <int D> struct AttnCfg {
  // Ring depths.  TMEM allows two CTAs per SM; the loads run far ahead of their use at any depth from 2
  // to 6 (same time within noise), so the rings are kept short and the shared memory left over is
  // requested back as L1 (carve-out attribute at launch) for the schedule entries and k-block scales.
  static constexpr int K_STAGES = (D == 128) ? 3 : 4;
  static constexpr int V_STAGES = (D == 128) ? 3 : 4;
  // The commit barriers are indexed by step modulo STEP_BARS, and a ring stage is handed back to its
  // producer through the commit barrier of the tile that used it: a producer can only tell that
  // barrier's phases apart while the ring is no deeper than STEP_BARS.
  static constexpr int STEP_BARS = 4;
  static_assert(K_STAGES <= STEP_BARS && V_STAGES <= STEP_BARS, "ring deeper than the commit barriers can tell apart");
  static constexpr int K_BYTES = 64 * D;
  static constexpr int V_BYTES = D * 128;   // D rows of 64 bf16
  static constexpr int TILE_BYTES = K_STAGES * K_BYTES + V_STAGES * V_BYTES;
  static constexpr int AUX_BYTES = 4096;    // barriers, TMEM pointer, abort flag, v_scale, vm, row exchange
  static constexpr int SMEM_BYTES = TILE_BYTES + AUX_BYTES + 1024 /* alignment slack */;
};

#define ATT_WAIT(bar, parity, where, iter)                                   \
  if (!mbar_wait_bounded((bar), (parity), abort_flag, WAIT_LIMIT)) {         \
    report_timeout(p, abort_flag, (where), (iter));                          \
    break;                                                                   \
  }

// FIXED = false: exact running row maximum (online softmax, lazy rescaling of O).
// FIXED = true:  the row's reference exponent is fixed when its FIRST kept block has been seen (that
//   block's maximum + REF_OFFSET) and P = 2^(s - m_ref) is kept in bf16 (8 exponent bits) and summed in
//   fp32, so scores up to 2^100 above the first block are representable and nothing is ever rescaled:
//   no per-step maximum, no maximum handed between the warp sets, no accumulator read-modify-write.
//   A step whose row sum leaves that range (or is not finite) makes the CTA give its work item back
//   through the redo list instead of storing it; the exact walk then computes that pair.
template <int D, typename OutT, bool FIXED>
__global__ void __launch_bounds__(ATT_THREADS, 2)
sparse_attn_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                         const AttnParams p) {
  using Cfg = AttnCfg<D>;
  constexpr int KST = Cfg::K_STAGES, VST = Cfg::V_STAGES;
  // second launch of a call: only the work items the fixed-reference walk gave back
  if (p.from_list && (int)blockIdx.x >= *reinterpret_cast<volatile int32_t*>(p.redo)) return;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* sK = smem;
  uint8_t* sV = sK + KST * Cfg::K_BYTES;
  uint8_t* aux = smem + Cfg::TILE_BYTES;
  // mbarriers.  [h][par]: one per half of the pair and per parity of the step index, so that each
  // barrier is arrived on and waited for by the same parties in every phase.
  uint64_t* bar_q = reinterpret_cast<uint64_t*>(aux);   // [1]     Q tile stored in TMEM
  uint64_t* bar_kfull = bar_q + 1;                      // [KST]   K tile landed
  uint64_t* bar_vfull = bar_kfull + KST;                // [VST]   V tile landed
  uint64_t* bar_sready = bar_vfull + VST;               // [2][4]  scores of (half, step mod 4) in TMEM: the Q.K^T
                                                        //         finished, so its K stage is free as well
  uint64_t* bar_pvdone = bar_sready + 8;                // [2][4]  P.V of (half, step mod 4) finished: P may be
                                                        //         rewritten, the V stage is free
  uint64_t* bar_sfree = bar_pvdone + 8;                 // [2][2]  scores of (half, step parity) copied to registers
  uint64_t* bar_pready = bar_sfree + 4;                 // [2][2]  P of (half, step parity) written
  uint64_t* bar_drain = bar_pready + 4;                 // [2]     issuers' MMAs retired (abort path only)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bar_drain + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* s_drain = abort_flag + 1;                  // 1: an earlier launch or CTA failed, leave at once
  volatile int* s_redo = s_drain + 1;                      // 1: a row sum left the fixed-reference range
  volatile int* s_mstep = s_redo + 1;                      // [4]  steps whose row maxima are published, per quadrant
  float* s_vscale = reinterpret_cast<float*>(aux + 512);   // [D]
  float* s_vm = s_vscale + D;                              // [D]
  volatile float* s_mrow = reinterpret_cast<volatile float*>(aux + 1536);   // [128] running row maximum
  float* s_xl = reinterpret_cast<float*>(aux + 2048);                       // [2][128] row-sum exchange
  static_assert(512 + 2 * D * 4 <= 1536 && 2048 + 2 * 128 * 4 <= Cfg::AUX_BYTES, "aux area too small");
  static_assert((27 + KST + VST) * 8 + 8 + 28 <= 512, "barrier area too small");

  // (the warp index through a shuffle: provably the same in all lanes, so the role branches are uniform)
  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
  // one thread decides for the whole CTA whether an earlier failure makes this launch drain (every
  // thread reading the word for itself could split the CTA around the collective operations below)
  if (threadIdx.x == 0) *s_drain = *reinterpret_cast<volatile int32_t*>(p.status) != 0;
  __syncthreads();
  if (*s_drain) return;
  const int item = p.from_list ? p.redo[REDO_HEADER + blockIdx.x] : (int)blockIdx.x;
  const int bh = item / p.npairs, pair = item % p.npairs;
  const int slice = bh % p.plan_slices;
  // The pair's schedule: entry i = kbA | kbB << 16 (0xFFFF: no tile for that half in step i).  First
  // the k-blocks both halves keep (kbA == kbB: one K/V tile, one full-height MMA group), then the
  // halves' remaining blocks side by side; each half's steps are contiguous from step 0.
  const int prow = slice * p.npairs + pair;
  const uint32_t* sched = p.sched + p.pair_ptr[prow];
  // per half: steps in the low 16 bits; the high 16 bits are 0 (the pair is q-blocks 2p and 2p+1) or hold
  // 1 + the q-block the half stands for, when the plan paired q-blocks by the k-blocks they share
  const uint32_t cnt_a = (uint32_t)p.sched_cnt[2 * prow], cnt_b = (uint32_t)p.sched_cnt[2 * prow + 1];
  const int n_a = (int)(cnt_a & 0xFFFFu), n_b = (int)(cnt_b & 0xFFFFu);
  const int n_steps = max(n_a, n_b);
  // A step has one MMA group of each kind per tile: group 0 serves the upper half, or both halves
  // when the tile is shared (kbA == kbB); group 1 serves the lower half.  Sharing halves the tensor
  // work of such a step but makes the two halves wait for each other in it.  (With single-lane
  // issuers that wait cost more than it saved at D = 64; with the issuers running warp-wide sharing
  // wins there too: 3.85 vs 3.96 ms on the CogVideoX shape.)
  constexpr bool SHARE_TILES = true;
  // Issuing a side-by-side step's two tiles in one burst (see `both` below) is slower at D = 128, where the
  // tensor pipe is what the issuers wait for (21.5 vs 21.1 ms on the Wan-14B shape), and a little faster at
  // D = 64.
  constexpr bool FUSE_STEPS = (D == 64);
#define PARO_STEP_GROUPS(e)                                                        \
  const int ka_ = (int)((e) & 0xFFFFu), kb_ = (int)((e) >> 16);                    \
  const bool shared_ = SHARE_TILES && ka_ == kb_;                                  \
  const bool act_[2] = {ka_ != 0xFFFF, !shared_ && kb_ != 0xFFFF};                 \
  [[maybe_unused]] const int kblk_[2] = {ka_, kb_};                                \
  [[maybe_unused]] const int which_[2] = {shared_ ? 2 : 0, 1};

  if (threadIdx.x == 0) {
    mbar_init(bar_q, 4);
    for (int i = 0; i < KST; ++i) mbar_init(bar_kfull + i, 1);
    for (int i = 0; i < VST; ++i) mbar_init(bar_vfull + i, 1);
    for (int i = 0; i < 8; ++i) {
      mbar_init(bar_sready + i, 1);
      mbar_init(bar_pvdone + i, 1);
    }
    for (int i = 0; i < 4; ++i) {
      mbar_init(bar_sfree + i, 2);    // the two warps (lane quadrants) of a half in one warp set
      mbar_init(bar_pready + i, 2);
      s_mstep[i] = 0;
    }
    mbar_init(bar_drain, 1);
    mbar_init(bar_drain + 1, 1);
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
  const uint32_t tS = tmem_base, tP = tmem_base + 64u, tQ = tmem_base + 96u, tO = tmem_base + 128u;

  if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 32;");
    if (warp == 8 && lane == 0) {
      // ---------------------------------------------------------------- TMA producer: K ring
      tma_prefetch_desc(&tm_k);
      bool ok = true;
      int t = 0;   // tiles so far = position in the ring
      // a stage is free again when the Q.K^T of the tile that held it has finished: the scores-ready
      // commit of that tile (no commit of its own for the ring)
      const uint32_t a_done = smem_u32(bar_sready);
      ReleaseFifo<KST> held;
      // schedule entries are fetched two steps ahead of their use
      uint32_t e_cur = n_steps > 0 ? sched[0] : 0u, e_nxt = n_steps > 1 ? sched[1] : 0u;
      for (int i = 0; i < n_steps && ok; ++i) {
        PARO_STEP_GROUPS(e_cur)
        e_cur = e_nxt;
        if (i + 2 < n_steps) e_nxt = ld_pinned_u32(sched + i + 2);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          if (!act_[j]) continue;
          const int st = t % KST;
          TR(0, i, 2 * j);
          if (t >= KST && !mbar_wait_bounded_at(held.oldest() & 0x7fffffffu, held.oldest() >> 31, abort_flag, WAIT_LIMIT)) {
            report_timeout(p, abort_flag, 1, i);
            ok = false;
            break;
          }
          held.push(commit_token(a_done, j, i));   // (a tile shared by both halves commits to both: j = 0 is watched)
          ++t;
          TR(0, i, 2 * j + 1);
          mbar_arrive_expect_tx(bar_kfull + st, Cfg::K_BYTES);
          tma_load_3d(sK + st * Cfg::K_BYTES, &tm_k, 0, kblk_[j] * 64, bh, bar_kfull + st);
        }
      }
      if (*abort_flag)   // leaving early: the copies this thread started must have landed first
        for (int u = max(0, t - KST); u < t; ++u) mbar_wait_plain_bounded(bar_kfull + u % KST, (u / KST) & 1, WAIT_LIMIT);
    } else if (warp == 9 && lane == 0) {
      // ---------------------------------------------------------------- TMA producer: V ring
      tma_prefetch_desc(&tm_v);
      bool ok = true;
      int t = 0;
      const uint32_t a_done = smem_u32(bar_pvdone);   // the P.V commit of the tile that held the stage
      ReleaseFifo<VST> held;
      uint32_t e_cur = n_steps > 0 ? sched[0] : 0u, e_nxt = n_steps > 1 ? sched[1] : 0u;
      for (int i = 0; i < n_steps && ok; ++i) {
        PARO_STEP_GROUPS(e_cur)
        e_cur = e_nxt;
        if (i + 2 < n_steps) e_nxt = ld_pinned_u32(sched + i + 2);
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          if (!act_[j]) continue;
          const int st = t % VST;
          TR(1, i, 2 * j);
          if (t >= VST && !mbar_wait_bounded_at(held.oldest() & 0x7fffffffu, held.oldest() >> 31, abort_flag, WAIT_LIMIT)) {
            report_timeout(p, abort_flag, 9, i);
            ok = false;
            break;
          }
          held.push(commit_token(a_done, j, i));
          ++t;
          TR(1, i, 2 * j + 1);
          mbar_arrive_expect_tx(bar_vfull + st, Cfg::V_BYTES);
          tma_load_3d(sV + st * Cfg::V_BYTES, &tm_v, kblk_[j] * 64, 0, bh, bar_vfull + st);
        }
      }
      if (*abort_flag)
        for (int u = max(0, t - VST); u < t; ++u) mbar_wait_plain_bounded(bar_vfull + u % VST, (u / VST) & 1, WAIT_LIMIT);
    } else if (warp == 10) {
      // ---------------------------------------------------------------- MMA issuer: S = Q.K^T
      // (the two issuers are separate warps so that a P.V group waiting for room in the tensor
      // queue does not hold back the next scores, and vice versa)
      // Every tile of the walk passes through an issuer, so its instruction count per tile is on the
      // kernel's critical path.  Hence: barrier addresses and the stage-0 descriptor are formed once,
      // the polls of a tile's barriers are issued together, ring position and phase are counters, and
      // the lane masks are compile-time constants of three instantiations of the tile code (W = 0
      // upper half, 1 lower half, 2 both halves, unmasked form).
      // The whole warp runs this loop converged (values below are made warp-uniform with a shuffle from
      // lane 0, every decision is a vote), so that descriptors and addresses live in uniform registers;
      // the tcgen05 instructions themselves are guarded by the elected lane's predicate.
      constexpr uint32_t IDESC_QK = instr_desc(2, 1, 1, 128, 64);  // s32 += s8 * s8
      const uint32_t lead = elect_one();
      const int n_steps_u = __shfl_sync(0xffffffffu, n_steps, 0);
      const uint32_t tS_u = __shfl_sync(0xffffffffu, tS, 0), tQ_u = tS_u + 96u;
      do {
        if (!__all_sync(0xffffffffu, mbar_wait_bounded(bar_q, 0, abort_flag, WAIT_LIMIT))) {
          report_timeout(p, abort_flag, 2, -1);
          break;
        }
        const uint32_t a_sfree = smem_u32(bar_sfree), a_sready = smem_u32(bar_sready);
        const uint32_t a_kfull = smem_u32(bar_kfull);
        const uint64_t dK0 = smem_desc(smem_u32(sK), D);
        uint32_t st = 0, kph = 0;   // ring stage of the next tile and the parity of its current use
        // the MMAs of one tile and their commit
        auto issue = [&](auto wtag, const int i, const uint32_t stage) {
          constexpr int W = decltype(wtag)::value;
          const uint64_t dK = dK0 + (uint64_t)(stage * (uint32_t)(Cfg::K_BYTES >> 4));
#pragma unroll
          for (int k = 0; k < D / 32; ++k) {
            if (W == 2) mma_i8_ts_p(lead, tS_u, tQ_u + 8 * k, desc_advance(dK, 32 * k), IDESC_QK, k > 0);
            else if (W == 0)   // lanes NOT written: the rows of the half the tile does not serve
              mma_i8_ts_masked_p(lead, tS_u, tQ_u + 8 * k, desc_advance(dK, 32 * k), IDESC_QK, k > 0, 0u, 0u, 0xffffffffu, 0xffffffffu);
            else
              mma_i8_ts_masked_p(lead, tS_u, tQ_u + 8 * k, desc_advance(dK, 32 * k), IDESC_QK, k > 0, 0xffffffffu, 0xffffffffu, 0u, 0u);
          }
          // one commit per half served: the softmax warps wait on it for the scores, the K producer for the stage
          if (W != 1) mma_commit_at_p(lead, a_sready + 8u * (uint32_t)(i & 3));
          if (W != 0) mma_commit_at_p(lead, a_sready + 32u + 8u * (uint32_t)(i & 3));
        };
        auto tile = [&](auto wtag, const int i, const int ev) -> bool {
          constexpr int W = decltype(wtag)::value;
          // the scores of step i-1 of the halves served are in registers: their rows of S may be
          // overwritten.  (i = 0 asks an unused barrier for parity 1, which passes at once.)
          const uint32_t par = (uint32_t)(i - 1) & 1u, ph = ((uint32_t)(i - 1) >> 1) & 1u;
          TRL(2, i, ev + 0);
          const bool r0 = W == 1 || mbar_poll(a_sfree + 8u * par, ph);
          const bool r1 = W == 0 || mbar_poll(a_sfree + 16u + 8u * par, ph);
          const bool r2 = mbar_poll(a_kfull + 8u * st, kph);
          if (!__all_sync(0xffffffffu, r0 && r1 && r2)) {
            bool good = true;
            if (W != 1) good = mbar_wait_bounded(bar_sfree + par, ph, abort_flag, WAIT_LIMIT);
            if (W != 0) good = good && mbar_wait_bounded(bar_sfree + 2 + par, ph, abort_flag, WAIT_LIMIT);
            good = good && mbar_wait_bounded(bar_kfull + st, kph, abort_flag, WAIT_LIMIT);
            if (!__all_sync(0xffffffffu, good)) return false;
          }
          TRL(2, i, ev + 1);
          tc_fence_after();
          issue(wtag, i, st);
          if (++st == KST) {
            st = 0;
            kph ^= 1u;
          }
          TRL(2, i, ev + 3);
          return true;
        };
        // A side-by-side step (one tile per half) whose four barriers are all complete -- the usual case
        // while this thread is what the walk waits for -- is issued as straight-line code: one branch for
        // the step instead of one per poll, tile and ring wrap (a taken branch costs a lone thread
        // about as much as issuing an MMA).
        auto both = [&](const int i) -> bool {
          const uint32_t par = (uint32_t)(i - 1) & 1u, ph = ((uint32_t)(i - 1) >> 1) & 1u;
          const uint32_t wrap1 = st + 1 == KST ? 1u : 0u, st1 = wrap1 ? 0u : st + 1, ph1 = kph ^ wrap1;
          TRL(2, i, 0);
          const bool r0 = mbar_poll(a_sfree + 8u * par, ph), r1 = mbar_poll(a_sfree + 16u + 8u * par, ph);
          const bool r2 = mbar_poll(a_kfull + 8u * st, kph), r3 = mbar_poll(a_kfull + 8u * st1, ph1);
          if (!__all_sync(0xffffffffu, r0 & r1 & r2 & r3)) return false;
          TRL(2, i, 1);
          tc_fence_after();
          issue(std::integral_constant<int, 0>{}, i, st);
          TRL(2, i, 3);
          issue(std::integral_constant<int, 1>{}, i, st1);
          const uint32_t wrap2 = st1 + 1 == KST ? 1u : 0u;
          st = wrap2 ? 0u : st1 + 1;
          kph = ph1 ^ wrap2;
          TRL(2, i, 7);
          return true;
        };
        uint32_t e_cur = n_steps_u > 0 ? sched[0] : 0u, e_nxt = n_steps_u > 1 ? sched[1] : 0u;
        for (int i = 0; i < n_steps_u; ++i) {
          const uint32_t e_u = __shfl_sync(0xffffffffu, e_cur, 0);
          const uint32_t ka = e_u & 0xFFFFu, kb = e_u >> 16;
          e_cur = e_nxt;
          if (i + 2 < n_steps_u) e_nxt = ld_pinned_u32(sched + i + 2);
          bool good;
          if (SHARE_TILES && ka == kb && ka != 0xFFFFu) {
            good = tile(std::integral_constant<int, 2>{}, i, 0);
          } else {
            if (FUSE_STEPS && ka != 0xFFFFu && kb != 0xFFFFu && both(i)) continue;
            good = ka == 0xFFFFu || tile(std::integral_constant<int, 0>{}, i, 0);
            good = good && (kb == 0xFFFFu || tile(std::integral_constant<int, 1>{}, i, 4));
          }
          if (!good) {
            report_timeout(p, abort_flag, 3, i);
            break;
          }
        }
      } while (false);
      if (*abort_flag) {   // the MMAs issued so far must retire before tensor memory is freed
        if (lead) mma_commit(bar_drain);
        mbar_wait_plain_bounded(bar_drain, 0, WAIT_LIMIT);
      }
    } else if (warp == 11) {
      // ---------------------------------------------------------------- MMA issuer: O += P.V
      constexpr uint32_t IDESC_PV = instr_desc(1, 1, 1, 128, D);   // f32 += bf16 * bf16
      const uint32_t lead = elect_one();
      const int n_steps_u = __shfl_sync(0xffffffffu, n_steps, 0);
      const uint32_t tS_u = __shfl_sync(0xffffffffu, tS, 0), tP_u = tS_u + 64u, tO_u = tS_u + 128u;
      const uint32_t a_pready = smem_u32(bar_pready), a_pvdone = smem_u32(bar_pvdone);
      const uint32_t a_vfull = smem_u32(bar_vfull);
      const uint64_t dV0 = smem_desc(smem_u32(sV), 128);
      uint32_t st = 0, vph = 0;
      auto issue = [&](auto wtag, const int i, const uint32_t stage) {
        constexpr int W = decltype(wtag)::value;
        const uint64_t dV = dV0 + (uint64_t)(stage * (uint32_t)(Cfg::V_BYTES >> 4));
        // both halves start at step 0, so a tile that serves both never mixes a first with a later step
        const uint32_t acc0 = i > 0 ? 1u : 0u;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          const uint32_t acc = k > 0 ? 1u : acc0;
          if (W == 2) mma_f16_ts_p(lead, tO_u, tP_u + 8 * k, desc_advance(dV, 32 * k), IDESC_PV, acc);
          else if (W == 0)
            mma_f16_ts_masked_p(lead, tO_u, tP_u + 8 * k, desc_advance(dV, 32 * k), IDESC_PV, acc, 0u, 0u, 0xffffffffu, 0xffffffffu);
          else
            mma_f16_ts_masked_p(lead, tO_u, tP_u + 8 * k, desc_advance(dV, 32 * k), IDESC_PV, acc, 0xffffffffu, 0xffffffffu, 0u, 0u);
        }
        // one commit per half served: P of that half may be rewritten, and the V producer takes it for the stage
        if (W != 1) mma_commit_at_p(lead, a_pvdone + 8u * (uint32_t)(i & 3));
        if (W != 0) mma_commit_at_p(lead, a_pvdone + 32u + 8u * (uint32_t)(i & 3));
      };
      auto tile = [&](auto wtag, const int i, const int ev) -> bool {
        constexpr int W = decltype(wtag)::value;
        const uint32_t par = (uint32_t)i & 1u, ph = ((uint32_t)i >> 1) & 1u;
        TRL(3, i, ev + 0);
        const bool r0 = W == 1 || mbar_poll(a_pready + 8u * par, ph);
        const bool r1 = W == 0 || mbar_poll(a_pready + 16u + 8u * par, ph);
        const bool r2 = mbar_poll(a_vfull + 8u * st, vph);
        if (!__all_sync(0xffffffffu, r0 && r1 && r2)) {
          bool good = true;
          if (W != 1) good = mbar_wait_bounded(bar_pready + par, ph, abort_flag, WAIT_LIMIT);
          if (W != 0) good = good && mbar_wait_bounded(bar_pready + 2 + par, ph, abort_flag, WAIT_LIMIT);
          good = good && mbar_wait_bounded(bar_vfull + st, vph, abort_flag, WAIT_LIMIT);
          if (!__all_sync(0xffffffffu, good)) return false;
        }
        TRL(3, i, ev + 1);
        tc_fence_after();
        issue(wtag, i, st);
        if (++st == VST) {
          st = 0;
          vph ^= 1u;
        }
        TRL(3, i, ev + 3);
        return true;
      };
      auto both = [&](const int i) -> bool {   // (as in the Q.K^T issuer)
        const uint32_t par = (uint32_t)i & 1u, ph = ((uint32_t)i >> 1) & 1u;
        const uint32_t wrap1 = st + 1 == VST ? 1u : 0u, st1 = wrap1 ? 0u : st + 1, ph1 = vph ^ wrap1;
        TRL(3, i, 0);
        const bool r0 = mbar_poll(a_pready + 8u * par, ph), r1 = mbar_poll(a_pready + 16u + 8u * par, ph);
        const bool r2 = mbar_poll(a_vfull + 8u * st, vph), r3 = mbar_poll(a_vfull + 8u * st1, ph1);
        if (!__all_sync(0xffffffffu, r0 & r1 & r2 & r3)) return false;
        TRL(3, i, 1);
        tc_fence_after();
        issue(std::integral_constant<int, 0>{}, i, st);
        TRL(3, i, 3);
        issue(std::integral_constant<int, 1>{}, i, st1);
        const uint32_t wrap2 = st1 + 1 == VST ? 1u : 0u;
        st = wrap2 ? 0u : st1 + 1;
        vph = ph1 ^ wrap2;
        TRL(3, i, 7);
        return true;
      };
      uint32_t e_cur = n_steps_u > 0 ? sched[0] : 0u, e_nxt = n_steps_u > 1 ? sched[1] : 0u;
      for (int i = 0; i < n_steps_u; ++i) {
        const uint32_t e_u = __shfl_sync(0xffffffffu, e_cur, 0);
        const uint32_t ka = e_u & 0xFFFFu, kb = e_u >> 16;
        e_cur = e_nxt;
        if (i + 2 < n_steps_u) e_nxt = ld_pinned_u32(sched + i + 2);
        bool good;
        if (SHARE_TILES && ka == kb && ka != 0xFFFFu) {
          good = tile(std::integral_constant<int, 2>{}, i, 0);
        } else {
          if (FUSE_STEPS && ka != 0xFFFFu && kb != 0xFFFFu && both(i)) continue;
          good = ka == 0xFFFFu || tile(std::integral_constant<int, 0>{}, i, 0);
          good = good && (kb == 0xFFFFu || tile(std::integral_constant<int, 1>{}, i, 4));
        }
        if (!good) {
          report_timeout(p, abort_flag, 5, i);
          break;
        }
      }
      if (*abort_flag) {
        if (lead) mma_commit(bar_drain + 1);
        mbar_wait_plain_bounded(bar_drain + 1, 0, WAIT_LIMIT);
      }
    }
  } else {
    // ------------------------------------------------------------------ softmax + epilogue
    asm volatile("setmaxnreg.inc.sync.aligned.u32 104;");
    const int qd = warp & 3;                 // TMEM lane quadrant this warp may touch
    const int set = warp >> 2;               // warp set: steps of this parity; also which half of O's columns
    const int r = qd * 32 + lane;            // row inside the 128-row tile
    const int half = qd >> 1;                // which q-block of the pair
    const uint32_t lane_off = (uint32_t)(qd * 32) << 16;
    const int n_mine = half ? n_b : n_a;
    auto my_kb = [&](int i) { return (int)((sched[i] >> (16 * half)) & 0xFFFFu); };   // this half's k-block of step i
    if (threadIdx.x < D) {
      s_vscale[threadIdx.x] = p.v_scale[(size_t)bh * D + threadIdx.x];
      s_vm[threadIdx.x] = p.vm ? p.vm[(size_t)bh * D + threadIdx.x] : 0.f;
    }
    named_barrier(1, ATT_SOFTMAX_THREADS);

    const uint32_t cnt_mine = half ? cnt_b : cnt_a;
    const int qblk = (cnt_mine >> 16) ? (int)(cnt_mine >> 16) - 1 : 2 * pair + half;
    const int tok = qblk * 64 + (r & 63);
    if (set == 0) {
      // this thread's query row goes to TMEM (four int8 per 32-bit column); rows past the end are zero
      uint32_t qrow[D / 4];
      const uint4* src = reinterpret_cast<const uint4*>(p.q8 + ((size_t)bh * p.N + (tok < p.N ? tok : 0)) * D);
#pragma unroll
      for (int j = 0; j < D / 16; ++j) {
        const uint4 v4 = tok < p.N ? src[j] : make_uint4(0, 0, 0, 0);
        qrow[4 * j] = v4.x; qrow[4 * j + 1] = v4.y; qrow[4 * j + 2] = v4.z; qrow[4 * j + 3] = v4.w;
      }
      if (D == 128) tmem_st32(tQ + lane_off, qrow); else tmem_st16(tQ + lane_off, qrow);
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      mbar_arrive_if(bar_q, lane == 0);
    }
    const int per_bh = p.nb * (64 / p.q_group);
    // rows past the end of the sequence: scale 0, or (fixed reference) a tiny positive one -- there the
    // -inf of masked columns times 0 would be a NaN that reads as a row sum out of range
    const float rowscale = tok < p.N ? p.q_scale[(size_t)bh * per_bh + tok / p.q_group] * p.scale_log2
                                     : (FIXED ? 1e-30f : 0.f);
    // l: this thread's share of the row sum (the steps of its parity), relative to the maximum m_l
    // (exact walk) or to the row's fixed reference exponent m_ref
    float m_l = -INFINITY, l = 0.f, m_ref = 0.f;
    bool ok = true, redo = false;
    auto wait_bar = [&](uint32_t bar_saddr, int phase, int code, int i) {
      const bool good = __all_sync(0xffffffffu, mbar_wait_bounded_at(bar_saddr, phase & 1, abort_flag, WAIT_LIMIT));
      if (!good) report_timeout(p, abort_flag, code, i);
      tc_fence_after();
      return good;
    };
    uint64_t* const my_sfree = bar_sfree + 2 * half + set;
    uint64_t* const my_pready = bar_pready + 2 * half + set;
    const uint32_t my_sready = smem_u32(bar_sready + 4 * half), my_pvdone = smem_u32(bar_pvdone + 4 * half);   // [step mod 4]
    const float* kscale_bh = p.k_scale + (size_t)bh * p.nb;
    // (a k-block id beyond the sequence can only come from a malformed plan; clamped so that the scale
    // look-up stays inside its array)
    int kb_next = set < n_mine ? min(my_kb(set), p.nb - 1) : 0;
    float ks_next = set < n_mine ? kscale_bh[kb_next] : 0.f;
    // One step of this thread's half (the two halves only meet in the issuers' queues).  `first` is a
    // compile-time tag: the thread's first step, where the fixed-reference walk settles the row's
    // reference exponent; every later step of that walk is straight-line code from scores to P.
    auto do_step = [&](const int i, auto first) -> bool {
      [[maybe_unused]] constexpr bool FIRST = decltype(first)::value;
      const int kb = kb_next;
      const float kscale = ks_next;
      if (i + 2 < n_mine) {   // fetched one step ahead so that the loads are off the critical path
        kb_next = min(my_kb(i + 2), p.nb - 1);
        ks_next = kscale_bh[kb_next];
      }
      [[maybe_unused]] const int trole = 4 + warp;
      TR(trole, i, 0);
      if (!wait_bar(my_sready + 8u * (i & 3), i >> 2, 6, i)) return false;
      TR(trole, i, 1);
      float f[64];
      {
        uint32_t s[64];
        tmem_ld32(tS + lane_off, s);
        tmem_ld32(tS + lane_off + 32u, s + 32);
        tmem_wait_ld();
        TR(trole, i, 2);
        // the scores are in registers: let the issuer overwrite S with this half's next step
        tc_fence_before();
        __syncwarp();
        mbar_arrive_if(my_sfree, lane == 0);
        // A branch on a value read after the arrival ends the basic block here.  Without it the
        // arrival, which nothing below depends on, is scheduled at the END of the straight-line code
        // that follows (after the step's exponentials), and the next Q.K^T starts that much later.
        if (*abort_flag) return false;
        // int32 scores -> fp32 by an integer addition instead of a conversion: the bit pattern
        // 0x4B400000 + s is the float SCORE_BIAS + s exactly (|s| <= 127 * 127 * D < 2^22).  The bias is
        // monotonic, so the row maximum is taken over the biased values, and it is folded into the
        // constant of the multiply-add that forms the exponent; that constant is rounded once, to
        // within 0.75 of one integer score step, common to the row and step.
#pragma unroll
        for (int j = 0; j < 64; ++j) f[j] = __int_as_float((int)s[j] + 0x4B400000);
      }
      const int valid = min(64, p.N - kb * 64);   // columns inside the sequence
      const float sc = rowscale * kscale;
      if (!FIXED && valid < 64) {   // (the fixed-reference walk corrects its row sum instead, below)
#pragma unroll
        for (int j = 0; j < 64; ++j)
          if (j >= valid) f[j] = -INFINITY;
      }
      auto row_max = [&]() {   // maximum of the step's scores, in the exponent's units
        float mx4[4] = {f[0], f[1], f[2], f[3]};   // four independent chains of 3-input max
#pragma unroll
        for (int j = 4; j < 64; j += 8) {
          mx4[0] = max3(mx4[0], f[j], f[j + 1]);
          mx4[1] = max3(mx4[1], f[j + 2], f[j + 3]);
          if (j + 4 < 64) {
            mx4[2] = max3(mx4[2], f[j + 4], f[j + 5]);
            mx4[3] = max3(mx4[3], f[j + 6], f[j + 7]);
          }
        }
        return (fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) - SCORE_BIAS) * sc;
      };
      float m_new;
      bool pv_consumed = FIXED ? (FIRST && set == 0) : (i == 0);   // step 0: nothing to wait for
      if constexpr (FIXED) {
        if (FIRST && set == 0) {
          m_ref = row_max() + REF_OFFSET;
          s_mrow[r] = m_ref;
          __syncwarp();
          st_release_shared_if(s_mstep + qd, 1, lane == 0);
        } else if (FIRST) {   // (step 1) the other warp set fixed the reference in step 0
          bool seen = ld_acquire_shared(s_mstep + qd) != 0;
          if (!seen) {
            const long long t0 = clock64();
            while (!(seen = ld_acquire_shared(s_mstep + qd) != 0)) {
              if (*abort_flag || clock64() - t0 > WAIT_LIMIT) break;
            }
          }
          if (!__all_sync(0xffffffffu, seen)) {
            report_timeout(p, abort_flag, 10, i);
            return false;
          }
          m_ref = s_mrow[r];
        }
        m_new = m_ref;
      } else {
      const float mx = row_max();
      // The running maximum of the row passes between the two threads that share it through shared
      // memory: step i reads what step i-1 (the other warp set) published.
      float m_old = -INFINITY;
      if (i > 0) {
        bool seen = ld_acquire_shared(s_mstep + qd) >= i;
        if (!seen) {
          const long long t0 = clock64();
          while (!(seen = ld_acquire_shared(s_mstep + qd) >= i)) {
            if (*abort_flag || clock64() - t0 > WAIT_LIMIT) break;
          }
        }
        if (!__all_sync(0xffffffffu, seen)) {
          report_timeout(p, abort_flag, 10, i);
          return false;
        }
        m_old = s_mrow[r];
      }
      m_new = m_old;
      bool resc = false;
      if (mx > m_old + RESCALE_TAU) {   // lazy: the maximum only moves when it grows by more than 2^tau
        m_new = mx;
        resc = m_old > -INFINITY;
      }
      s_mrow[r] = m_new;
      __syncwarp();
      st_release_shared_if(s_mstep + qd, i + 1, lane == 0);
      if (m_new != m_l) {
        l *= ex2_approx(m_l - m_new);     // 0 when m_l = -inf
        m_l = m_new;
      }
      if (__any_sync(0xffffffffu, resc)) {  // O may only be touched once this half's previous P.V has landed
        pv_consumed = true;
        if (!wait_bar(my_pvdone + 8u * ((i - 1) & 3), (i - 1) >> 2, 7, i)) return false;
        const float alpha = resc ? ex2_approx(m_old - m_new) : 1.f;
        // (rare, and deliberately not unrolled: unrolled, this loop costs the hot path 19 spilled registers)
#pragma unroll 1
        for (int c = 0; c < D / 16; ++c) {  // the thread whose step moved the maximum rescales the whole row
          uint32_t o[16];
          const uint32_t addr = tO + lane_off + (uint32_t)(16 * c);
          tmem_ld16(addr, o);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 16; ++j) o[j] = __float_as_uint(__uint_as_float(o[j]) * alpha);
          tmem_st16(addr, o);
        }
        tmem_wait_st();
      }
      }   // exact walk
      const float xoff = fmaf(-SCORE_BIAS, sc, -m_new);   // (bias + s) * sc + xoff = s * sc - m
      const uint64_t sc2 = pack2(sc, sc), negm2 = pack2(xoff, xoff);
      uint64_t sum2[2] = {0ull, 0ull};
      uint32_t pk[32];   // bf16 P: two values per 32-bit column
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        float x0, x1;
        unpack2(fma2(pack2(f[2 * j], f[2 * j + 1]), sc2, negm2), x0, x1);
        const float p0 = ex2_approx(x0), p1 = ex2_approx(x1);   // 2^-inf = 0 for masked columns
        sum2[j & 1] = add2(sum2[j & 1], pack2(p0, p1));
        pk[j] = pack_bf16x2(p0, p1);
      }
      // P of this half is rewritten only after the P.V that read its previous contents (the other warp
      // set's step) has finished.  All of the step's arithmetic is done by now: between that P.V's
      // completion and this step's P being ready for the issuer lie one store and one arrival.
      TR(trole, i, 3);
      if (!pv_consumed && !wait_bar(my_pvdone + 8u * ((i - 1) & 3), (i - 1) >> 2, 7, i)) return false;
      TR(trole, i, 4);
      tmem_st32(tP + lane_off, pk);
      float sa, sb;
      unpack2(add2(sum2[0], sum2[1]), sa, sb);
      if constexpr (FIXED) redo = redo || !(sa + sb < ROWSUM_LIMIT);   // out of range, or NaN
      l += sa + sb;
      // Fixed-reference walk: the columns past the end of the sequence were not masked.  Their K rows
      // arrive as zeros, so each of them scored exactly 0 and contributed the same P to the sum, which
      // is taken out here; in P.V they meet the zero padding of V.
      if (FIXED && valid < 64) l -= (float)(64 - valid) * ex2_approx(fmaf(SCORE_BIAS, sc, xoff));
      tmem_wait_st();
      tc_fence_before();
      __syncwarp();
      mbar_arrive_if(my_pready, lane == 0);   // one arrival per warp
      TR(trole, i, 5);
      return true;
    };
    if constexpr (FIXED) {
      if (set < n_mine) ok = do_step(set, std::true_type{});
      for (int i = set + 2; ok && i < n_mine; i += 2) ok = do_step(i, std::false_type{});
    } else {
      for (int i = set; ok && i < n_mine; i += 2) ok = do_step(i, std::false_type{});
    }

    // epilogue (the TMEM loads are warp-collective: every lane of the warp executes them, rows past
    // the end of the sequence only skip the store)
    if (ok && n_mine > 0) ok = wait_bar(my_pvdone + 8u * ((n_mine - 1) & 3), (n_mine - 1) >> 2, 8, n_mine);
    // final maximum and row sum = both threads' shares (reached by every softmax thread, also
    // after a failed wait)
    if (FIXED && redo) *s_redo = 1;
    named_barrier(1, ATT_SOFTMAX_THREADS);
    const float m = n_mine > 0 ? s_mrow[r] : -INFINITY;
    if (!FIXED && m_l != m) l *= ex2_approx(m_l - m);
    s_xl[set * 128 + r] = l;
    named_barrier(1, ATT_SOFTMAX_THREADS);
    l += s_xl[(set ^ 1) * 128 + r];
    ok = ok && !*abort_flag;
    const bool give_back = FIXED && *s_redo != 0;
    if (ok && give_back && threadIdx.x == 0) {
      const int slot = atomicAdd(p.redo, 1);
      p.redo[REDO_HEADER + slot] = item;
    }
    if (ok && !give_back) {
      const int b = bh / p.H, h = bh % p.H;
      const bool live = tok < p.N;
      int dst = tok;
      if (live && p.inv_idx && tok >= p.n_text)
        dst = p.n_text + p.inv_idx[(size_t)h * (p.N - p.n_text) + (tok - p.n_text)];
      OutT* orow = static_cast<OutT*>(p.out) + b * p.osb + h * p.osh + (int64_t)dst * p.osn + set * (D / 2);
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        uint32_t o[32];
        if (n_mine > 0) {
          tmem_ld32(tO + lane_off + (uint32_t)(set * (D / 2) + 32 * c), o);
          tmem_wait_ld();
        } else {
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = 0u;
        }
        uint32_t w[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int d0 = set * (D / 2) + 32 * c + 2 * j;
          const float a0f = l > 0.f ? fmaf(__uint_as_float(o[2 * j]) * inv_l, s_vscale[d0], s_vm[d0]) : 0.f;
          const float a1f = l > 0.f ? fmaf(__uint_as_float(o[2 * j + 1]) * inv_l, s_vscale[d0 + 1], s_vm[d0 + 1]) : 0.f;
          OutT t2[2] = {F16Traits<OutT>::from_float(a0f), F16Traits<OutT>::from_float(a1f)};
          w[j] = *reinterpret_cast<const uint32_t*>(t2);
        }
        if (live) {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            *reinterpret_cast<uint4*>(orow + 32 * c + 8 * j) = make_uint4(w[4 * j], w[4 * j + 1], w[4 * j + 2], w[4 * j + 3]);
        }
      }
      if (live && set == 0 && p.lse)
        p.lse[(size_t)bh * p.N + dst] = l > 0.f ? (log2f(l) + m) * 0.6931471805599453f : -INFINITY;
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 10) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

// ---------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// 3-D tensor map over a tensor [d2][d1][d0] of `esize`-byte elements, box [1][box1][box0].
static int make_tensor_map(CUtensorMap* map, CUtensorMapDataType dt, int esize, const void* base, uint64_t d0, uint64_t d1,
                    uint64_t d2, uint32_t box0, uint32_t box1, CUtensorMapSwizzle swz) {
  EncodeTiledFn fn = encode_fn();
  PARO_REQUIRE(fn != nullptr, PARO_ECUDA, "cuTensorMapEncodeTiled is not available from this driver");
  cuuint64_t dims[3] = {d0, d1, d2};
  cuuint64_t strides[2] = {d0 * esize, d0 * d1 * esize};
  cuuint32_t box[3] = {box0, box1, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult rc = fn(map, dt, 3, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  PARO_REQUIRE(rc == CUDA_SUCCESS, PARO_ECUDA, "cuTensorMapEncodeTiled failed with code %d", (int)rc);
  return PARO_OK;
}

template <int D, typename OutT, bool FIXED>
static int launch_walk(const int8_t* k8, const uint16_t* v16, const AttnParams& p, unsigned ctas, cudaStream_t s) {
  using Cfg = AttnCfg<D>;
  const uint64_t BH = (uint64_t)p.B * p.H;
  const uint64_t npad = (uint64_t)p.nb * 64;
  const CUtensorMapSwizzle swz_qk = D == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B;
  CUtensorMap tk, tv;
  if (int rc = make_tensor_map(&tk, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, k8, D, p.N, BH, D, 64, swz_qk)) return rc;
  if (int rc = make_tensor_map(&tv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, v16, npad, D, BH, 64, D, CU_TENSOR_MAP_SWIZZLE_128B))
    return rc;
  auto kern = sparse_attn_kernel<D, OutT, FIXED>;
  PARO_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM_BYTES));
  // shared memory for two CTAs per SM and no more: the rest of the 256 KB serves as L1
  constexpr int carveout_pct = (2 * (Cfg::SMEM_BYTES + 1024) * 100 + 228 * 1024 - 1) / (228 * 1024);
  PARO_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, carveout_pct < 100 ? carveout_pct : 100));
  kern<<<ctas, ATT_THREADS, Cfg::SMEM_BYTES, s>>>(tk, tv, p);
  return check_launch("sparse_attn_kernel");
}

static int launch_attn_exact(const int8_t* k8, const uint16_t* v16, const AttnParams& p, int D, int out_dtype, unsigned ctas,
                      cudaStream_t s) {
  if (D == 128)
    return out_dtype == PARO_F16 ? launch_walk<128, __half, false>(k8, v16, p, ctas, s)
                                 : launch_walk<128, __nv_bfloat16, false>(k8, v16, p, ctas, s);
  return out_dtype == PARO_F16 ? launch_walk<64, __half, false>(k8, v16, p, ctas, s)
                               : launch_walk<64, __nv_bfloat16, false>(k8, v16, p, ctas, s);
}

static int launch_attn_fixed(const int8_t* k8, const uint16_t* v16, const AttnParams& p, int D, int out_dtype, unsigned ctas,
                      cudaStream_t s) {
  if (D == 128)
    return out_dtype == PARO_F16 ? launch_walk<128, __half, true>(k8, v16, p, ctas, s)
                                 : launch_walk<128, __nv_bfloat16, true>(k8, v16, p, ctas, s);
  return out_dtype == PARO_F16 ? launch_walk<64, __half, true>(k8, v16, p, ctas, s)
                               : launch_walk<64, __nv_bfloat16, true>(k8, v16, p, ctas, s);
}

}  // namespace paro

using namespace paro;

extern "C" size_t paro_sparse_attn_redo_bytes(int B, int H, int N) {
  if (B <= 0 || H <= 0 || N <= 0) return 0;
  const size_t nb = ((size_t)N + 63) / 64;
  return sizeof(int32_t) * (REDO_HEADER + (size_t)B * H * ((nb + 1) / 2));
}

extern "C" int paro_sparse_attn(const int8_t* q8, const int8_t* k8, const uint16_t* v16,
                                const float* q_scale, int q_group, const float* k_scale,
                                const float* v_scale, const float* vm,
                                const int32_t* pair_ptr, const uint32_t* sched, const int32_t* sched_cnt,
                                int plan_slices,
                                const int32_t* inv_idx, int n_text,
                                void* out, int out_dtype,
                                int64_t out_stride_b, int64_t out_stride_h, int64_t out_stride_n,
                                float* lse, int B, int H, int N, int D, float sm_scale, int mode,
                                int32_t* redo, size_t redo_bytes,
                                int32_t* status, paro_stream_t stream) {
  PARO_REQUIRE(q8 && k8 && v16 && q_scale && k_scale && v_scale && pair_ptr && sched && sched_cnt && out && status, PARO_EINVAL,
               "paro_sparse_attn: null pointer");
  PARO_REQUIRE(B > 0 && H > 0 && N > 0, PARO_ESHAPE, "paro_sparse_attn: empty problem");
  PARO_REQUIRE(D == 64 || D == 128, PARO_ESHAPE, "paro_sparse_attn: head_dim %d unsupported (64 or 128)", D);
  PARO_REQUIRE(q_group == 32 || q_group == 64, PARO_EINVAL, "paro_sparse_attn: q_group must be 32 or 64");
  PARO_REQUIRE(out_dtype == PARO_F16 || out_dtype == PARO_BF16, PARO_EINVAL, "paro_sparse_attn: bad out_dtype");
  PARO_REQUIRE(plan_slices == H || plan_slices == B * H, PARO_ESHAPE,
               "paro_sparse_attn: plan_slices must be H or B*H (got %d)", plan_slices);
  PARO_REQUIRE(n_text >= 0 && n_text <= N, PARO_ESHAPE, "paro_sparse_attn: n_text out of range");
  PARO_REQUIRE(aligned16(q8) && aligned16(k8) && aligned16(v16) && aligned16(out), PARO_EALIGN,
               "paro_sparse_attn: q8/k8/v16/out must be 16-byte aligned");
  PARO_REQUIRE(out_stride_b % 8 == 0 && out_stride_h % 8 == 0 && out_stride_n % 8 == 0 && out_stride_n >= D,
               PARO_EALIGN, "paro_sparse_attn: output strides must be multiples of 8 elements");
  PARO_REQUIRE(sm_scale > 0.f, PARO_EINVAL, "paro_sparse_attn: sm_scale must be positive");
  PARO_REQUIRE(mode == PARO_ATTN_FAST || mode == PARO_ATTN_EXACT, PARO_EINVAL, "paro_sparse_attn: unknown mode %d", mode);
  PARO_REQUIRE(mode == PARO_ATTN_EXACT || (redo && redo_bytes >= paro_sparse_attn_redo_bytes(B, H, N)), PARO_ECAP,
               "paro_sparse_attn: PARO_ATTN_FAST needs a redo work space of paro_sparse_attn_redo_bytes() bytes");
  AttnParams p;
  p.q8 = q8; p.q_scale = q_scale; p.k_scale = k_scale; p.v_scale = v_scale; p.vm = vm;
  p.pair_ptr = pair_ptr; p.sched = sched; p.sched_cnt = sched_cnt; p.inv_idx = inv_idx;
  p.out = out; p.lse = lse; p.status = status; p.redo = redo;
  p.osb = out_stride_b; p.osh = out_stride_h; p.osn = out_stride_n;
  p.plan_slices = plan_slices; p.q_group = q_group; p.n_text = n_text;
  p.B = B; p.H = H; p.N = N; p.nb = (N + 63) / 64; p.npairs = (p.nb + 1) / 2;
  p.from_list = 0;
  p.scale_log2 = sm_scale * 1.44269504f;
  cudaStream_t s = (cudaStream_t)stream;
  const uint64_t ctas = (uint64_t)B * H * p.npairs;
  PARO_REQUIRE(ctas < (1ull << 31), PARO_ESHAPE, "paro_sparse_attn: too many work items");
  if (mode == PARO_ATTN_EXACT) return launch_attn_exact(k8, v16, p, D, out_dtype, (unsigned)ctas, s);
  // fixed-reference walk over every work item, then the exact walk over the items it gave back (usually none:
  // the second launch's CTAs then leave at once)
  PARO_CUDA_OK(cudaMemsetAsync(redo, 0, sizeof(int32_t) * REDO_HEADER, s));
  if (int rc = launch_attn_fixed(k8, v16, p, D, out_dtype, (unsigned)ctas, s)) return rc;
  p.from_list = 1;
  return launch_attn_exact(k8, v16, p, D, out_dtype, (unsigned)ctas, s);
}


extern "C" int paro_status_poll(const int32_t* status, int32_t* host_out, paro_stream_t stream) {
  PARO_REQUIRE(status, PARO_EINVAL, "paro_status_poll: null pointer");
  int32_t w[4] = {0, 0, 0, 0};
  PARO_CUDA_OK(cudaMemcpyAsync(w, status, sizeof(w), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
  PARO_CUDA_OK(cudaStreamSynchronize((cudaStream_t)stream));
  if (host_out)
    for (int i = 0; i < 4; ++i) host_out[i] = w[i];
  if (w[0] != 0)
    return fail(PARO_ETIMEOUT, "sparse attention wait expired: role %d, work item %d, tile %d", w[1], w[2], w[3]);
  return PARO_OK;
}

#ifdef PARO_TRACE
// Copies the trace table to the host and clears it on the device (synchronises).
extern "C" int paro_debug_trace(long long* host_out) {
  void* dev = nullptr;
  if (cudaMemcpyFromSymbol(host_out, paro::g_trace, sizeof(paro::g_trace)) != cudaSuccess) return -1;
  if (cudaGetSymbolAddress(&dev, paro::g_trace) != cudaSuccess) return -1;
  return cudaMemset(dev, 0, sizeof(paro::g_trace)) == cudaSuccess ? 0 : -1;
}
#endif
