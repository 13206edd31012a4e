// Persistent tcgen05 recurrence kernels for 16-bit LSTM layers.
//
// Forward (replaces persistent_fwd_kernel, fastlstm/kernels.py:414-663):
//   CTA (pb, ht) owns UH hidden units (their 4 gate rows of Wh: N = 4*UH rows, all
//   K = H columns) and keeps that slice RESIDENT in shared memory for the whole
//   sequence.  Per (timestep, batch tile of 128 rows) it computes
//       D[128, N] = h[t][tile rows, :] (TMA-streamed, K-major)  x  Wh_slice^T
//   with tcgen05.mma into a TMEM accumulator, then the epilogue warps add the
//   projected pre-activations, write the final pre-activations back (saved for
//   backward), apply the gates with c carried in fp32 registers, and publish
//   h[t+1] / c[t+1].  h is exchanged between the CTAs of a batch tile through
//   global memory (L2): one arrival counter per (timestep, batch tile), released
//   by the epilogue warps (or, with interleaved tiles, by a publisher warp on their
//   behalf) and acquired (bounded spin) by the TMA producer of each CTA before it
//   streams h[t+1].  Each CTA interleaves up to four independent batch tiles so the
//   hand-off latency of one hides behind the work of the others.
//
//   warp 0        TMA producer (flag wait, h tiles, Wh slice once)
//   warps 1..NACC tcgen05.mma issuers (each owns whole K chunks and its own TMEM
//                 accumulator; warp 1 owns the TMEM allocation)
//   next warp     publisher (interleaved tiles only): proxy fence + release per item
//   last 4 or 8   epilogue: thread = batch row x 8 or 16 hidden units x 4 gates
#include <stdio.h>
#include <algorithm>
#include <atomic>
#include <stdlib.h>

#include "generic.cuh"
#include "sm100.cuh"
#include "sm100_common.cuh"
#include "sm100_rec_util.cuh"

namespace blstm {
namespace sm100 {

constexpr int RB = 128;                 // batch rows per tile (MMA M)
constexpr int RK = 64;                  // K chunk (one 128-byte swizzle row)
constexpr int R_MAX_STAGES = 16;
constexpr int R_STAGE_BYTES = RB * RK * 2;   // 16 KB: what an M = 128 MMA reads of a stage's activation rows

// Ring depth R and number of concurrent TMA-issuing lanes / MMA-issuing warps NI.  Every stage
// barrier must always be waited on by the SAME thread of each role (a parity wait cannot tell
// phase n from phase n+2, so two threads sharing a barrier could lap each other): stage s belongs
// to lane / issuer s % NI, which needs NI | R.  NI is also capped by the TMEM accumulators
// available (max_ni) and by the chunks per item (an issuer without work would leave a stale
// accumulator).
static bool pick_ring(size_t fixed_bytes, size_t stage_bytes, int max_ni, int kc, int* stages, int* ni) {
  // Prefer many concurrent issuers, but only count them fully when the ring holds two rounds of
  // their chunks (R >= 2 NI): with R == NI the loads of one round cannot overlap the MMAs of the
  // previous one.
  const int cand[7] = {16, 12, 8, 6, 4, 3, 2};
  int best_r = 0, best_n = 0, best_score = -1;
  for (int i = 0; i < 7; ++i) {
    const int r = cand[i];
    if (fixed_bytes + (size_t)r * stage_bytes > 232448) continue;
    for (int n = 4; n >= 1; --n) {
      if (n > max_ni || n > kc || r % n != 0) continue;
      const int score = (r >= 2 * n) ? 2 * n : n;
      if (score > best_score) { best_score = score; best_r = r; best_n = n; }
    }
  }
  if (!best_r) return false;
  *stages = best_r;
  *ni = best_n;
  return true;
}

struct RecPlan {
  bool ok;
  int UH, N, nh, nbt, nb_par, ntl, TI, grid, epi_warps, threads, stages, ni, nl, ws;
  int npb;                  // interleaved tiles: TMA landing buffers per epilogue warp (1 or 2), else 0
  int kr;                   // K chunks of the Wh slice that stay resident (all of them unless ws)
  int hb;                   // bytes of the h rows in a ring stage: 128 rows, or a single smaller tile's own rows
  size_t w_bytes, stage_bytes, smem, ep_bytes;
  size_t off_flags, n_flags, ws_bytes;
};

// Geometry follows the SM count of the current device (a B200 with all 148 SMs when no device can
// be queried, e.g. when only a workspace size is asked for on a host without a GPU); the
// cooperative launch refuses if the device cannot hold the grid.
static RecPlan make_plan(const blstm_desc& d, int phase) {
  RecPlan p{};
  p.ok = false;
  if (d.flags & BLSTM_FLAG_FORCE_GENERIC) return p;
  if (phase != BLSTM_PHASE_FWD) return p;
  if (d.dtype != BLSTM_F16 && d.dtype != BLSTM_BF16) return p;
  const int H = d.hidden_size, B = d.batch;
  if (H % 64 != 0 || H < 64 || H > 2048) return p;
  p.nbt = cdiv(B, RB);
  int UH = 16;
  // Wider slices when they fill the GPU AND leave every CTA two or more tiles to interleave (a single
  // tile of 32 units per CTA is latency bound and measured slower than two interleaved tiles of 16:
  // 2.12 against 1.87 ms at B=1024, H=512, T=256).
  const int sm_share = (d.flags & BLSTM_FLAG_HALF_DEVICE) ? 2 : 1;   // half the device: two kernels side by side
  if (H <= 512 && p.nbt * (H / 32) >= 74) {
    const int sms32 = plan_sm_count() / sm_share;
    int par32 = sms32 / (H / 32);
    if (par32 > p.nbt) par32 = p.nbt;
    if (par32 > 0 && cdiv(p.nbt, par32) >= 2) UH = 32;
  }
  p.UH = UH;
  p.N = 4 * UH;
  p.nh = H / UH;
  const int sms = plan_sm_count() / sm_share;
  if (p.nh > sms) return p;
  p.nb_par = sms / p.nh;
  if (p.nb_par > p.nbt) p.nb_par = p.nbt;
  p.ntl = cdiv(p.nbt, p.nb_par);
  p.TI = p.ntl >= 3 ? 4 : p.ntl >= 2 ? 2 : 1;     // batch tiles interleaved per CTA (state: cell rows in registers)
  p.grid = p.nh * p.nb_par;
  p.epi_warps = (UH == 16 && p.TI == 1) ? 4 : 8;
  // a single 16-unit tile in flight is latency bound: four issuers next to one epilogue warpgroup
  // (9 warps); otherwise two issuers, eight epilogue warps and, for interleaved tiles, the publisher
  // (interleaved 32-unit slices: N = 128 runs the tensor pipe at full rate from ONE issuing thread, and a
  // single accumulator per item leaves tensor-memory columns for the cell rows of four tiles)
  const int n_issuers = (UH == 16 && p.TI == 1) ? 4 : (UH == 32 && p.TI >= 2) ? 1 : 2;
  const int n_publisher = p.TI >= 2 ? 1 : 0;
  p.threads = 32 * (1 + n_issuers + n_publisher + p.epi_warps);   // producer + MMA issuers [+ publisher] + epilogue
  // Wh slice resident in shared memory when it fits next to a useful ring; otherwise (H > 1024) it is
  // streamed through the ring with h, chunk by chunk, every step (it stays in L2).  A single batch tile
  // of fewer than 128 rows only stages its own rows (the MMA's rows past them read whatever follows:
  // accumulator rows nobody uses), which makes room for up to 16 stages.
  p.w_bytes = (size_t)p.N * H * 2;
  p.ws = p.w_bytes > 128 * 1024 ? 1 : 0;
  p.hb = (p.nbt == 1 ? (int)round_up((size_t)B, 8) : RB) * 128;
  const size_t w_chunk = (size_t)p.N * 128;
  p.stage_bytes = p.hb + (p.ws ? w_chunk : 0);
  // (a stage that holds fewer than 128 rows is still READ as 128 rows by the MMA: the ring is followed by
  //  enough shared memory for the last stage's read to stay inside the allocation)
  const size_t tail_pad = p.stage_bytes < (size_t)R_STAGE_BYTES ? R_STAGE_BYTES - p.stage_bytes : 0;
  // Streamed means ALL of it: keeping 18 of H=2048's 32 chunks resident (6-stage ring) measured 10.2 ms
  // against 8.1 ms with none resident and a 16-stage ring - the depth of the ring is worth more than
  // the bytes saved.  (The kernel handles any split; `kr` chunks are resident.)
  p.kr = p.ws ? 0 : H / RK;
  // Interleaved tiles: the epilogue's gate traffic goes through TMA.  Every epilogue warp owns
  // landing buffers for its 32 rows' projected pre-activations (4 gates x NU units; the final
  // pre-activations are written back in place and leave from there).
  // Two landing buffers per warp (the next item's box is fetched a whole item ahead) when the ring
  // still gets four stages, else one.
  p.npb = 0;
  p.ep_bytes = 0;
  size_t fixed = 1024 + (size_t)p.kr * w_chunk + 512 + tail_pad;
  if (p.TI >= 2) {
    const int NU = 4 * UH / p.epi_warps;
    const size_t pb = 256 * (size_t)NU;
    p.npb = (fixed + p.epi_warps * 2 * pb + 4 * p.stage_bytes <= 232448) ? 2 : 1;
    p.ep_bytes = p.epi_warps * p.npb * pb;
    fixed += p.ep_bytes;
  }
  if (!pick_ring(fixed, p.stage_bytes, n_issuers, H / RK, &p.stages, &p.ni)) return p;
  // TMA-issuing lanes of the producer warp (they split the ring's stages; nl | stages).  As many as
  // issuers by default; measured exceptions (3-4 % each): two interleaved tiles do better with more lanes
  // (B=2048: 2.55 -> 2.46 ms, B=1024: 1.89 -> 1.78 ms), a single tile on a six-stage ring with fewer
  // (H=1024: 3.89 -> 3.75 ms).
  p.nl = p.ni;
  if (p.TI == 2) p.nl = UH == 32 ? 2 : 4;
  if (p.TI == 1 && p.stages == 6) p.nl = 2;
  if (p.stages % p.nl != 0 || p.nl > H / RK) p.nl = p.ni;
  p.smem = fixed + (size_t)p.stages * p.stage_bytes;
  p.n_flags = (size_t)(d.seq_len + 1) * p.nbt;
  p.off_flags = sizeof(Control);
  p.ws_bytes = p.off_flags + round_up(p.n_flags * sizeof(int), 256);
  p.ok = true;
  return p;
}

struct FwdParams {
  int T, B, H;
  int nbt, nh, nb_par, ntl;
  int stages;
  int ni;                   // MMA-issuing warps in use
  int nl;                   // TMA-issuing lanes of the producer warp (nl divides the ring depth)
  int ws;                   // 1: part of the Wh slice streamed through the ring instead of resident
  int kr;                   // resident K chunks of the Wh slice
  int hb;                   // bytes of the h rows in a ring stage
  int stage_bytes;
  int fmt;
  int no_arrive;
  int inference;            // skip the stores that only backward needs
  int flag_target;          // arrivals that complete a flag: nh CTAs per batch tile [x epilogue warps]
  int cta_publish;          // 1: one arrival per CTA and item, 0: one per epilogue warp
  int npb;                  // TMA landing buffers per epilogue warp (interleaved tiles)
  int ep_bytes;             // bytes of the epilogue's TMA buffers (between the weights and the ring)
  unsigned long long limit_ns;
  Control* ctl;
  int* flags;
  void* ifgo;               // [T,B,4H] in/out
  void* out;                // [T+1,B,H]
  void* cell;               // [T+1,B,H]
};

// Position in a CTA's sequence of work items, which every role walks in the same order:
//   for chunk (TI tiles) : for step in [0, steps) : for j in [0, TI) : tile pb + (chunk*TI + j)*nb_par
// (tiles past the last one are skipped).  next() moves to the following existing item.
template <int TI>
struct ItemCursor {
  int ch, t, j;
  __device__ __forceinline__ void init() { ch = 0; t = 0; j = -1; }
  __device__ __forceinline__ bool next(int pb, int nb_par, int nbt, int n_chunks, int steps) {
    for (;;) {
      if (++j == TI) { j = 0; if (++t == steps) { t = 0; ++ch; } }
      if (ch >= n_chunks) return false;
      if (pb + (ch * TI + j) * nb_par < nbt) return true;
    }
  }
  __device__ __forceinline__ int tile(int pb, int nb_par) const { return pb + (ch * TI + j) * nb_par; }
};

// UH: hidden units per CTA (16 or 32).  TI: batch tiles interleaved per CTA (1, 2 or 4).
// Warps: 1 TMA producer, NACC MMA issuers, with interleaved tiles one publisher warp, 4 or 8 epilogue
// warps - at most 12 (3 per SM sub-partition), which leaves 168 registers per thread; a 13th would cap
// them at 128.  The epilogue must not spill.
template <int UH, int TI, typename T16>
__global__ void __launch_bounds__(32 * (UH == 16 && TI == 1 ? 9 : (TI >= 2 ? (UH == 32 ? 11 : 12) : 11)), 1)
fwd_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmH,
           const __grid_constant__ CUtensorMap tmP, const FwdParams p) {
  constexpr int N = 4 * UH;
  // Interleaved tiles are throughput bound, and there the epilogue's row-strided 16-byte global
  // accesses (a thread owns a batch row: 32 sectors per warp instruction) were the bottleneck: the
  // projected pre-activations come in as TMA boxes through shared memory, one set of buffers per
  // epilogue warp (tmP: ifgo as {unit, row, gate, step}), and the final pre-activations go out from
  // the same buffers (16 units per thread: coalesced plain stores; 8 units: a TMA box): eight of the
  // twelve 16-byte accesses a thread makes per 8 units.  h keeps its direct stores (they are what
  // the step hand-off orders) and so do the cell rows (a buffer for them would cost a ring stage).
  constexpr bool TMAEP = (TI >= 2);
  // Epilogue warps.  A single tile of 16 units is latency bound and runs best as one warpgroup with
  // 16 units per thread next to four issuers (9 warps); every other shape uses two warpgroups that
  // split the CTA's units (8 or 16 per thread), which keeps interleaved tiles free of spills.
  constexpr int EW = (UH == 16 && TI == 1) ? 4 : 8;
  constexpr int NU = 4 * UH / EW;                   // units per epilogue thread
  constexpr int NV = NU / 8;                        // 16-byte pieces per operand per thread
  // Which side runs the generic->async proxy fence of the hand-off.  One tile in flight: the READER, after
  // it has seen the counter (traced: the writers' release then waits for their h stores alone, 1.5 k clk
  // instead of fence 1.8 k + release 1.5 k, against 0.8 k for the fence on the reading side).  Interleaved
  // tiles: the writers' publisher warp.
  constexpr bool WRITER_FENCE = false;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int H = p.H;
  const int KC = H / RK;                            // K chunks
  uint8_t* w_s = smem;                              // [KC][N rows][128 B]
  const int R_STAGES = p.stages;
  const int SB = p.stage_bytes;                     // h chunk (16 KB) [+ Wh chunk when streamed]
  uint8_t* ep_s = smem + (size_t)p.kr * N * 128;          // epilogue TMA buffers (interleaved tiles)
  const int HB = p.hb;                                    // h rows of a stage; a streamed Wh chunk follows them
  uint8_t* a_s = ep_s + p.ep_bytes;                       // [stages][h chunk | optional Wh chunk]
  uint64_t* bars = reinterpret_cast<uint64_t*>(a_s + (size_t)R_STAGES * SB);
  uint64_t* full = bars;                            // [R_MAX_STAGES]
  uint64_t* empty = bars + R_MAX_STAGES;            // [R_MAX_STAGES]
  uint64_t* acc_full = bars + 2 * R_MAX_STAGES;     // [2]
  uint64_t* acc_empty = acc_full + 2;               // [2]
  uint64_t* w_full = acc_empty + 2;                 // [1]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(w_full + 1);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* pub_cnt = const_cast<int*>(dead) + 1;        // [4] arrivals of the epilogue warps, by item index mod 4
  uint64_t* pub_bar = reinterpret_cast<uint64_t*>(pub_cnt + 4);   // [4] item stored? by item index mod 4
  uint64_t* pre_full = pub_bar + 4;                 // [8 epilogue warps][2] landing buffer filled

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ht = blockIdx.x % p.nh, pb = blockIdx.x / p.nh;
  // One thread can issue a tcgen05.mma only every ~150 clocks whatever its shape, far below
  // what these small-N shapes need, so NACC warps issue concurrently: warp x takes the x-th
  // K=16 slice(s) of every chunk into its own TMEM accumulator, and the epilogue adds them up.
  // With interleaved tiles the epilogue warps are the bottleneck and the release that publishes an item
  // stalls its thread for a memory round trip, so a PUBLISHER warp does the releasing (and the proxy
  // fence of the hand-off): the epilogue warps only arrive on a CTA-local barrier after storing h.
  constexpr bool PUBLISHER = (TI >= 2);
  constexpr int NACC = (UH == 16 && TI == 1) ? 4 : (UH == 32 && TI >= 2) ? 1 : 2;   // issuer warps / partial accumulators
  constexpr int FIRST_EPI = 1 + NACC + (PUBLISHER ? 1 : 0);   // first epilogue warp
  // Columns per item buffer (NACC * N <= 256).  Interleaved tiles pack the two buffers into the first
  // 256 columns and keep the tiles' cell rows (fp32, a column per unit) in the columns behind them.
  constexpr int ACC_STRIDE = (TI >= 2) ? NACC * N : 256;
  constexpr int C_BASE = 2 * ACC_STRIDE;
  static_assert(TI == 1 || C_BASE + TI * UH <= 512, "cell rows do not fit the tensor memory");
  constexpr uint32_t TMEM_COLS = 512;
  const int nacc = p.ni;                             // accumulators / issuers / TMA lanes in use

  if (threadIdx.x == 0) {
    // full[s] is armed (arrive + expected bytes) for its first use here and re-armed by the MMA issuer
    // that consumed it for every later use, which keeps that work out of the latency-bound TMA producer loop
    for (int s = 0; s < R_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], nacc); mbar_init(&acc_empty[a], EW); }
    mbar_init(w_full, 1);
    *dead = 0;
    for (int i = 0; i < 4; ++i) pub_cnt[i] = 0;
    for (int i = 0; i < 4; ++i) mbar_init(&pub_bar[i], EW);
    for (int i = 0; i < 16; ++i) mbar_init(&pre_full[i], 1);
    fence_mbar_init();
    // (stage s is first used by chunk s; with streamed weights there are more chunks than stages)
    for (int s = 0; s < R_STAGES; ++s) mbar_expect_tx(&full[s], (p.ws && s % KC >= p.kr) ? SB : HB);
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmH);
    if (TMAEP) tma_prefetch_desc(&tmP);
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  WaitCtx wc{dead, p.ctl, p.limit_ns, -1, (int)blockIdx.x};

  // Work items of this CTA, in the order every role walks them:
  //   for chunk (TI tiles) : for t in [0,T) : for j in [0,TI) : (t, bt = pb + (chunk*TI + j) * nb_par)
  const int n_chunks = (p.ntl + TI - 1) / TI;

  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    // One thread needs a few hundred clocks per cp.async.bulk.tensor issue, so p.ni lanes issue in
    // lockstep, each owning the ring stages congruent to its lane index.
    if (lane == 0 && p.kr > 0) {
      // resident part of the Wh slice: rows (gate g, unit ht*UH + u), K chunks [0, kr) of [N][64]
      mbar_expect_tx(w_full, (uint32_t)((size_t)p.kr * N * 128));
      for (int kc = 0; kc < p.kr; ++kc) tma_load_3d(w_s + (size_t)kc * N * 128, &tmW, w_full, kc * RK, ht * UH, 0);
    }
    int gs = 0;                // ring position of the current item's chunk 0
    uint32_t gph = 0;
    bool ok = true;
    // With interleaved tiles an item's arrival counter is usually complete long before its turn, and
    // what costs is the round trip of looking: lane 31 reads the NEXT item's counter while the other
    // lanes issue the current item's loads, and lane 0 only spins when that early look found it incomplete.
    ItemCursor<TI> nx;
    nx.init();
    bool nx_valid = nx.next(pb, p.nb_par, p.nbt, n_chunks, p.T);   // the first item itself
    int early = 0;             // lane 31: early reading of the next item's counter
    for (int ch = 0; ch < n_chunks && ok; ++ch) {
      for (int t = 0; t < p.T && ok; ++t) {
        for (int j = 0; j < TI && ok; ++j) {
          const int bt = pb + (ch * TI + j) * p.nb_par;
          if (bt >= p.nbt) continue;
          // what lane 31 read for this item while the previous item's loads were being issued
          const int early_now = (TI >= 2) ? __shfl_sync(0xffffffffu, early, 31) : 0;
          if (TI >= 2) nx_valid = nx_valid && nx.next(pb, p.nb_par, p.nbt, n_chunks, p.T);
          bool lane_ok = true;
          // One tile in flight: the wait for each issuing lane's first ring stage (half a thousand clocks
          // even when the stage is long free) is taken BEFORE the counter, off the step's chain.
          const int nl = p.nl;                 // TMA-issuing lanes: lane l owns the ring stages == l (mod nl)
          const int kc_first = (lane + nl - gs % nl) % nl;
          if (TI == 1 && lane < nl && kc_first < KC) {
            int s = gs + kc_first;
            uint32_t ph = gph;
            while (s >= R_STAGES) { s -= R_STAGES; ph ^= 1; }
            lane_ok = mbar_wait(&empty[s], ph ^ 1, wc);
          }
          if (t > 0) {   // h[t] of this batch tile complete: every epilogue warp of every hidden tile arrived
            int seen = 1;
            if (lane == 0 && !(TI >= 2 && early_now >= p.flag_target)) {
              wc.d0 = t; wc.d1 = bt;
              seen = wait_flag_ge(&p.flags[(size_t)t * p.nbt + bt], p.flag_target, p.ctl, p.limit_ns, t, bt) ? 1 : 0;
            }
            seen = __shfl_sync(0xffffffffu, seen, 0);
            if (!seen) { *dead = 1; ok = false; break; }
            // One proxy fence must lie between the peers' generic-proxy stores and this warp's TMA
            // reads: here for a single tile in flight, in the writers' publisher warp otherwise (this
            // loop then streams h without a break).
            if (!WRITER_FENCE && !PUBLISHER) fence_proxy_async();
          }
          const int row0 = bt * RB;
          if (lane < nl && lane_ok) {
            // this lane owns ring stages == lane (mod nl): the item's chunks that land there
            for (int kc = kc_first; kc < KC; kc += nl) {
              int s = gs + kc;
              uint32_t ph = gph;
              while (s >= R_STAGES) { s -= R_STAGES; ph ^= 1; }
              if (!(TI == 1 && kc == kc_first) && !mbar_wait(&empty[s], ph ^ 1, wc)) { lane_ok = false; break; }
              tma_load_3d(a_s + (size_t)s * SB, &tmH, &full[s], kc * RK, row0, t);
              if (kc >= p.kr) tma_load_3d(a_s + (size_t)s * SB + HB, &tmW, &full[s], kc * RK, ht * UH, 0);
            }
          } else if (TI >= 2 && lane == 31) {
            // (the other arm of the same branch: the issuing lanes do not wait for this read)
            early = 0;
            if (nx_valid && nx.t > 0) early = ld_acquire_gpu(&p.flags[(size_t)nx.t * p.nbt + nx.tile(pb, p.nb_par)]);
          }
          if (__any_sync(0xffffffffu, !lane_ok)) { ok = false; break; }
          gs += KC;
          while (gs >= R_STAGES) { gs -= R_STAGES; gph ^= 1; }
        }
      }
    }
  } else if (PUBLISHER && warp == 1 + NACC) {
    // ---------------------------------------------------------------- publisher
    // Walks the items in the epilogue's order; when all epilogue warps have stored an item's h rows
    // (their arrival on pub_bar is a CTA-scope release, this wait the acquire), the proxy fence of the
    // hand-off and one release at GPU scope count this CTA in on the item's arrival counter.  An
    // epilogue warp can be at most four items ahead (it needs the counters this thread completes),
    // so four barriers never mix items.
    if (lane == 0) {
      int k = 0;
      bool ok = true;
      for (int ch = 0; ch < n_chunks && ok; ++ch) {
        for (int t = 0; t < p.T && ok; ++t) {
          for (int j = 0; j < TI && ok; ++j) {
            const int bt = pb + (ch * TI + j) * p.nb_par;
            if (bt >= p.nbt) continue;
            wc.d0 = t; wc.d1 = bt;
            if (!mbar_wait(&pub_bar[k & 3], (uint32_t)(k >> 2) & 1u, wc)) { ok = false; break; }
            fence_proxy_async();
            if (!p.no_arrive) red_release_gpu_add(&p.flags[(size_t)(t + 1) * p.nbt + bt], 1);
            ++k;
          }
        }
      }
    }
  } else if (warp < 1 + NACC) {
    // ---------------------------------------------------------------- MMA issuers
    const int x = warp - 1;                 // accumulator / K-slice index of this issuer
    if (lane == 0) {
      constexpr uint64_t descK = smem_desc_base(16, 1024);
      const uint32_t idesc = instr_desc(p.fmt, 0, 0, RB, N);
      // Every tcgen05 instruction (mma or commit) costs this thread ~150 clocks of issue time, so
      // issuer x owns WHOLE chunks (kc = x, x+NACC, ...): four MMAs and one commit per chunk,
      // in parallel with the other issuers, each into its own accumulator.
      bool ok = (x < nacc) && (p.kr == 0 || mbar_wait(w_full, 0, wc));
      int gs = 0;
      uint32_t gph = 0;
      uint32_t acc_ph[2] = {0, 0};
      int it = 0;
      const uint32_t w_addr = smem_u32(w_s);
      for (int ch = 0; ch < n_chunks && ok; ++ch) {
        for (int t = 0; t < p.T && ok; ++t) {
          for (int j = 0; j < TI && ok; ++j) {
            const int bt = pb + (ch * TI + j) * p.nb_par;
            if (bt >= p.nbt) continue;
            const int a = it & 1;
            ++it;
            if (!mbar_wait(&acc_empty[a], acc_ph[a] ^ 1, wc)) { ok = false; break; }
            acc_ph[a] ^= 1;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + a * ACC_STRIDE + x * N;
            uint32_t acc_on = 0;   // first MMA of the item overwrites this issuer's accumulator
            for (int kc = (x + nacc - gs % nacc) % nacc; kc < KC; kc += nacc) {
              int s = gs + kc;
              uint32_t ph = gph;
              while (s >= R_STAGES) { s -= R_STAGES; ph ^= 1; }
              if (!mbar_wait_spin(&full[s], ph, wc)) { ok = false; break; }
              // arm the stage's next use: R_STAGES chunks further on (chunks wrap around within an item)
              mbar_expect_tx(&full[s], (p.ws && (kc + R_STAGES) % KC >= p.kr) ? SB : HB);
              tc_fence_after();
              const uint32_t sa = smem_u32(a_s + (size_t)s * SB);
              const uint32_t sb = kc >= p.kr ? sa + HB : w_addr + (uint32_t)kc * N * 128;
#pragma unroll
              for (int k = 0; k < RK / 16; ++k)
                umma_f16(d_tmem, smem_desc(descK, sa + k * 32), smem_desc(descK, sb + k * 32), idesc,
                         (k > 0) ? 1u : acc_on);
              acc_on = 1;
              umma_commit(&empty[s]);
            }
            if (ok) umma_commit(&acc_full[a]);
            gs += KC;
            while (gs >= R_STAGES) { gs -= R_STAGES; gph ^= 1; }
          }
        }
      }
    }
  } else if constexpr (TMAEP) {
    // ---------------------------------------------------------------- epilogue, interleaved tiles
    // thread = (batch row, NU units), worked in passes of 8 units.  Each warp owns `npb` landing
    // buffers [4 gates][32 rows][NU units]: rows of 16 bytes lie back to back, rows of 32 bytes carry
    // the 32-byte swizzle, so the 32 lanes' 16-byte pieces of one gate fall into different banks.
    // Lane 0 issues the warp's TMA loads (`npb` items ahead) and stores.
    constexpr int PB_BYTES = 256 * NU, NPIECE = NU / 8;
    const int ew = warp - FIRST_EPI;
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int ug = ew >> 2;
    const int row_in_tile = q * 32 + lane;
    const int unit0 = ht * UH + ug * NU;
    const int npb = p.npb;
    uint8_t* pbuf = ep_s + (size_t)ew * npb * PB_BYTES;
    uint64_t* pfull = pre_full + 2 * ew;
    T16* out = reinterpret_cast<T16*>(p.out);
    T16* cell = reinterpret_cast<T16*>(p.cell);
    auto c_off = [&](int v) { return (NU == 16) ? lane * 32 + ((v ^ ((lane >> 2) & 1)) * 16) : lane * 16; };
    auto p_off = [&](int g, int v) { return g * (64 * NU) + c_off(v); };
    // the load cursor runs `npb` items ahead of the item being worked on (lane 0 only)
    ItemCursor<TI> lc;
    lc.init();
    bool lc_valid = lc.next(pb, p.nb_par, p.nbt, n_chunks, p.T);
    int n_loaded = 0;
    auto issue_load = [&]() {
      if (!lc_valid) return;
      const int b = (npb == 2) ? (n_loaded & 1) : 0;
      mbar_expect_tx(&pfull[b], PB_BYTES);
      tma_load_4d(pbuf + (size_t)b * PB_BYTES, &tmP, &pfull[b], unit0, lc.tile(pb, p.nb_par) * RB + q * 32, 0, lc.t);
      ++n_loaded;
      lc_valid = lc.next(pb, p.nb_par, p.nbt, n_chunks, p.T);
    };
    if (lane == 0)
      for (int i = 0; i < npb; ++i) issue_load();
    int it = 0;                             // items consumed
    bool ok = true;
    // cell rows of this thread's (row, NU units) for tile slot j: tensor-memory columns behind the accumulators
    const uint32_t c_taddr = tmem_base + C_BASE + (uint32_t(q * 32) << 16) + ug * NU;
    for (int ch = 0; ch < n_chunks && ok; ++ch) {
#pragma unroll
      for (int j = 0; j < TI; ++j) {
        const int bt = pb + (ch * TI + j) * p.nb_par;
        const int row = bt * RB + row_in_tile;
#pragma unroll
        for (int v = 0; v < NPIECE; ++v) {
          float c0[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) c0[u] = 0.f;
          if (bt < p.nbt && row < p.B) unpack8<T16>(ldg16(cell + (size_t)row * H + unit0 + 8 * v), c0);
          uint32_t cr[8];
#pragma unroll
          for (int u = 0; u < 8; ++u) cr[u] = __float_as_uint(c0[u]);
          tmem_st_32x8(c_taddr + j * UH + 8 * v, cr);
        }
      }
      tmem_st_wait();
      for (int t = 0; t < p.T && ok; ++t) {
#pragma unroll
        for (int j = 0; j < TI; ++j) {
          const int bt = pb + (ch * TI + j) * p.nb_par;
          if (bt >= p.nbt) continue;
          const int a = it & 1;
          const uint32_t a_ph = (uint32_t)(it >> 1) & 1u;
          const int b = (npb == 2) ? (it & 1) : 0;
          const uint32_t b_ph = (npb == 2) ? ((uint32_t)(it >> 1) & 1u) : ((uint32_t)it & 1u);
          ++it;
          const int row = bt * RB + row_in_tile;
          const bool row_ok = row < p.B;
          wc.d0 = t; wc.d1 = bt;
          if (!mbar_wait(&acc_full[a], a_ph, wc)) { ok = false; break; }
          if (!mbar_wait(&pfull[b], b_ph, wc)) { ok = false; break; }
          tc_fence_after();
          const uint32_t taddr = tmem_base + a * ACC_STRIDE + (uint32_t(q * 32) << 16) + ug * NU;
          uint8_t* pbb = pbuf + (size_t)b * PB_BYTES;
          const size_t o1 = ((size_t)(t + 1) * p.B + row) * H + unit0;
#pragma unroll
          for (int v = 0; v < NPIECE; ++v) {
            float pa[4][8];
            uint32_t cr[8];
            tmem_ld_32x8(c_taddr + j * UH + 8 * v, cr);
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              uint32_t acc[NACC][8];
#pragma unroll
              for (int x = 0; x < NACC; ++x) tmem_ld_32x8(taddr + x * N + g * UH + 8 * v, acc[x]);
              tmem_ld_wait();
#pragma unroll
              for (int u = 0; u < 8; ++u) {
                float s0 = __uint_as_float(acc[0][u]);
#pragma unroll
                for (int x = 1; x < NACC; ++x)
                  if (x < nacc) s0 += __uint_as_float(acc[x][u]);
                pa[g][u] = s0;
              }
            }
            if (v == NPIECE - 1) {
              // the accumulator is in registers: hand the TMEM buffer back to the MMA warps
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&acc_empty[a]);
            }
#pragma unroll
            for (int g = 0; g < 4; ++g) {
              const uint4 pw4 = *reinterpret_cast<const uint4*>(pbb + p_off(g, v));
              const uint32_t w[4] = {pw4.x, pw4.y, pw4.z, pw4.w};
#pragma unroll
              for (int u = 0; u < 4; ++u) {
                const float2 f2 = cvt2<T16>(w[u]);
                pa[g][2 * u] += f2.x;
                pa[g][2 * u + 1] += f2.y;
              }
            }
            float hv[8], cv[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
              const float cn = sigmoid_fast(pa[1][u]) * __uint_as_float(cr[u]) + sigmoid_fast(pa[0][u]) * tanh_fast(pa[2][u]);
              cv[u] = cn;
              cr[u] = __float_as_uint(cn);
              hv[u] = sigmoid_fast(pa[3][u]) * tanh_fast(cn);
            }
            tmem_st_32x8(c_taddr + j * UH + 8 * v, cr);
            if (row_ok) store8<T16>(out + o1 + 8 * v, hv);
            // final pre-activations back in place (16-bit, as stored)
#pragma unroll
            for (int g = 0; g < 4; ++g)
              *reinterpret_cast<uint4*>(pbb + p_off(g, v)) =
                  make_uint4(pk2<T16>(pa[g][0], pa[g][1]), pk2<T16>(pa[g][2], pa[g][3]), pk2<T16>(pa[g][4], pa[g][5]),
                             pk2<T16>(pa[g][6], pa[g][7]));
            if (row_ok && (!p.inference || t == p.T - 1)) store8<T16>(cell + o1 + 8 * v, cv);
          }
          tmem_st_wait();
          // publish h[t+1] first (it is all the peers wait for): the publisher warp fences and releases
          __syncwarp();
          if (lane == 0) mbar_arrive(&pub_bar[(it - 1) & 3]);
          // then the final pre-activations leave the landing buffer, and the box of the item `npb` ahead is
          // fetched into it
          if constexpr (NU == 16) {
            // Plain stores, NOT a TMA store: an SM's TMA unit writes only ~29 B/clk and the stores queue in
            // front of the h loads (measured: 8 such boxes per item cut a concurrent h stream from 71 to
            // 33 B/clk).  Two lanes cover a row's 32 bytes, so a warp instruction writes 16 full sectors:
            // instruction k = (gate k/2, rows 16*(k%2) ...), lane = (row, 16-byte piece).
            if (!p.inference) {
              T16* gbase = reinterpret_cast<T16*>(p.ifgo) + ((size_t)t * p.B + (size_t)bt * RB + q * 32) * (4 * (size_t)H) + unit0;
              const int r_lo = lane >> 1, v = lane & 1;
#pragma unroll
              for (int k = 0; k < 8; ++k) {
                const int g = k >> 1, r = (k & 1) * 16 + r_lo;
                const uint4 w = *reinterpret_cast<const uint4*>(pbb + g * (64 * NU) + r * 32 + ((v ^ ((r >> 2) & 1)) * 16));
                if (bt * RB + q * 32 + r < p.B) stg16(gbase + (size_t)r * (4 * (size_t)H) + (size_t)g * H + v * 8, w);
              }
            }
            fence_proxy_async_smem();      // the buffer's reads come before the next box is written into it
            __syncwarp();
            if (lane == 0) issue_load();
          } else {
            fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              const int row0 = bt * RB + q * 32;
              if (!p.inference) tma_store_4d(&tmP, pbb, unit0, row0, 0, t);
              tma_store_commit();
              tma_store_wait_read<0>();
              issue_load();
            }
          }
          __syncwarp();
        }
      }
    }
    if (lane == 0) tma_store_wait<0>();
  } else {
    // ---------------------------------------------------------------- epilogue
    // thread = (batch row, NU units): warpgroup `ug` takes the ug-th group of NU of the CTA's UH units
    const int ew = warp - FIRST_EPI;
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const int ug = ew >> 2;
    const int row_in_tile = q * 32 + lane;
    const int unit0 = ht * UH + ug * NU;
    const size_t H4 = 4 * (size_t)H;
    T16* ifgo = reinterpret_cast<T16*>(p.ifgo);
    T16* out = reinterpret_cast<T16*>(p.out);
    T16* cell = reinterpret_cast<T16*>(p.cell);
    int it = 0;                             // items consumed: TMEM buffer it & 1, on its (it >> 1)-th use
    bool ok = true;
    for (int ch = 0; ch < n_chunks && ok; ++ch) {
      float c[TI][NU];
      uint4 pre[4 * NV];                    // projected pre-activations of the NEXT item: 4 gates x NU units
      // initial cell state of this chunk's tiles
#pragma unroll
      for (int j = 0; j < TI; ++j) {
        const int bt = pb + (ch * TI + j) * p.nb_par;
        const int row = bt * RB + row_in_tile;
#pragma unroll
        for (int u = 0; u < NU; ++u) c[j][u] = 0.f;
        if (bt < p.nbt && row < p.B) {
#pragma unroll
          for (int v = 0; v < NV; ++v) unpack8<T16>(ldg16(cell + (size_t)row * H + unit0 + 8 * v), &c[j][8 * v]);
        }
      }
      auto load_pre = [&](int t, int bt) {
        const int row = bt * RB + row_in_tile;
        if (t < p.T && bt < p.nbt && row < p.B) {
          const T16* src = ifgo + ((size_t)t * p.B + row) * H4 + unit0;
#pragma unroll
          for (int g = 0; g < 4; ++g)
#pragma unroll
            for (int v = 0; v < NV; ++v) pre[g * NV + v] = ldg16(src + (size_t)g * H + 8 * v);
        }
      };
      load_pre(0, pb + (ch * TI) * p.nb_par);   // pre-activations of the first item
      for (int t = 0; t < p.T && ok; ++t) {
#pragma unroll
        for (int j = 0; j < TI; ++j) {
          const int bt = pb + (ch * TI + j) * p.nb_par;
          if (bt >= p.nbt) continue;
          const int a = it & 1;
          const uint32_t a_ph = (uint32_t)(it >> 1) & 1u;
          ++it;
          const int row = bt * RB + row_in_tile;
          const bool row_ok = row < p.B;
          wc.d0 = t; wc.d1 = bt;
          if (!mbar_wait(&acc_full[a], a_ph, wc)) { ok = false; break; }
          tc_fence_after();
          const uint32_t taddr = tmem_base + a * ACC_STRIDE + (uint32_t(q * 32) << 16) + ug * NU;
          // The thread's NU units are worked in passes of PW: accumulator read-out (the issuers' partial
          // sums, gate by gate, XG of them per wait so that at most 48 values are in flight), gate
          // maths, h store.  Two interleaved tiles of 16 units per thread take two passes of 8 -
          // a single pass would not fit the register file - and save the final pre-activations
          // inside the pass; every other shape takes one pass and saves them after the release.
          constexpr int PW = (NU == 16 && TI >= 2) ? 8 : NU;
          constexpr int XG = (NACC * PW > 48) ? 2 : NACC;
          const size_t o1 = ((size_t)(t + 1) * p.B + row) * H + unit0;
          T16* gdst = ifgo + ((size_t)t * p.B + row) * H4 + unit0;
          float pa[4][PW];
#pragma unroll
          for (int h0 = 0; h0 < NU; h0 += PW) {
#pragma unroll
            for (int g = 0; g < 4; ++g) {
#pragma unroll
              for (int x0 = 0; x0 < NACC; x0 += XG) {
                uint32_t v[XG][PW];
#pragma unroll
                for (int x = 0; x < XG; ++x) tmem_ld_cols<PW>(taddr + (x0 + x) * N + g * UH + h0, v[x]);
                tmem_ld_wait();
#pragma unroll
                for (int u = 0; u < PW; ++u) {
                  float s0 = (x0 == 0) ? 0.f : pa[g][u];
#pragma unroll
                  for (int x = 0; x < XG; ++x)
                    if (x0 + x < nacc) s0 += __uint_as_float(v[x][u]);
                  pa[g][u] = s0;
                }
              }
            }
            if (h0 + PW == NU) {
              // the accumulator is in registers: hand the TMEM buffer back to the MMA warps
              tc_fence_before();
              __syncwarp();
              if (lane == 0) mbar_arrive(&acc_empty[a]);
            }
#pragma unroll
            for (int g = 0; g < 4; ++g)
#pragma unroll
              for (int v = 0; v < PW / 8; ++v) {
                const uint4 pw4 = pre[g * NV + h0 / 8 + v];
                const uint32_t w[4] = {pw4.x, pw4.y, pw4.z, pw4.w};
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                  const float2 f2 = cvt2<T16>(w[u]);
                  pa[g][8 * v + 2 * u] += f2.x;
                  pa[g][8 * v + 2 * u + 1] += f2.y;
                }
              }
            float hv[PW];
#pragma unroll
            for (int u = 0; u < PW; ++u) {
              const float cn = sigmoid_fast(pa[1][u]) * c[j][h0 + u] + sigmoid_fast(pa[0][u]) * tanh_fast(pa[2][u]);
              c[j][h0 + u] = cn;
              hv[u] = sigmoid_fast(pa[3][u]) * tanh_fast(cn);
            }
            if (row_ok) {
#pragma unroll
              for (int v = 0; v < PW / 8; ++v) store8<T16>(out + o1 + h0 + 8 * v, &hv[8 * v]);
              if (PW < NU && !p.inference) {
#pragma unroll
                for (int g = 0; g < 4; ++g) store8<T16>(gdst + (size_t)g * H + h0, pa[g]);
              }
            }
          }
          // publish h[t+1] first (it is all the peers wait for): generic-proxy stores -> proxy fence
          // (here or on the reading side) -> warp-level arrival with release semantics; peers read
          // the rows through TMA
          if (WRITER_FENCE) fence_proxy_async();
          __syncwarp();
          // arrival per warp, or (cta_publish) one per CTA and item: the last epilogue warp to get here
          // publishes for all (a warp can be at most two items ahead of another, so four counters
          // never mix items)
          if (lane == 0) {
            if constexpr (PUBLISHER) {
              mbar_arrive(&pub_bar[(it - 1) & 3]);     // the publisher warp releases for the CTA
            } else {
              const bool pub = !p.cta_publish || (smem_count_arrive(&pub_cnt[it & 3]) & (EW - 1)) == EW - 1;
              if (pub && !p.no_arrive) red_release_gpu_add(&p.flags[(size_t)(t + 1) * p.nbt + bt], 1);
            }
          }
          // only now (after the release: a fence would otherwise wait for these loads) fetch the NEXT
          // item's projected pre-activations; they land while the peers run their step
          {
            int nj = j + 1, nt = t;
            if (nj == TI || pb + (ch * TI + nj) * p.nb_par >= p.nbt) { nj = 0; nt = t + 1; }
            load_pre(nt, pb + (ch * TI + nj) * p.nb_par);
            // the item after that: only pull its lines into L2 (a 32-byte sector covers both
            // warpgroups' pieces when each takes 16 bytes, so one of them asks)
            int fj = nj + 1, ft = nt;
            if (fj == TI || pb + (ch * TI + fj) * p.nb_par >= p.nbt) { fj = 0; ft = nt + 1; }
            const int fbt = pb + (ch * TI + fj) * p.nb_par;
            const int frow = fbt * RB + row_in_tile;
            if (ft < p.T && fbt < p.nbt && frow < p.B && (NV == 2 || ug == 0)) {
              const T16* src = ifgo + ((size_t)ft * p.B + frow) * H4 + unit0;
#pragma unroll
              for (int g = 0; g < 4; ++g) prefetch_l2(src + (size_t)g * H);
            }
          }
          // off the critical path: final pre-activations and c[t+1], saved for backward
          // (inference: only the last cell state is needed, as c_n)
          if (row_ok && (!p.inference || t == p.T - 1)) {
#pragma unroll
            for (int v = 0; v < NV; ++v) store8<T16>(cell + o1 + 8 * v, &c[j][8 * v]);
          }
          if (PW == NU && row_ok && !p.inference) {
#pragma unroll
            for (int g = 0; g < 4; ++g)
#pragma unroll
              for (int v = 0; v < NV; ++v) store8<T16>(gdst + (size_t)g * H + 8 * v, &pa[g][8 * (v % (PW / 8))]);
          }
        }
      }
    }
  }
  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int UH, int TI, typename T16>
static int launch_fwd_t(const RecPlan& pl, const CUtensorMap& tw, const CUtensorMap& th, const CUtensorMap& tp,
                        FwdParams& p, cudaStream_t st) {
  auto kern = fwd_kernel<UH, TI, T16>;
  BLSTM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
  void* args[] = {(void*)&tw, (void*)&th, (void*)&tp, (void*)&p};
  BLSTM_CUDA_OK(cudaLaunchCooperativeKernel((void*)kern, dim3(pl.grid), dim3(pl.threads), args, pl.smem, st));
  count_launch();
  return BLSTM_OK;
}


// =====================================================================================
// Backward (replaces lstm_persistent_seq_bwd, fastlstm/kernels.py:1201-1409)
//
// dh_{t-1}[B,H] = d_ifgo[t][B,4H] x Wh[4H,H] has K = 4H.  A cluster of four CTAs owns 64
// output units of one batch tile; CTA r of the cluster takes gate r's K range (H rows of
// Wh, resident in shared memory as an N-major operand) and streams the matching H columns
// of d_ifgo[t] through TMA.  Each CTA ends a step with a partial [128 x 64] fp32 product in
// TMEM; the four partials are reduce-scattered through distributed shared memory (each CTA
// receives the three 16-unit slices it needs, 24 KB per step) so that CTA r finishes with
// dh for units [16r, 16r+16) of the cluster's 64 - the units whose gate maths it then
// does (thread = batch row x 8 units: dc carried in fp32 registers, d_ifgo[t-1] written and
// published with the same per-(step, batch tile) arrival counters as the forward kernel).
// =====================================================================================
constexpr int DB_PARTS = 1024;            // row groups of the bias-gradient column sum
constexpr int XROW_BYTES = 64;            // one row of a slice: 16 fp32; its four 16-byte pieces are XOR-swizzled
constexpr int XSLOT_BYTES = RB * XROW_BYTES;  // one exchanged slice: 128 rows x 16 fp32 = 8 KB

struct BwdPlan {
  bool ok;
  int nug, nbt, nb_par, ntl, TI, grid, threads, stages, ni, nl, ws, alias;
  int kr;                   // K chunks of the Wh slice that stay resident (all of them unless ws)
  int hb;                   // bytes of the d_ifgo rows in a ring stage (128 rows, or a single smaller tile's own)
  size_t w_bytes, recv_bytes, stage_bytes, smem, ep_bytes;
  size_t off_flags, n_flags, off_db, ws_bytes;
};

// CTAs of the backward kernel that can be resident at once.  Clusters of four do not tile every GPC
// without a remainder: a B200 with 148 SMs holds 33 of them, 132 CTAs (asked of the occupancy
// calculator once per process, for the kernel's largest shared-memory footprint; defined behind the kernel).
static int bwd_cta_capacity();

static BwdPlan make_bwd_plan(const blstm_desc& d) {
  BwdPlan p{};
  p.ok = false;
  if (d.flags & BLSTM_FLAG_FORCE_GENERIC) return p;
  if (d.dtype != BLSTM_F16 && d.dtype != BLSTM_BF16) return p;
  const int H = d.hidden_size, B = d.batch;
  if (H % 64 != 0 || H < 64 || H > 2048) return p;
  p.nbt = cdiv(B, RB);
  p.nug = H / 64;
  const int per_tile = p.nug * 4;
  const int sms = std::min(plan_sm_count(), bwd_cta_capacity()) / ((d.flags & BLSTM_FLAG_HALF_DEVICE) ? 2 : 1);
  if (per_tile > sms) return p;
  p.nb_par = sms / per_tile;
  if (p.nb_par > p.nbt) p.nb_par = p.nbt;
  p.ntl = cdiv(p.nbt, p.nb_par);
  // Batch tiles interleaved per CTA.  Their only per-tile state is the carries in registers: the
  // exchange buffers below are indexed by item parity, not by tile.
  p.TI = p.ntl >= 3 ? 4 : p.ntl >= 2 ? 2 : 1;
  p.grid = p.nb_par * per_tile;
  p.threads = 0;                          // set below
  p.w_bytes = (size_t)H * 128;
  p.ws = p.w_bytes > 128 * 1024 ? 1 : 0;                   // stream the Wh slice through the ring
  p.hb = (p.nbt == 1 ? (int)round_up((size_t)B, 8) : RB) * 128;
  p.stage_bytes = p.hb + (p.ws ? 8192 : 0);
  const int KCp = H / RK;
  // (a stage that holds fewer than 128 rows is still READ as 128 rows by the MMA: the ring is followed by
  //  enough shared memory for the last stage's read to stay inside the allocation)
  const size_t tail_pad = p.stage_bytes < (size_t)R_STAGE_BYTES ? R_STAGE_BYTES - p.stage_bytes : 0;
  // Streamed means all of it (the depth of the ring is worth more than the bytes a resident part saves:
  // H=2048 measured 12.5 ms with 18 of 32 chunks resident against 11.5 ms with none); the kernel handles
  // any split, `kr` chunks are resident.
  auto resident_chunks = [&](size_t) { return p.ws ? 0 : KCp; };
  // Cluster exchange: receive slots (3 peers x 8 KB) and send staging (3 x 8 KB), one set.  With
  // interleaved tiles a CTA tells its three peers when it has consumed an item's slices, and nobody
  // stages or ships the next item before all three have said so (`consumed` in the kernel).
  // Interleaved tiles also move the epilogue's gate traffic through TMA: three landing buffers per pair
  // of epilogue warps (32 rows x 4 gates x 16 units; d_ifgo is written back in place and stored from there).
  p.recv_bytes = (size_t)2 * 3 * XSLOT_BYTES;
  p.ep_bytes = p.TI >= 2 ? (size_t)4 * 3 * 4096 : 0;
  p.kr = resident_chunks(1024 + p.recv_bytes + p.ep_bytes + 1024);
  if (1024 + (size_t)p.kr * 8192 + p.recv_bytes + p.ep_bytes + 1024 + 3 * p.stage_bytes > 232448 && p.TI >= 2) {
    p.TI = 1;                                               // not enough room to interleave tiles
    p.ep_bytes = 0;
    p.kr = resident_chunks(1024 + p.recv_bytes + 1024);
  }
  size_t wres = (size_t)p.kr * 8192;
  size_t fixed = 1024 + wres + p.recv_bytes + p.ep_bytes + 1024 + tail_pad;  // 1024: barriers and counters behind the ring
  // warps: 1 producer + 3 MMA issuers (or 2 + a publisher warp when tiles are interleaved) + 2 epilogue
  // warpgroups = 12 (3 per SM sub-partition, 168 registers each); a 13th warp would cap every thread
  // at 128 registers.
  const int n_issuers = p.TI >= 2 ? 2 : 3;
  p.threads = 32 * 12;
  if (!pick_ring(fixed, p.stage_bytes, n_issuers, H / RK, &p.stages, &p.ni)) return p;
  // One tile in flight and a shallow ring (H = 768, 1024: the resident weights leave three stages):
  // the ring is idle while an item's slices cross the cluster, so the exchange buffers are laid over
  // its first stages and the ring gets their 48 KB.  A peer may then write a slice only after this
  // CTA has finished the item's MMAs, which each CTA tells its peers (see `rdy` in the kernel).
  p.alias = 0;
  if (p.TI == 1 && p.stages < 6) {
    int st2 = 0, ni2 = 0;
    const size_t fixed2 = 1024 + wres + 1024 + tail_pad;
    if (pick_ring(fixed2, p.stage_bytes, n_issuers, H / RK, &st2, &ni2) && st2 > p.stages &&
        (size_t)st2 * p.stage_bytes >= p.recv_bytes) {
      p.alias = 1; p.stages = st2; p.ni = ni2; fixed = fixed2;
    }
  }
  // TMA-issuing lanes of the producer warp (nl | stages): four interleaved tiles do better with four
  // (B=4096, H=512: 8.5 -> 8.1 ms), a single tile on a six-stage ring with two (H=1024: 5.33 -> 5.22 ms)
  p.nl = p.ni;
  if (p.TI == 4) p.nl = 4;
  if (p.TI == 1 && p.stages == 6) p.nl = 2;
  if (p.stages % p.nl != 0 || p.nl > H / RK) p.nl = p.ni;
  p.smem = fixed + (size_t)p.stages * p.stage_bytes;
  p.n_flags = (size_t)d.seq_len * p.nbt;
  p.off_flags = sizeof(Control);
  p.off_db = p.off_flags + round_up(p.n_flags * sizeof(int), 256);
  p.ws_bytes = p.off_db + round_up((size_t)DB_PARTS * 4 * H * sizeof(float), 256);
  p.ok = true;
  return p;
}

struct BwdParams {
  int T, B, H;
  int nbt, nug, nb_par, ntl;
  int stages;
  int ni;
  int nl;                   // TMA-issuing lanes of the producer warp (nl divides the ring depth)
  int ws;
  int kr;                   // resident K chunks of the Wh slice
  int hb;                   // bytes of the d_ifgo rows in a ring stage
  int stage_bytes;
  int fmt;
  int no_arrive;
  int flag_target;          // arrivals that complete a flag: H/16 CTAs per batch tile [x 8 epilogue warps]
  int cta_publish;          // 1: one arrival per CTA and item, 0: one per epilogue warp
  int alias;                // 1: exchange buffers laid over the first ring stages (one tile in flight)
  int ep_bytes;             // bytes of the epilogue's TMA buffers (interleaved tiles)
  unsigned long long limit_ns;
  Control* ctl;
  int* flags;               // [T][nbt]: arrivals for d_ifgo[t]
  const void* dout;         // [T,B,H]
  const void* dh_n;         // [B,H] or null
  const void* dc_n;         // [B,H] or null
  const void* ifgo;         // [T,B,4H]
  const void* cell;         // [T+1,B,H]
  void* d_ifgo;             // [T,B,4H]
  void* dh0;                // [B,H]
  void* dc0;                // [B,H]
  float* db_part;           // [nb_par * 4][4H] bias-gradient partial sums (one row per CTA group and row quarter), or null
};

template <typename T16>
__device__ __forceinline__ void unpack16(const uint4& v0, const uint4& v1, float (&f)[16]) {
  const uint32_t w[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
  for (int u = 0; u < 8; ++u) { const float2 t = cvt2<T16>(w[u]); f[2 * u] = t.x; f[2 * u + 1] = t.y; }
}
template <typename T16>
__device__ __forceinline__ void store16(T16* dst, const float (&f)[16]) {
  uint32_t w[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) w[u] = pk2<T16>(f[2 * u], f[2 * u + 1]);
  stg16(dst, make_uint4(w[0], w[1], w[2], w[3]));
  stg16(dst + 8, make_uint4(w[4], w[5], w[6], w[7]));
}

template <int TI, typename T16>
__global__ void __launch_bounds__(384, 1)
bwd_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmG,
           const __grid_constant__ CUtensorMap tmI, const __grid_constant__ CUtensorMap tmD, const BwdParams p) {
  // Warps: 0 = TMA producer, then NACC MMA issuers, then (interleaved tiles only) one PUBLISHER warp,
  // then 8 epilogue warps from warp 4 on - 12 in all either way.
  // With interleaved tiles the epilogue warps are the bottleneck, and the release that publishes an
  // item stalls its thread for a memory round trip: there a thread of its own does the releasing
  // (the epilogue warps only arrive on a CTA-local barrier after their stores), which costs one issuer.
  constexpr bool PUBLISHER = (TI >= 2);
  constexpr int N = 64, NACC = PUBLISHER ? 2 : 3, ACC_STRIDE = 256;   // NACC: MMA issuer warps
  constexpr int FIRST_EPI = 4;
  constexpr bool WRITER_FENCE = false;            // the proxy fence of the hand-off: reader (one tile) or publisher warp
  constexpr int ITEM_WARPS = 8;                   // epilogue warps, all working on every item
  // Interleaved tiles are throughput bound and the epilogue's row-strided 16-byte global accesses were
  // the bottleneck there: the saved pre-activations come in, and d_ifgo goes out, as TMA boxes through
  // shared memory, one pair of landing buffers per epilogue warp (tmI: ifgo, tmD: d_ifgo, both
  // as {unit, row, gate, step}).  The TMA store of d_ifgo[t] is also what the peers' producers read
  // next, so a warp counts its item in only after its store has completed.
  constexpr bool TMAEP = (TI >= 2);
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int H = p.H;
  const int KC = H / RK;
  const int R_STAGES = p.stages;
  uint8_t* w_s = smem;                                        // [KC][64 k rows][128 B]
  const int SB = p.stage_bytes;                               // d_ifgo chunk (16 KB) [+ Wh chunk when streamed]
  const int HB = p.hb;                                        // d_ifgo rows of a stage; a streamed Wh chunk follows
  uint8_t* recv = smem + (size_t)p.kr * 8192;                 // [3 senders][128 rows][64 B]
  constexpr int XB = 1;                                       // one set of exchange buffers
  uint8_t* stage = recv + (size_t)XB * 3 * XSLOT_BYTES;      // [3 receivers][128 rows][64 B]
  uint8_t* ep_s = stage + (size_t)XB * 3 * XSLOT_BYTES;      // epilogue TMA buffers [4 warp pairs][3][4 KB]
  uint8_t* a_s = p.alias ? recv : ep_s + p.ep_bytes;         // ring (over the exchange buffers if aliased)
  uint64_t* bars = reinterpret_cast<uint64_t*>(a_s + (size_t)R_STAGES * SB);
  uint64_t* full = bars;
  uint64_t* empty = bars + R_MAX_STAGES;
  uint64_t* acc_full = bars + 2 * R_MAX_STAGES;
  uint64_t* acc_empty = acc_full + 2;
  uint64_t* w_full = acc_empty + 2;
  uint64_t* xchg = w_full + 1;                                // [2]
  uint64_t* staged = xchg + 2;                                // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(staged + 2);
  volatile int* dead = reinterpret_cast<volatile int*>(tmem_slot + 1);
  int* pub_cnt = const_cast<int*>(dead) + 1;        // [4] arrivals of the epilogue warps, by item index mod 4
  uint64_t* pub_bar = reinterpret_cast<uint64_t*>(pub_cnt + 4);   // [4] item published? by item index mod 4
  uint64_t* rdy = pub_bar + 4;                                 // aliased buffers: the 3 peers are done with their MMAs
  uint64_t* consumed = rdy + 1;                                // interleaved tiles: the 3 peers' 8 warps read an item's slices
  uint64_t* pre_full = consumed + 1;                           // [4 warp pairs][3] landing buffer filled
  uint64_t* pre_done = pre_full + 12;                          // [4 warp pairs][3] both warps wrote their d_ifgo halves
  uint64_t* pre_free = pre_full + 24;                          // [4 warp pairs][3] landing buffer may be refilled

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t r = cluster_ctarank();                       // gate whose K range this CTA owns
  const int cid = blockIdx.x >> 2;
  const int ugc = cid % p.nug, pb = cid / p.nug;
  constexpr uint32_t TMEM_COLS = 512;
  const int nacc = p.ni;                             // accumulators / issuers / TMA lanes in use

  if (threadIdx.x == 0) {
    // full[s] is armed (arrive + expected bytes) for its first use here and re-armed by the MMA issuer
    // that consumed it for every later use, which keeps that work out of the latency-bound TMA producer loop
    for (int s = 0; s < R_STAGES; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int a = 0; a < 2; ++a) { mbar_init(&acc_full[a], nacc); mbar_init(&acc_empty[a], ITEM_WARPS); }
    mbar_init(w_full, 1);
    for (int j = 0; j < 2; ++j) { mbar_init(&xchg[j], 1); mbar_init(&staged[j], ITEM_WARPS); }   // xchg: one expect_tx arrival + tx bytes
    *dead = 0;
    for (int i = 0; i < 4; ++i) pub_cnt[i] = 0;
    for (int i = 0; i < 4; ++i) mbar_init(&pub_bar[i], TMAEP ? 4 : ITEM_WARPS);   // (interleaved: one arrival per warp pair)
    mbar_init(rdy, 3);
    mbar_init(consumed, 3 * ITEM_WARPS);
    for (int i = 0; i < 24; ++i) { mbar_init(&pre_full[i], i < 12 ? 1 : 2); mbar_init(&pre_free[i], 1); }
    fence_mbar_init();
    for (int s = 0; s < R_STAGES; ++s) mbar_expect_tx(&full[s], (p.ws && s % KC >= p.kr) ? SB : HB);
    tma_prefetch_desc(&tmW);
    tma_prefetch_desc(&tmG);
    if (TMAEP) { tma_prefetch_desc(&tmI); tma_prefetch_desc(&tmD); }
  }
  if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  cluster_sync_all();                 // peers' barriers exist before anyone arrives on them remotely
  const uint32_t tmem_base = *tmem_slot;
  WaitCtx wc{dead, p.ctl, p.limit_ns, -1, (int)blockIdx.x};
  const int n_chunks = (p.ntl + TI - 1) / TI;
  const int T = p.T;

  // Items of a chunk: for s in [0,T] : for j in [0,TI).  Item (s,j) first (s > 0) forms
  // dh = d_ifgo[T-s] x Wh for its tile, then (s < T) does the gate maths of step t = T-1-s.
  if (warp == 0) {
    // ---------------------------------------------------------------- TMA producer
    if (lane == 0 && p.kr > 0) {
      mbar_expect_tx(w_full, (uint32_t)((size_t)p.kr * 8192));
      for (int kc = 0; kc < p.kr; ++kc)
        tma_load_2d(w_s + (size_t)kc * 8192, &tmW, w_full, ugc * 64, (int)r * H + kc * RK);
    }
    int gs = 0;
    uint32_t gph = 0;
    bool ok = true;
    // With interleaved tiles an item's arrival counter is usually complete long before its turn, and
    // what costs is the round trip of looking: lane 31 reads the NEXT item's counter while the other
    // lanes issue the current item's loads, and lane 0 only spins when that early look found it incomplete.
    ItemCursor<TI> nx;
    nx.init();
    bool nx_valid = nx.next(pb, p.nb_par, p.nbt, n_chunks, T);   // the first item itself
    int early = 0;             // lane 31: early reading of the next item's counter
    for (int ch = 0; ch < n_chunks && ok; ++ch) {
      for (int st = 1; st <= T && ok; ++st) {
        const int tg = T - st;      // timestep whose d_ifgo is streamed
        for (int j = 0; j < TI && ok; ++j) {
          const int bt = pb + (ch * TI + j) * p.nb_par;
          if (bt >= p.nbt) continue;
          const int early_now = (TI >= 2) ? __shfl_sync(0xffffffffu, early, 31) : 0;
          if (TI >= 2) nx_valid = nx_valid && nx.next(pb, p.nb_par, p.nbt, n_chunks, T);
          int seen = 1;
          if (lane == 0 && !(TI >= 2 && early_now >= p.flag_target)) {
            wc.d0 = tg; wc.d1 = bt;
            seen = wait_flag_ge(&p.flags[(size_t)tg * p.nbt + bt], p.flag_target, p.ctl, p.limit_ns, tg, bt) ? 1 : 0;
          }
          seen = __shfl_sync(0xffffffffu, seen, 0);
          if (!seen) { *dead = 1; ok = false; break; }
          // One proxy fence must lie between the peers' generic-proxy stores and the TMA reads below:
          // here for a single tile in flight (the writers' release then waits for their stores alone),
          // in the writers' publisher warp for interleaved tiles (this loop then streams without a break).
          if (!WRITER_FENCE && !PUBLISHER) fence_proxy_async();
          const int row0 = bt * RB, col0 = (int)r * H;
          bool lane_ok = true;
          const int nl = p.nl;                 // TMA-issuing lanes: lane l owns the ring stages == l (mod nl)
          if (lane < nl) {
            // this lane owns ring stages == lane (mod nl): the item's chunks that land there
            for (int kc = (lane + nl - gs % nl) % nl; kc < KC; kc += nl) {
              int s = gs + kc;
              uint32_t ph = gph;
              while (s >= R_STAGES) { s -= R_STAGES; ph ^= 1; }
              if (!mbar_wait(&empty[s], ph ^ 1, wc)) { lane_ok = false; break; }
              tma_load_3d(a_s + (size_t)s * SB, &tmG, &full[s], col0 + kc * RK, row0, tg);
              if (kc >= p.kr) tma_load_2d(a_s + (size_t)s * SB + HB, &tmW, &full[s], ugc * 64, col0 + kc * RK);
            }
          } else if (TI >= 2 && lane == 31) {
            // (the other arm of the same branch: the issuing lanes do not wait for this read)
            early = 0;
            if (nx_valid) early = ld_acquire_gpu(&p.flags[(size_t)(T - 1 - nx.t) * p.nbt + nx.tile(pb, p.nb_par)]);
          }
          if (__any_sync(0xffffffffu, !lane_ok)) { ok = false; break; }
          gs += KC;
          while (gs >= R_STAGES) { gs -= R_STAGES; gph ^= 1; }
        }
      }
    }
  } else if (PUBLISHER && warp == 1 + NACC) {
    // ---------------------------------------------------------------- publisher
    // Walks the gate-maths items in the epilogue's order; when all eight epilogue warps have stored
    // an item's d_ifgo rows (their arrival on pub_bar is a CTA-scope release, this wait the acquire),
    // one release at GPU scope counts this CTA in on the item's arrival counter.  An epilogue warp can
    // be at most four items ahead of the slowest (it needs the counters this thread completes), so
    // four barriers never mix items.
    if (lane == 0) {
      int k = 0;
      bool ok = true;
      for (int ch = 0; ch < n_chunks && ok; ++ch) {
        for (int st = 0; st < T && ok; ++st) {
          for (int j = 0; j < TI && ok; ++j) {
            const int bt = pb + (ch * TI + j) * p.nb_par;
            if (bt >= p.nbt) continue;
            wc.d0 = T - 1 - st; wc.d1 = bt;
            if (!mbar_wait(&pub_bar[k & 3], (uint32_t)(k >> 2) & 1u, wc)) { ok = false; break; }
            // the generic->async proxy fence of the hand-off runs here, on the causality path between
            // the epilogue warps' stores (ordered before this thread by the barrier) and the release
            fence_proxy_async();
            if (!p.no_arrive) red_release_gpu_add(&p.flags[(size_t)(T - 1 - st) * p.nbt + bt], 1);
            ++k;
          }
        }
      }
    } else if (TMAEP && lane <= 4) {
      // ------------------------------------------------------------ gate loaders (lanes 1..4)
      // Lane 1+w fetches the gate boxes of the two epilogue warps of row quarter w (all 16 units: 32-byte
      // rows), up to three gate-maths items ahead, into the pair's three landing buffers in turn; a
      // buffer is refilled once the pair has said that the d_ifgo box it held has been written
      // (pre_free).  Issuing these loads from here rather than from the epilogue warps matters: a TMA
      // issue waits for room behind the producer's 16 KB boxes (about a thousand clocks), which the
      // epilogue warps cannot afford.
      const int w = lane - 1;
      const int gq = w;                                         // the pair's row quarter
      const int g_unit0 = ugc * 64 + (int)r * 16;
      uint8_t* g_buf = ep_s + (size_t)w * 3 * 4096;
      ItemCursor<TI> lc;
      lc.init();
      int n = 0;
      bool ok = true;
      while (ok && lc.next(pb, p.nb_par, p.nbt, n_chunks, T)) {
        const int b = n % 3;
        wc.d0 = T - 1 - lc.t; wc.d1 = lc.tile(pb, p.nb_par);
        if (n >= 3 && !mbar_wait(&pre_free[3 * w + b], (uint32_t)(n / 3 - 1) & 1u, wc)) { ok = false; break; }
        mbar_expect_tx(&pre_full[3 * w + b], 4096);
        tma_load_4d(g_buf + b * 4096, &tmI, &pre_full[3 * w + b], g_unit0, lc.tile(pb, p.nb_par) * RB + gq * 32, 0,
                    T - 1 - lc.t);
        ++n;
      }
    }
  } else if (warp < 1 + NACC) {
    // ---------------------------------------------------------------- MMA issuers (own whole chunks)
    const int x = warp - 1;
    if (lane == 0) {
      constexpr uint64_t descA = smem_desc_base(16, 1024);       // d_ifgo tile, K-major
      constexpr uint64_t descB = smem_desc_base(8192, 1024);     // Wh chunk, N-major (64 units wide)
      const uint32_t idesc = instr_desc(p.fmt, 0, 1, RB, N);
      bool ok = (x < nacc) && (p.kr == 0 || mbar_wait(w_full, 0, wc));
      int gs = 0;
      uint32_t gph = 0;
      uint32_t acc_ph[2] = {0, 0};
      int it = 0;
      const uint32_t w_addr = smem_u32(w_s);
      for (int ch = 0; ch < n_chunks && ok; ++ch) {
        for (int st = 1; st <= T && ok; ++st) {
          for (int j = 0; j < TI && ok; ++j) {
            const int bt = pb + (ch * TI + j) * p.nb_par;
            if (bt >= p.nbt) continue;
            const int a = it & 1;
            ++it;
            if (!mbar_wait(&acc_empty[a], acc_ph[a] ^ 1, wc)) { ok = false; break; }
            acc_ph[a] ^= 1;
            tc_fence_after();
            const uint32_t d_tmem = tmem_base + a * ACC_STRIDE + x * N;
            uint32_t acc_on = 0;
            for (int kc = (x + nacc - gs % nacc) % nacc; kc < KC; kc += nacc) {
              int s = gs + kc;
              uint32_t ph = gph;
              while (s >= R_STAGES) { s -= R_STAGES; ph ^= 1; }
              if (!mbar_wait_spin(&full[s], ph, wc)) { ok = false; break; }
              // arm the stage's next use: R_STAGES chunks further on (chunks wrap around within an item)
              mbar_expect_tx(&full[s], (p.ws && (kc + R_STAGES) % KC >= p.kr) ? SB : HB);
              tc_fence_after();
              const uint32_t sa = smem_u32(a_s + (size_t)s * SB);
              const uint32_t sb = kc >= p.kr ? sa + HB : w_addr + (uint32_t)kc * 8192;
#pragma unroll
              for (int k = 0; k < RK / 16; ++k)
                umma_f16(d_tmem, smem_desc(descA, sa + k * 32), smem_desc(descB, sb + k * 2048), idesc,
                         (k > 0) ? 1u : acc_on);
              acc_on = 1;
              umma_commit(&empty[s]);
            }
            if (ok) umma_commit(&acc_full[a]);
            gs += KC;
            while (gs >= R_STAGES) { gs -= R_STAGES; gph ^= 1; }
          }
        }
      }
    }
  } else {
    // ---------------------------------------------------------------- epilogue: two warpgroups
    // thread = (batch row, 8 units): the two warpgroups split the CTA's 16 units of every item, which
    // halves the serial path of a step (accumulator read-out, gate maths) and keeps it free of spills.
    constexpr int NU = 8;                        // units per thread
    const int g = (warp - FIRST_EPI) >> 2;       // warpgroup = which half of the 16 units
    const int uoff = g * NU;
    const int q = warp & 3;
    const int row_in_tile = q * 32 + lane;
    const int unit0 = ugc * 64 + (int)r * 16 + uoff;
    const int swz = (row_in_tile >> 1) & 3;   // bank swizzle of the exchanged slices
    const size_t H4 = 4 * (size_t)H;
    const T16* ifgo = reinterpret_cast<const T16*>(p.ifgo);
    const T16* cell = reinterpret_cast<const T16*>(p.cell);
    const T16* dout = reinterpret_cast<const T16*>(p.dout);
    T16* dg = reinterpret_cast<T16*>(p.d_ifgo);
    const bool shipper = (warp == FIRST_EPI) && lane == 0;   // sends the staged slices
    // Bias gradient (replaces the reduction of fastlstm/lstm.py:497 and a separate pass over d_ifgo):
    // every thread adds the d_ifgo values it stores - as stored, i.e. rounded - to 32 fp32 sums of its
    // own (4 gates x 8 units) that live in the tensor-memory columns behind the accumulators, one
    // 32-column block per warpgroup; after the last step the 32 rows of a warp are added up with
    // shuffles and lane 0 writes the warp's partial sums.
    constexpr int DB_COL = 192;                  // NACC * N <= 192 columns per accumulator buffer are in use
    const uint32_t db_taddr = tmem_base + DB_COL + g * 32 + (uint32_t(q * 32) << 16);
    const bool want_db = p.db_part != nullptr;
    if (want_db) {
      uint32_t z[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) z[u] = 0u;
#pragma unroll
      for (int k = 0; k < 4; ++k) tmem_st_32x8(db_taddr + 8 * k, z);
      tmem_st_wait();
    }
    int it = 0;                 // MMA items consumed so far: TMEM buffer it & 1, on its (it >> 1)-th use
    int pub_it = 0;             // gate-maths items published so far
    bool ok = true;
    // Interleaved tiles: the two warps of a row quarter (one per unit half) share three landing buffers
    // [4 gates][32 rows][16 units] (32-byte rows with the 32-byte swizzle: a warp's 16-byte pieces of one
    // gate fall into different banks), used in turn by consecutive gate-maths items.  Whole 32-byte
    // segments matter: an SM's TMA unit is what bounds an item, and its cost goes by row segments - eight
    // boxes of 16-byte segments in and eight out per item cost it about twice the item's 128 KB of d_ifgo
    // chunks.  A lane of the publisher warp issues the pair's TMA loads; lane 0 of the pair's first warp
    // issues its store once both warps have written their halves (pre_done); when the store has completed
    // the buffer is handed back to the loader and the pair counts the item in.
    uint8_t* pbuf = ep_s + (size_t)q * 3 * 4096;
    uint64_t* pfull = pre_full + 3 * q;
    uint64_t* pdone = pre_done + 3 * q;
    auto p_off = [&](int k) { return k * 1024 + lane * 32 + ((g ^ ((lane >> 2) & 1)) * 16); };
    uint64_t* pfree = pre_free + 3 * q;
    for (int ch = 0; ch < n_chunks && ok; ++ch) {
      // dc is carried per interleaved tile; dh is rebuilt from the accumulator in every item, so one
      // copy serves all tiles (its first value, the gradient of h_n, is fetched in the tile's first item)
      float dc[TI][NU], dhc[NU];
      uint4 pf[7];       // next item's inputs: gates i,f,g,o, c[t+1], c[t], dout[t]
#pragma unroll
      for (int j = 0; j < TI; ++j) {
        const int bt = pb + (ch * TI + j) * p.nb_par;
        const int row = bt * RB + row_in_tile;
        const bool rok = bt < p.nbt && row < p.B;
#pragma unroll
        for (int u = 0; u < NU; ++u) dc[j][u] = 0.f;
        if (rok && p.dc_n) unpack8<T16>(ldg16(reinterpret_cast<const T16*>(p.dc_n) + (size_t)row * H + unit0), dc[j]);
      }
      auto prefetch = [&](int t, int bt) {
        const int row = bt * RB + row_in_tile;
        if (bt < p.nbt && row < p.B) {
          if constexpr (!TMAEP) {
            const T16* gsrc = ifgo + ((size_t)t * p.B + row) * H4 + unit0;
#pragma unroll
            for (int k = 0; k < 4; ++k) pf[k] = ldg16(gsrc + (size_t)k * H);
          }
          pf[4] = ldg16(cell + ((size_t)(t + 1) * p.B + row) * H + unit0);
          pf[5] = ldg16(cell + ((size_t)t * p.B + row) * H + unit0);
          pf[6] = ldg16(dout + ((size_t)t * p.B + row) * H + unit0);
        }
      };
      // two items ahead the same inputs are only pulled into L2 (no registers to hold them yet);
      // a 32-byte sector covers both warpgroups' halves, so one warpgroup issues them
      auto prefetch_far = [&](int t, int bt) {
        const int row = bt * RB + row_in_tile;
        if (g == 0 && bt < p.nbt && row < p.B) {
          if constexpr (!TMAEP) {
            const T16* gsrc = ifgo + ((size_t)t * p.B + row) * H4 + unit0;
#pragma unroll
            for (int k = 0; k < 4; ++k) prefetch_l2(gsrc + (size_t)k * H);
          }
          prefetch_l2(cell + ((size_t)t * p.B + row) * H + unit0);
          prefetch_l2(dout + ((size_t)t * p.B + row) * H + unit0);
        }
      };
      // Everything in the gate maths that does not depend on dh is worked out ahead of the accumulator:
      //   dh = dout + dh_carry;  dcv = dh*fA + dc;  d_i = dcv*fBi;  d_f = dcv*fBf;  d_g = dcv*fBg;
      //   d_o = dh*fBo;  dc' = dcv*fSf
      // With one tile in flight that happens as soon as the prefetched inputs land (the warps would
      // only wait for the next accumulator); with interleaved tiles it fills the cluster exchange.
      constexpr bool USE_FACTORS = (TI <= 2);
      constexpr bool EARLY_FACTORS = (TI == 1);
      constexpr int NF = USE_FACTORS ? NU : 1;
      float fA[NF], fBi[NF], fBf[NF], fBg[NF], fBo[NF], fSf[NF], fDd[NF];
      auto factors = [&]() {
        if constexpr (USE_FACTORS) {
        const uint32_t wi[4] = {pf[0].x, pf[0].y, pf[0].z, pf[0].w};
        const uint32_t wf[4] = {pf[1].x, pf[1].y, pf[1].z, pf[1].w};
        const uint32_t wg[4] = {pf[2].x, pf[2].y, pf[2].z, pf[2].w};
        const uint32_t wo[4] = {pf[3].x, pf[3].y, pf[3].z, pf[3].w};
        const uint32_t w1[4] = {pf[4].x, pf[4].y, pf[4].z, pf[4].w};
        const uint32_t w0[4] = {pf[5].x, pf[5].y, pf[5].z, pf[5].w};
        const uint32_t wd[4] = {pf[6].x, pf[6].y, pf[6].z, pf[6].w};
#pragma unroll
        for (int w = 0; w < 4; ++w) {
          const float2 pi = cvt2<T16>(wi[w]), pff = cvt2<T16>(wf[w]), pg = cvt2<T16>(wg[w]), po = cvt2<T16>(wo[w]);
          const float2 c1 = cvt2<T16>(w1[w]), c0 = cvt2<T16>(w0[w]), dd = cvt2<T16>(wd[w]);
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            const int u = 2 * w + e;
            const float si = sigmoid_fast(e ? pi.y : pi.x), sf = sigmoid_fast(e ? pff.y : pff.x);
            const float so = sigmoid_fast(e ? po.y : po.x);
            const float tg = tanh_fast(e ? pg.y : pg.x), tc = tanh_fast(e ? c1.y : c1.x);
            fA[u] = so * (1.f - tc * tc);
            fBi[u] = tg * si * (1.f - si);
            fBf[u] = (e ? c0.y : c0.x) * sf * (1.f - sf);
            fBg[u] = si * (1.f - tg * tg);
            fBo[u] = tc * so * (1.f - so);
            fSf[u] = sf;
            fDd[u] = e ? dd.y : dd.x;
          }
        }
        }
      };
      // interleaved tiles: the gates of the item whose maths comes next, out of its landing buffer
      auto fetch_gates = [&]() -> bool {
        if constexpr (TMAEP) {
          if (!mbar_wait(&pfull[pub_it % 3], (uint32_t)(pub_it / 3) & 1u, wc)) return false;
          const uint8_t* pbb = pbuf + (pub_it % 3) * 4096;
#pragma unroll
          for (int k = 0; k < 4; ++k) pf[k] = *reinterpret_cast<const uint4*>(pbb + p_off(k));
        }
        return true;
      };
      prefetch(T - 1, pb + (ch * TI) * p.nb_par);
      if (USE_FACTORS && EARLY_FACTORS) factors();
      for (int st = 0; st <= T && ok; ++st) {
#pragma unroll
        for (int j = 0; j < TI; ++j) {
          const int bt = pb + (ch * TI + j) * p.nb_par;
          if (bt >= p.nbt) continue;
          const int row = bt * RB + row_in_tile;
          const bool row_ok = row < p.B;
          if (st > 0) {
            // ---- dh = (sum over the cluster's four K ranges of) d_ifgo[T-st] x Wh
            const int a = it & 1;
            const uint32_t a_ph = (uint32_t)(it >> 1) & 1u;
            // one set of exchange buffers: its barriers change phase with every item
            constexpr int xb = 0;
            const uint32_t x_ph = (uint32_t)it & 1u;
            ++it;
            wc.d0 = T - st; wc.d1 = bt;
            if (!mbar_wait(&acc_full[a], a_ph, wc)) { ok = false; break; }
            if constexpr (TI >= 2) {
              // the previous item's slices have been read by all three peers (so the staging below
              // overwrites nothing a copy still reads, and the peers' receive slots are free again)
              // (no data rides on this barrier, so a plain CTA-scope wait will do)
              if (it > 1 && !mbar_wait(consumed, (uint32_t)it & 1u, wc)) { ok = false; break; }
            }
            if (p.alias && shipper) {
              // this item's MMAs are done (their reads of the ring completed before acc_full did), so
              // the ring - and the exchange buffers laid over it - is idle until the next item: tell
              // the three peers they may write their slices.  Nothing of this thread is published by
              // the signal, hence relaxed.
#pragma unroll
              for (int dst = 0; dst < 4; ++dst)
                if (dst != (int)r) mbar_arrive_remote_relaxed(mapa_shared(smem_u32(rdy), dst));
            }
            tc_fence_after();
            const uint32_t taddr = tmem_base + a * ACC_STRIDE + (uint32_t(q * 32) << 16) + uoff;
#pragma unroll
            for (int dst = 0; dst < 4; ++dst) {
              // the issuers' partial accumulators for these units: NACC loads, ONE wait
              uint32_t v[NACC][NU];
#pragma unroll
              for (int xx = 0; xx < NACC; ++xx) tmem_ld_32x8(taddr + xx * N + dst * 16, v[xx]);
              tmem_ld_wait();
              float sum[NU];
#pragma unroll
              for (int u = 0; u < NU; ++u) {
                float a0 = __uint_as_float(v[0][u]);
                if (nacc > 1) a0 += __uint_as_float(v[1][u]);
                if (NACC > 2 && nacc > 2) a0 += __uint_as_float(v[NACC - 1][u]);
                sum[u] = a0;
              }
              if (dst == (int)r) {
#pragma unroll
                for (int u = 0; u < NU; ++u) dhc[u] = sum[u];   // last step's carry is dead by now
              } else {
                // stage the slice for peer `dst` locally (row = 64 B, 16-byte pieces XOR-swizzled)
                uint8_t* sp = stage + ((size_t)xb * 3 + (dst < (int)r ? dst : dst - 1)) * XSLOT_BYTES +
                              row_in_tile * XROW_BYTES;
#pragma unroll
                for (int c4 = 0; c4 < NU / 4; ++c4)
                  *reinterpret_cast<float4*>(sp + (((uoff >> 2) + c4) ^ swz) * 16) =
                      make_float4(sum[4 * c4], sum[4 * c4 + 1], sum[4 * c4 + 2], sum[4 * c4 + 3]);
              }
            }
            tc_fence_before();
            fence_proxy_async_smem();                 // staged slices -> visible to the bulk-copy engine
            __syncwarp();
            if (lane == 0) { mbar_arrive(&acc_empty[a]); mbar_arrive(&staged[xb]); }
            // one thread ships the three slices once all eight epilogue warps have staged their part
            // (bounded mbarrier wait, never a named barrier: a warp that gave up must not strand the rest)
            if (shipper && mbar_wait(&staged[xb], x_ph, wc) &&
                (!p.alias || mbar_wait_cluster(rdy, x_ph, wc))) {   // aliased: every peer's ring is idle
              mbar_expect_tx(&xchg[xb], 3 * XSLOT_BYTES);      // what this CTA is about to receive
#pragma unroll
              for (int dst = 0; dst < 4; ++dst)
                if (dst != (int)r) {
                  // this CTA is sender number `slot` among peer dst's three; addresses mapped on the
                  // spot (only this thread needs them)
                  const int slot = (int)r < dst ? (int)r : (int)r - 1;
                  dsmem_bulk_copy(mapa_shared(smem_u32(recv) + (xb * 3 + slot) * XSLOT_BYTES, dst),
                                  stage + ((size_t)xb * 3 + (dst < (int)r ? dst : dst - 1)) * XSLOT_BYTES,
                                  XSLOT_BYTES, mapa_shared(smem_u32(&xchg[xb]), dst));
                }
            }
            if (USE_FACTORS && !EARLY_FACTORS && st < T) {               // fills the wait for the peers' slices
              if (!fetch_gates()) { ok = false; break; }
              factors();
            }
            if (!mbar_wait_cluster(&xchg[xb], x_ph, wc)) { ok = false; break; }
            const uint8_t* rv = recv + (size_t)xb * (3 * XSLOT_BYTES) + row_in_tile * XROW_BYTES;
#pragma unroll
            for (int c4 = 0; c4 < NU / 4; ++c4) {
              const int off = (((uoff >> 2) + c4) ^ swz) * 16;
              const float4 s0 = *reinterpret_cast<const float4*>(rv + off);
              const float4 s1 = *reinterpret_cast<const float4*>(rv + XSLOT_BYTES + off);
              const float4 s2 = *reinterpret_cast<const float4*>(rv + 2 * XSLOT_BYTES + off);
              dhc[4 * c4 + 0] += s0.x + s1.x + s2.x;
              dhc[4 * c4 + 1] += s0.y + s1.y + s2.y;
              dhc[4 * c4 + 2] += s0.z + s1.z + s2.z;
              dhc[4 * c4 + 3] += s0.w + s1.w + s2.w;
            }
            if constexpr (TI >= 2) {
              // this warp has read the item's slices (the sums above hold them): tell the three peers.
              // Nothing is published by the signal, hence relaxed.
              __syncwarp();
              if (lane == 0) {
#pragma unroll
                for (int dst = 0; dst < 4; ++dst)
                  if (dst != (int)r) mbar_arrive_remote_relaxed(mapa_shared(smem_u32(consumed), dst));
              }
            }
          }
          if (st == 0) {
#pragma unroll
            for (int u = 0; u < NU; ++u) dhc[u] = 0.f;
            if (row_ok && p.dh_n) unpack8<T16>(ldg16(reinterpret_cast<const T16*>(p.dh_n) + (size_t)row * H + unit0), dhc);
          }
          if (st < T) {
            // ---- gate maths of step t for this thread's row and 8 units, two per packed word
            const int t = T - 1 - st;
            uint32_t qi[4], qf[4], qg[4], qo[4];
            if constexpr (USE_FACTORS) {
              if (!EARLY_FACTORS && st == 0) {            // later items computed them during the exchange
                if (!fetch_gates()) { ok = false; break; }
                factors();
              }
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                float r_[2][4];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                  const int u = 2 * w + e;
                  const float dh = fDd[u] + dhc[u];
                  const float dcv = fmaf(dh, fA[u], dc[j][u]);
                  r_[e][0] = dcv * fBi[u];
                  r_[e][1] = dcv * fBf[u];
                  r_[e][2] = dcv * fBg[u];
                  r_[e][3] = dh * fBo[u];
                  dc[j][u] = dcv * fSf[u];
                }
                qi[w] = pk2<T16>(r_[0][0], r_[1][0]);
                qf[w] = pk2<T16>(r_[0][1], r_[1][1]);
                qg[w] = pk2<T16>(r_[0][2], r_[1][2]);
                qo[w] = pk2<T16>(r_[0][3], r_[1][3]);
              }
            } else {
              // four interleaved tiles leave no registers for the factors: all of the maths here
              if (!fetch_gates()) { ok = false; break; }
              const uint32_t wi[4] = {pf[0].x, pf[0].y, pf[0].z, pf[0].w};
              const uint32_t wf[4] = {pf[1].x, pf[1].y, pf[1].z, pf[1].w};
              const uint32_t wg[4] = {pf[2].x, pf[2].y, pf[2].z, pf[2].w};
              const uint32_t wo[4] = {pf[3].x, pf[3].y, pf[3].z, pf[3].w};
              const uint32_t w1[4] = {pf[4].x, pf[4].y, pf[4].z, pf[4].w};
              const uint32_t w0[4] = {pf[5].x, pf[5].y, pf[5].z, pf[5].w};
              const uint32_t wd[4] = {pf[6].x, pf[6].y, pf[6].z, pf[6].w};
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                const float2 pi = cvt2<T16>(wi[w]), pff = cvt2<T16>(wf[w]), pg = cvt2<T16>(wg[w]), po = cvt2<T16>(wo[w]);
                const float2 c1 = cvt2<T16>(w1[w]), c0 = cvt2<T16>(w0[w]), dd = cvt2<T16>(wd[w]);
                float r_[2][4];
#pragma unroll
                for (int e = 0; e < 2; ++e) {
                  const int u = 2 * w + e;
                  const float si = sigmoid_fast(e ? pi.y : pi.x), sf = sigmoid_fast(e ? pff.y : pff.x);
                  const float so = sigmoid_fast(e ? po.y : po.x);
                  const float tg = tanh_fast(e ? pg.y : pg.x), tc = tanh_fast(e ? c1.y : c1.x);
                  const float dh = (e ? dd.y : dd.x) + dhc[u];
                  const float dcv = fmaf(dh * so, 1.f - tc * tc, dc[j][u]);
                  r_[e][0] = dcv * (tg * si * (1.f - si));
                  r_[e][1] = dcv * ((e ? c0.y : c0.x) * sf * (1.f - sf));
                  r_[e][2] = dcv * (si * (1.f - tg * tg));
                  r_[e][3] = dh * (tc * so * (1.f - so));
                  dc[j][u] = dcv * sf;
                }
                qi[w] = pk2<T16>(r_[0][0], r_[1][0]);
                qf[w] = pk2<T16>(r_[0][1], r_[1][1]);
                qg[w] = pk2<T16>(r_[0][2], r_[1][2]);
                qo[w] = pk2<T16>(r_[0][3], r_[1][3]);
              }
            }
            if constexpr (TMAEP) {
              // d_ifgo[t] goes back into the landing buffer the gates came from and leaves as one box.
              // The PREVIOUS item's box has been written by now: its buffer takes the gates of the item
              // two ahead, and (the peers' producers read d_ifgo next) the warp counts that item in.
              uint8_t* pbb = pbuf + (pub_it % 3) * 4096;
              *reinterpret_cast<uint4*>(pbb + p_off(0)) = make_uint4(qi[0], qi[1], qi[2], qi[3]);
              *reinterpret_cast<uint4*>(pbb + p_off(1)) = make_uint4(qf[0], qf[1], qf[2], qf[3]);
              *reinterpret_cast<uint4*>(pbb + p_off(2)) = make_uint4(qg[0], qg[1], qg[2], qg[3]);
              *reinterpret_cast<uint4*>(pbb + p_off(3)) = make_uint4(qo[0], qo[1], qo[2], qo[3]);
              fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) mbar_arrive(&pdone[pub_it % 3]);      // this warp's half of the box is in place
              if (lane == 0 && g == 0 && mbar_wait(&pdone[pub_it % 3], (uint32_t)(pub_it / 3) & 1u, wc)) {
                tma_store_4d(&tmD, pbb, unit0, bt * RB + q * 32, 0, t);      // (g == 0: unit0 is the pair's first unit)
                tma_store_commit();
                // The peers' producers read d_ifgo[t] next, so the pair counts the item in only once the
                // store has completed, and it waits for that at once: putting the wait off by an item (when
                // it costs nothing) lengthens every tile's hand-off chain by that item, and the chain is
                // what bounds the step even with four tiles interleaved (B=4096, H=512: 8.28 -> 7.75 ms).
                tma_store_wait<0>();
                mbar_arrive(&pfree[pub_it % 3]);
                mbar_arrive(&pub_bar[pub_it & 3]);
              }
            } else if (row_ok) {
              T16* dstp = dg + ((size_t)t * p.B + row) * H4 + unit0;
              stg16(dstp, make_uint4(qi[0], qi[1], qi[2], qi[3]));
              stg16(dstp + (size_t)H, make_uint4(qf[0], qf[1], qf[2], qf[3]));
              stg16(dstp + 2 * (size_t)H, make_uint4(qg[0], qg[1], qg[2], qg[3]));
              stg16(dstp + 3 * (size_t)H, make_uint4(qo[0], qo[1], qo[2], qo[3]));
            }
            // publish d_ifgo[t] rows of this warp, then (after the release) fetch the next item's inputs
            if (WRITER_FENCE) fence_proxy_async();
            __syncwarp();
            // interleaved tiles: hand the item to the publisher warp.  One tile: arrival per warp, or
            // (cta_publish) one per CTA and item - the last epilogue warp to get here publishes for all
            // (a warp can be at most four items ahead of another - the maths-only items that open a
            // chunk - so four counters never mix items)
            if (lane == 0) {
              if constexpr (TMAEP) {
                // counted in above, once the store has completed
              } else if constexpr (PUBLISHER) {
                mbar_arrive(&pub_bar[pub_it & 3]);      // the publisher warp releases for the CTA
              } else {
                const bool pub = !p.cta_publish ||
                                 (smem_count_arrive(&pub_cnt[pub_it & 3]) & (ITEM_WARPS - 1)) == ITEM_WARPS - 1;
                if (pub && !p.no_arrive) red_release_gpu_add(&p.flags[(size_t)t * p.nbt + bt], 1);
              }
            }
            ++pub_it;
            // bias-gradient sums: after the publication, off the hand-off chain
            if (want_db) {   // warp-uniform: tensor-memory loads and stores need the whole warp; rows past B add 0
              const uint32_t* qs[4] = {qi, qf, qg, qo};
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                uint32_t acc[8];
                tmem_ld_32x8(db_taddr + 8 * k, acc);
                tmem_ld_wait();
#pragma unroll
                for (int w = 0; w < 4; ++w) {
                  const float2 f2 = cvt2<T16>(qs[k][w]);
                  acc[2 * w] = __float_as_uint(__uint_as_float(acc[2 * w]) + (row_ok ? f2.x : 0.f));
                  acc[2 * w + 1] = __float_as_uint(__uint_as_float(acc[2 * w + 1]) + (row_ok ? f2.y : 0.f));
                }
                tmem_st_32x8(db_taddr + 8 * k, acc);
              }
              tmem_st_wait();
            }
            {
              int nj = j + 1, ns = st;
              if (nj == TI || pb + (ch * TI + nj) * p.nb_par >= p.nbt) { nj = 0; ns = st + 1; }
              if (ns < T) {
                prefetch(T - 1 - ns, pb + (ch * TI + nj) * p.nb_par);
                if (USE_FACTORS && EARLY_FACTORS) factors();
              }
              int fj = nj + 1, fs = ns;
              if (fj == TI || pb + (ch * TI + fj) * p.nb_par >= p.nbt) { fj = 0; fs = ns + 1; }
              if (fs < T) prefetch_far(T - 1 - fs, pb + (ch * TI + fj) * p.nb_par);
            }
          } else if (row_ok) {
            // ---- after the last step: the carries are the gradients of the initial state
            store8<T16>(reinterpret_cast<T16*>(p.dh0) + (size_t)row * H + unit0, dhc);
            store8<T16>(reinterpret_cast<T16*>(p.dc0) + (size_t)row * H + unit0, dc[j]);
          }
        }
      }
    }
    if (want_db) {
      float* dst = p.db_part + ((size_t)pb * 4 + q) * H4 + unit0;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        uint32_t acc[8];
        tmem_ld_32x8(db_taddr + 8 * k, acc);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          float v = __uint_as_float(acc[u]);
#pragma unroll
          for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
          if (lane == 0) dst[(size_t)k * H + u] = v;
        }
      }
    }
  }
  // ---------------------------------------------------------------- teardown
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
  cluster_sync_all();   // no CTA leaves while a peer may still write into its shared memory
}

// Column sums of d_ifgo [rows, cols] (16-bit) over DB_PARTS interleaved row groups -> part[DB_PARTS][cols].
// HBM-bound (the whole d_ifgo is read once): a thread owns 8 adjacent columns (one 16-byte load per
// row, a warp covers 512 contiguous bytes) and keeps 8 row loads in flight.
template <typename T16>
__global__ void __launch_bounds__(128) colsum_kernel(const T16* __restrict__ g, int rows, int cols, float* __restrict__ part) {
  const int col = (blockIdx.x * 128 + threadIdx.x) * 8;
  if (col >= cols) return;
  float s[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) s[u] = 0.f;
  const T16* src = g + col;
  int rr = blockIdx.y;
  for (; rr + 7 * DB_PARTS < rows; rr += 8 * DB_PARTS) {
    uint4 v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = ldg16(src + (size_t)(rr + i * DB_PARTS) * cols);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint32_t w[4] = {v[i].x, v[i].y, v[i].z, v[i].w};
#pragma unroll
      for (int u = 0; u < 4; ++u) { const float2 f = cvt2<T16>(w[u]); s[2 * u] += f.x; s[2 * u + 1] += f.y; }
    }
  }
  for (; rr < rows; rr += DB_PARTS) {
    const uint4 v = ldg16(src + (size_t)rr * cols);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int u = 0; u < 4; ++u) { const float2 f = cvt2<T16>(w[u]); s[2 * u] += f.x; s[2 * u + 1] += f.y; }
  }
  float* dst = part + (size_t)blockIdx.y * cols + col;
  *reinterpret_cast<float4*>(dst) = make_float4(s[0], s[1], s[2], s[3]);
  *reinterpret_cast<float4*>(dst + 4) = make_float4(s[4], s[5], s[6], s[7]);
}

static int bwd_cta_capacity() {
  static std::atomic<int> cached{0};
  int c = cached.load(std::memory_order_relaxed);
  if (c > 0) return c;
  int cap = 132;
  DeviceInfo di;
  if (get_device_info(&di) == BLSTM_OK && di.sm_count > 0) {
    cap = di.sm_count * 132 / 148 / 4 * 4;
    auto kern = bwd_kernel<1, __half>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448) == cudaSuccess) {
      cudaLaunchConfig_t cfg = {};
      cfg.gridDim = dim3(di.sm_count / 4 * 4);
      cfg.blockDim = dim3(384);
      cfg.dynamicSmemBytes = 232448;
      cudaLaunchAttribute attr;
      attr.id = cudaLaunchAttributeClusterDimension;
      attr.val.clusterDim.x = 4;
      attr.val.clusterDim.y = 1;
      attr.val.clusterDim.z = 1;
      cfg.attrs = &attr;
      cfg.numAttrs = 1;
      int mc = 0;
      if (cudaOccupancyMaxActiveClusters(&mc, kern, &cfg) == cudaSuccess && mc > 0) cap = mc * 4;
    }
    (void)cudaGetLastError();
  }
  cached.store(cap, std::memory_order_relaxed);
  return cap;
}

template <int TI, typename T16>
static int launch_bwd_t(const BwdPlan& pl, const CUtensorMap& tw, const CUtensorMap& tg, const CUtensorMap& ti,
                        const CUtensorMap& td, BwdParams& p, cudaStream_t st) {
  auto kern = bwd_kernel<TI, T16>;
  BLSTM_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)pl.smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(pl.grid);
  cfg.blockDim = dim3(pl.threads);
  cfg.dynamicSmemBytes = pl.smem;
  cfg.stream = st;
  cudaLaunchAttribute attrs[2];
  attrs[0].id = cudaLaunchAttributeClusterDimension;
  attrs[0].val.clusterDim.x = 4;
  attrs[0].val.clusterDim.y = 1;
  attrs[0].val.clusterDim.z = 1;
  attrs[1].id = cudaLaunchAttributeCooperative;
  attrs[1].val.cooperative = 1;
  cfg.attrs = attrs;
  // FASTLSTM_B200_NO_COOP=1 drops the cooperative attribute (profilers that replay kernels refuse
  // a cooperative cluster launch); co-residency then rests on the occupancy check below alone.
  static const bool no_coop = [] { const char* e = getenv("FASTLSTM_B200_NO_COOP"); return e && e[0] == '1'; }();
  cfg.numAttrs = no_coop ? 1 : 2;
  // every CTA spins on its peers: the whole grid has to be resident at once
  int max_clusters = 0;
  BLSTM_CUDA_OK(cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg));
  if (max_clusters * 4 < pl.grid) return BLSTM_E_NOT_CORESIDENT;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kern, tw, tg, ti, td, p);
  if (cfg.numAttrs == 2 && (e == cudaErrorNotSupported || e == cudaErrorCooperativeLaunchTooLarge)) {
    // Only when the driver refuses the cooperative + cluster combination as such is the cooperative
    // attribute dropped (co-residency then rests on the occupancy check above); any other launch error
    // is reported as it is.
    (void)cudaGetLastError();
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, kern, tw, tg, ti, td, p);
  }
  BLSTM_CUDA_OK(e);
  count_launch();
  return BLSTM_OK;
}

}  // namespace sm100

using namespace sm100;

bool sm100_recurrence_supported(const blstm_desc& d, int phase) {
  return phase == BLSTM_PHASE_BWD ? make_bwd_plan(d).ok : make_plan(d, phase).ok;
}
size_t sm100_recurrence_workspace(const blstm_desc& d, int phase) {
  return phase == BLSTM_PHASE_BWD ? make_bwd_plan(d).ws_bytes : make_plan(d, phase).ws_bytes;
}

int sm100_plan_detail(const blstm_desc& d, int phase, char* buf, size_t n) {
  if (phase == BLSTM_PHASE_BWD) {
    const BwdPlan p = make_bwd_plan(d);
    if (!p.ok) return 0;
    char wh[48];
    if (p.ws) snprintf(wh, sizeof(wh), "%d/%d chunks resident, rest streamed", p.kr, d.hidden_size / RK);
    else snprintf(wh, sizeof(wh), "resident");
    return snprintf(buf, n, "sm100 bwd cluster=4 units_per_cluster=64 TI=%d grid=%d threads=%d stages=%d issuers=%d "
                    "loaders=%d rows_per_stage=%d wh=%s alias=%d smem=%zu", p.TI, p.grid, p.threads, p.stages, p.ni, p.nl,
                    p.hb / 128, wh, p.alias, p.smem);
  }
  const RecPlan p = make_plan(d, phase);
  if (!p.ok) return 0;
  if (sm100_fwd_cluster_shape(d))
    return snprintf(buf, n, "sm100 fwd cluster=%d (one per batch tile, h handed over in shared memory) UH=16 TI=1 grid=%d "
                    "threads=288 wh=resident", d.hidden_size / 16, d.hidden_size / 16 * p.nbt);
  char wh[48];
  if (p.ws) snprintf(wh, sizeof(wh), "%d/%d chunks resident, rest streamed", p.kr, d.hidden_size / RK);
  else snprintf(wh, sizeof(wh), "resident");
  return snprintf(buf, n, "sm100 fwd UH=%d TI=%d grid=%d threads=%d stages=%d issuers=%d loaders=%d rows_per_stage=%d wh=%s smem=%zu",
                  p.UH, p.TI, p.grid, p.threads, p.stages, p.ni, p.nl, p.hb / 128, wh, p.smem);
}

int sm100_fwd_recurrence(const blstm_desc& d, void* ifgo, const void* Wh, void* out, void* cell, void* ws,
                         size_t ws_bytes, cudaStream_t st) {
  const RecPlan pl = make_plan(d, BLSTM_PHASE_FWD);
  if (!pl.ok) return BLSTM_E_UNSUPPORTED;
  if (ws_bytes < pl.ws_bytes) return BLSTM_E_WORKSPACE;
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc) return rc;
  if (!di.coop || pl.grid > di.sm_count) return BLSTM_E_NOT_CORESIDENT;
  const int H = d.hidden_size, B = d.batch, T = d.seq_len;
  CUtensorMap tw, th;
  {  // Wh [4H,H] as {k, unit row, gate}
    uint64_t dims[3] = {(uint64_t)H, (uint64_t)H, 4};
    uint64_t str[2] = {(uint64_t)H * 2, (uint64_t)H * H * 2};
    uint32_t box[3] = {RK, (uint32_t)pl.UH, 4};
    rc = encode_tensor_map(&tw, Wh, 3, dims, str, box);
    if (rc) return rc;
  }
  {  // out [T+1,B,H] as {k, batch row, t}: rows past B are zero-filled, never another timestep
    uint64_t dims[3] = {(uint64_t)H, (uint64_t)B, (uint64_t)(T + 1)};
    uint64_t str[2] = {(uint64_t)H * 2, (uint64_t)B * H * 2};
    uint32_t box[3] = {RK, (uint32_t)(pl.hb / 128), 1};
    rc = encode_tensor_map(&th, out, 3, dims, str, box);
    if (rc) return rc;
  }
  CUtensorMap tp = th;              // only read by the kernels that interleave tiles
  if (pl.TI >= 2) {
    const int NU = 4 * pl.UH / pl.epi_warps;
    {  // ifgo [T,B,4H] as {unit, batch row, gate, t}: a box is one warp's 4 gates x 32 rows x NU units;
       // the box's inner extent equals the swizzle span (32 bytes) or is a single 16-byte piece (none)
      uint64_t dims[4] = {(uint64_t)H, (uint64_t)B, 4, (uint64_t)T};
      uint64_t str[3] = {(uint64_t)4 * H * 2, (uint64_t)H * 2, (uint64_t)B * 4 * H * 2};
      uint32_t box[4] = {(uint32_t)NU, 32, 4, 1};
      rc = encode_tensor_map(&tp, ifgo, 4, dims, str, box, 2, NU == 16 ? 32 : 0);
      if (rc) return rc;
    }
  }
  BLSTM_CUDA_OK(cudaMemsetAsync(ws, 0, pl.ws_bytes, st));
  {  // small hidden sizes with few batch tiles: hand-off inside one cluster per tile
    bool taken = false;
    rc = sm100_fwd_cluster(d, ifgo, Wh, out, cell, ws, st, &taken);
    if (rc || taken) return rc;
  }
  FwdParams p;
  p.npb = pl.npb;
  p.ep_bytes = (int)pl.ep_bytes;
  p.T = T; p.B = B; p.H = H;
  p.nbt = pl.nbt; p.nh = pl.nh; p.nb_par = pl.nb_par; p.ntl = pl.ntl;
  p.stages = pl.stages;
  p.ni = pl.ni;
  p.nl = pl.nl;
  p.ws = pl.ws;
  p.kr = pl.kr;
  p.hb = pl.hb;
  p.stage_bytes = (int)pl.stage_bytes;
  p.fmt = d.dtype == BLSTM_BF16 ? 1 : 0;
  p.no_arrive = (d.flags & BLSTM_FLAG_TEST_NO_ARRIVE) ? 1 : 0;
  p.inference = (d.flags & BLSTM_FLAG_INFERENCE) ? 1 : 0;
  // One arrival per CTA and item (the last epilogue warp to finish publishes for all; with interleaved
  // tiles the publisher warp).  Measured 3-7 % faster than one arrival per warp from 64 arrivals per
  // counter on (B=512 H=512: 1.43 -> 1.33 ms; H=1024: 4.06 -> 3.95 ms; H=2048: 9.4 -> 9.0 ms): the
  // same-address reductions serialise in L2 and the counter completes with the slowest of them.
  p.cta_publish = (pl.nh * pl.epi_warps >= 64 || pl.TI >= 2) ? 1 : 0;
  p.flag_target = p.cta_publish ? pl.nh : pl.nh * pl.epi_warps;
  p.limit_ns = d.wait_limit_us > 0 ? (unsigned long long)d.wait_limit_us * 1000ull : kDefaultWaitNs;
  p.ctl = reinterpret_cast<Control*>(ws);
  p.flags = reinterpret_cast<int*>(static_cast<char*>(ws) + pl.off_flags);
  p.ifgo = ifgo; p.out = out; p.cell = cell;
  const bool bf = d.dtype == BLSTM_BF16;
#define BLSTM_FWD_CASE(U, I)                                                                         \
  if (pl.UH == U && pl.TI == I)                                                                      \
    return bf ? launch_fwd_t<U, I, __nv_bfloat16>(pl, tw, th, tp, p, st)                             \
              : launch_fwd_t<U, I, __half>(pl, tw, th, tp, p, st);
  BLSTM_FWD_CASE(16, 1)
  BLSTM_FWD_CASE(16, 2)
  BLSTM_FWD_CASE(16, 4)
  BLSTM_FWD_CASE(32, 1)
  BLSTM_FWD_CASE(32, 2)
  BLSTM_FWD_CASE(32, 4)
#undef BLSTM_FWD_CASE
  return BLSTM_E_UNSUPPORTED;
}

int sm100_bwd_recurrence(const blstm_desc& d, const void* dout, const void* dh_n, const void* dc_n,
                         const void* ifgo, const void* cell, const void* Wh, void* d_ifgo, void* dh0, void* dc0,
                         float* db, void* ws, size_t ws_bytes, cudaStream_t st) {
  const BwdPlan pl = make_bwd_plan(d);
  if (!pl.ok) return BLSTM_E_UNSUPPORTED;
  if (ws_bytes < pl.ws_bytes) return BLSTM_E_WORKSPACE;
  DeviceInfo di;
  int rc = get_device_info(&di);
  if (rc) return rc;
  if (!di.coop || pl.grid > di.sm_count) return BLSTM_E_NOT_CORESIDENT;
  const int H = d.hidden_size, B = d.batch, T = d.seq_len;
  CUtensorMap tw, tg;
  {  // Wh [4H,H] row-major: rows are K (gate-major), columns the output units (N-major operand)
    uint64_t dims[2] = {(uint64_t)H, (uint64_t)4 * H};
    uint64_t str[1] = {(uint64_t)H * 2};
    uint32_t box[2] = {64, 64};
    rc = encode_tensor_map(&tw, Wh, 2, dims, str, box);
    if (rc) return rc;
  }
  {  // d_ifgo [T,B,4H] as {k, batch row, t}
    uint64_t dims[3] = {(uint64_t)4 * H, (uint64_t)B, (uint64_t)T};
    uint64_t str[2] = {(uint64_t)4 * H * 2, (uint64_t)B * 4 * H * 2};
    uint32_t box[3] = {RK, (uint32_t)(pl.hb / 128), 1};
    rc = encode_tensor_map(&tg, d_ifgo, 3, dims, str, box);
    if (rc) return rc;
  }
  CUtensorMap ti = tg, td = tg;     // only read by the kernels that interleave tiles
  if (pl.TI >= 2) {
    // ifgo and d_ifgo [T,B,4H] as {unit, batch row, gate, t}: a box is a warp pair's 4 gates x 32 rows x 16 units
    // (32-byte rows, 32-byte swizzle)
    uint64_t dims[4] = {(uint64_t)H, (uint64_t)B, 4, (uint64_t)T};
    uint64_t str[3] = {(uint64_t)4 * H * 2, (uint64_t)H * 2, (uint64_t)B * 4 * H * 2};
    uint32_t box[4] = {16, 32, 4, 1};
    rc = encode_tensor_map(&ti, ifgo, 4, dims, str, box, 2, 32);
    if (rc) return rc;
    rc = encode_tensor_map(&td, d_ifgo, 4, dims, str, box, 2, 32);
    if (rc) return rc;
  }
  BLSTM_CUDA_OK(cudaMemsetAsync(ws, 0, pl.off_db, st));
  BwdParams p;
  p.ep_bytes = (int)pl.ep_bytes;
  p.T = T; p.B = B; p.H = H;
  p.nbt = pl.nbt; p.nug = pl.nug; p.nb_par = pl.nb_par; p.ntl = pl.ntl; p.stages = pl.stages; p.ni = pl.ni;
  p.nl = pl.nl;
  p.ws = pl.ws; p.kr = pl.kr; p.hb = pl.hb; p.stage_bytes = (int)pl.stage_bytes;
  p.alias = pl.alias;
  p.fmt = d.dtype == BLSTM_BF16 ? 1 : 0;
  p.no_arrive = (d.flags & BLSTM_FLAG_TEST_NO_ARRIVE) ? 1 : 0;
  // One arrival per epilogue warp up to about a thousand per counter, one per CTA beyond that and
  // whenever tiles are interleaved.  (Unlike in the forward kernel, per-CTA arrivals measured 2-5 %
  // SLOWER here below that size: eight warps elect the publisher instead of four.)
  p.cta_publish = ((H / 16) * 8 >= 1024 || pl.TI >= 2) ? 1 : 0;
  p.flag_target = p.cta_publish ? H / 16 : (H / 16) * 8;
  p.limit_ns = d.wait_limit_us > 0 ? (unsigned long long)d.wait_limit_us * 1000ull : kDefaultWaitNs;
  p.ctl = reinterpret_cast<Control*>(ws);
  p.flags = reinterpret_cast<int*>(static_cast<char*>(ws) + pl.off_flags);
  p.dout = dout; p.dh_n = dh_n; p.dc_n = dc_n; p.ifgo = ifgo; p.cell = cell;
  p.d_ifgo = d_ifgo; p.dh0 = dh0; p.dc0 = dc0;
  p.db_part = db ? reinterpret_cast<float*>(static_cast<char*>(ws) + pl.off_db) : nullptr;
  const bool bf = d.dtype == BLSTM_BF16;
  if (pl.TI == 1)      rc = bf ? launch_bwd_t<1, __nv_bfloat16>(pl, tw, tg, ti, td, p, st) : launch_bwd_t<1, __half>(pl, tw, tg, ti, td, p, st);
  else if (pl.TI == 2) rc = bf ? launch_bwd_t<2, __nv_bfloat16>(pl, tw, tg, ti, td, p, st) : launch_bwd_t<2, __half>(pl, tw, tg, ti, td, p, st);
  else                 rc = bf ? launch_bwd_t<4, __nv_bfloat16>(pl, tw, tg, ti, td, p, st) : launch_bwd_t<4, __half>(pl, tw, tg, ti, td, p, st);
  if (rc) return rc;
  if (db) return reduce_db(p.db_part, pl.nb_par * 4, 4 * H, db, st);   // the kernel left one row per CTA group and row quarter
  return BLSTM_OK;
}

int sm100_bias_grad(const blstm_desc& d, const void* d_ifgo, float* db, void* ws, size_t ws_bytes, cudaStream_t st) {
  const BwdPlan pl = make_bwd_plan(d);
  if (!pl.ok) return BLSTM_E_UNSUPPORTED;
  if (ws_bytes < pl.ws_bytes) return BLSTM_E_WORKSPACE;
  float* part = reinterpret_cast<float*>(static_cast<char*>(ws) + pl.off_db);
  const int rows = d.seq_len * d.batch, cols = 4 * d.hidden_size;
  dim3 grid(cdiv(cols, 1024), DB_PARTS);
  if (d.dtype == BLSTM_BF16) colsum_kernel<__nv_bfloat16><<<grid, 128, 0, st>>>((const __nv_bfloat16*)d_ifgo, rows, cols, part);
  else                       colsum_kernel<__half><<<grid, 128, 0, st>>>((const __half*)d_ifgo, rows, cols, part);
  BLSTM_CUDA_OK(cudaGetLastError());
  count_launch();
  return reduce_db(part, DB_PARTS, cols, db, st);
}

}  // namespace blstm
