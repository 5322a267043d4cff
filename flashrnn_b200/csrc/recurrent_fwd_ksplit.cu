// Persistent forward recurrence for heads too wide for one CTA's tensor memory (sm_100a).
//
// A (head, batch tile) group is a 2-D grid of CTAs: D/32 row tiles (32 hidden units = GR*32 rows
// of the recurrent matrix each) times KS splits of the contraction dimension. CTA (rt, ks) keeps
// R[rows of tile rt, K-chunk ks] in tensor memory for the whole sequence. Per step:
//   1. tcgen05.mma over its K-chunk of round_bf16(h_{t-1})            -> partial gates [rows x batch]
//   2. the KS CTAs of a row tile form a thread-block cluster; every accumulator row is sent with
//      asynchronous DSMEM stores to the CTA that owns its unit (32/KS units each), which adds the
//      KS partial sums in a fixed order                               -> gates of the owned units
//   3. cell epilogue for the owned units, states to global memory
//   4. round_bf16(h_t) of the owned units goes to the group's operand buffer in global memory; there
//      is no flag: a receiver polls the data words, which differ from the all-ones fill once
//      written, and copies its K-chunk into shared memory as operand B of the next step.
// All CTAs of the launch must be resident at the same time (cooperative launch).
//
// Same arithmetic as reference.recurrence (flashrnn/flashrnn2/reference.py:72-114); the 2-D
// decomposition follows the idea of the reference's hybrid kernel (flashrnn/flashrnn2/hybrid_fw2d.cu:404-419).
#include "frnn_common.cuh"

namespace frnn {

namespace {

constexpr int kEpiThreads = 128;
constexpr int kThreads = 192;  // 4 epilogue warps + MMA warp + TMA warp
constexpr int kWxStages = 4;
constexpr int kMaxKc = 896;    // K-chunk bound: its R tile (Kc/2 columns) plus the accumulator fit 512 TMEM columns

template <int CELL, int BV, int KS, bool WX_BF16>
struct KsCfg {
  using CT = CellTraits<CELL>;
  static constexpr int U = 32;                  // units per row tile
  static constexpr int UO = U / KS;             // units whose gates this CTA sums up and owns
  static constexpr int BT = 16;                 // UMMA N (M = 128 needs a multiple of 16)
  static constexpr int ROWS = CT::GR * U;       // accumulator rows in use
  static constexpr int RPP = kEpiThreads / UO;  // batch rows covered by one pass of the epilogue threads
  static constexpr int NI = BV / RPP < 1 ? 1 : BV / RPP;  // (batch row, unit) items per thread
  static constexpr int A_COL0 = 32;
  static constexpr int WX_ES = WX_BF16 ? 2 : 4;
  static constexpr int WX_STAGE_BYTES = BV * CT::GW * UO * WX_ES;
  static constexpr int PART_FLOATS = KS * CT::GR * BV * UO;  // one parity: [source][gate][batch][unit]
  static constexpr int PART_BYTES = PART_FLOATS * 4;
  static_assert(BV == 8 || BV == 16, "batch tile");
  static_assert(ROWS <= 128, "one accumulator tile");
  static_assert(KS == 2 || KS == 4, "cluster width");
};

__device__ __forceinline__ void report_ks(int* err, int code, int detail) {
  if (atomicCAS(err, 0, code) == 0) {
    err[1] = detail;
    err[2] = static_cast<int>(blockIdx.x);
  }
  __threadfence();
}

// EXT: the call is one chunk of a longer sequence (T_total, t0), stores bf16 snapshots or clips h_t; the plain
// instantiation folds all three away.
template <int CELL, int BV, int KS, bool WX_BF16, bool EXT>
__global__ void __launch_bounds__(kThreads, 1)
frnn_fwd_ks_kernel(const FwdParams p, const __grid_constant__ CUtensorMap wx_map) {
  using Cfg = KsCfg<CELL, BV, KS, WX_BF16>;
  using CT = typename Cfg::CT;
  constexpr int BT = Cfg::BT, UO = Cfg::UO, NI = Cfg::NI, RPP = Cfg::RPP;

  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) uint64_t s_hbar[2];
  __shared__ __align__(8) uint64_t s_mma_bar;
  __shared__ __align__(8) uint64_t s_part_bar[2];
  __shared__ __align__(8) uint64_t s_wx_full[kWxStages];
  __shared__ __align__(8) uint64_t s_wx_empty[kWxStages];
  __shared__ uint32_t s_tmem_base;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long t_entry = clock64();
  const int D = p.D, N = p.N, T = p.T, B = p.B;
  const int RT = D / 32;
  const int ks = static_cast<int>(blockIdx.x % KS);  // == rank inside the cluster
  const int rt = static_cast<int>((blockIdx.x / KS) % RT);
  const int gid = static_cast<int>(blockIdx.x / (KS * RT));
  const int n = gid % N;
  const int b0 = (gid / N) * BV;
  const int bv = min(BV, B - b0);
  const int Kc = D / KS;
  const int hbuf_bytes = BT * Kc * 2;
  uint8_t* const hbuf = smem;
  float* const part = reinterpret_cast<float*>(smem + 2 * hbuf_bytes);
  uint8_t* const wxs = smem + ((2 * hbuf_bytes + 2 * Cfg::PART_BYTES + 127) & ~127);
  const volatile int* abort_flag = p.err;
  const uint64_t limit = p.wait_limit_ns;
  // four operand slots per group in global memory, each [K-chunk][BT x Kc, K-major]; h_t goes to slot (t + 1) % 4
  uint8_t* const xg_h = p.xg_data + static_cast<size_t>(gid) * 4 * (static_cast<size_t>(BT) * D * 2);
  const size_t slot_bytes = static_cast<size_t>(BT) * D * 2;
  const int mute_from = p.err[4] != 0 ? p.err[5] : 0x7fffffff;  // test hook: nobody publishes from this step on
  // Second test hook, race verification by delay injection (err[6] = seed, see jitter_stall). It is compiled into the
  // fp32-Wx instantiations only: the exchange code is the same for both Wx types, and even the untaken per-step test
  // costs the bf16 backward more than 1 %.
  constexpr bool kJitter = !WX_BF16;
  const uint32_t jitter = kJitter ? static_cast<uint32_t>(p.err[6]) : 0u;
  const bool zero_first = p.zero_first_dev != nullptr ? *p.zero_first_dev != 0 : p.slstm_zero_first != 0;
  const int hist_states = p.output_mode == 0 ? CT::S : (p.output_mode == 1 ? 1 : 0);  // state planes written per step
  const bool prof = p.err[3] != 0 && blockIdx.x == 0 && lane == 0 && (warp == 0 || warp == 4);
  uint32_t tmem_cols = 64;
  while (tmem_cols < static_cast<uint32_t>(Cfg::A_COL0 + Kc / 2)) tmem_cols <<= 1;

  // ---------------- prologue ----------------
  if (tid == 0) {
    mbar_init(smem_u32(&s_hbar[0]), kEpiThreads);
    mbar_init(smem_u32(&s_hbar[1]), kEpiThreads);
    mbar_init(smem_u32(&s_mma_bar), 1);
    mbar_init(smem_u32(&s_part_bar[0]), 1);
    mbar_init(smem_u32(&s_part_bar[1]), 1);
    for (int s = 0; s < kWxStages; ++s) {
      mbar_init(smem_u32(&s_wx_full[s]), 1);
      mbar_init(smem_u32(&s_wx_empty[s]), kEpiThreads);
    }
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(&s_tmem_base), tmem_cols);
    tmem_relinquish_alloc();
  }
  for (int i = tid; i < 2 * hbuf_bytes / 16; i += kThreads) reinterpret_cast<uint4*>(hbuf)[i] = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();
  // round_bf16(initial h) of this CTA's K-chunk -> operand buffer 0
  for (int i = tid; i < bv * (Kc / 2); i += kThreads) {
    const int b = i / (Kc / 2), k = 2 * (i % (Kc / 2));
    const float2 v = *reinterpret_cast<const float2*>(p.initial + (static_cast<size_t>(b0 + b) * N + n) * D + ks * Kc + k);
    *reinterpret_cast<uint32_t*>(hbuf + kmajor_offset(BT, b, k)) = pack_bf16x2(v.x, v.y);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = s_tmem_base;

  if (warp < 4) {
    // rows (gate g, unit u) of the tile, K-chunk ks -> tensor memory (lane = row, column = two k)
    const bool valid = tid < Cfg::ROWS;
    const int g = valid ? tid / 32 : 0, u = tid % 32;
    const __nv_bfloat16* src = p.R + ((static_cast<size_t>(g) * N + n) * D + rt * 32 + u) * D + ks * Kc;
    for (int c0 = 0; c0 < Kc / 2; c0 += 8) {
      uint32_t r[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
      if (valid) {
        const uint4 lo = __ldg(reinterpret_cast<const uint4*>(src + 2 * c0));
        const uint4 hi = __ldg(reinterpret_cast<const uint4*>(src + 2 * c0 + 8));
        r[0] = lo.x; r[1] = lo.y; r[2] = lo.z; r[3] = lo.w;
        r[4] = hi.x; r[5] = hi.y; r[6] = hi.z; r[7] = hi.w;
      }
      tmem_st_x8(tmem_addr(tbase, 32 * warp, Cfg::A_COL0 + c0), r);
    }
    tmem_st_wait();
  }

  // cell items of this thread: unit `ul` of the owned slice, batch rows ib0 + j * RPP
  const int ul = tid % UO, ib0 = tid / UO;
  const int d0 = rt * 32 + ks * UO + ul;  // unit inside the head
  float st[NI][CT::S];
  float bias[CT::GB];
  bool act[NI];
  const int Tt = EXT ? p.T_total : T, t0 = EXT ? p.t0 : 0;
  const bool out_bf16 = EXT && p.out_bf16 != 0;
  const size_t sBTND = static_cast<size_t>(B) * Tt * N * D;
  const size_t ND = static_cast<size_t>(N) * D;
#pragma unroll
  for (int j = 0; j < NI; ++j) {
    const int ib = ib0 + j * RPP;
    act[j] = warp < 4 && ib < bv;
#pragma unroll
    for (int s = 0; s < CT::S; ++s)
      st[j][s] = act[j] ? p.initial[static_cast<size_t>(s) * B * ND + (static_cast<size_t>(b0 + ib)) * ND + n * D + d0] : 0.0f;
    if (act[j] && p.hbf != nullptr)
      p.hbf[((static_cast<size_t>(b0 + ib) * (T + 1)) * N + n) * D + d0] = __float2bfloat16_rn(st[j][0]);
  }
#pragma unroll
  for (int g = 0; g < CT::GB; ++g) bias[g] = warp < 4 ? p.bias[(static_cast<size_t>(g) * N + n) * D + d0] : 0.0f;
  constexpr uint32_t part_tx = static_cast<uint32_t>(KS) * CT::GR * UO * BV * 4u;
  if (warp == 4 && lane == 0) {
    mbar_arrive_expect_tx(smem_u32(&s_part_bar[0]), part_tx);
    if (T >= 2) mbar_arrive_expect_tx(smem_u32(&s_part_bar[1]), part_tx);
    tma_prefetch_desc(&wx_map);
  }
  fence_proxy_async();
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();
  if (prof && warp == 0) p.err[20] = static_cast<int>(clock64() - t_entry);

  // ---------------- main loops ----------------
  if (warp == 4) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(128, BT, false, false);
      long long pw = 0, pi = 0;
      int committed = 0;  // steps whose tcgen05.mma have been issued and committed
      for (int t = 0; t < T; ++t) {
        if (kJitter && jitter != 0u) jitter_stall(jitter, 1u, static_cast<uint32_t>(t));
        const int pb = t & 1;
        const long long m0 = prof ? clock64() : 0;
        if (t >= 1 && !mbar_wait_bounded<false, true>(smem_u32(&s_hbar[pb]), ((t - 1) >> 1) & 1, limit, abort_flag)) {
          report_ks(p.err, kErrWaitH, t);
          break;
        }
        fence_proxy_async_smem();
        tc_fence_after_sync();
        const long long m1 = prof ? clock64() : 0;
        const uint32_t hb = smem_u32(hbuf + pb * hbuf_bytes);
        for (int kk = 0; kk < Kc / 16; ++kk) {
          const uint64_t bdesc = umma_smem_desc(hb + kk * 2 * (BT * 16), BT * 16, 128);
          umma_bf16_ts(tbase, tbase + Cfg::A_COL0 + kk * 8, bdesc, idesc, kk > 0 ? 1u : 0u);
        }
        umma_commit(smem_u32(&s_mma_bar));
        ++committed;
        if (prof) { pw += m1 - m0; pi += clock64() - m1; }
      }
      // Before the CTA may release its tensor memory and shared memory every issued tcgen05.mma must
      // have finished. Normally the epilogue has waited for the last commit already; after a failed
      // wait it has not (it stops waiting), so the issuing thread waits here itself. The commit
      // completes without any other party, hence no abort flag and a plain bound.
      if (committed > 0) mbar_wait_bounded<false, true>(smem_u32(&s_mma_bar), (committed - 1) & 1, limit, nullptr);
      if (prof) { p.err[16] = static_cast<int>(pw); p.err[17] = static_cast<int>(pi); }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      const uint32_t stage_tx = static_cast<uint32_t>(p.wx_box_b) * CT::GW * UO * Cfg::WX_ES;
      for (int t = 0; t < T; ++t) {
        const int s = t % kWxStages;
        if (t >= kWxStages) {
          if (!mbar_wait_bounded<false>(smem_u32(&s_wx_empty[s]), ((t / kWxStages) - 1) & 1, limit, abort_flag)) {
            report_ks(p.err, kErrWaitEmpty, t);
            break;
          }
        }
        // Once any wait of the grid has run out, the epilogue threads stop waiting for the stages and
        // release them early, so "released" no longer implies that the previous copy into this stage
        // has landed; arming its barrier again could then be a second arrival in one phase. The flag
        // is set before any thread skips a wait, so checking it after the wait above is enough.
        if (*abort_flag != 0) break;
        mbar_arrive_expect_tx(smem_u32(&s_wx_full[s]), stage_tx);
        tma_load_5d(smem_u32(wxs + s * Cfg::WX_STAGE_BYTES), &wx_map, smem_u32(&s_wx_full[s]), rt * 32 + ks * UO, n, 0, t0 + t, b0);
      }
    }
  } else {
    // accumulator row of this thread: gate g_row, unit u_row of the tile; its sums go to the owner of the unit
    const bool row_valid = tid < Cfg::ROWS;
    const int g_row = tid / 32, u_row = tid % 32;
    const int owner = u_row / UO;
    const uint32_t part_local = smem_u32(part) + static_cast<uint32_t>((ks * CT::GR + g_row) * BV * UO + (u_row % UO)) * 4u;
    const uint32_t part_remote = map_to_cta(part_local, owner);
    const uint32_t bar_remote0 = map_to_cta(smem_u32(&s_part_bar[0]), owner);
    const uint32_t bar_remote1 = map_to_cta(smem_u32(&s_part_bar[1]), owner);
    // packet (8 units of one batch row) this thread publishes when it is the first lane of its group of eight
    const int chunk = d0 / Kc, kin = d0 % Kc;
    const size_t pub_base = static_cast<size_t>(chunk) * hbuf_bytes + static_cast<size_t>(kin >> 3) * (BT * 16);
    // packets this thread fetches from the group's operand buffer: rows `prow`, k-groups kg0 + j * KG_STEP
    constexpr int KG_STEP = kEpiThreads / BV;
    constexpr int XCH = (kMaxKc / 8 + KG_STEP - 1) / KG_STEP;
    const int prow = tid % BV, kg0 = tid / BV;
    const size_t poll_base = static_cast<size_t>(ks) * hbuf_bytes + static_cast<size_t>(kg0) * (BT * 16) + prow * 16;
    long long pc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    bool dead = false;  // after a failed wait the warp keeps walking through the loop without waiting
    for (int t = 0; t < T; ++t) {
      if (kJitter && jitter != 0u) jitter_stall(jitter, 0u, static_cast<uint32_t>(t));
      const int s = t % kWxStages, pb = t & 1;
      const long long c0 = prof ? clock64() : 0;
      if (!dead && !mbar_wait_bounded<false, true>(smem_u32(&s_wx_full[s]), (t / kWxStages) & 1, limit, abort_flag)) {
        report_ks(p.err, kErrWaitWx, t);
        dead = true;
      }
      float wx[NI][CT::GW];
#pragma unroll
      for (int j = 0; j < NI; ++j) {
        const int ib = ib0 + j * RPP;
#pragma unroll
        for (int g = 0; g < CT::GW; ++g) {
          const int e = (ib * CT::GW + g) * UO + ul;
          if (ib < BV) {
            if constexpr (WX_BF16) wx[j][g] = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(wxs + s * Cfg::WX_STAGE_BYTES)[e]);
            else wx[j][g] = reinterpret_cast<const float*>(wxs + s * Cfg::WX_STAGE_BYTES)[e];
          } else {
            wx[j][g] = 0.0f;
          }
        }
      }
      mbar_arrive(smem_u32(&s_wx_empty[s]));
      const long long c1 = prof ? clock64() : 0;
      if (!dead && !mbar_wait_bounded<false, true>(smem_u32(&s_mma_bar), t & 1, limit, abort_flag)) {
        report_ks(p.err, kErrWaitMma, t);
        dead = true;
      }
      tc_fence_after_sync();
      const long long c2 = prof ? clock64() : 0;
      // partial gates of this row for all batch columns -> the owner's buffer [source][gate][batch][unit]
      {
        uint32_t r[BV / 8][8];
#pragma unroll
        for (int c = 0; c < BV / 8; ++c) tmem_ld_x8(tmem_addr(tbase, 32 * warp, 8 * c), r[c]);
        tmem_ld_wait();
        tc_fence_before_sync();
        if (row_valid && !dead) {
          const uint32_t dst = part_remote + static_cast<uint32_t>(pb) * Cfg::PART_BYTES;
          const uint32_t bar = pb ? bar_remote1 : bar_remote0;
#pragma unroll
          for (int c = 0; c < BV / 8; ++c)
#pragma unroll
            for (int q = 0; q < 8; ++q) st_async_b32(dst + (8 * c + q) * UO * 4, r[c][q], bar);
        }
      }
      const long long c3 = prof ? clock64() : 0;
      if (!dead && !mbar_wait_bounded<true, true>(smem_u32(&s_part_bar[pb]), (t >> 1) & 1, limit, abort_flag)) {
        report_ks(p.err, kErrWaitPart, t);
        dead = true;
      }
      const long long c4 = prof ? clock64() : 0;
      float ry[NI][CT::GR];
      {
        const float* pbuf = part + pb * Cfg::PART_FLOATS;
#pragma unroll
        for (int j = 0; j < NI; ++j) {
          const int ib = ib0 + j * RPP;
#pragma unroll
          for (int g = 0; g < CT::GR; ++g) {
            float acc = 0.0f;
            if (ib < BV) {
#pragma unroll
              for (int src = 0; src < KS; ++src) acc += pbuf[((src * CT::GR + g) * BV + ib) * UO + ul];
            }
            ry[j][g] = acc;
          }
        }
      }
      // the buffer of this parity is free again: arm its barrier for step t + 2 (only a barrier whose
      // phase has completed may be armed again, hence not after a failed wait)
      if (tid == 0 && !dead && t + 2 < T) mbar_arrive_expect_tx(smem_u32(&s_part_bar[pb]), part_tx);
      float cv[NI][CT::GC];
      uint32_t hb16[NI];
      const bool take_i = CELL == kSLSTM && t0 + t == 0 && zero_first;
#pragma unroll
      for (int j = 0; j < NI; ++j) {
        cell_forward<CELL>(ry[j], wx[j], bias, st[j], cv[j], take_i);
        if constexpr (EXT) st[j][0] = fminf(fmaxf(st[j][0], -p.fwd_clip), p.fwd_clip);  // +inf when the clip is off
        hb16[j] = act[j] ? static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(st[j][0]))) : 0u;
      }
      const long long c5 = prof ? clock64() : 0;
      // publish round_bf16(h_t): eight neighbouring lanes hold one 16-byte packet (8 units of a batch row)
      const bool publish = !dead && t + 1 < T && t < mute_from;
#pragma unroll
      for (int j = 0; j < NI; ++j) {
        const uint32_t w0 = hb16[j] | (__shfl_down_sync(0xffffffffu, hb16[j], 1) << 16);
        const uint32_t w1 = __shfl_down_sync(0xffffffffu, w0, 2);
        const uint32_t w2 = __shfl_down_sync(0xffffffffu, w0, 4);
        const uint32_t w3 = __shfl_down_sync(0xffffffffu, w1, 4);
        if (act[j] && publish && (lane & 7) == 0) {
          // The data words double as arrival flags (they differ from the all-ones fill); the packet of
          // slot (t + 3) % 4, which held h_{t-2} and has been consumed by every CTA, is refilled, and the
          // fence at the end of the step orders the refill before this thread's next data store.
          const size_t at = pub_base + static_cast<size_t>(ib0 + j * RPP) * 16;
          st_relaxed_gpu_v4(xg_h + static_cast<size_t>((t + 1) & 3) * slot_bytes + at,
                            make_uint4(xg_clean(w0), xg_clean(w1), xg_clean(w2), xg_clean(w3)));
          st_relaxed_gpu_v4(xg_h + static_cast<size_t>((t + 3) & 3) * slot_bytes + at,
                            make_uint4(kXgFill, kXgFill, kXgFill, kXgFill));
        }
      }
      const long long c6 = prof ? clock64() : 0;
      if (t + 1 < T) {
        // fetch this CTA's K-chunk of h_t from slot (t + 1) % 4 into the operand buffer of the next step
        const uint8_t* src = xg_h + static_cast<size_t>((t + 1) & 3) * slot_bytes + poll_base;
        uint8_t* dst = hbuf + ((t + 1) & 1) * hbuf_bytes + kg0 * (BT * 16) + prow * 16;
        uint32_t pend = 0;
        if (prow < bv && !dead) {
#pragma unroll
          for (int j = 0; j < XCH; ++j)
            if (kg0 + j * KG_STEP < Kc / 8) pend |= 1u << j;
        }
        uint64_t t0 = 0;
        uint32_t poll_rounds = 0;
        while (pend != 0u) {
          uint4 v[XCH];
#pragma unroll
          for (int j = 0; j < XCH; ++j)
            if ((pend >> j) & 1u) v[j] = ld_relaxed_gpu_v4(src + j * (KG_STEP * BT * 16));
#pragma unroll
          for (int j = 0; j < XCH; ++j) {
            if (((pend >> j) & 1u) && xg_arrived(v[j])) {
              *reinterpret_cast<uint4*>(dst + j * (KG_STEP * BT * 16)) = v[j];
              pend &= ~(1u << j);
            }
          }
          // the global timer is slow to read: look at it (and at the abort flag) only every 16th round
          if (pend != 0u && (++poll_rounds & 15u) == 0u) {
            const uint64_t now = global_timer_ns();
            if (t0 == 0) t0 = now;
            if (*abort_flag != 0 || now - t0 > limit) {
              report_ks(p.err, kErrWaitH, t + 1);
              dead = true;
              break;
            }
          }
        }
        // a wait that ran out in some lanes only must not leave the warp divided: the warp-wide
        // tcgen05.ld of the next step needs all lanes on one path
        dead = __any_sync(0xffffffffu, dead);
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(&s_hbar[(t + 1) & 1]));
        fence_acq_rel_gpu();
      }
      const long long c7 = prof ? clock64() : 0;
#pragma unroll
      for (int j = 0; j < NI; ++j) {
        if (act[j]) {
          const size_t row = (static_cast<size_t>(b0 + ib0 + j * RPP) * T + t);       // cache / hbf: whole-sequence calls only
          const size_t hrow = (static_cast<size_t>(b0 + ib0 + j * RPP) * Tt + t0 + t);
#pragma unroll
          for (int q = 0; q < CT::S; ++q) {
            if (q < hist_states) {
              if (out_bf16) reinterpret_cast<__nv_bfloat16*>(p.history)[q * sBTND + hrow * ND + n * D + d0] = __float2bfloat16_rn(st[j][q]);
              else p.history[q * sBTND + hrow * ND + n * D + d0] = st[j][q];
            }
          }
          if (p.cache != nullptr && CELL != kElman) {
#pragma unroll
            for (int q = 0; q < CT::GC; ++q) st_cache<CT::CES>(p.cache, (row * CT::GC + q) * ND + n * D + d0, cv[j][q]);
          }
          if (p.hbf != nullptr)
            p.hbf[((static_cast<size_t>(b0 + ib0 + j * RPP) * (T + 1) + t + 1) * N + n) * D + d0] =
                __ushort_as_bfloat16(static_cast<unsigned short>(hb16[j]));
        }
      }
      if (prof) {
        pc[0] += c1 - c0; pc[1] += c2 - c1; pc[2] += c3 - c2; pc[3] += c4 - c3; pc[4] += c5 - c4;
        pc[5] += c6 - c5; pc[6] += c7 - c6; pc[7] += clock64() - c7;
      }
    }
    if (prof) {
#pragma unroll
      for (int q = 0; q < 8; ++q) p.err[8 + q] = static_cast<int>(pc[q]);
    }
#pragma unroll
    for (int j = 0; j < NI; ++j) {
      if (act[j]) {
#pragma unroll
        for (int q = 0; q < CT::S; ++q)
          p.carry[static_cast<size_t>(q) * B * ND + static_cast<size_t>(b0 + ib0 + j * RPP) * ND + n * D + d0] = st[j][q];
        if (p.output_mode == 2) {  // "last": h of the final step as [B][1][N][D]
          const size_t at = static_cast<size_t>(b0 + ib0 + j * RPP) * ND + n * D + d0;
          if (out_bf16) reinterpret_cast<__nv_bfloat16*>(p.history)[at] = __float2bfloat16_rn(st[j][0]);
          else p.history[at] = st[j][0];
        }
      }
    }
  }

  // ---------------- teardown ----------------
  if (*abort_flag != 0) {
    // give copies that are still in flight time to land before shared memory is released
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 4) tmem_dealloc(tbase, tmem_cols);
}

template <int CELL, int BV, int KS, bool WX_BF16, bool EXT>
int launch_fwd_ks_ext(const FwdParams& p, const void* wx, cudaStream_t stream, int* capacity_only) {
  using Cfg = KsCfg<CELL, BV, KS, WX_BF16>;
  using CT = typename Cfg::CT;
  if (p.D % 32 != 0 || p.D % KS != 0 || (p.D / KS) % 16 != 0 || p.D / KS > kMaxKc) return -2;
  if (capacity_only == nullptr && p.xg_data == nullptr) return -2;
  const int Kc = p.D / KS;
  const int hbuf_bytes = Cfg::BT * Kc * 2;
  int smem = ((2 * hbuf_bytes + 2 * Cfg::PART_BYTES + 127) & ~127) + kWxStages * Cfg::WX_STAGE_BYTES;
  CUtensorMap map;
  const uint64_t dims[5] = {static_cast<uint64_t>(p.D), static_cast<uint64_t>(p.N), static_cast<uint64_t>(CT::GW),
                            static_cast<uint64_t>(p.T_total), static_cast<uint64_t>(p.B)};
  const uint32_t box[5] = {static_cast<uint32_t>(Cfg::UO), 1u, static_cast<uint32_t>(CT::GW), 1u, static_cast<uint32_t>(p.wx_box_b)};
  if (capacity_only == nullptr && make_tensor_map(&map, wx, Cfg::WX_ES, 5, dims, box) != 0) return -4;
  auto kern = frnn_fwd_ks_kernel<CELL, BV, KS, WX_BF16, EXT>;
  const int fit = fit_tmem_budget(kern, kThreads, tmem_cols_pow2(Cfg::A_COL0 + Kc / 2, 64u), &smem);
  if (fit != 0) return fit;
  cudaError_t e = cudaSuccess;
  const int n_btiles = (p.B + BV - 1) / BV;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(p.N * n_btiles * (p.D / 32) * KS));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  // clusters of KS CTAs (the K-split partners of a row tile); all CTAs wait on one another through
  // global memory, so the whole grid must be resident: cooperative launch
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = KS;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeCooperative;
  attr[1].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  int max_clusters = 0;
  e = cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (capacity_only != nullptr) {
    *capacity_only = max_clusters * KS;
    return 0;
  }
  if (max_clusters * KS < static_cast<int>(cfg.gridDim.x)) return -2;
  e = cudaLaunchKernelEx(&cfg, kern, p, map);
  return static_cast<int>(e);
}

template <int CELL, int BV, int KS, bool WX_BF16>
int launch_fwd_ks(const FwdParams& p, const void* wx, cudaStream_t stream, int* capacity_only = nullptr) {
  const bool ext = p.T_total != p.T || p.t0 != 0 || p.out_bf16 != 0 || p.fwd_clip < INFINITY;
  return ext ? launch_fwd_ks_ext<CELL, BV, KS, WX_BF16, true>(p, wx, stream, capacity_only)
             : launch_fwd_ks_ext<CELL, BV, KS, WX_BF16, false>(p, wx, stream, capacity_only);
}

template <int CELL, int KS>
int launch_fwd_ks_cell(const FwdParams& p, const void* wx, int wx_bf16, int bv, cudaStream_t s, int* cap) {
  if (bv == 8) return wx_bf16 ? launch_fwd_ks<CELL, 8, KS, true>(p, wx, s, cap) : launch_fwd_ks<CELL, 8, KS, false>(p, wx, s, cap);
  if (bv == 16) return wx_bf16 ? launch_fwd_ks<CELL, 16, KS, true>(p, wx, s, cap) : launch_fwd_ks<CELL, 16, KS, false>(p, wx, s, cap);
  return -2;
}

}  // namespace

// Forward launch for heads split over row tiles and K-chunks (ksplit = CTAs per row tile).
int forward_ksplit_dispatch(int cell, const FwdParams& p, const void* wx, int wx_bf16, int bv, int ksplit, cudaStream_t s,
                            int* capacity_only) {
  if (ksplit == 2) {
    switch (cell) {
      case kLSTM: return launch_fwd_ks_cell<kLSTM, 2>(p, wx, wx_bf16, bv, s, capacity_only);
      case kSLSTM: return launch_fwd_ks_cell<kSLSTM, 2>(p, wx, wx_bf16, bv, s, capacity_only);
      case kGRU: return launch_fwd_ks_cell<kGRU, 2>(p, wx, wx_bf16, bv, s, capacity_only);
      case kElman: return launch_fwd_ks_cell<kElman, 2>(p, wx, wx_bf16, bv, s, capacity_only);
      default: return -1;
    }
  }
  if (ksplit == 4) {
    switch (cell) {
      case kLSTM: return launch_fwd_ks_cell<kLSTM, 4>(p, wx, wx_bf16, bv, s, capacity_only);
      case kSLSTM: return launch_fwd_ks_cell<kSLSTM, 4>(p, wx, wx_bf16, bv, s, capacity_only);
      case kGRU: return launch_fwd_ks_cell<kGRU, 4>(p, wx, wx_bf16, bv, s, capacity_only);
      case kElman: return launch_fwd_ks_cell<kElman, 4>(p, wx, wx_bf16, bv, s, capacity_only);
      default: return -1;
    }
  }
  return -2;
}

// How many CTAs of the forward launch for this shape the device can hold at once (clusters are placed
// inside one GPC, so this can be less than the SM count); <= 0 if unknown.
int forward_ksplit_capacity(int cell, int bv, int ksplit, int D) {
  FwdParams p{};
  p.B = bv; p.T = 1; p.N = 1; p.D = D;
  p.T_total = 1;
  p.fwd_clip = INFINITY;  // the plain instantiation
  p.wx_box_b = bv;
  int cap = 0;
  const int rc = forward_ksplit_dispatch(cell, p, nullptr, 1, bv, ksplit, nullptr, &cap);
  return rc == 0 ? cap : 0;
}

}  // namespace frnn
