// Persistent forward recurrence for sm_100a.
//
// One thread-block cluster of C CTAs handles one (head, batch tile) for the whole sequence.
// CTA `rank` owns U = D / C hidden units: its GR*U rows of the head's recurrent matrix are
// loaded once into tensor memory and stay there (operand A of every tcgen05.mma), the rounded
// hidden state of the previous step is operand B in shared memory, and the fp32 accumulator
// lives in tensor memory too. Per step: UMMA -> tcgen05.ld -> cell epilogue (adds Wx_t + b,
// applies the cell) -> stores all states -> pushes round_bf16(h_t) of its units into the
// operand buffer of every CTA of the cluster with asynchronous DSMEM stores that complete on the
// receiver's mbarrier. Wx_t tiles are prefetched by TMA through a small ring.
//
// Replaces FLASHRNNCellFusedForward (flashrnn/flashrnn/fused/flashrnn_fused_forward.cu:147-660)
// with the arithmetic of reference.recurrence (flashrnn/flashrnn2/reference.py:72-114).
#include "frnn_common.cuh"

namespace frnn {

namespace {

constexpr int kEpiThreads = 128;
constexpr int kFwdThreads = 192;  // 4 epilogue warps + MMA warp + TMA warp
constexpr int kWxStages = 4;

template <int CELL, int BV, int U, bool WX_BF16>
struct FwdCfg {
  using CT = CellTraits<CELL>;
  static constexpr int BT = BV < 16 ? 16 : BV;  // UMMA N (M=128 needs a multiple of 16)
  static constexpr int ROWS = CT::GR * U;       // rows of R owned by the CTA, gate-major
  static constexpr int MT = (ROWS + 127) / 128;
  static constexpr int IPT = (U * BV / kEpiThreads) < 2 ? 2 : (U * BV / kEpiThreads);
  static constexpr int TPB = U / IPT;  // threads per batch row in the cell phase
  static constexpr int ACC_COLS = MT * BT;
  static constexpr int A_COL0 = (ACC_COLS + 31) / 32 * 32;
  static constexpr int WX_ES = WX_BF16 ? 2 : 4;
  static constexpr int WX_STAGE_BYTES = BV * CT::GW * U * WX_ES;
  static constexpr int GROW = MT * 128;  // floats per batch row of the gate buffer
  static constexpr int GBUF_BYTES = BV * GROW * 4;
  static_assert(IPT == 2 || IPT == 4 || IPT == 8, "items per thread");
  static_assert(U % IPT == 0 && BV * TPB <= kEpiThreads, "item mapping");
};

__device__ __forceinline__ void report(int* err, int code, int detail) {
  if (atomicCAS(err, 0, code) == 0) {
    err[1] = detail;
    err[2] = static_cast<int>(blockIdx.x);
  }
  __threadfence();
}

// EXT: the call is one chunk of a longer sequence (T_total, t0), stores bf16 snapshots or clips h_t; the plain
// instantiation folds all three away (they cost the narrow heads, whose step is the epilogue loop, 3 - 5 %).
template <int CELL, int BV, int U, bool WX_BF16, bool XG, bool EXT>
__global__ void __launch_bounds__(kFwdThreads, 1)
frnn_fwd_kernel(const FwdParams p, const __grid_constant__ CUtensorMap wx_map) {
  using Cfg = FwdCfg<CELL, BV, U, WX_BF16>;
  using CT = typename Cfg::CT;
  constexpr int BT = Cfg::BT, MT = Cfg::MT, IPT = Cfg::IPT, TPB = Cfg::TPB;

  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) uint64_t s_hbar[2];
  __shared__ __align__(8) uint64_t s_mma_bar;
  __shared__ __align__(8) uint64_t s_wx_full[kWxStages];
  __shared__ __align__(8) uint64_t s_wx_empty[kWxStages];
  __shared__ uint32_t s_tmem_base;
  __shared__ long long s_prof_clk[2];  // [0] last MMA commit, [1] last h push (phase timers only)

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long t_entry = clock64();
  const int D = p.D, N = p.N, T = p.T, B = p.B, C = p.C;
  const int rank = static_cast<int>(blockIdx.x % C);  // == rank inside the cluster when there is one
  const int gid = blockIdx.x / C;
  const int n = gid % N;
  const int b0 = (gid / N) * BV;
  const int bv = min(BV, B - b0);
  const int hbuf_bytes = BT * D * 2;
  uint8_t* const hbuf = smem;
  float* const gbuf = reinterpret_cast<float*>(smem + 2 * hbuf_bytes);
  uint8_t* const wxs = smem + ((2 * hbuf_bytes + Cfg::GBUF_BYTES + 127) & ~127);
  const volatile int* abort_flag = p.err;
  const uint64_t limit = p.wait_limit_ns;
  constexpr bool xg = XG;  // exchange h through global memory instead of DSMEM
  // four operand slots per group in global memory: h_t goes to slot (t + 1) % 4, see the epilogue
  uint8_t* const xg_h = xg ? p.xg_data + static_cast<size_t>(gid) * 4 * hbuf_bytes : nullptr;
  // test hook: with err[4] = 1 no CTA publishes h from step err[5] on, so the next operand wait runs out
  const int mute_from = p.err[4] != 0 ? p.err[5] : 0x7fffffff;  // test hook: nobody publishes from this step on
  // Second test hook, race verification by delay injection (err[6] = seed, see jitter_stall). It is compiled into the
  // fp32-Wx instantiations only: the exchange code is the same for both Wx types, and even the untaken per-step test
  // costs the bf16 backward more than 1 %.
  constexpr bool kJitter = !WX_BF16;
  const uint32_t jitter = kJitter ? static_cast<uint32_t>(p.err[6]) : 0u;
  const bool zero_first = p.zero_first_dev != nullptr ? *p.zero_first_dev != 0 : p.slstm_zero_first != 0;
  const int hist_states = p.output_mode == 0 ? CT::S : (p.output_mode == 1 ? 1 : 0);  // state planes written per step
  const bool prof = p.err[3] != 0 && blockIdx.x == 0 && lane == 0 && (warp == 0 || warp == 4);
  const int a_cols = MT * (D / 2);
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(Cfg::A_COL0 + a_cols)) tmem_cols <<= 1;

  // ---------------- prologue ----------------
  if (tid == 0) {
    // cluster exchange: one arming arrival + the bytes pushed by the peers; global exchange: the
    // epilogue threads copy the operand in and arrive themselves
    mbar_init(smem_u32(&s_hbar[0]), xg ? kEpiThreads : 1);
    mbar_init(smem_u32(&s_hbar[1]), xg ? kEpiThreads : 1);
    mbar_init(smem_u32(&s_mma_bar), 1);
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
  for (int i = tid; i < 2 * hbuf_bytes / 16; i += kFwdThreads)
    reinterpret_cast<uint4*>(hbuf)[i] = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();
  // round_bf16(initial h) of the whole head for this batch tile -> operand buffer 0
  for (int i = tid; i < bv * (D / 2); i += kFwdThreads) {
    const int b = i / (D / 2), k = 2 * (i % (D / 2));
    const float2 v = *reinterpret_cast<const float2*>(p.initial + (static_cast<size_t>(b0 + b) * N + n) * D + k);
    *reinterpret_cast<uint32_t*>(hbuf + kmajor_offset(BT, b, k)) = pack_bf16x2(v.x, v.y);
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = s_tmem_base;

  if (warp < 4) {
    // R rows of this CTA -> tensor memory (lane = row, 32-bit column = two consecutive k)
    for (int j = 0; j < MT; ++j) {
      const int rr = j * 128 + tid;
      const bool valid = rr < Cfg::ROWS;
      const int g = valid ? rr / U : 0, u = valid ? rr % U : 0;
      const __nv_bfloat16* src = p.R + ((static_cast<size_t>(g) * N + n) * D + rank * U + u) * D;
      for (int c0 = 0; c0 < D / 2; c0 += 8) {
        uint32_t r[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
        if (valid) {
          const uint4 lo = __ldg(reinterpret_cast<const uint4*>(src + 2 * c0));
          const uint4 hi = __ldg(reinterpret_cast<const uint4*>(src + 2 * c0 + 8));
          r[0] = lo.x; r[1] = lo.y; r[2] = lo.z; r[3] = lo.w;
          r[4] = hi.x; r[5] = hi.y; r[6] = hi.z; r[7] = hi.w;
        }
        tmem_st_x8(tmem_addr(tbase, 32 * warp, Cfg::A_COL0 + j * (D / 2) + c0), r);
      }
    }
    tmem_st_wait();
  }

  // cell-phase item of this thread: batch row `ib`, units [d0, d0 + IPT) of the head
  const int ib = tid / TPB, uq = tid % TPB;
  const bool active = warp < 4 && tid < BV * TPB && ib < bv;
  const int ul = uq * IPT;          // unit offset inside the CTA's slice
  const int d0 = rank * U + ul;     // unit offset inside the head
  float st[CT::S][IPT];
  float bias[CT::GB][IPT];
  const int Tt = EXT ? p.T_total : T, t0 = EXT ? p.t0 : 0;
  const bool out_bf16 = EXT && p.out_bf16 != 0;
  const size_t sBTND = static_cast<size_t>(B) * Tt * N * D;
  const size_t item_bn = (static_cast<size_t>(b0 + ib) * N + n) * D + d0;  // into [B][1][N][D]
  if (active) {
#pragma unroll
    for (int s = 0; s < CT::S; ++s)
      ld_f32_vec<IPT>(p.initial + static_cast<size_t>(s) * B * N * D + item_bn, st[s]);
#pragma unroll
    for (int g = 0; g < CT::GB; ++g)
      ld_f32_vec<IPT>(p.bias + (static_cast<size_t>(g) * N + n) * D + d0, bias[g]);
    if (p.hbf != nullptr) {
      __nv_bfloat16* dst = p.hbf + ((static_cast<size_t>(b0 + ib) * (T + 1)) * N + n) * D + d0;
#pragma unroll
      for (int j = 0; j < IPT; j += 2)
        *reinterpret_cast<uint32_t*>(dst + j) = pack_bf16x2(st[0][j], st[0][j + 1]);
    }
  }
  const uint32_t h_tx_bytes = static_cast<uint32_t>(D) * bv * 2u;
  if (warp == 4 && lane == 0) {
    if (!xg && T >= 2) mbar_arrive_expect_tx(smem_u32(&s_hbar[1]), h_tx_bytes);
    if (!xg && T >= 3) mbar_arrive_expect_tx(smem_u32(&s_hbar[0]), h_tx_bytes);
    tma_prefetch_desc(&wx_map);
  }
  fence_proxy_async();
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();

  if (prof && warp == 0) p.err[20] = static_cast<int>(clock64() - t_entry);  // prologue cycles
  // ---------------- main loops ----------------
  if (warp == 4) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(128, BT, false, false);
      long long pw = 0, pi = 0, px = 0, pf = 0;
      int committed = 0;  // steps whose tcgen05.mma have been issued and committed
      for (int t = 0; t < T; ++t) {
        if (kJitter && jitter != 0u) jitter_stall(jitter, 1u, static_cast<uint32_t>(t));
        const int pb = t & 1;
        const long long m0 = prof ? clock64() : 0;
        if (t >= 1) {
          if (!mbar_wait_bounded<true, true>(smem_u32(&s_hbar[pb]), ((t - 1) >> 1) & 1, limit, abort_flag)) {
            report(p.err, kErrWaitH, t);
            break;
          }
        }
        const long long mw = prof ? clock64() : 0;
        fence_proxy_async_smem();
        tc_fence_after_sync();
        const long long m1 = prof ? clock64() : 0;
        if (prof) pf += m1 - mw;
        const uint32_t hb = smem_u32(hbuf + pb * hbuf_bytes);
        for (int j = 0; j < MT; ++j) {
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint64_t bdesc = umma_smem_desc(hb + kk * 2 * (BT * 16), BT * 16, 128);
            umma_bf16_ts(tbase + j * BT, tbase + Cfg::A_COL0 + j * (D / 2) + kk * 8, bdesc, idesc,
                         kk > 0 ? 1u : 0u);
          }
        }
        umma_commit(smem_u32(&s_mma_bar));
        ++committed;
        // arm this parity's operand barrier for its next use (step t + 2), after the issue so that it
        // is off the critical path; its current phase has completed (we waited for it above)
        if (!xg && t >= 1 && t + 2 <= T - 1) mbar_arrive_expect_tx(smem_u32(&s_hbar[pb]), h_tx_bytes);
        if (prof) {
          const long long m2 = clock64();
          pw += m1 - m0; pi += m2 - m1;
          if (t >= 1) px += m1 - *reinterpret_cast<volatile long long*>(&s_prof_clk[1]);
          *reinterpret_cast<volatile long long*>(&s_prof_clk[0]) = m2;
        }
      }
      // Before the CTA may release its tensor memory and shared memory every issued tcgen05.mma must
      // have finished. Normally the epilogue has waited for the last commit already; after a failed
      // wait it has not (it stops waiting), so the issuing thread waits here itself. The commit
      // completes without any other party, hence no abort flag and a plain bound.
      if (committed > 0) mbar_wait_bounded<false, true>(smem_u32(&s_mma_bar), (committed - 1) & 1, limit, nullptr);
      if (prof) { p.err[16] = static_cast<int>(pw); p.err[17] = static_cast<int>(pi); p.err[18] = static_cast<int>(px); p.err[19] = static_cast<int>(pf); }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      const uint32_t stage_tx = static_cast<uint32_t>(p.wx_box_b) * CT::GW * U * Cfg::WX_ES;
      for (int t = 0; t < T; ++t) {
        const int s = t % kWxStages;
        if (t >= kWxStages) {
          if (!mbar_wait_bounded<false>(smem_u32(&s_wx_empty[s]), ((t / kWxStages) - 1) & 1, limit, abort_flag)) {
            report(p.err, kErrWaitEmpty, t);
            break;
          }
        }
        // Once any wait of the grid has run out, the epilogue threads stop waiting for the stages and
        // release them early, so "released" no longer implies that the previous copy into this stage
        // has landed; arming its barrier again could then be a second arrival in one phase. The flag
        // is set before any thread skips a wait, so checking it after the wait above is enough.
        if (*abort_flag != 0) break;
        mbar_arrive_expect_tx(smem_u32(&s_wx_full[s]), stage_tx);
        tma_load_5d(smem_u32(wxs + s * Cfg::WX_STAGE_BYTES), &wx_map, smem_u32(&s_wx_full[s]), rank * U, n, 0, t0 + t, b0);
      }
    }
  } else {
    const size_t hist_off = ((static_cast<size_t>(b0 + ib) * Tt + t0) * N + n) * D + d0;  // elements, fp32 or bf16
    float* hist = p.history + hist_off;
    const size_t cache_off = ((static_cast<size_t>(b0 + ib) * T * CT::GC) * N + n) * D + d0;  // elements
    __nv_bfloat16* hbf = p.hbf == nullptr ? nullptr : p.hbf + ((static_cast<size_t>(b0 + ib) * (T + 1) + 1) * N + n) * D + d0;
    const uint32_t h_off = kmajor_offset(BT, ib, d0);
    // Peers this lane pushes to (it shares the cluster with the other lanes of its packet group)
    // and the distance from this CTA's shared window to theirs, constant for the whole kernel.
    constexpr int LPP = 8 / IPT;  // lanes that together hold one 16-byte packet of h
    constexpr int NPEER = 16 / LPP;
    uint32_t peer_delta[NPEER];
    {
      const uint32_t base = smem_u32(smem);
#pragma unroll
      for (int i = 0; i < NPEER; ++i) {
        const int d = i * LPP + (lane & (LPP - 1));
        peer_delta[i] = (!xg && d < C) ? map_to_cta(base, d) - base : 0u;
      }
    }
    const size_t ND = static_cast<size_t>(N) * D;
    long long pc[7] = {0, 0, 0, 0, 0, 0, 0};
    long long pd = 0;
    // After a wait has failed (`dead`), the warp keeps walking through the loop so that the
    // named barrier below always sees all 128 threads; waits return at once because the abort
    // flag is set, and nothing that is computed from then on matters.
    bool dead = false;
    for (int t = 0; t < T; ++t) {
      if (kJitter && jitter != 0u) jitter_stall(jitter, 0u, static_cast<uint32_t>(t));
      const int s = t % kWxStages;
      const long long c0 = prof ? clock64() : 0;
      if (!dead && !mbar_wait_bounded<false, true>(smem_u32(&s_wx_full[s]), (t / kWxStages) & 1, limit, abort_flag)) {
        report(p.err, kErrWaitWx, t);
        dead = true;
      }
      const long long c1 = prof ? clock64() : 0;
      float wx[CT::GW][IPT];
      if (active) {
        const uint8_t* ws = wxs + s * Cfg::WX_STAGE_BYTES;
#pragma unroll
        for (int g = 0; g < CT::GW; ++g) {
          const int e = (ib * CT::GW + g) * U + ul;
          if constexpr (WX_BF16) ld_bf16_vec<IPT>(reinterpret_cast<const __nv_bfloat16*>(ws) + e, wx[g]);
          else ld_f32_vec<IPT>(reinterpret_cast<const float*>(ws) + e, wx[g]);
        }
      }
      mbar_arrive(smem_u32(&s_wx_empty[s]));
      if (!dead && !mbar_wait_bounded<false, true>(smem_u32(&s_mma_bar), t & 1, limit, abort_flag)) {
        report(p.err, kErrWaitMma, t);
        dead = true;
      }
      tc_fence_after_sync();
      const long long c2 = prof ? clock64() : 0;
      if (prof) pd += c2 - *reinterpret_cast<volatile long long*>(&s_prof_clk[0]);
      // phase 1: accumulator rows (lane = gate row) -> gate buffer [batch][row]
      {
        uint32_t r[MT][BV / 8][8];
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
          for (int c = 0; c < BV / 8; ++c) tmem_ld_x8(tmem_addr(tbase, 32 * warp, j * BT + 8 * c), r[j][c]);
        tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < MT; ++j)
#pragma unroll
          for (int c = 0; c < BV / 8; ++c)
#pragma unroll
            for (int q = 0; q < 8; ++q) gbuf[(8 * c + q) * Cfg::GROW + j * 128 + tid] = __uint_as_float(r[j][c][q]);
      }
      tc_fence_before_sync();
      const long long c3 = prof ? clock64() : 0;
      asm volatile("bar.sync 1, 128;" ::: "memory");  // the four epilogue warps only
      const long long c4 = prof ? clock64() : 0;
      // phase 2: the cell, for IPT consecutive units of one batch row
      long long c5 = 0, c6 = 0;
      float cv[CT::GC][IPT];
      uint32_t hp[IPT / 2];
#pragma unroll
      for (int j = 0; j < IPT / 2; ++j) hp[j] = 0u;
      if (active) {
        float ry[CT::GR][IPT];
#pragma unroll
        for (int g = 0; g < CT::GR; ++g) ld_f32_vec<IPT>(gbuf + ib * Cfg::GROW + g * U + ul, ry[g]);
        const bool take_i = CELL == kSLSTM && t0 + t == 0 && zero_first;
#pragma unroll
        for (int j = 0; j < IPT; ++j) {
          float ryj[CT::GR], wxj[CT::GW], bj[CT::GB], sj[CT::S], cj[CT::GC];
#pragma unroll
          for (int g = 0; g < CT::GR; ++g) ryj[g] = ry[g][j];
#pragma unroll
          for (int g = 0; g < CT::GW; ++g) wxj[g] = wx[g][j];
#pragma unroll
          for (int g = 0; g < CT::GB; ++g) bj[g] = bias[g][j];
#pragma unroll
          for (int q = 0; q < CT::S; ++q) sj[q] = st[q][j];
          cell_forward<CELL>(ryj, wxj, bj, sj, cj, take_i);
          if constexpr (EXT) sj[0] = fminf(fmaxf(sj[0], -p.fwd_clip), p.fwd_clip);  // +inf when the clip is off
#pragma unroll
          for (int q = 0; q < CT::S; ++q) st[q][j] = sj[q];
#pragma unroll
          for (int q = 0; q < CT::GC; ++q) cv[q][j] = cj[q];
        }
#pragma unroll
        for (int j = 0; j < IPT; j += 2) hp[j / 2] = pack_bf16x2(st[0][j], st[0][j + 1]);
      }
      if (prof) c5 = clock64();
      // push round_bf16(h_t): LPP neighbouring lanes first gather one 16-byte packet (8 units of one
      // batch row), then share the peers among themselves, so a thread issues C / LPP stores.
      {
        uint32_t pk[4];
        if constexpr (LPP == 4) {
          const uint32_t a = hp[0];
          const uint32_t b1 = __shfl_xor_sync(0xffffffffu, a, 1);
          const uint32_t lo = (lane & 1) ? b1 : a, hi = (lane & 1) ? a : b1;
          const uint32_t lo2 = __shfl_xor_sync(0xffffffffu, lo, 2), hi2 = __shfl_xor_sync(0xffffffffu, hi, 2);
          pk[0] = (lane & 2) ? lo2 : lo; pk[1] = (lane & 2) ? hi2 : hi;
          pk[2] = (lane & 2) ? lo : lo2; pk[3] = (lane & 2) ? hi : hi2;
        } else if constexpr (LPP == 2) {
          const uint32_t o0 = __shfl_xor_sync(0xffffffffu, hp[0], 1), o1 = __shfl_xor_sync(0xffffffffu, hp[IPT / 2 - 1], 1);
          pk[0] = (lane & 1) ? o0 : hp[0]; pk[1] = (lane & 1) ? o1 : hp[IPT / 2 - 1];
          pk[2] = (lane & 1) ? hp[0] : o0; pk[3] = (lane & 1) ? hp[IPT / 2 - 1] : o1;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j) pk[j] = hp[j % (IPT / 2)];
        }
        const bool publish = !dead && t + 1 < T && t < mute_from;
        if (!xg) {
          if (active && publish) {
            const uint32_t dst = smem_u32(hbuf + ((t + 1) & 1) * hbuf_bytes) + (h_off & ~15u);
            const uint32_t bar = smem_u32(&s_hbar[(t + 1) & 1]);
            const int first = lane & (LPP - 1);
#pragma unroll
            for (int i = 0; i < NPEER; ++i) {
              if (i * LPP + first < C)
                st_async_v4_b32(dst + peer_delta[i], pk[0], pk[1], pk[2], pk[3], bar + peer_delta[i]);
            }
          }
        } else {
          // One lane of each packet group stores the packet into slot (t + 1) % 4 of the group's
          // global operand buffer; there is no separate flag: receivers poll the data words, which
          // differ from the all-ones fill once written (two bf16 NaNs with all-ones payload never
          // come out of the rounding). The same lane then refills its packet of slot (t + 3) % 4,
          // which held h_{t-2}: every CTA has consumed that (it published h_{t-1} afterwards, and
          // this CTA has consumed all of h_{t-1}). The fence at the end of the step orders the
          // refill before this thread's next data store, so a receiver that has seen h_{t+1} of
          // this packet position can no longer see h_{t-2} where it waits for h_{t+2}.
          if (active && publish && (lane & (LPP - 1)) == 0) {
            const size_t at = h_off & ~15u;
            st_relaxed_gpu_v4(xg_h + static_cast<size_t>((t + 1) & 3) * hbuf_bytes + at, make_uint4(pk[0], pk[1], pk[2], pk[3]));
            st_relaxed_gpu_v4(xg_h + static_cast<size_t>((t + 3) & 3) * hbuf_bytes + at,
                              make_uint4(kXgFill, kXgFill, kXgFill, kXgFill));
          }
        }
      }
      if (prof) { c6 = clock64(); *reinterpret_cast<volatile long long*>(&s_prof_clk[1]) = c6; }
      if (xg && t + 1 < T) {
        // Fetch the whole operand h_t of the group from slot (t + 1) % 4 into this CTA's operand
        // buffer: thread `tid` owns the 16-byte packets tid, tid + 128, ... of the active batch
        // rows, polls them until none shows the fill pattern and copies them to shared memory.
        constexpr int KG_STEP = kEpiThreads / BV;            // k-groups between two packets of a thread
        constexpr int XCH = (960 / 8 + KG_STEP - 1) / KG_STEP;  // packets per thread at the widest head this kernel takes (D/2 + 32 TMEM columns <= 512)
        const int row = tid % BV, kg0 = tid / BV;
        const uint8_t* src = xg_h + static_cast<size_t>((t + 1) & 3) * hbuf_bytes + kg0 * (BT * 16) + row * 16;
        uint8_t* dst = hbuf + ((t + 1) & 1) * hbuf_bytes + kg0 * (BT * 16) + row * 16;
        uint32_t pend = 0;
        if (row < bv && !dead) {
#pragma unroll
          for (int j = 0; j < XCH; ++j)
            if (kg0 + j * KG_STEP < D / 8) pend |= 1u << j;
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
              report(p.err, kErrWaitH, t + 1);
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
        fence_acq_rel_gpu();  // orders this step's refill and observations before the next step's (see above)
      }
      if (active) {
#pragma unroll
        for (int q = 0; q < CT::S; ++q) {
          if (q < hist_states) {
            // bf16 snapshots: the same element offsets from the same base, two bytes each (keeps one pointer live)
            if (out_bf16) st_bf16_vec<IPT>(reinterpret_cast<__nv_bfloat16*>(p.history) + (hist - p.history) + q * sBTND + t * ND, st[q]);
            else st_f32_vec<IPT>(hist + q * sBTND + t * ND, st[q]);
          }
        }
        if (p.cache != nullptr && CELL != kElman) {
#pragma unroll
          for (int q = 0; q < CT::GC; ++q)
            st_cache_vec<IPT, CT::CES>(p.cache, cache_off + (static_cast<size_t>(t) * CT::GC + q) * ND, cv[q]);
        }
        if (hbf != nullptr) {
#pragma unroll
          for (int j = 0; j < IPT; j += 2) *reinterpret_cast<uint32_t*>(hbf + t * ND + j) = hp[j / 2];
        }
      }
      if (prof) {
        pc[0] += c1 - c0; pc[1] += c2 - c1; pc[2] += c3 - c2; pc[3] += c4 - c3; pc[4] += c5 - c4;
        pc[5] += c6 - c5; pc[6] += clock64() - c6;
      }
    }
    if (prof) {
#pragma unroll
      for (int q = 0; q < 7; ++q) p.err[8 + q] = static_cast<int>(pc[q]);
      p.err[15] = static_cast<int>(pd);
    }
    if (active) {
#pragma unroll
      for (int q = 0; q < CT::S; ++q) st_f32_vec<IPT>(p.carry + static_cast<size_t>(q) * B * N * D + item_bn, st[q]);
      if (p.output_mode == 2) {  // "last": h of the final step as [B][1][N][D]
        if (out_bf16) st_bf16_vec<IPT>(reinterpret_cast<__nv_bfloat16*>(p.history) + item_bn, st[0]);
        else st_f32_vec<IPT>(p.history + item_bn, st[0]);
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

template <int CELL, int BV, int U, bool WX_BF16, bool XG, bool EXT>
int launch_fwd_ext(const FwdParams& p, const void* wx, cudaStream_t stream) {
  using Cfg = FwdCfg<CELL, BV, U, WX_BF16>;
  using CT = typename Cfg::CT;
  const int hbuf_bytes = Cfg::BT * p.D * 2;
  int smem = ((2 * hbuf_bytes + Cfg::GBUF_BYTES + 127) & ~127) + kWxStages * Cfg::WX_STAGE_BYTES;
  if (Cfg::A_COL0 + Cfg::MT * (p.D / 2) > 512) return -3;
  CUtensorMap map;
  const uint64_t dims[5] = {static_cast<uint64_t>(p.D), static_cast<uint64_t>(p.N), static_cast<uint64_t>(CT::GW),
                            static_cast<uint64_t>(p.T_total), static_cast<uint64_t>(p.B)};
  const uint32_t box[5] = {static_cast<uint32_t>(U), 1u, static_cast<uint32_t>(CT::GW), 1u, static_cast<uint32_t>(p.wx_box_b)};
  if (make_tensor_map(&map, wx, Cfg::WX_ES, 5, dims, box) != 0) return -4;
  auto kern = frnn_fwd_kernel<CELL, BV, U, WX_BF16, XG, EXT>;
  const int fit = fit_tmem_budget(kern, kFwdThreads, tmem_cols_pow2(Cfg::A_COL0 + Cfg::MT * (p.D / 2), 32u), &smem);
  if (fit != 0) return fit;
  cudaError_t e = cudaSuccess;
  if (p.C > 8 && !XG) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const int n_btiles = (p.B + BV - 1) / BV;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(p.N * n_btiles * p.C));
  cfg.blockDim = dim3(kFwdThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (!XG) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = static_cast<unsigned>(p.C);
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
  } else {
    // the CTAs of a group wait on one another through global memory: all must be resident
    attr[0].id = cudaLaunchAttributeCooperative;
    attr[0].val.cooperative = 1;
  }
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  if (!XG && p.C > 1) {
    // a cluster that cannot be placed (too many CTAs or too much shared memory per GPC) is reported, not launched
    int max_clusters = 0;
    e = cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg);
    if (e != cudaSuccess) return static_cast<int>(e);
    if (max_clusters < 1) return -2;
  }
  e = cudaLaunchKernelEx(&cfg, kern, p, map);
  return static_cast<int>(e);
}

template <int CELL, int BV, int U, bool WX_BF16, bool XG>
int launch_fwd(const FwdParams& p, const void* wx, cudaStream_t stream) {
  const bool ext = p.T_total != p.T || p.t0 != 0 || p.out_bf16 != 0 || p.fwd_clip < INFINITY;
  return ext ? launch_fwd_ext<CELL, BV, U, WX_BF16, XG, true>(p, wx, stream)
             : launch_fwd_ext<CELL, BV, U, WX_BF16, XG, false>(p, wx, stream);
}

template <int CELL, int BV, int U>
int launch_fwd_dt(const FwdParams& p, const void* wx, int wx_bf16, cudaStream_t s) {
  if constexpr (U == 32) {  // groups wider than a cluster exchange through global memory (32-unit slices only)
    if (p.xg_data != nullptr)
      return wx_bf16 ? launch_fwd<CELL, BV, U, true, true>(p, wx, s) : launch_fwd<CELL, BV, U, false, true>(p, wx, s);
  }
  if (p.xg_data != nullptr) return -2;
  return wx_bf16 ? launch_fwd<CELL, BV, U, true, false>(p, wx, s) : launch_fwd<CELL, BV, U, false, false>(p, wx, s);
}
template <int CELL>
int launch_fwd_cell(const FwdParams& p, const void* wx, int wx_bf16, int bv, int unit, cudaStream_t s) {
  if (bv == 8 && unit == 32) return launch_fwd_dt<CELL, 8, 32>(p, wx, wx_bf16, s);
  if (bv == 16 && unit == 32) return launch_fwd_dt<CELL, 16, 32>(p, wx, wx_bf16, s);
  if (bv == 8 && unit == 16) return launch_fwd_dt<CELL, 8, 16>(p, wx, wx_bf16, s);
  if (bv == 16 && unit == 16) return launch_fwd_dt<CELL, 16, 16>(p, wx, wx_bf16, s);
  return -2;
}

}  // namespace

int forward_dispatch(int cell, const FwdParams& p, const void* wx, int wx_bf16, int bv, int unit, cudaStream_t s) {
  switch (cell) {
    case kLSTM: return launch_fwd_cell<kLSTM>(p, wx, wx_bf16, bv, unit, s);
    case kSLSTM: return launch_fwd_cell<kSLSTM>(p, wx, wx_bf16, bv, unit, s);
    case kGRU: return launch_fwd_cell<kGRU>(p, wx, wx_bf16, bv, unit, s);
    case kElman: return launch_fwd_cell<kElman>(p, wx, wx_bf16, bv, unit, s);
    default: return -1;
  }
}

}  // namespace frnn
