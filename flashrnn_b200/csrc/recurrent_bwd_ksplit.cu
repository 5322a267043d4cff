// Persistent BPTT recurrence for wide heads (sm_100a): every CTA owns columns of R.
//
// dh_{t-1} = sum over all recurrent gate rows k = (g, o) of dG_t[k] * R[g, o, p]. A (head, batch
// tile) group is a 2-D grid of CTAs: D/128 tiles of 128 hidden units p times KS splits of the
// K = GR*D gate rows. CTA (pt, ks) keeps R[k in chunk ks, p in tile pt] transposed in tensor
// memory (lane = p) for the whole sequence. Per step, going backwards in time:
//   1. the owner of a unit adds dH_t, the carried gradient and the KS partial sums of dh_t that its
//      cluster partners sent, runs the cell's backward formulas            -> dG_t of its units
//   2. dG_t (bf16) goes to the group's operand buffer in global memory (no flag: receivers poll the
//      data words, which differ from the all-ones fill once written), to dgr / dWx, and into db
//   3. every CTA copies its K-chunk of dG_t into shared memory and runs tcgen05.mma over it
//                                                                          -> partial dh_{t-1} [128 x batch]
//   4. each accumulator row is sent with asynchronous DSMEM stores to the cluster partner that
//      owns the unit (128/KS units each).
// All CTAs of the launch must be resident at the same time (cooperative launch).
//
// Replaces FLASHRNNCellFusedBackward (flashrnn/flashrnn/fused/flashrnn_fused_backward.cu) for wide
// heads; the exchange of dG instead of partial dh follows the reference's hybrid kernel
// (flashrnn/flashrnn2/hybrid_bw2d.cu:664-678). Gradient formulas: cells.cuh.
#include "frnn_common.cuh"

namespace frnn {

namespace {

constexpr int kEpiThreads = 128;
constexpr int kThreads = 192;  // 4 epilogue warps + MMA warp + TMA warp
constexpr int kMaxKc = 896;    // K-chunk bound: Kc/2 columns of R plus the accumulator fit 512 TMEM columns

template <int CELL, int BV, int KS, bool WX_BF16>
struct BksCfg {
  using CT = CellTraits<CELL>;
  static constexpr int UO = 128 / KS;           // units owned by one CTA
  static constexpr int BT = 16;                 // UMMA N
  static constexpr int RPP = kEpiThreads / UO;  // batch rows covered by one pass of the epilogue threads
  static constexpr int NI = BV / RPP < 1 ? 1 : BV / RPP;  // (batch row, unit) items per thread
  static constexpr int A_COL0 = 32;
  static constexpr int GCL = CELL == kElman ? 0 : CT::GC;  // cached gates actually loaded
  static constexpr int CACHE_BYTES = GCL * BV * UO * CT::CES;  // the cached gates come first in a stage
  static constexpr int STAGE_BYTES = CACHE_BYTES + 3 * CT::S * BV * UO * 4;
  static_assert(CACHE_BYTES % 128 == 0, "TMA destinations after the cached gates stay 128-byte aligned");
  static constexpr int NST = STAGE_BYTES * 4 <= 65536 ? 4 : (STAGE_BYTES * 3 <= 65536 ? 3 : 2);
  static constexpr int PART_FLOATS = KS * BV * UO;  // one parity: [source][batch][unit]
  static constexpr int PART_BYTES = PART_FLOATS * 4;
  static constexpr int DBUF_BYTES = BV * CT::GB * UO * 4;
  static_assert(BV == 8 || BV == 16, "batch tile");
  static_assert(KS == 2 || KS == 4 || KS == 8, "cluster width");
  static_assert(UO % 8 == 0, "packets of eight units");
};

__device__ __forceinline__ void report_bks(int* err, int code, int detail) {
  if (atomicCAS(err, 0, code) == 0) {
    err[1] = detail;
    err[2] = static_cast<int>(blockIdx.x);
  }
  __threadfence();
}

// OPTS: one of the v1 options (recurrent-gradient clip / cut, v1 sLSTM convention) is set; the plain instantiation
// folds them away.
template <int CELL, int BV, int KS, bool WX_BF16, bool OPTS>
__global__ void __launch_bounds__(kThreads, 1)
frnn_bwd_ks_kernel(const BwdParams p, const __grid_constant__ CUtensorMap cache_map,
                   const __grid_constant__ CUtensorMap hist_map, const __grid_constant__ CUtensorMap init_map,
                   const __grid_constant__ CUtensorMap dhist_map) {
  using Cfg = BksCfg<CELL, BV, KS, WX_BF16>;
  using CT = typename Cfg::CT;
  constexpr int BT = Cfg::BT, UO = Cfg::UO, NI = Cfg::NI, RPP = Cfg::RPP, S = CT::S, GCL = Cfg::GCL;

  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) uint64_t s_dg_bar[2];
  __shared__ __align__(8) uint64_t s_mma_bar;
  __shared__ __align__(8) uint64_t s_part_bar[2];
  __shared__ __align__(8) uint64_t s_full[4];
  __shared__ __align__(8) uint64_t s_empty[4];
  __shared__ uint32_t s_tmem_base;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long t_entry = clock64();
  const int D = p.D, N = p.N, T = p.T, B = p.B;
  const int PT = D / 128;
  const int ks = static_cast<int>(blockIdx.x % KS);  // == rank inside the cluster
  const int pt = static_cast<int>((blockIdx.x / KS) % PT);
  const int gid = static_cast<int>(blockIdx.x / (KS * PT));
  const int n = gid % N;
  const int btile = gid / N;
  const int b0 = btile * BV;
  const int bv = min(BV, B - b0);
  const int K = CT::GR * D;
  const int Kc = K / KS;
  const int dg_bytes = BT * Kc * 2;
  uint8_t* const dgbuf = smem;  // two operand buffers [BT x Kc] K-major
  float* const part = reinterpret_cast<float*>(smem + 2 * dg_bytes);
  float* const dbuf = reinterpret_cast<float*>(smem + 2 * dg_bytes + 2 * Cfg::PART_BYTES);
  uint8_t* const stages = smem + ((2 * dg_bytes + 2 * Cfg::PART_BYTES + Cfg::DBUF_BYTES + 127) & ~127);
  const volatile int* abort_flag = p.err;
  const uint64_t limit = p.wait_limit_ns;
  // four operand slots per group in global memory, each [K-chunk][BT x Kc, K-major]; dG of iteration i goes to slot i % 4
  const size_t slot_bytes = static_cast<size_t>(BT) * K * 2;
  uint8_t* const xg_dg = p.xg_data + static_cast<size_t>(gid) * 4 * slot_bytes;
  const int mute_from = p.err[4] != 0 ? p.err[5] : 0x7fffffff;  // test hook: nobody publishes from this step on
  // Second test hook, race verification by delay injection (err[6] = seed, see jitter_stall). It is compiled into the
  // fp32-Wx instantiations only: the exchange code is the same for both Wx types, and even the untaken per-step test
  // costs the bf16 backward more than 1 %.
  constexpr bool kJitter = !WX_BF16;
  const uint32_t jitter = kJitter ? static_cast<uint32_t>(p.err[6]) : 0u;
  const bool prof = p.err[3] != 0 && blockIdx.x == 0 && lane == 0 && (warp == 0 || warp == 4);
  uint32_t tmem_cols = 64;
  while (tmem_cols < static_cast<uint32_t>(Cfg::A_COL0 + Kc / 2)) tmem_cols <<= 1;

  // ---------------- prologue ----------------
  if (tid == 0) {
    mbar_init(smem_u32(&s_dg_bar[0]), kEpiThreads);
    mbar_init(smem_u32(&s_dg_bar[1]), kEpiThreads);
    mbar_init(smem_u32(&s_mma_bar), 1);
    mbar_init(smem_u32(&s_part_bar[0]), 1);
    mbar_init(smem_u32(&s_part_bar[1]), 1);
    for (int s = 0; s < Cfg::NST; ++s) {
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&s_empty[s]), kEpiThreads);
    }
    fence_mbar_init();
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(&s_tmem_base), tmem_cols);
    tmem_relinquish_alloc();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = s_tmem_base;

  if (warp < 4) {
    // R[k, p in tile] for the chunk's gate rows k -> tensor memory, lane = p, column c packs k = 2c, 2c + 1.
    // Sixteen rows of R (128 consecutive p each) are staged in shared memory with coalesced loads
    // (the operand buffers are still idle) and read back column-wise.
    __nv_bfloat16* const rbuf = reinterpret_cast<__nv_bfloat16*>(dgbuf);  // [16][128]
    for (int c0 = 0; c0 < Kc / 2; c0 += 8) {
      for (int v = tid; v < 16 * 16; v += kEpiThreads) {
        const int kk = v / 16, pv = v % 16;
        const int k = ks * Kc + 2 * c0 + kk;
        const int g = k / D, o = k % D;
        const __nv_bfloat16* src = p.R + ((static_cast<size_t>(g) * N + n) * D + o) * D + pt * 128 + pv * 8;
        reinterpret_cast<uint4*>(rbuf)[v] = __ldg(reinterpret_cast<const uint4*>(src));
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      uint32_t r[8];
#pragma unroll
      for (int q = 0; q < 8; ++q)
        r[q] = static_cast<uint32_t>(__bfloat16_as_ushort(rbuf[(2 * q) * 128 + tid])) |
               (static_cast<uint32_t>(__bfloat16_as_ushort(rbuf[(2 * q + 1) * 128 + tid])) << 16);
      tmem_st_x8(tmem_addr(tbase, 32 * warp, Cfg::A_COL0 + c0), r);
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    tmem_st_wait();
    // the operand buffers start as zeros (batch rows past the tile's end stay zero)
    for (int i = tid; i < 2 * dg_bytes / 16; i += kEpiThreads) reinterpret_cast<uint4*>(dgbuf)[i] = make_uint4(0u, 0u, 0u, 0u);
  }

  // cell items of this thread: unit `ul` of the owned slice, batch rows ib0 + j * RPP
  const int ul = tid % UO, ib0 = tid / UO;
  const int u0 = pt * 128 + ks * UO;  // first owned unit inside the head
  const int d0 = u0 + ul;
  const size_t ND = static_cast<size_t>(N) * D;
  const size_t BND = static_cast<size_t>(B) * ND;
  bool act[NI];
  float dcar[NI][S];
  float dbacc[NI][CT::GB];
#pragma unroll
  for (int j = 0; j < NI; ++j) {
    const int ib = ib0 + j * RPP;
    act[j] = warp < 4 && ib < bv;
#pragma unroll
    for (int q = 0; q < S; ++q)
      dcar[j][q] = act[j] ? p.d_carry[q * BND + static_cast<size_t>(b0 + ib) * ND + n * D + d0] : 0.0f;
#pragma unroll
    for (int g = 0; g < CT::GB; ++g) dbacc[j][g] = 0.0f;
  }
  constexpr uint32_t part_tx = static_cast<uint32_t>(KS) * BV * UO * 4u;
  if (warp == 4 && lane == 0) {
    mbar_arrive_expect_tx(smem_u32(&s_part_bar[1]), part_tx);              // consumed in iteration 1
    if (T >= 2) mbar_arrive_expect_tx(smem_u32(&s_part_bar[0]), part_tx);  // iteration 2
  }
  if (warp == 5 && lane == 0) {
    tma_prefetch_desc(&cache_map);
    tma_prefetch_desc(&hist_map);
    tma_prefetch_desc(&init_map);
    tma_prefetch_desc(&dhist_map);
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
      for (int it = 0; it < T; ++it) {
        if (kJitter && jitter != 0u) jitter_stall(jitter, 1u, static_cast<uint32_t>(it));
        const int pb = it & 1;
        const long long m0 = prof ? clock64() : 0;
        if (!mbar_wait_bounded<false, true>(smem_u32(&s_dg_bar[pb]), (it >> 1) & 1, limit, abort_flag)) {
          report_bks(p.err, kErrWaitDg, it);
          break;
        }
        fence_proxy_async_smem();
        tc_fence_after_sync();
        const long long m1 = prof ? clock64() : 0;
        const uint32_t db = smem_u32(dgbuf + pb * dg_bytes);
        for (int kk = 0; kk < Kc / 16; ++kk) {
          const uint64_t bdesc = umma_smem_desc(db + kk * 2 * (BT * 16), BT * 16, 128);
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
      const uint32_t stage_tx = static_cast<uint32_t>(p.box_b) * UO * (GCL * CT::CES + 3 * S * 4);
      const int sbu = p.box_b * UO;  // floats per state plane in a stage
      for (int it = 0; it < T; ++it) {
        const int s = it % Cfg::NST;
        const int t = T - 1 - it;
        if (it >= Cfg::NST) {
          if (!mbar_wait_bounded<false>(smem_u32(&s_empty[s]), ((it / Cfg::NST) - 1) & 1, limit, abort_flag)) {
            report_bks(p.err, kErrWaitEmpty, it);
            break;
          }
        }
        // after a failed wait anywhere the stages are released early: do not arm a barrier whose
        // previous copy may still be in flight (the flag is set before any thread skips a wait)
        if (*abort_flag != 0) break;
        const uint32_t bar = smem_u32(&s_full[s]);
        uint8_t* sb = stages + s * Cfg::STAGE_BYTES;
        mbar_arrive_expect_tx(bar, stage_tx);
        if (GCL > 0) tma_load_5d(smem_u32(sb), &cache_map, bar, u0, n, 0, t, b0);
        float* q = reinterpret_cast<float*>(sb + GCL * sbu * CT::CES);
        tma_load_5d(smem_u32(q), &hist_map, bar, u0, n, t, b0, 0);
        q += S * sbu;
        if (t > 0) tma_load_5d(smem_u32(q), &hist_map, bar, u0, n, t - 1, b0, 0);
        else tma_load_5d(smem_u32(q), &init_map, bar, u0, n, 0, b0, 0);
        q += S * sbu;
        tma_load_5d(smem_u32(q), &dhist_map, bar, u0, n, t, b0, 0);
      }
    }
  } else {
    const int sbu = p.box_b * UO;
    // accumulator row of this thread: unit p_row of the tile; its partial sums go to the unit's owner
    const int owner = tid / UO;
    const uint32_t part_local = smem_u32(part) + static_cast<uint32_t>(ks * BV * UO + (tid % UO)) * 4u;
    const uint32_t part_remote = map_to_cta(part_local, owner);
    const uint32_t bar_remote0 = map_to_cta(smem_u32(&s_part_bar[0]), owner);
    const uint32_t bar_remote1 = map_to_cta(smem_u32(&s_part_bar[1]), owner);
    // packets this thread fetches from the group's operand buffer: rows `prow`, k-groups kg0 + j * KG_STEP
    constexpr int KG_STEP = kEpiThreads / BV;
    constexpr int XCH = (kMaxKc / 8 + KG_STEP - 1) / KG_STEP;
    const int prow = tid % BV, kg0 = tid / BV;
    const size_t poll_base = static_cast<size_t>(ks) * dg_bytes + static_cast<size_t>(kg0) * (BT * 16) + prow * 16;
    long long pc[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    int rounds = 0;
    // Packets (eight units of one gate and batch row) of the staging layout [gate][batch][unit] that
    // this thread moves, and where each lives inside an operand slot (gate row k = g * D + unit,
    // K-chunk k / Kc, then K-major with 16-byte packets per batch row). The staging area is the
    // buffer of the final db reduction, unused until then.
    constexpr int PPR = UO / 8;                 // packets per (gate, batch row)
    constexpr int NPK = CT::GR * BV * PPR;      // packets per step
    constexpr int NPT = (NPK + kEpiThreads - 1) / kEpiThreads;
    __nv_bfloat16* const pubbuf = reinterpret_cast<__nv_bfloat16*>(dbuf);
    __nv_bfloat16* const pubw = pubbuf + CT::GR * BV * UO;
    static_assert((CT::GR + (CELL == kGRU ? CT::GW : 0)) * 2 <= CT::GB * 4, "staging fits the db buffer");
    uint32_t pk_at[NPT];
#pragma unroll
    for (int q = 0; q < NPT; ++q) {
      const int pi = tid + q * kEpiThreads;
      const int k = (pi / (BV * PPR)) * D + u0 + (pi % PPR) * 8;
      pk_at[q] = pi < NPK ? static_cast<uint32_t>(k / Kc) * static_cast<uint32_t>(dg_bytes) +
                                static_cast<uint32_t>((k % Kc) >> 3) * (BT * 16)
                          : 0u;
    }
    bool dead = false;  // after a failed wait the warp keeps walking through the loop without waiting
    const bool clip_on = OPTS && p.grad_clip > 0.0f;
    const bool cut = OPTS && p.cut_recurrent != 0;
    const bool slstm_v1 = OPTS && p.slstm_v1 != 0;

    float cache[NI][CT::GC], sn[NI][S], sp[NI][S], dhs[NI][S];
    auto load_stage = [&](int it) {
      const int s = it % Cfg::NST;
      if (!dead && !mbar_wait_bounded<false, true>(smem_u32(&s_full[s]), (it / Cfg::NST) & 1, limit, abort_flag)) {
        report_bks(p.err, kErrWaitWx, it);
        dead = true;
      }
      const uint8_t* sb = stages + s * Cfg::STAGE_BYTES;
#pragma unroll
      for (int j = 0; j < NI; ++j) {
        const int ib = (ib0 + j * RPP) % BV;
#pragma unroll
        for (int g = 0; g < GCL; ++g) cache[j][g] = ld_cache<CT::CES>(sb, (ib * GCL + g) * UO + ul);
        const float* q = reinterpret_cast<const float*>(sb + GCL * sbu * CT::CES);
#pragma unroll
        for (int k = 0; k < S; ++k) {
          sn[j][k] = q[k * sbu + ib * UO + ul];
          sp[j][k] = q[(S + k) * sbu + ib * UO + ul];
          dhs[j][k] = q[(2 * S + k) * sbu + ib * UO + ul];
        }
      }
      mbar_arrive(smem_u32(&s_empty[s]));
    };
    load_stage(0);

    for (int it = 0; it <= T; ++it) {
      if (kJitter && jitter != 0u) jitter_stall(jitter, 0u, static_cast<uint32_t>(it));
      const int t = T - 1 - it;
      const int pb = it & 1;
      const long long c0 = prof ? clock64() : 0;
      float ds[NI][S];
#pragma unroll
      for (int j = 0; j < NI; ++j)
#pragma unroll
        for (int q = 0; q < S; ++q) ds[j][q] = dcar[j][q] + (it < T ? dhs[j][q] : 0.0f);
      if (it >= 1) {
        // partial dh of this step from the KS CTAs of the cluster
        if (!dead && !mbar_wait_bounded<true, true>(smem_u32(&s_part_bar[pb]), ((it - 1) >> 1) & 1, limit, abort_flag)) {
          report_bks(p.err, kErrWaitPart, it);
          dead = true;
        }
        const float* pbuf = part + pb * Cfg::PART_FLOATS;
#pragma unroll
        for (int j = 0; j < NI; ++j) {
          const int ib = (ib0 + j * RPP) % BV;
          if (!cut) {
#pragma unroll
            for (int src = 0; src < KS; ++src) ds[j][0] += pbuf[(src * BV + ib) * UO + ul];
          }
        }
        // the buffer of this parity is free again: arm its barrier for iteration it + 2 (only a barrier
        // whose phase has completed may be armed again, hence not after a failed wait)
        if (tid == 0 && !dead && it + 2 <= T) mbar_arrive_expect_tx(smem_u32(&s_part_bar[pb]), part_tx);
      }
      if (clip_on && it >= 1 && it < T) {
        // the gradient carried into h_t from step t + 1 (total minus the external part) is complete here: clip it
#pragma unroll
        for (int j = 0; j < NI; ++j) ds[j][0] = clip_sym(ds[j][0] - dhs[j][0], p.grad_clip) + dhs[j][0];
      }
      const long long c1 = prof ? clock64() : 0;
      if (it == T) {
#pragma unroll
        for (int j = 0; j < NI; ++j) {
          if (act[j]) {
#pragma unroll
            for (int q = 0; q < S; ++q)
              p.d_initial[q * BND + static_cast<size_t>(b0 + ib0 + j * RPP) * ND + n * D + d0] = ds[j][q];
          }
        }
        break;
      }
      float gr[NI][CT::GR], gw[NI][CT::GW];
      const bool take_i = CELL == kSLSTM && t == 0 && p.slstm_zero_first != 0;
#pragma unroll
      for (int j = 0; j < NI; ++j) {
        float gb[CT::GB];
        cell_backward<CELL>(cache[j], sp[j], sn[j], ds[j], gr[j], gw[j], gb, take_i, slstm_v1);
#pragma unroll
        for (int q = 0; q < S; ++q) dcar[j][q] = ds[j][q];
        if (!act[j]) {
#pragma unroll
          for (int g = 0; g < CT::GR; ++g) gr[j][g] = 0.0f;
#pragma unroll
          for (int g = 0; g < CT::GW; ++g) gw[j][g] = 0.0f;
        } else {
#pragma unroll
          for (int g = 0; g < CT::GB; ++g) dbacc[j][g] += gb[g];
        }
      }
      const long long c2 = prof ? clock64() : 0;
      // round_bf16(dG_t) of the owned units is first laid out in shared memory as [gate][batch][unit], so
      // that all 128 threads then move 16-byte packets (eight units of one gate and batch row): to the
      // group's operand slot, to dgr for the dR contraction, and (bf16 Wx) to dWx.
      const bool publish = !dead && it < mute_from;
#pragma unroll
      for (int j = 0; j < NI; ++j) {
        const int ib = ib0 + j * RPP;
#pragma unroll
        for (int g = 0; g < CT::GR; ++g) pubbuf[(g * BV + ib) * UO + ul] = __float2bfloat16_rn(gr[j][g]);
        if constexpr (WX_BF16 && CELL == kGRU) {
#pragma unroll
          for (int g = 0; g < CT::GW; ++g) pubw[(g * BV + ib) * UO + ul] = __float2bfloat16_rn(gw[j][g]);
        }
        if constexpr (!WX_BF16) {
          if (act[j]) {
            const size_t row = static_cast<size_t>(b0 + ib) * T + t;
#pragma unroll
            for (int g = 0; g < CT::GW; ++g) static_cast<float*>(p.dwx)[(row * CT::GW + g) * ND + n * D + d0] = gw[j][g];
          }
        }
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
#pragma unroll
      for (int q = 0; q < NPT; ++q) {
        const int pi = tid + q * kEpiThreads;
        const int b = (pi % (BV * PPR)) / PPR;
        if (pi < NPK && b < bv) {
          const int g = pi / (BV * PPR), u8 = pi % PPR;
          const uint4 pk = reinterpret_cast<const uint4*>(pubbuf)[pi];
          if (publish) {
            // The data words double as arrival flags; the packet of slot (it + 2) % 4, which held dG of
            // iteration it - 2 and has been consumed by every CTA, is refilled, and the fence after the
            // poll below orders the refill before this thread's next data store to that slot.
            const size_t at = pk_at[q] + b * 16;
            st_relaxed_gpu_v4(xg_dg + static_cast<size_t>(it & 3) * slot_bytes + at,
                              make_uint4(xg_clean(pk.x), xg_clean(pk.y), xg_clean(pk.z), xg_clean(pk.w)));
            st_relaxed_gpu_v4(xg_dg + static_cast<size_t>((it + 2) & 3) * slot_bytes + at,
                              make_uint4(kXgFill, kXgFill, kXgFill, kXgFill));
          }
          const size_t off = ((static_cast<size_t>(b0 + b) * T + t) * CT::GR + g) * ND + n * D + u0 + u8 * 8;
          *reinterpret_cast<uint4*>(p.dgr + off) = pk;
          if constexpr (WX_BF16 && CELL != kGRU) {  // W-gate and R-gate gradients coincide, and so do the layouts
            if (p.dwx != static_cast<void*>(p.dgr)) *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.dwx) + off) = pk;
          }
        }
      }
      if constexpr (WX_BF16 && CELL == kGRU) {
        constexpr int NPKW = CT::GW * BV * PPR;
#pragma unroll
        for (int q = 0; q < (NPKW + kEpiThreads - 1) / kEpiThreads; ++q) {
          const int pi = tid + q * kEpiThreads;
          const int b = (pi % (BV * PPR)) / PPR;
          if (pi < NPKW && b < bv) {
            const int g = pi / (BV * PPR), u8 = pi % PPR;
            const size_t off = ((static_cast<size_t>(b0 + b) * T + t) * CT::GW + g) * ND + n * D + u0 + u8 * 8;
            *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.dwx) + off) = reinterpret_cast<const uint4*>(pubw)[pi];
          }
        }
      }
      // While the packets of the other CTAs are on their way: next step's inputs into registers. Polling
      // right away would only add a wasted round trip to the far L2.
      if (it + 1 < T) load_stage(it + 1);
      const long long c3 = prof ? clock64() : 0;
      {
        // fetch this CTA's K-chunk of dG_t from slot it % 4 into the operand buffer
        const uint8_t* src = xg_dg + static_cast<size_t>(it & 3) * slot_bytes + poll_base;
        uint8_t* dst = dgbuf + pb * dg_bytes + kg0 * (BT * 16) + prow * 16;
        uint32_t pend = 0;
        if (prow < bv && !dead) {
#pragma unroll
          for (int j = 0; j < XCH; ++j)
            if (kg0 + j * KG_STEP < Kc / 8) pend |= 1u << j;
        }
        uint64_t t0 = 0;
        uint32_t poll_rounds = 0;
        while (pend != 0u) {
          if (prof) ++rounds;
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
              report_bks(p.err, kErrWaitDg, it);
              dead = true;
              break;
            }
          }
        }
        // a wait that ran out in some lanes only must not leave the warp divided: the warp-wide
        // tcgen05.ld of the next step needs all lanes on one path
        dead = __any_sync(0xffffffffu, dead);
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(&s_dg_bar[pb]));
        fence_acq_rel_gpu();
      }
      const long long c4 = prof ? clock64() : 0;
      const long long c5 = c4;
      if (!dead && !mbar_wait_bounded<false, true>(smem_u32(&s_mma_bar), it & 1, limit, abort_flag)) {
        report_bks(p.err, kErrWaitMma, it);
        dead = true;
      }
      tc_fence_after_sync();
      const long long c6 = prof ? clock64() : 0;
      {
        // partial dh_{t-1} of this row for all batch columns -> the owner's buffer [source][batch][unit]
        uint32_t r[BV / 8][8];
#pragma unroll
        for (int c = 0; c < BV / 8; ++c) tmem_ld_x8(tmem_addr(tbase, 32 * warp, 8 * c), r[c]);
        tmem_ld_wait();
        tc_fence_before_sync();
        if (!dead) {
          const uint32_t dst = part_remote + static_cast<uint32_t>((it + 1) & 1) * Cfg::PART_BYTES;
          const uint32_t bar = ((it + 1) & 1) ? bar_remote1 : bar_remote0;
#pragma unroll
          for (int c = 0; c < BV / 8; ++c)
#pragma unroll
            for (int q = 0; q < 8; ++q) st_async_b32(dst + (8 * c + q) * UO * 4, r[c][q], bar);
        }
      }
      if (prof) {
        pc[0] += c1 - c0; pc[1] += c2 - c1; pc[2] += c3 - c2; pc[3] += c4 - c3; pc[4] += c5 - c4;
        pc[5] += c6 - c5; pc[6] += clock64() - c6;
      }
    }
    if (prof) {
#pragma unroll
      for (int q = 0; q < 8; ++q) p.err[8 + q] = static_cast<int>(pc[q]);
      p.err[18] = rounds;
    }
    // bias gradient: per-thread sums -> shared memory, reduced over the batch rows below
#pragma unroll
    for (int j = 0; j < NI; ++j) {
      const int ib = ib0 + j * RPP;
      if (ib < BV) {
#pragma unroll
        for (int g = 0; g < CT::GB; ++g) dbuf[(ib * CT::GB + g) * UO + ul] = act[j] ? dbacc[j][g] : 0.0f;
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
  for (int i = tid; i < CT::GB * UO; i += kThreads) {
    float acc = 0.0f;
    for (int b = 0; b < bv; ++b) acc += dbuf[b * CT::GB * UO + i];
    const int g = i / UO, u = i % UO;
    p.db_part[((static_cast<size_t>(btile) * CT::GB + g) * N + n) * D + u0 + u] = acc;
  }
  cluster_sync_all();
  if (warp == 4) tmem_dealloc(tbase, tmem_cols);
}

template <int CELL, int BV, int KS, bool WX_BF16, bool OPTS>
int launch_bwd_ks_opt(const BwdParams& p, const void* cache, const float* history, const float* initial,
                      const float* d_history, cudaStream_t stream, int* capacity_only) {
  using Cfg = BksCfg<CELL, BV, KS, WX_BF16>;
  using CT = typename Cfg::CT;
  const int K = CT::GR * p.D;
  if (p.D % 128 != 0 || K % (KS * 16) != 0 || K / KS > kMaxKc) return -2;
  if (capacity_only == nullptr && p.xg_data == nullptr) return -2;
  const int Kc = K / KS;
  const int dg_bytes = Cfg::BT * Kc * 2;
  int smem = ((2 * dg_bytes + 2 * Cfg::PART_BYTES + Cfg::DBUF_BYTES + 127) & ~127) + Cfg::NST * Cfg::STAGE_BYTES;
  if (smem > 227 * 1024) return -2;
  const uint64_t uD = p.D, uN = p.N, uT = p.T, uB = p.B;
  const uint32_t ub = static_cast<uint32_t>(p.box_b);
  const uint32_t uo = static_cast<uint32_t>(Cfg::UO);
  CUtensorMap cache_map, hist_map, init_map, dhist_map;
  if (capacity_only == nullptr) {
    const uint64_t dims[5] = {uD, uN, static_cast<uint64_t>(Cfg::GCL > 0 ? Cfg::GCL : 1), uT, uB};
    const uint32_t box[5] = {uo, 1u, static_cast<uint32_t>(Cfg::GCL > 0 ? Cfg::GCL : 1), 1u, ub};
    // Elman has no cache: describe the history instead so that the (unused) map is valid.
    const void* base = Cfg::GCL > 0 ? static_cast<const void*>(cache) : static_cast<const void*>(history);
    if (make_tensor_map(&cache_map, base, Cfg::GCL > 0 ? CT::CES : 4, 5, dims, box) != 0) return -4;
  }
  if (capacity_only == nullptr) {
    const uint64_t dims[5] = {uD, uN, uT, uB, static_cast<uint64_t>(CT::S)};
    const uint32_t box[5] = {uo, 1u, 1u, ub, static_cast<uint32_t>(CT::S)};
    if (make_tensor_map(&hist_map, history, 4, 5, dims, box) != 0) return -4;
    if (make_tensor_map(&dhist_map, d_history, 4, 5, dims, box) != 0) return -4;
    const uint64_t dims1[5] = {uD, uN, 1u, uB, static_cast<uint64_t>(CT::S)};
    if (make_tensor_map(&init_map, initial, 4, 5, dims1, box) != 0) return -4;
  }
  auto kern = frnn_bwd_ks_kernel<CELL, BV, KS, WX_BF16, OPTS>;
  const int fit = fit_tmem_budget(kern, kThreads, tmem_cols_pow2(Cfg::A_COL0 + Kc / 2, 64u), &smem);
  if (fit != 0) return fit;
  cudaError_t e = cudaSuccess;
  const int n_btiles = (p.B + BV - 1) / BV;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(p.N * n_btiles * (p.D / 128) * KS));
  cfg.blockDim = dim3(kThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  // clusters of KS CTAs (the K-split partners of a unit tile); all CTAs wait on one another through
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
  e = cudaLaunchKernelEx(&cfg, kern, p, cache_map, hist_map, init_map, dhist_map);
  return static_cast<int>(e);
}

template <int CELL, int BV, int KS, bool WX_BF16>
int launch_bwd_ks(const BwdParams& p, const void* cache, const float* history, const float* initial,
                  const float* d_history, cudaStream_t stream, int* capacity_only = nullptr) {
  const bool opts = p.grad_clip > 0.0f || p.cut_recurrent != 0 || p.slstm_v1 != 0;
  return opts ? launch_bwd_ks_opt<CELL, BV, KS, WX_BF16, true>(p, cache, history, initial, d_history, stream, capacity_only)
              : launch_bwd_ks_opt<CELL, BV, KS, WX_BF16, false>(p, cache, history, initial, d_history, stream, capacity_only);
}

template <int CELL, int KS>
int launch_bwd_ks_bv(const BwdParams& p, const void* cache, const float* history, const float* initial,
                     const float* d_history, int wx_bf16, int bv, cudaStream_t s, int* cap) {
  if (bv == 8)
    return wx_bf16 ? launch_bwd_ks<CELL, 8, KS, true>(p, cache, history, initial, d_history, s, cap)
                   : launch_bwd_ks<CELL, 8, KS, false>(p, cache, history, initial, d_history, s, cap);
  if (bv == 16)
    return wx_bf16 ? launch_bwd_ks<CELL, 16, KS, true>(p, cache, history, initial, d_history, s, cap)
                   : launch_bwd_ks<CELL, 16, KS, false>(p, cache, history, initial, d_history, s, cap);
  return -2;
}
template <int CELL> constexpr bool CT_GR_IS_ONE = CellTraits<CELL>::GR == 1;
template <int CELL>
int launch_bwd_ks_cell(const BwdParams& p, const void* cache, const float* history, const float* initial,
                       const float* d_history, int wx_bf16, int bv, int ksplit, cudaStream_t s, int* cap) {
  if constexpr (CT_GR_IS_ONE<CELL>) {  // only a single-gate cell is narrow enough in K for two chunks
    if (ksplit == 2) return launch_bwd_ks_bv<CELL, 2>(p, cache, history, initial, d_history, wx_bf16, bv, s, cap);
  }
  if (ksplit == 4) return launch_bwd_ks_bv<CELL, 4>(p, cache, history, initial, d_history, wx_bf16, bv, s, cap);
  if (ksplit == 8) return launch_bwd_ks_bv<CELL, 8>(p, cache, history, initial, d_history, wx_bf16, bv, s, cap);
  return -2;
}

}  // namespace

// Smallest cluster width over which the K = gates_r * D gate rows of the backward contraction can be
// split so that one chunk of R fits a CTA's tensor memory; 0 if the head cannot be split this way.
int backward_ksplit_width(int gates_r, int D) {
  if (D % 128 != 0) return 0;
  const int K = gates_r * D;
  for (int ks = 2; ks <= 8; ks *= 2)
    if (K % (ks * 16) == 0 && K / ks <= kMaxKc) return ks;
  return 0;
}
// Can the gate rows be split over exactly `ks` CTAs (a wider split than necessary shortens the
// tensor-core chain of a step and the operand chunk every CTA has to fetch)?
bool backward_ksplit_valid(int cell, int gates_r, int D, int ks) {
  if (D % 128 != 0 || (ks != 2 && ks != 4 && ks != 8)) return false;
  if (ks == 2 && gates_r != 1) return false;  // two chunks are only compiled for the single-gate cell
  const int K = gates_r * D;
  (void)cell;
  return K % (ks * 16) == 0 && K / ks <= kMaxKc;
}

int backward_ksplit_dispatch(int cell, const BwdParams& p, const void* cache, const float* history,
                             const float* initial, const float* d_history, int wx_bf16, int bv, int ksplit,
                             cudaStream_t s, int* capacity_only) {
  switch (cell) {
    case kLSTM: return launch_bwd_ks_cell<kLSTM>(p, cache, history, initial, d_history, wx_bf16, bv, ksplit, s, capacity_only);
    case kSLSTM: return launch_bwd_ks_cell<kSLSTM>(p, cache, history, initial, d_history, wx_bf16, bv, ksplit, s, capacity_only);
    case kGRU: return launch_bwd_ks_cell<kGRU>(p, cache, history, initial, d_history, wx_bf16, bv, ksplit, s, capacity_only);
    case kElman: return launch_bwd_ks_cell<kElman>(p, cache, history, initial, d_history, wx_bf16, bv, ksplit, s, capacity_only);
    default: return -1;
  }
}

// How many CTAs of the backward launch for this shape the device can hold at once (clusters of
// `ksplit` CTAs are placed inside one GPC, so this can be less than the SM count); <= 0 if unknown.
int backward_ksplit_capacity(int cell, int bv, int ksplit, int D) {
  BwdParams p{};
  p.B = bv; p.T = 1; p.N = 1; p.D = D;
  p.box_b = bv;
  int cap = 0;
  const int rc = backward_ksplit_dispatch(cell, p, nullptr, nullptr, nullptr, nullptr, 1, bv, ksplit, nullptr, &cap);
  return rc == 0 ? cap : 0;
}

}  // namespace frnn
