// Persistent BPTT recurrence of ONE wide head whose units are split over the GPUs of a node: every rank owns
// the COLUMNS of R that belong to its units.
//
// dh_{t-1}[p] = sum over all recurrent gate rows k = (g, o) of dG_t[k] * R[g, o, p]. Rank r owns units
// p in [r*Dl, (r+1)*Dl); its CTAs form a 2-D grid: Dl/128 unit tiles times KS chunks of K = GR*D. CTA (ut, ks)
// keeps R[k in chunk ks, p in tile ut] transposed on the SM for the whole sequence: the first k_tmem rows in
// tensor memory, the rest in a ring of MN-major, 128-byte-swizzled shared-memory stages filled by TMA (streamed
// again every step when the ring is too short). Per step, going backwards in time:
//   1. the owner of (unit, batch row) adds dH_t, the carried gradient and the KS partial sums of dh_t that its
//      cluster partners sent, and runs the cell's backward formulas              -> dG_t of its units
//   2. round_bf16(dG_t) is stored into the dG history of EVERY rank (peer stores; see recurrent_mg_common.cuh),
//      dWx and db are kept locally
//   3. every CTA stages its K-chunk of dG_t from this rank's own history in sub-chunks of 512 k and multiplies
//                                                                                -> partial dh_{t-1} [128 x batch]
//   4. batch columns [ks'*BO, (ks'+1)*BO) of every accumulator row go to cluster partner ks' (async DSMEM stores).
// The dG history [B][T][GR*D] is afterwards operand A of the dR contraction (rows of this rank's units only).
//
// Reference: flashrnn/flashrnn2/hybrid_bw2d.cu:507-552,645-661 (the _mg backward with peer tables);
// gradient formulas: cells.cuh.
#include "recurrent_mg_common.cuh"

namespace frnn {

namespace {

constexpr int kEpi = 128;
constexpr int kMgThreads = 224;  // 4 epilogue warps, MMA warp, state TMA warp, weight-ring TMA warp

template <int CELL, int KS, bool WX_BF16>
struct MgBwdCfg {
  using CT = CellTraits<CELL>;
  static constexpr int BO = kMgBT / KS;  // batch rows owned by one CTA of the cluster; thread tid owns unit tid of all of them
  static constexpr int GCL = CELL == kElman ? 0 : CT::GC;
  static constexpr int CACHE_BYTES = GCL * BO * 128 * CT::CES;  // the cached gates come first in a stage
  static constexpr int STAGE_BYTES = CACHE_BYTES + 3 * CT::S * BO * 128 * 4;
  static_assert(CACHE_BYTES % 128 == 0, "TMA destinations after the cached gates stay 128-byte aligned");
  static constexpr int NST = STAGE_BYTES * 4 <= 49152 ? 4 : (STAGE_BYTES * 3 <= 65536 ? 3 : 2);
  static constexpr int PART_FLOATS = KS * 128 * BO;  // one parity: [source][unit][owned batch row]
  static constexpr int PART_BYTES = PART_FLOATS * 4;
  static constexpr int PUBW = (WX_BF16 && CELL == kGRU) ? CT::GW : 0;  // separate staging of the W-gate gradients
  static constexpr int PUB_BYTES = (CT::GR + PUBW) * BO * 128 * 2;     // [gate][batch row][unit] bf16
  static_assert(KS == 4 || KS == 8 || KS == 16, "cluster width");
};

template <int CELL, int KS, bool WX_BF16>
__global__ void __launch_bounds__(kMgThreads, 1)
frnn_bwd_mg_kernel(const MgBwdParams p, const __grid_constant__ CUtensorMap cache_map,
                   const __grid_constant__ CUtensorMap hist_map, const __grid_constant__ CUtensorMap init_map,
                   const __grid_constant__ CUtensorMap dhist_map, const __grid_constant__ CUtensorMap r_map) {
  using Cfg = MgBwdCfg<CELL, KS, WX_BF16>;
  using CT = typename Cfg::CT;
  constexpr int BT = kMgBT, BO = Cfg::BO, S = CT::S, GCL = Cfg::GCL;

  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) uint64_t s_dgbar[2];
  __shared__ __align__(8) uint64_t s_dgfree[2];
  __shared__ __align__(8) uint64_t s_mma_bar;
  __shared__ __align__(8) uint64_t s_part_bar[2];
  __shared__ __align__(8) uint64_t s_full[4];
  __shared__ __align__(8) uint64_t s_empty[4];
  __shared__ __align__(8) uint64_t s_afull[kMgMaxRing];
  __shared__ __align__(8) uint64_t s_aempty[kMgMaxRing];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_ready_ok;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int D = p.D, T = p.T, B = p.B, Dl = p.Dl, ldx = p.ldx, P = p.P;
  const int per_rank = (Dl / 128) * KS;
  const int lr = static_cast<int>(blockIdx.x) / per_rank;
  const int rank = p.rank0 + lr;
  const int cta = static_cast<int>(blockIdx.x) % per_rank;
  const int ks = cta % KS;  // == rank inside the cluster
  const int ut = cta / KS;
  const int xu = lr * p.x_rank_stride + ut * 128;  // first unit of the tile inside the local tensors
  const int ug = rank * Dl + ut * 128;             // first unit of the tile inside the head
  const int K = CT::GR * D;
  const int Kc = K / KS;
  const int SCK = Kc < kMgSubK ? Kc : kMgSubK;
  const int NSC = Kc / SCK;
  const int dg_bytes = mg_operand_bytes(SCK);
  const int k_tmem = p.k_tmem, n_ring = p.n_ring, NA = p.ring_stages;
  const bool resident = p.resident != 0;
  uint8_t* const ring = smem;
  uint8_t* const dgbuf = smem + NA * kMgRingBytes;
  float* const part = reinterpret_cast<float*>(dgbuf + 2 * dg_bytes);
  __nv_bfloat16* const pub = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(part) + 2 * Cfg::PART_BYTES);
  uint8_t* const stages = reinterpret_cast<uint8_t*>(pub) + ((Cfg::PUB_BYTES + 127) & ~127);
  const volatile int* abort_flag = p.err;
  const uint64_t limit = p.wait_limit_ns;
  const int mute_from = p.err[4] != 0 ? p.err[5] : 0x7fffffff;  // test hook: nobody publishes from this step on
  // Second test hook, race verification by delay injection (err[6] = seed, see jitter_stall). It is compiled into the
  // fp32-Wx instantiations only: the exchange code is the same for both Wx types, and even the untaken per-step test
  // costs the bf16 backward more than 1 %.
  constexpr bool kJitter = !WX_BF16;
  const uint32_t jitter = kJitter ? static_cast<uint32_t>(p.err[6]) : 0u;
  constexpr uint32_t tmem_cols = 512;
  const size_t grow = static_cast<size_t>(T) * K;  // elements per batch row of a dG history buffer

  // ---------------- prologue ----------------
  if (tid == 0) {
    mbar_init(smem_u32(&s_dgbar[0]), kEpi);
    mbar_init(smem_u32(&s_dgbar[1]), kEpi);
    mbar_init(smem_u32(&s_dgfree[0]), 1);
    mbar_init(smem_u32(&s_dgfree[1]), 1);
    mbar_init(smem_u32(&s_mma_bar), 1);
    mbar_init(smem_u32(&s_part_bar[0]), 1);
    mbar_init(smem_u32(&s_part_bar[1]), 1);
    for (int s = 0; s < Cfg::NST; ++s) {
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&s_empty[s]), kEpi);
    }
    for (int s = 0; s < kMgMaxRing; ++s) {
      mbar_init(smem_u32(&s_afull[s]), 1);
      mbar_init(smem_u32(&s_aempty[s]), 1);
    }
    fence_mbar_init();
    s_ready_ok = 1;
    if (p.ranks_here < P && !mg_handshake(p.ready, rank, P, p.epoch, cta == 0, limit, abort_flag)) {
      mg_report(p.err, kErrWaitReady, 0);
      s_ready_ok = 0;
    }
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(&s_tmem_base), tmem_cols);
    tmem_relinquish_alloc();
  }
  for (int i = tid; i < 2 * dg_bytes / 16; i += kMgThreads) reinterpret_cast<uint4*>(dgbuf)[i] = make_uint4(0u, 0u, 0u, 0u);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = s_tmem_base;
  const bool ready_ok = s_ready_ok != 0;

  if (warp < 4) {
    // R[k, p in tile] for the first k_tmem gate rows of the chunk -> tensor memory, lane = p, column c packs
    // k = 2c, 2c + 1. Sixteen rows of R (128 consecutive p each) are staged in shared memory with coalesced
    // loads (the partial-sum buffers are still idle) and read back column-wise.
    __nv_bfloat16* const rbuf = reinterpret_cast<__nv_bfloat16*>(part);  // [16][128]
    for (int c0 = 0; c0 < k_tmem / 2; c0 += 8) {
      for (int v = tid; v < 16 * 16; v += kEpi) {
        const int kk = v / 16, pv = v % 16;
        const size_t k = static_cast<size_t>(ks) * Kc + 2 * c0 + kk;
        reinterpret_cast<uint4*>(rbuf)[v] = __ldg(reinterpret_cast<const uint4*>(p.Rc + k * ldx + xu + pv * 8));
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      uint32_t r[8];
#pragma unroll
      for (int q = 0; q < 8; ++q)
        r[q] = static_cast<uint32_t>(__bfloat16_as_ushort(rbuf[(2 * q) * 128 + tid])) |
               (static_cast<uint32_t>(__bfloat16_as_ushort(rbuf[(2 * q + 1) * 128 + tid])) << 16);
      tmem_st_x8(tmem_addr(tbase, 32 * warp, BT + c0), r);
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    tmem_st_wait();
  }

  // thread tid owns unit tid of the tile for the batch rows ks*BO + j, j < BO
  float dcar[BO][S];
  float dbacc[BO][CT::GB];
#pragma unroll
  for (int j = 0; j < BO; ++j) {
    const int b = ks * BO + j;
#pragma unroll
    for (int q = 0; q < S; ++q)
      dcar[j][q] = (warp < 4 && b < B) ? p.d_carry[(static_cast<size_t>(q) * B + b) * ldx + xu + tid] : 0.0f;
#pragma unroll
    for (int g = 0; g < CT::GB; ++g) dbacc[j][g] = 0.0f;
  }
  constexpr uint32_t part_tx = static_cast<uint32_t>(KS) * 128u * BO * 4u;
  if (warp == 4 && lane == 0) {
    mbar_arrive_expect_tx(smem_u32(&s_part_bar[1]), part_tx);              // consumed in iteration 1
    if (T >= 2) mbar_arrive_expect_tx(smem_u32(&s_part_bar[0]), part_tx);  // iteration 2
  }
  if (warp == 5 && lane == 0) {
    tma_prefetch_desc(&cache_map);
    tma_prefetch_desc(&hist_map);
    tma_prefetch_desc(&init_map);
    tma_prefetch_desc(&dhist_map);
    tma_prefetch_desc(&r_map);
  }
  fence_proxy_async();
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  tc_fence_after_sync();

  // ---------------- main loops ----------------
  if (warp == 4) {
    if (lane == 0 && ready_ok) {
      const uint32_t idesc_ts = umma_idesc_bf16(128, BT, false, false);
      const uint32_t idesc_ss = umma_idesc_bf16(128, BT, true, false);  // ring stages hold R^T MN-major
      int committed = 0;
      int ring_stage = 0;        // next stage of the weight ring to consume, and the phase its barrier is in
      uint32_t ring_phase = 0;
      bool ok = true;
      for (int it = 0; it < T && ok; ++it) {
        if (kJitter && jitter != 0u) jitter_stall(jitter, 1u, static_cast<uint32_t>(it));
        for (int sc = 0; sc < NSC && ok; ++sc) {
          const long long q = static_cast<long long>(it) * NSC + sc;
          const int buf = static_cast<int>(q & 1);
          if (!mbar_wait_bounded<false, true>(smem_u32(&s_dgbar[buf]), static_cast<uint32_t>((q >> 1) & 1), limit, abort_flag)) {
            mg_report(p.err, kErrWaitDg, it);
            ok = false;
            break;
          }
          fence_proxy_async_smem();
          tc_fence_after_sync();
          // Descriptors advance by constants: 16 k = 32 B inside a 128-byte swizzled row of the operand (2 in units of
          // 16 B), the next 64-k block is 4096 B further (256); eight 32-bit columns of tensor memory; 16 k rows of
          // 128 B (2048 B = 128) inside each box of a weight stage.
          const uint64_t bdesc0 = umma_smem_desc_k_sw128(smem_u32(dgbuf + buf * dg_bytes));
          const int k0 = sc * SCK;
          int n_ts = (k_tmem - k0) / 16;
          n_ts = n_ts < 0 ? 0 : (n_ts > SCK / 16 ? SCK / 16 : n_ts);
          uint32_t acol = tbase + BT + k0 / 2;
          int kk = 0;
#pragma unroll 4
          for (; kk < n_ts; ++kk) {
            umma_bf16_ts(tbase, acol, bdesc0 + (kk >> 2) * 256 + (kk & 3) * 2, idesc_ts, (k0 | kk) != 0 ? 1u : 0u);
            acol += 8;
          }
          for (; kk < SCK / 16; kk += kMgRingK / 16) {
            if (!resident || it == 0) {
              if (!mbar_wait_bounded<false, true>(smem_u32(&s_afull[ring_stage]), ring_phase, limit, abort_flag)) {
                mg_report(p.err, kErrWaitRing, it);
                ok = false;
                break;
              }
              tc_fence_after_sync();
            }
            uint64_t adesc = umma_smem_desc_mn_sw128(smem_u32(ring + ring_stage * kMgRingBytes), 8192u);
            uint64_t bdesc = bdesc0 + (kk >> 2) * 256;
#pragma unroll
            for (int i = 0; i < kMgRingK / 16; ++i) {
              umma_bf16_ss(tbase, adesc, bdesc, idesc_ss, (k0 | kk | i) != 0 ? 1u : 0u);
              adesc += 128;
              bdesc += 2;
            }
            if (!resident) umma_commit(smem_u32(&s_aempty[ring_stage]));
            if (++ring_stage == NA) {
              ring_stage = 0;
              ring_phase ^= 1u;
            }
          }
          if (!ok) break;
          umma_commit(smem_u32(&s_dgfree[buf]));
        }
        if (!ok) break;
        umma_commit(smem_u32(&s_mma_bar));
        ++committed;
      }
      if (!ok) {
        umma_commit(smem_u32(&s_mma_bar));
        ++committed;
      }
      if (committed > 0) mbar_wait_bounded<false, true>(smem_u32(&s_mma_bar), (committed - 1) & 1, limit, nullptr);
    }
  } else if (warp == 5) {
    if (lane == 0 && ready_ok) {
      constexpr uint32_t stage_tx = static_cast<uint32_t>(Cfg::STAGE_BYTES);
      constexpr int sbu = BO * 128;  // floats per state plane in a stage
      for (int it = 0; it < T; ++it) {
        const int s = it % Cfg::NST;
        const int t = T - 1 - it;
        if (it >= Cfg::NST &&
            !mbar_wait_bounded<false>(smem_u32(&s_empty[s]), ((it / Cfg::NST) - 1) & 1, limit, abort_flag)) {
          mg_report(p.err, kErrWaitEmpty, it);
          break;
        }
        if (*abort_flag != 0) break;  // stages are released early after a failed wait: do not arm a busy barrier
        const uint32_t bar = smem_u32(&s_full[s]);
        uint8_t* sb = stages + s * Cfg::STAGE_BYTES;
        mbar_arrive_expect_tx(bar, stage_tx);
        if (GCL > 0) tma_load_5d(smem_u32(sb), &cache_map, bar, xu, 0, 0, t, ks * BO);
        float* q = reinterpret_cast<float*>(sb + Cfg::CACHE_BYTES);
        tma_load_5d(smem_u32(q), &hist_map, bar, xu, 0, t, ks * BO, 0);
        q += S * sbu;
        if (t > 0) tma_load_5d(smem_u32(q), &hist_map, bar, xu, 0, t - 1, ks * BO, 0);
        else tma_load_5d(smem_u32(q), &init_map, bar, xu, 0, 0, ks * BO, 0);
        q += S * sbu;
        tma_load_5d(smem_u32(q), &dhist_map, bar, xu, 0, t, ks * BO, 0);
      }
    }
  } else if (warp == 6) {
    if (lane == 0 && ready_ok && n_ring > 0) {
      const int k_base = ks * Kc + k_tmem;
      auto load_stage = [&](int stage, int j) {
        const uint32_t bar = smem_u32(&s_afull[stage]);
        const uint32_t dst = smem_u32(ring + stage * kMgRingBytes);
        mbar_arrive_expect_tx(bar, static_cast<uint32_t>(kMgRingBytes));
        tma_load_3d(dst, &r_map, bar, xu, k_base + j * kMgRingK, 0);
        tma_load_3d(dst + 8192u, &r_map, bar, xu + 64, k_base + j * kMgRingK, 0);
      };
      if (resident) {
        for (int j = 0; j < n_ring; ++j) load_stage(j, j);
      } else {
        int stage = 0;
        uint32_t phase = 1;  // parity of the release this stage's next refill waits for (none before the first lap)
        bool first_lap = true, ok = true;
        for (int it = 0; it < T && ok; ++it) {
          for (int j = 0; j < n_ring; ++j) {
            if (!first_lap && !mbar_wait_bounded<false, true>(smem_u32(&s_aempty[stage]), phase, limit, abort_flag)) {
              mg_report(p.err, kErrWaitRing, it);
              ok = false;
              break;
            }
            // (a bounded wait that returned true saw no abort; the flag itself is read only once per step)
            if (j == 0 && *abort_flag != 0) { ok = false; break; }
            load_stage(stage, j);
            if (++stage == NA) {
              stage = 0;
              phase ^= 1u;
              first_lap = false;
            }
          }
        }
      }
    }
  } else if (ready_ok) {
    const uint32_t part_local = smem_u32(part) + static_cast<uint32_t>((ks * 128 + tid) * BO) * 4u;
    bool dead = false;
    __nv_bfloat16* const pubw = pub + CT::GR * BO * 128;

    // this CTA's K-chunk of dG of step `t` -> operand buffers, one sub-chunk at a time (iteration `it`)
    auto fetch = [&](int it, int t) {
      for (int sc = 0; sc < NSC; ++sc) {
        const long long q = static_cast<long long>(it) * NSC + sc;
        const int buf = static_cast<int>(q & 1);
        if (q >= 2 && !dead &&
            !mbar_wait_bounded<false, true>(smem_u32(&s_dgfree[buf]), static_cast<uint32_t>(((q >> 1) - 1) & 1), limit, abort_flag)) {
          mg_report(p.err, kErrWaitMma, it);
          dead = true;
        }
        if (!dead && !mg_fetch_subchunk(p.dgr[rank] + static_cast<size_t>(t) * K + static_cast<size_t>(ks) * Kc + sc * SCK, grow,
                                        dgbuf + buf * dg_bytes, SCK, B, warp, lane, limit, abort_flag)) {
          mg_report(p.err, kErrWaitDg, it);
          dead = true;
        }
        dead = __any_sync(0xffffffffu, dead);
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(&s_dgbar[buf]));
      }
    };

    for (int it = 0; it <= T; ++it) {
      if (kJitter && jitter != 0u) jitter_stall(jitter, 0u, static_cast<uint32_t>(it));
      const int t = T - 1 - it;
      const int pb = it & 1;
      if (it >= 1 && !dead &&
          !mbar_wait_bounded<true, true>(smem_u32(&s_part_bar[pb]), ((it - 1) >> 1) & 1, limit, abort_flag)) {
        mg_report(p.err, kErrWaitPart, it);
        dead = true;
      }
      const int s = it % Cfg::NST;
      if (it < T && !dead && !mbar_wait_bounded<false, true>(smem_u32(&s_full[s]), (it / Cfg::NST) & 1, limit, abort_flag)) {
        mg_report(p.err, kErrWaitWx, it);
        dead = true;
      }
      const uint8_t* sb = stages + s * Cfg::STAGE_BYTES;
      const float* pbuf = part + pb * Cfg::PART_FLOATS;
      const bool take_i = CELL == kSLSTM && t == 0 && p.slstm_zero_first != 0;
#pragma unroll
      for (int j = 0; j < BO; ++j) {
        const int b = ks * BO + j;
        const bool act = b < B;
        float ds[S];
#pragma unroll
        for (int q = 0; q < S; ++q) ds[q] = dcar[j][q];
        if (it >= 1) {
#pragma unroll
          for (int src = 0; src < KS; ++src) ds[0] += pbuf[(src * 128 + tid) * BO + j];
        }
        if (it == T) {
          if (act) {
#pragma unroll
            for (int q = 0; q < S; ++q) p.d_initial[(static_cast<size_t>(q) * B + b) * ldx + xu + tid] = ds[q];
          }
          continue;
        }
        float cache[CT::GC], sn[S], sp[S];
#pragma unroll
        for (int g = 0; g < GCL; ++g) cache[g] = ld_cache<CT::CES>(sb, (j * GCL + g) * 128 + tid);
        const float* q0 = reinterpret_cast<const float*>(sb + Cfg::CACHE_BYTES);
#pragma unroll
        for (int k = 0; k < S; ++k) {
          sn[k] = q0[(k * BO + j) * 128 + tid];
          sp[k] = q0[((S + k) * BO + j) * 128 + tid];
          ds[k] += q0[((2 * S + k) * BO + j) * 128 + tid];
        }
        float gr[CT::GR], gw[CT::GW], gb[CT::GB];
        cell_backward<CELL>(cache, sp, sn, ds, gr, gw, gb, take_i);
#pragma unroll
        for (int q = 0; q < S; ++q) dcar[j][q] = ds[q];
        if (act) {
#pragma unroll
          for (int g = 0; g < CT::GB; ++g) dbacc[j][g] += gb[g];
        }
#pragma unroll
        for (int g = 0; g < CT::GR; ++g) pub[(g * BO + j) * 128 + tid] = __float2bfloat16_rn(act ? gr[g] : 0.0f);
        if constexpr (WX_BF16 && CELL == kGRU) {
#pragma unroll
          for (int g = 0; g < CT::GW; ++g) pubw[(g * BO + j) * 128 + tid] = __float2bfloat16_rn(act ? gw[g] : 0.0f);
        }
        if constexpr (!WX_BF16) {
          if (act) {
            const size_t row = static_cast<size_t>(b) * T + t;
#pragma unroll
            for (int g = 0; g < CT::GW; ++g) static_cast<float*>(p.dwx)[(row * CT::GW + g) * ldx + xu + tid] = gw[g];
          }
        }
      }
      if (it == T) break;
      mbar_arrive(smem_u32(&s_empty[s]));
      // The partial-sum buffer of this parity is free again (all threads pass the barrier below before dG_t
      // leaves, and nobody can send the sums of iteration it + 2 before it has seen dG of iteration it + 1).
      if (tid == 0 && it >= 1 && !dead && it + 2 <= T) mbar_arrive_expect_tx(smem_u32(&s_part_bar[pb]), part_tx);
      asm volatile("bar.sync 1, 128;" ::: "memory");
      {
        // packets of eight units of one gate and batch row: to the dG history of every rank and (bf16 Wx) to dWx
        const bool on = !dead && it < mute_from;
        constexpr int NPKT = CT::GR * BO * 16;
        for (int job = tid; job < NPKT * P; job += kEpi) {
          const int pk = job % NPKT, q = job / NPKT;
          const int g = pk / (BO * 16), bl = (pk / 16) % BO, u8 = pk % 16;
          const int b = ks * BO + bl;
          if (b < B) {
            const uint4 v = *reinterpret_cast<const uint4*>(pub + (g * BO + bl) * 128 + u8 * 8);
            if (on)
              st_relaxed_sys_v4(p.dgr[q] + static_cast<size_t>(b) * grow + static_cast<size_t>(t) * K +
                                    static_cast<size_t>(g) * D + ug + u8 * 8,
                                make_uint4(xg_clean(v.x), xg_clean(v.y), xg_clean(v.z), xg_clean(v.w)));
            if constexpr (WX_BF16 && CELL != kGRU) {  // W-gate and R-gate gradients coincide
              if (q == 0)
                *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.dwx) +
                                          ((static_cast<size_t>(b) * T + t) * CT::GW + g) * ldx + xu + u8 * 8) = v;
            }
          }
        }
        if constexpr (WX_BF16 && CELL == kGRU) {
          constexpr int NPKW = CT::GW * BO * 16;
          for (int pk = tid; pk < NPKW; pk += kEpi) {
            const int g = pk / (BO * 16), bl = (pk / 16) % BO, u8 = pk % 16;
            const int b = ks * BO + bl;
            if (b < B)
              *reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(p.dwx) +
                                        ((static_cast<size_t>(b) * T + t) * CT::GW + g) * ldx + xu + u8 * 8) =
                  *reinterpret_cast<const uint4*>(pubw + (g * BO + bl) * 128 + u8 * 8);
          }
        }
      }
      fetch(it, t);
      if (!dead && !mbar_wait_bounded<false, true>(smem_u32(&s_mma_bar), it & 1, limit, abort_flag)) {
        mg_report(p.err, kErrWaitMma, it);
        dead = true;
      }
      tc_fence_after_sync();
      {
        // partial dh_{t-1} of unit `tid`: batch columns [d*BO, (d+1)*BO) go to CTA d of the cluster
        uint32_t r[4][8];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_x8(tmem_addr(tbase, 32 * warp, 8 * c), r[c]);
        tmem_ld_wait();
        tc_fence_before_sync();
        if (!dead) {
          const uint32_t off = static_cast<uint32_t>((it + 1) & 1) * Cfg::PART_BYTES;
          const uint32_t bar_local = smem_u32(&s_part_bar[(it + 1) & 1]);
#pragma unroll
          for (int d = 0; d < KS; ++d) {
            const uint32_t dst = map_to_cta(part_local + off, d);
            const uint32_t bar = map_to_cta(bar_local, d);
            if constexpr (BO >= 4) {
#pragma unroll
              for (int v = 0; v < BO / 4; ++v) {
                const int c0 = d * BO + 4 * v;
                st_async_v4_b32(dst + v * 16, r[c0 / 8][c0 % 8], r[c0 / 8][c0 % 8 + 1], r[c0 / 8][c0 % 8 + 2],
                                r[c0 / 8][c0 % 8 + 3], bar);
              }
            } else {
              const int c0 = d * BO;
              st_async_v2_b32(dst, r[c0 / 8][c0 % 8], r[c0 / 8][c0 % 8 + 1], bar);
            }
          }
        }
      }
    }
    // bias gradient of unit `tid`, summed over this CTA's batch rows
#pragma unroll
    for (int g = 0; g < CT::GB; ++g) {
      float acc = 0.0f;
#pragma unroll
      for (int j = 0; j < BO; ++j) acc += dbacc[j][g];
      p.db_part[(static_cast<size_t>(ks) * CT::GB + g) * ldx + xu + tid] = acc;
    }
  } else if (warp < 4) {
    // the handshake failed: the outputs of this call are invalid; keep db_part defined
    for (int g = 0; g < CT::GB; ++g) p.db_part[(static_cast<size_t>(ks) * CT::GB + g) * ldx + xu + tid] = 0.0f;
  }

  // ---------------- teardown ----------------
  if (*abort_flag != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 4) tmem_dealloc(tbase, tmem_cols);
}

template <int CELL, int KS, bool WX_BF16>
int launch_bwd_mg(const MgBwdParams& p, cudaStream_t stream, int* capacity_only) {
  using Cfg = MgBwdCfg<CELL, KS, WX_BF16>;
  using CT = typename Cfg::CT;
  const int K = CT::GR * p.D;
  const int Kc = K / KS;
  const int SCK = Kc < kMgSubK ? Kc : kMgSubK;
  int smem = p.ring_stages * kMgRingBytes + 2 * mg_operand_bytes(SCK) + 2 * Cfg::PART_BYTES + ((Cfg::PUB_BYTES + 127) & ~127) +
             Cfg::NST * Cfg::STAGE_BYTES;
  if (smem > 227 * 1024) return -2;
  CUtensorMap cache_map, hist_map, init_map, dhist_map, r_map;
  if (capacity_only == nullptr) {
    const uint64_t ux = static_cast<uint64_t>(p.ldx), uT = static_cast<uint64_t>(p.T), uB = static_cast<uint64_t>(p.B);
    const uint32_t bo = static_cast<uint32_t>(Cfg::BO);
    {
      const uint64_t dims[5] = {ux, 1u, static_cast<uint64_t>(Cfg::GCL > 0 ? Cfg::GCL : 1), uT, uB};
      const uint32_t box[5] = {128u, 1u, static_cast<uint32_t>(Cfg::GCL > 0 ? Cfg::GCL : 1), 1u, bo};
      // Elman has no cache: describe the history instead so that the (unused) map is valid.
      const void* base = Cfg::GCL > 0 ? static_cast<const void*>(p.cache) : static_cast<const void*>(p.history);
      if (make_tensor_map(&cache_map, base, Cfg::GCL > 0 ? CT::CES : 4, 5, dims, box) != 0) return -4;
    }
    {
      const uint64_t dims[5] = {ux, 1u, uT, uB, static_cast<uint64_t>(CT::S)};
      const uint32_t box[5] = {128u, 1u, 1u, bo, static_cast<uint32_t>(CT::S)};
      if (make_tensor_map(&hist_map, p.history, 4, 5, dims, box) != 0) return -4;
      if (make_tensor_map(&dhist_map, p.d_history, 4, 5, dims, box) != 0) return -4;
      const uint64_t dims1[5] = {ux, 1u, 1u, uB, static_cast<uint64_t>(CT::S)};
      if (make_tensor_map(&init_map, p.initial, 4, 5, dims1, box) != 0) return -4;
    }
    {
      // columns of R as (p, k = gate row, 1): a box is 64 k rows of 64 p (128 bytes), MN-major for the tensor core
      const uint64_t dims[3] = {ux, static_cast<uint64_t>(K), 1u};
      const uint32_t box[3] = {64u, static_cast<uint32_t>(kMgRingK), 1u};
      if (make_tensor_map(&r_map, p.Rc, 2, 3, dims, box, true) != 0) return -4;
    }
  }
  auto kern = frnn_bwd_mg_kernel<CELL, KS, WX_BF16>;
  const int fit = fit_tmem_budget(kern, kMgThreads, 512u, &smem);
  if (fit != 0) return fit;
  cudaError_t e = cudaSuccess;
  if (KS > 8) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(p.ranks_here * (p.Dl / 128) * KS));
  cfg.blockDim = dim3(kMgThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = KS;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
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
  e = cudaLaunchKernelEx(&cfg, kern, p, cache_map, hist_map, init_map, dhist_map, r_map);
  return static_cast<int>(e);
}

template <int CELL, int KS>
int launch_bwd_mg_dt(const MgBwdParams& p, int wx_bf16, cudaStream_t s, int* cap) {
  return wx_bf16 ? launch_bwd_mg<CELL, KS, true>(p, s, cap) : launch_bwd_mg<CELL, KS, false>(p, s, cap);
}
template <int CELL>
int launch_bwd_mg_ks(const MgBwdParams& p, int wx_bf16, int ks, cudaStream_t s, int* cap) {
  switch (ks) {
    case 4: return launch_bwd_mg_dt<CELL, 4>(p, wx_bf16, s, cap);
    case 8: return launch_bwd_mg_dt<CELL, 8>(p, wx_bf16, s, cap);
    case 16: return launch_bwd_mg_dt<CELL, 16>(p, wx_bf16, s, cap);
    default: return -2;
  }
}

// R_cols[k][pl] = R[g, o, rank*Dl + pl] (k = g*D + o) gathered from the row slices the ranks hold:
// rows o in [q*Dl, (q+1)*Dl) live on rank q as R_rows_q[g][o - q*Dl][:]. Plain peer loads, once per call.
struct GatherParams {
  const __nv_bfloat16* rows[kMgMaxRanks];
  __nv_bfloat16* cols;
  int GR, D, Dl, ld_rows, ld_cols, x_rank_stride, rank0, ranks_here, P;
};
__global__ void gather_columns_kernel(const GatherParams p) {
  const int vec_per_row = p.Dl / 8;
  const long long per_rank = static_cast<long long>(p.GR) * p.D * vec_per_row;
  const long long total = per_rank * p.ranks_here;
  for (long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int lr = static_cast<int>(i / per_rank);
    const long long r = i % per_rank;
    const int v = static_cast<int>(r % vec_per_row);
    const long long k = r / vec_per_row;
    const int g = static_cast<int>(k / p.D), o = static_cast<int>(k % p.D);
    const int rank = p.rank0 + lr;
    const int q = o / p.Dl, ol = o % p.Dl;
    // the owner's buffer holds its rows at row offset (its slot in its own launch) * x_rank_stride
    const int row_off = p.ranks_here == p.P ? q * p.x_rank_stride : 0;
    const __nv_bfloat16* src = p.rows[q] + (static_cast<size_t>(g) * p.ld_rows + row_off + ol) * p.D + rank * p.Dl + v * 8;
    __nv_bfloat16* dst = p.cols + static_cast<size_t>(k) * p.ld_cols + lr * p.x_rank_stride + v * 8;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(src);
  }
}

}  // namespace

int backward_mg_dispatch(int cell, const MgBwdParams& p, int wx_bf16, int ksplit, cudaStream_t s, int* capacity_only) {
  switch (cell) {
    case kLSTM: return launch_bwd_mg_ks<kLSTM>(p, wx_bf16, ksplit, s, capacity_only);
    case kSLSTM: return launch_bwd_mg_ks<kSLSTM>(p, wx_bf16, ksplit, s, capacity_only);
    case kGRU: return launch_bwd_mg_ks<kGRU>(p, wx_bf16, ksplit, s, capacity_only);
    case kElman: return launch_bwd_mg_ks<kElman>(p, wx_bf16, ksplit, s, capacity_only);
    default: return -1;
  }
}

int backward_mg_fixed_smem(int cell, int ksplit, int D, int wx_bf16) {
  const int gr = cell == kGRU ? 3 : (cell == kElman ? 1 : 4);
  const int s = cell == kSLSTM ? 4 : (cell == kLSTM ? 2 : 1);
  const int gcl = cell == kElman ? 0 : 4;
  const int gw = cell == kGRU ? 3 : (cell == kElman ? 1 : 4);
  const int bo = kMgBT / ksplit;
  const int Kc = gr * D / ksplit;
  const int SCK = Kc < kMgSubK ? Kc : kMgSubK;
  const int ces = (cell == kLSTM || cell == kGRU) ? 2 : 4;
  const int stage = (gcl * ces + 3 * s * 4) * bo * 128;
  const int nst = stage * 4 <= 49152 ? 4 : (stage * 3 <= 65536 ? 3 : 2);
  const int pub = (gr + ((wx_bf16 && cell == kGRU) ? gw : 0)) * bo * 128 * 2;
  return 2 * mg_operand_bytes(SCK) + 2 * (ksplit * 128 * bo * 4) + ((pub + 127) & ~127) + nst * stage;
}

int gather_columns_launch(const void* const* rows, void* cols, int gr, int D, int Dl, int P, int rank0, int ranks_here,
                          cudaStream_t s) {
  GatherParams g{};
  for (int q = 0; q < P; ++q) g.rows[q] = static_cast<const __nv_bfloat16*>(rows[q]);
  g.cols = static_cast<__nv_bfloat16*>(cols);
  g.GR = gr; g.D = D; g.Dl = Dl; g.P = P; g.rank0 = rank0; g.ranks_here = ranks_here;
  const bool together = ranks_here == P && P > 1;
  g.ld_rows = together ? D : Dl;
  g.ld_cols = together ? D : Dl;
  g.x_rank_stride = together ? Dl : 0;
  gather_columns_kernel<<<592, 256, 0, s>>>(g);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace frnn
