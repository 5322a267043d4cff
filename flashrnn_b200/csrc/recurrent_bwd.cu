// Persistent reverse-time (BPTT) recurrence for sm_100a.
//
// Same decomposition as the forward kernel: a cluster of C CTAs per (head, batch tile), CTA
// `rank` owns U hidden units and keeps the SAME GR*U rows of R resident in tensor memory, but
// transposed: operand A is R_slice^T [D x GR*U]. Per step t = T-1 .. 0 each CTA
//   1. sums the C partial dh_t contributions that arrived for its units (fixed order), adds the
//      history gradient and the pointwise carry, runs the cell backward -> dg_t,
//   2. streams dg_t out (dWx, bf16 copy for the dR contraction), keeps db in registers,
//   3. multiplies: partial dh_{t-1}[all D units] = R_slice^T * round_bf16(dg_t) on tcgen05,
//   4. scatters the partial rows to the CTAs that own those units (async DSMEM stores that
//      complete on the owner's mbarrier).
// No atomics anywhere; dR itself is a separate contraction over (b, t).
//
// Replaces FLASHRNNCellFusedBackward (flashrnn/flashrnn/fused/flashrnn_fused_backward.cu:130-625).
#include "frnn_common.cuh"

namespace frnn {

namespace {

constexpr int kEpiThreads = 128;
constexpr int kBwdThreads = 192;
constexpr int kMaxTiles = 16;  // 128-row tiles of the partial dh a CTA can produce (D <= 2048)
constexpr int kStages = 4;  // upper bound of the TMA ring depth (Cfg::NST is the depth in use)

template <int CELL, int BV, int U, bool WX_BF16>
struct BwdCfg {
  using CT = CellTraits<CELL>;
  static constexpr int BT = BV < 16 ? 16 : BV;
  static constexpr int ROWS = CT::GR * U;  // K of the backward contraction
  static constexpr int IPT = (U * BV / kEpiThreads) < 2 ? 2 : (U * BV / kEpiThreads);
  static constexpr int TPB = U / IPT;
  static constexpr int GCL = CELL == kElman ? 0 : CT::GC;  // cached gates actually loaded
  static constexpr int CACHE_BYTES = GCL * BV * U * CT::CES;  // the cached gates come first in a stage
  static constexpr int STAGE_BYTES = CACHE_BYTES + 3 * CT::S * BV * U * 4;
  static_assert(CACHE_BYTES % 128 == 0, "TMA destinations after the cached gates stay 128-byte aligned");
  // TMA ring depth: four stages unless a stage is so large (wide batch tiles, many states) that fewer
  // fit. 16-row tiles run where CTAs outnumber SMs, so their ring stays below 80 KB and two CTAs
  // share one SM's shared memory.
  static constexpr int RING_MAX = BV == 16 ? 81920 : 122880;
  static constexpr int NST = STAGE_BYTES * 4 <= (BV == 16 ? 81920 : 98304) ? 4 : (STAGE_BYTES * 3 <= RING_MAX ? 3 : 2);
  static constexpr int DGBUF_BYTES = BT * ROWS * 2;
  static constexpr int DBUF_BYTES = BV * CT::GB * U * 4;
  static_assert(ROWS % 16 == 0, "K must be a multiple of 16");
  static_assert(IPT == 2 || IPT == 4 || IPT == 8, "items per thread");
};

__device__ __forceinline__ void report(int* err, int code, int detail) {
  if (atomicCAS(err, 0, code) == 0) {
    err[1] = detail;
    err[2] = static_cast<int>(blockIdx.x);
  }
  __threadfence();
}

// OPTS: compiled with the v1 options (recurrent-gradient clip / cut, v1 sLSTM convention); the plain instantiation
// carries none of that code on its per-step critical path.
template <int CELL, int BV, int U, bool WX_BF16, bool XG, bool OPTS>
__global__ void __launch_bounds__(kBwdThreads, (BV == 16 && !XG) ? 2 : 1)  // 16-row tiles are chosen when CTAs outnumber SMs: let two share one
frnn_bwd_kernel(const BwdParams p, const __grid_constant__ CUtensorMap cache_map,
                const __grid_constant__ CUtensorMap hist_map, const __grid_constant__ CUtensorMap init_map,
                const __grid_constant__ CUtensorMap dhist_map) {
  using Cfg = BwdCfg<CELL, BV, U, WX_BF16>;
  using CT = typename Cfg::CT;
  constexpr int BT = Cfg::BT, IPT = Cfg::IPT, TPB = Cfg::TPB, ROWS = Cfg::ROWS, S = CT::S, GCL = Cfg::GCL;

  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) uint64_t s_part_bar[2];
  __shared__ __align__(8) uint64_t s_dg_bar;
  __shared__ __align__(8) uint64_t s_mma_bar[kMaxTiles];  // one per 128-row tile of the partial dh
  __shared__ __align__(8) uint64_t s_full[kStages];
  __shared__ __align__(8) uint64_t s_empty[kStages];
  __shared__ uint32_t s_tmem_base;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const long long t_entry = clock64();
  const int D = p.D, N = p.N, T = p.T, B = p.B, C = p.C;
  const int rank = static_cast<int>(blockIdx.x % C);  // == rank inside the cluster when there is one
  const int gid = blockIdx.x / C;
  const int n = gid % N;
  const int btile = gid / N;
  const int b0 = btile * BV;
  const int bv = min(BV, B - b0);
  const int MTB = (D + 127) / 128;
  const int a_col0 = (MTB * BT + 31) / 32 * 32;
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(a_col0 + MTB * (ROWS / 2))) tmem_cols <<= 1;

  // shared memory carve-up
  const int part_bytes = C * BV * U * 4;  // one parity buffer: [source CTA][batch][unit] fp32
  constexpr bool xg = XG;   // exchange partial dh through global memory instead of DSMEM
  const int part_bufs = xg ? 0 : 2;       // the global exchange is summed straight from global memory
  uint8_t* const dgbuf = smem;
  float* const part = reinterpret_cast<float*>(smem + Cfg::DGBUF_BYTES);
  float* const dbuf = reinterpret_cast<float*>(smem + Cfg::DGBUF_BYTES + part_bufs * part_bytes);
  uint8_t* const stages = smem + ((Cfg::DGBUF_BYTES + part_bufs * part_bytes + Cfg::DBUF_BYTES + 127) & ~127);
  // Global layout per group: [slot][dest CTA][source CTA][batch][unit] fp32, two slots; the
  // partial sums consumed in iteration i travel through slot i % 2. There is no separate flag:
  // the lowest mantissa bit of every word is replaced by a phase bit that flips each time the slot
  // is reused (the buffer starts as all ones), and the receiver polls the words themselves.
  uint8_t* const xg_p = xg ? p.xg_data + static_cast<size_t>(gid) * 2 * C * part_bytes : nullptr;
  const volatile int* abort_flag = p.err;
  const uint64_t limit = p.wait_limit_ns;
  // test hook: with err[4] = 1 no CTA scatters partial dh from iteration err[5] on, so the next wait runs out
  const int mute_from = p.err[4] != 0 ? p.err[5] : 0x7fffffff;  // test hook: nobody publishes from this step on
  // Second test hook, race verification by delay injection (err[6] = seed, see jitter_stall). It is compiled into the
  // fp32-Wx instantiations only: the exchange code is the same for both Wx types, and even the untaken per-step test
  // costs the bf16 backward more than 1 %.
  constexpr bool kJitter = !WX_BF16;
  const uint32_t jitter = kJitter ? static_cast<uint32_t>(p.err[6]) : 0u;
  const bool prof = p.err[3] != 0 && blockIdx.x == 0 && lane == 0 && (warp == 0 || warp == 4);
  const bool cut = OPTS && p.cut_recurrent != 0;
  const bool clip_on = OPTS && p.grad_clip > 0.0f;

  if (tid == 0) {
    mbar_init(smem_u32(&s_part_bar[0]), 1);
    mbar_init(smem_u32(&s_part_bar[1]), 1);
    mbar_init(smem_u32(&s_dg_bar), kEpiThreads);
    for (int j = 0; j < kMaxTiles; ++j) mbar_init(smem_u32(&s_mma_bar[j]), 1);
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
  for (int i = tid; i < Cfg::DGBUF_BYTES / 16; i += kBwdThreads)
    reinterpret_cast<uint4*>(dgbuf)[i] = make_uint4(0u, 0u, 0u, 0u);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = s_tmem_base;

  if (warp < 4) {
    // R_slice^T -> tensor memory: lane = input unit p, column c packs k = 2c, 2c+1 with
    // k = g*U + u indexing the CTA's rows of R. Sixteen rows of R at a time are staged in shared
    // memory with coalesced 16-byte loads (the TMA ring is still idle) and read back column-wise.
    __nv_bfloat16* const rbuf = reinterpret_cast<__nv_bfloat16*>(stages);  // [16][D]
    const int vec_per_row = D / 8;
    for (int c0 = 0; c0 < ROWS / 2; c0 += 8) {
      for (int v = tid; v < 16 * vec_per_row; v += kEpiThreads) {
        const int k = 2 * c0 + v / vec_per_row, pv = v % vec_per_row;
        const __nv_bfloat16* src = p.R + ((static_cast<size_t>(k / U) * N + n) * D + rank * U + (k % U)) * D + pv * 8;
        reinterpret_cast<uint4*>(rbuf)[v] = __ldg(reinterpret_cast<const uint4*>(src));
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      for (int j = 0; j < MTB; ++j) {
        const int pp = j * 128 + tid;
        uint32_t r[8];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          uint32_t v = 0u;
          if (pp < D) {
            v = static_cast<uint32_t>(__bfloat16_as_ushort(rbuf[(2 * q) * D + pp])) |
                (static_cast<uint32_t>(__bfloat16_as_ushort(rbuf[(2 * q + 1) * D + pp])) << 16);
          }
          r[q] = v;
        }
        tmem_st_x8(tmem_addr(tbase, 32 * warp, a_col0 + j * (ROWS / 2) + c0), r);
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
    }
    tmem_st_wait();
  }

  const int ib = tid / TPB, uq = tid % TPB;
  const bool active = warp < 4 && tid < BV * TPB && ib < bv;
  const int ul = uq * IPT;
  const int d0 = rank * U + ul;
  const size_t BND = static_cast<size_t>(B) * N * D;
  const size_t item_bn = (static_cast<size_t>(b0 + ib) * N + n) * D + d0;
  float dcar[S][IPT];      // gradient carried to the state of the step being processed
  float dbacc[CT::GB][IPT];
#pragma unroll
  for (int g = 0; g < CT::GB; ++g)
#pragma unroll
    for (int j = 0; j < IPT; ++j) dbacc[g][j] = 0.0f;
#pragma unroll
  for (int q = 0; q < S; ++q)
#pragma unroll
    for (int j = 0; j < IPT; ++j) dcar[q][j] = 0.0f;
  if (active) {
#pragma unroll
    for (int q = 0; q < S; ++q) ld_f32_vec<IPT>(p.d_carry + q * BND + item_bn, dcar[q]);
  }
  const uint32_t part_tx = static_cast<uint32_t>(C) * bv * U * 4u;
  if (tid == 0 && !xg) {
    mbar_arrive_expect_tx(smem_u32(&s_part_bar[1]), part_tx);                 // iteration 1 (or final if T == 1)
    if (T >= 2) mbar_arrive_expect_tx(smem_u32(&s_part_bar[0]), part_tx);     // iteration 2
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

  if (prof && warp == 0) p.err[20] = static_cast<int>(clock64() - t_entry);  // prologue cycles
  if (warp == 4) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(128, BT, false, false);
      const uint32_t db_addr = smem_u32(dgbuf);
      long long pw = 0, pi = 0;
      int committed = 0;  // iterations whose tcgen05.mma have been issued and committed
      for (int it = 0; it < T; ++it) {
        if (kJitter && jitter != 0u) jitter_stall(jitter, 1u, static_cast<uint32_t>(it));
        const long long m0 = prof ? clock64() : 0;
        if (!mbar_wait_bounded<false, true>(smem_u32(&s_dg_bar), it & 1, limit, abort_flag)) {
          report(p.err, kErrWaitDg, it);
          break;
        }
        tc_fence_after_sync();
        const long long m1 = prof ? clock64() : 0;
        for (int j = 0; j < MTB; ++j) {
          for (int kk = 0; kk < ROWS / 16; ++kk) {
            const uint64_t bdesc = umma_smem_desc(db_addr + kk * 2 * (BT * 16), BT * 16, 128);
            umma_bf16_ts(tbase + j * BT, tbase + a_col0 + j * (ROWS / 2) + kk * 8, bdesc, idesc, kk > 0 ? 1u : 0u);
          }
          // each tile gets its own completion barrier: its rows are scattered while the next tiles
          // are still on the tensor core
          umma_commit(smem_u32(&s_mma_bar[j]));
        }
        ++committed;
        if (prof) { pw += m1 - m0; pi += clock64() - m1; }
      }
      // Before the CTA may release its tensor memory and shared memory every issued tcgen05.mma must
      // have finished. Normally the epilogue has waited for the last commit already; after a failed
      // wait it has not (it stops waiting), so the issuing thread waits here itself. The commit
      // completes without any other party, hence no abort flag and a plain bound.
      if (committed > 0)
        mbar_wait_bounded<false, true>(smem_u32(&s_mma_bar[MTB - 1]), (committed - 1) & 1, limit, nullptr);
      if (prof) { p.err[16] = static_cast<int>(pw); p.err[17] = static_cast<int>(pi); }
    }
  } else if (warp == 5) {
    if (lane == 0) {
      const uint32_t stage_tx = static_cast<uint32_t>(p.box_b) * U * (GCL * CT::CES + 3 * S * 4);
      const int sbu = p.box_b * U;  // floats per state plane in a stage
      for (int it = 0; it < T; ++it) {
        const int s = it % Cfg::NST;
        const int t = T - 1 - it;
        if (it >= Cfg::NST) {
          if (!mbar_wait_bounded<false>(smem_u32(&s_empty[s]), ((it / Cfg::NST) - 1) & 1, limit, abort_flag)) {
            report(p.err, kErrWaitEmpty, it);
            break;
          }
        }
        // Once any wait of the grid has run out, the epilogue threads stop waiting for the stages and
        // release them early, so "released" no longer implies that the previous copy into this stage
        // has landed; arming its barrier again could then be a second arrival in one phase. The flag
        // is set before any thread skips a wait, so checking it after the wait above is enough.
        if (*abort_flag != 0) break;
        const uint32_t bar = smem_u32(&s_full[s]);
        uint8_t* sb = stages + s * Cfg::STAGE_BYTES;
        mbar_arrive_expect_tx(bar, stage_tx);
        if (GCL > 0) tma_load_5d(smem_u32(sb), &cache_map, bar, rank * U, n, 0, t, b0);
        float* q = reinterpret_cast<float*>(sb + GCL * sbu * CT::CES);
        tma_load_5d(smem_u32(q), &hist_map, bar, rank * U, n, t, b0, 0);
        q += S * sbu;
        if (t > 0) tma_load_5d(smem_u32(q), &hist_map, bar, rank * U, n, t - 1, b0, 0);
        else tma_load_5d(smem_u32(q), &init_map, bar, rank * U, n, 0, b0, 0);
        q += S * sbu;
        tma_load_5d(smem_u32(q), &dhist_map, bar, rank * U, n, t, b0, 0);
      }
    }
  } else {
    const size_t ND = static_cast<size_t>(N) * D;
    const int sbu = p.box_b * U;
    const uint32_t dg_off = kmajor_offset(BT, ib, ul);
    long long pc[5] = {0, 0, 0, 0, 0};
    long long pc5 = 0, pc6 = 0, pc7 = 0, pc8 = 0;
    // Once a wait has failed (`dead`) the warp keeps walking through the loop without waiting, so
    // that the warp-wide tcgen05.ld below is always executed by all of its lanes.
    bool dead = false;
    for (int it = 0; it <= T; ++it) {
      if (kJitter && jitter != 0u) jitter_stall(jitter, 0u, static_cast<uint32_t>(it));
      const int t = T - 1 - it;
      const long long c0 = prof ? clock64() : 0;
      float ds[S][IPT];
#pragma unroll
      for (int q = 0; q < S; ++q)
#pragma unroll
        for (int j = 0; j < IPT; ++j) ds[q][j] = dcar[q][j];
      float cache[CT::GC][IPT], sn[S][IPT], sp[S][IPT];
      float dh_ext[IPT];
#pragma unroll
      for (int j = 0; j < IPT; ++j) dh_ext[j] = 0.0f;
      if (it < T) {
        const int s = it % Cfg::NST;
        if (!dead && !mbar_wait_bounded<false, true>(smem_u32(&s_full[s]), (it / Cfg::NST) & 1, limit, abort_flag)) {
          report(p.err, kErrWaitWx, it);
          dead = true;
        }
        if (prof) pc6 += clock64() - c0;
        if (active) {
          const uint8_t* sb = stages + s * Cfg::STAGE_BYTES;
#pragma unroll
          for (int g = 0; g < GCL; ++g) ld_cache_vec<IPT, CT::CES>(sb, (ib * GCL + g) * U + ul, cache[g]);
          const float* q = reinterpret_cast<const float*>(sb + GCL * sbu * CT::CES);
#pragma unroll
          for (int k = 0; k < S; ++k) ld_f32_vec<IPT>(q + k * sbu + ib * U + ul, sn[k]);
          q += S * sbu;
#pragma unroll
          for (int k = 0; k < S; ++k) ld_f32_vec<IPT>(q + k * sbu + ib * U + ul, sp[k]);
          q += S * sbu;
#pragma unroll
          for (int k = 0; k < S; ++k) {
            float dhv[IPT];
            ld_f32_vec<IPT>(q + k * sbu + ib * U + ul, dhv);
#pragma unroll
            for (int j = 0; j < IPT; ++j) {
              ds[k][j] += dhv[j];
              if (k == 0 && clip_on) dh_ext[j] = dhv[j];  // kept aside: only the carried part is clipped below
            }
          }
        }
        mbar_arrive(smem_u32(&s_empty[s]));
      }
      const long long c1 = prof ? clock64() : 0;
      if (it >= 1) {
        // partial dh for this step from every CTA of the cluster
        const int pb = it & 1;
        if (xg) {
          // Global exchange: this thread's IPT floats of every source CTA's block are polled straight
          // into registers until each word shows this iteration's phase bit, then added in source
          // order. A slot is not rewritten before this CTA has scattered again, which it does only
          // after this poll, so a word with the right phase can only be this iteration's.
          constexpr int SB = IPT == 2 ? 32 : 12;  // sources per batch
          const uint32_t phase = static_cast<uint32_t>(((it - 1) >> 1) & 1);
          const uint8_t* src0 = xg_p + ((static_cast<size_t>(it & 1) * C + rank) * C) * (BV * U * 4) + (ib * U + ul) * 4;
          for (int s0 = 0; s0 < C; s0 += SB) {
            uint32_t v[SB][IPT];
            uint32_t pend = 0;
            if (active && !dead) {
#pragma unroll
              for (int k = 0; k < SB; ++k)
                if (s0 + k < C) pend |= 1u << k;
            }
            uint64_t t0 = 0;
            uint32_t poll_rounds = 0;
            while (pend != 0u) {
#pragma unroll
              for (int k = 0; k < SB; ++k) {
                if ((pend >> k) & 1u) {
                  const uint8_t* a = src0 + static_cast<size_t>(s0 + k) * (BV * U * 4);
                  if constexpr (IPT == 4) {
                    const uint4 w = ld_relaxed_gpu_v4(a);
                    v[k][0] = w.x; v[k][1] = w.y; v[k][2] = w.z; v[k][3] = w.w;
                  } else {
                    const uint2 w = ld_relaxed_gpu_v2(a);
                    v[k][0] = w.x; v[k][1] = w.y;
                  }
                }
              }
#pragma unroll
              for (int k = 0; k < SB; ++k) {
                if ((pend >> k) & 1u) {
                  bool ok = true;
#pragma unroll
                  for (int j = 0; j < IPT; ++j) ok = ok && (v[k][j] & 1u) == phase;
                  if (ok) pend &= ~(1u << k);
                }
              }
              // the global timer is slow to read: look at it (and at the abort flag) only every 16th round
              if (pend != 0u && (++poll_rounds & 15u) == 0u) {
                const uint64_t now = global_timer_ns();
                if (t0 == 0) t0 = now;
                if (*abort_flag != 0 || now - t0 > limit) {
                  report(p.err, kErrWaitPart, it);
                  dead = true;
                  break;
                }
              }
            }
            if (active && !dead && !cut) {
#pragma unroll
              for (int k = 0; k < SB; ++k)
                if (s0 + k < C) {
#pragma unroll
                  for (int j = 0; j < IPT; ++j) ds[0][j] += __uint_as_float(v[k][j] & ~1u);
                }
            }
          }
          // a wait that ran out in some lanes only must not leave the warp divided: the warp-wide
          // tcgen05.ld of the next step needs all lanes on one path
          dead = __any_sync(0xffffffffu, dead);
          if (prof) pc5 += clock64() - c1;
        } else if (!dead && !mbar_wait_bounded<true, true>(smem_u32(&s_part_bar[pb]), ((it - 1) >> 1) & 1, limit, abort_flag)) {
          report(p.err, kErrWaitPart, it);
          dead = true;
        }
        if (prof && !xg) pc5 += clock64() - c1;
        if (active && !xg && !cut) {
          const float* pbuf = part + static_cast<size_t>(pb) * (part_bytes / 4) + ib * U + ul;
          // fixed summation order; the loads of eight sources are issued together before the adds
          for (int s0 = 0; s0 < C; s0 += 8) {
            float v[8][IPT];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              if (s0 + k < C) {
                ld_f32_vec<IPT>(pbuf + (s0 + k) * BV * U, v[k]);
              } else {
#pragma unroll
                for (int j = 0; j < IPT; ++j) v[k][j] = 0.0f;
              }
            }
#pragma unroll
            for (int k = 0; k < 8; ++k)
#pragma unroll
              for (int j = 0; j < IPT; ++j) ds[0][j] += v[k][j];
          }
        }
      }
      if (clip_on && it >= 1 && it < T) {
        // the gradient carried into h_t from step t + 1 (total minus the external part) is complete here: clip it
#pragma unroll
        for (int j = 0; j < IPT; ++j) ds[0][j] = clip_sym(ds[0][j] - dh_ext[j], p.grad_clip) + dh_ext[j];
      }
      const long long c2 = prof ? clock64() : 0;
      if (it == T) {
        if (active) {
#pragma unroll
          for (int q = 0; q < S; ++q) st_f32_vec<IPT>(p.d_initial + q * BND + item_bn, ds[q]);
        }
        break;
      }
      uint32_t dgp[CT::GR][IPT / 2];
      float dgw[CT::GW][IPT];
      if (active) {
        float dgr[CT::GR][IPT];
        const bool take_i = CELL == kSLSTM && t == 0 && p.slstm_zero_first != 0;
#pragma unroll
        for (int j = 0; j < IPT; ++j) {
          float cj[CT::GC], snj[S], spj[S], dsj[S], gr[CT::GR], gw[CT::GW], gb[CT::GB];
#pragma unroll
          for (int g = 0; g < GCL; ++g) cj[g] = cache[g][j];
#pragma unroll
          for (int q = 0; q < S; ++q) { snj[q] = sn[q][j]; spj[q] = sp[q][j]; dsj[q] = ds[q][j]; }
          cell_backward<CELL>(cj, spj, snj, dsj, gr, gw, gb, take_i, OPTS && p.slstm_v1 != 0);
#pragma unroll
          for (int q = 0; q < S; ++q) dcar[q][j] = dsj[q];
#pragma unroll
          for (int g = 0; g < CT::GR; ++g) dgr[g][j] = gr[g];
#pragma unroll
          for (int g = 0; g < CT::GW; ++g) dgw[g][j] = gw[g];
#pragma unroll
          for (int g = 0; g < CT::GB; ++g) dbacc[g][j] += gb[g];
        }
#pragma unroll
        for (int g = 0; g < CT::GR; ++g)
#pragma unroll
          for (int j = 0; j < IPT; j += 2) dgp[g][j / 2] = pack_bf16x2(dgr[g][j], dgr[g][j + 1]);
        // operand B of the dh contraction: [batch rows x (g, u)] K-major
#pragma unroll
        for (int g = 0; g < CT::GR; ++g) {
          uint8_t* dst = dgbuf + dg_off + (g * U / 8) * (BT * 16);
          if constexpr (IPT == 2) *reinterpret_cast<uint32_t*>(dst) = dgp[g][0];
          else if constexpr (IPT == 4) *reinterpret_cast<uint2*>(dst) = make_uint2(dgp[g][0], dgp[g][1]);
          else *reinterpret_cast<uint4*>(dst) = make_uint4(dgp[g][0], dgp[g][1], dgp[g][2], dgp[g][3]);
        }
      }
      fence_proxy_async_smem();
      tc_fence_before_sync();
      mbar_arrive(smem_u32(&s_dg_bar));
      const long long c3 = prof ? clock64() : 0;
      // Re-arm the partial-dh barrier of this parity for its next use (iteration it + 2), off the
      // critical path; only a barrier whose phase has really completed may be armed again
      // (arriving twice in one phase is invalid), hence not after a failed wait.
      if (tid == 0 && it >= 1 && !dead && !xg && it + 2 <= T)
        mbar_arrive_expect_tx(smem_u32(&s_part_bar[it & 1]), part_tx);
      if (active) {
        // streams to global memory
        const size_t row = (static_cast<size_t>(b0 + ib) * T + t);
        __nv_bfloat16* dgr_g = p.dgr + (row * CT::GR * N + n) * D + d0;
#pragma unroll
        for (int g = 0; g < CT::GR; ++g)
#pragma unroll
          for (int j = 0; j < IPT; j += 2) *reinterpret_cast<uint32_t*>(dgr_g + g * ND + j) = dgp[g][j / 2];
        if constexpr (WX_BF16) {
          // A caller may pass one buffer as dwx and dgr where the two hold the same values in the same layout
          // (bf16 Wx, cells whose W-gates are their R-gates): written once.
          if (CELL == kGRU || p.dwx != static_cast<void*>(p.dgr)) {
            __nv_bfloat16* dwx_g = static_cast<__nv_bfloat16*>(p.dwx) + (row * CT::GW * N + n) * D + d0;
#pragma unroll
            for (int g = 0; g < CT::GW; ++g)
#pragma unroll
              for (int j = 0; j < IPT; j += 2)
                *reinterpret_cast<uint32_t*>(dwx_g + g * ND + j) = pack_bf16x2(dgw[g][j], dgw[g][j + 1]);
          }
        } else {
          float* dwx_g = static_cast<float*>(p.dwx) + (row * CT::GW * N + n) * D + d0;
#pragma unroll
          for (int g = 0; g < CT::GW; ++g) st_f32_vec<IPT>(dwx_g + g * ND, dgw[g]);
        }
      }
      long long c4 = 0;
      // scatter partial dh_{t-1} rows to the CTAs that own those units
      const int nb = (it + 1) & 1;
      const uint32_t part_base = smem_u32(part) + static_cast<uint32_t>(nb) * part_bytes + static_cast<uint32_t>(rank) * BV * U * 4;
      const uint32_t bar_local = smem_u32(&s_part_bar[nb]);
      for (int j = 0; j < MTB; ++j) {
        if (!dead && !mbar_wait_bounded<false, true>(smem_u32(&s_mma_bar[j]), it & 1, limit, abort_flag)) {
          report(p.err, kErrWaitMma, it);
          dead = true;
        }
        tc_fence_after_sync();
        if (prof && j == 0) c4 = clock64();
        uint32_t r[BV / 8][8];
#pragma unroll
        for (int c = 0; c < BV / 8; ++c) tmem_ld_x8(tmem_addr(tbase, 32 * warp, j * BT + 8 * c), r[c]);
        tmem_ld_wait();
        // This lane holds one unit's row (all batch columns); the owner wants rows of one batch
        // column over consecutive units. Four neighbouring lanes transpose 4 x 4 blocks with
        // shuffles, after which lane i of the quad holds batch columns 8c + i and 8c + 4 + i of the
        // quad's four units: two 16-byte packets per 8 columns.
        const int qi = lane & 3;
#pragma unroll
        for (int c = 0; c < BV / 8; ++c) {
#pragma unroll
          for (int h = 0; h < 8; h += 4) {
            uint32_t a = (qi & 1) ? r[c][h + 0] : r[c][h + 1], b = (qi & 1) ? r[c][h + 2] : r[c][h + 3];
            a = __shfl_xor_sync(0xffffffffu, a, 1);
            b = __shfl_xor_sync(0xffffffffu, b, 1);
            if (qi & 1) { r[c][h + 0] = a; r[c][h + 2] = b; } else { r[c][h + 1] = a; r[c][h + 3] = b; }
            a = (qi & 2) ? r[c][h + 0] : r[c][h + 2];
            b = (qi & 2) ? r[c][h + 1] : r[c][h + 3];
            a = __shfl_xor_sync(0xffffffffu, a, 2);
            b = __shfl_xor_sync(0xffffffffu, b, 2);
            if (qi & 2) { r[c][h + 0] = a; r[c][h + 1] = b; } else { r[c][h + 2] = a; r[c][h + 3] = b; }
          }
        }
        const int pp0 = j * 128 + (tid & ~3);  // first unit of the quad
        if (pp0 < D && !dead && it < mute_from) {
          const int dest = pp0 / U, pl0 = pp0 % U;
          if (!xg) {
            const uint32_t ra = map_to_cta(part_base + pl0 * 4, dest);
            const uint32_t rb = map_to_cta(bar_local, dest);
#pragma unroll
            for (int c = 0; c < BV / 8; ++c)
#pragma unroll
              for (int h = 0; h < 8; h += 4) {
                const int bcol = 8 * c + h + qi;
                if (bcol < bv) st_async_v4_b32(ra + bcol * U * 4, r[c][h], r[c][h + 1], r[c][h + 2], r[c][h + 3], rb);
              }
          } else {
            uint8_t* dst = xg_p + ((static_cast<size_t>((it + 1) & 1) * C + dest) * C + rank) * (BV * U * 4) + pl0 * 4;
            const uint32_t ph = static_cast<uint32_t>((it >> 1) & 1);  // phase of iteration it + 1
#pragma unroll
            for (int c = 0; c < BV / 8; ++c)
#pragma unroll
              for (int h = 0; h < 8; h += 4) {
                const int bcol = 8 * c + h + qi;
                if (bcol < bv)
                  st_relaxed_gpu_v4(dst + bcol * U * 4, make_uint4((r[c][h] & ~1u) | ph, (r[c][h + 1] & ~1u) | ph,
                                                                   (r[c][h + 2] & ~1u) | ph, (r[c][h + 3] & ~1u) | ph));
              }
          }
        }
      }
      if (prof) pc7 += clock64() - c4;
      tc_fence_before_sync();
      if (prof) {
        pc[0] += c1 - c0; pc[1] += c2 - c1; pc[2] += c3 - c2; pc[3] += c4 - c3; pc[4] += clock64() - c4;
      }
    }
    if (prof) {
#pragma unroll
      for (int q = 0; q < 5; ++q) p.err[8 + q] = static_cast<int>(pc[q]);
      p.err[13] = static_cast<int>(pc5);
      p.err[14] = static_cast<int>(pc6);
      p.err[18] = static_cast<int>(pc7);  // scatter without the refill
      p.err[19] = static_cast<int>(pc8);  // fence before the poll
    }
  }

  // bias gradient: reduce the per-thread sums over the batch rows of this tile
  if (active) {
#pragma unroll
    for (int g = 0; g < CT::GB; ++g) st_f32_vec<IPT>(dbuf + (ib * CT::GB + g) * U + ul, dbacc[g]);
  }
  if (*abort_flag != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  for (int i = tid; i < CT::GB * U; i += kBwdThreads) {
    float acc = 0.0f;
    for (int b = 0; b < bv; ++b) acc += dbuf[b * CT::GB * U + i];
    const int g = i / U, u = i % U;
    p.db_part[((static_cast<size_t>(btile) * CT::GB + g) * N + n) * D + rank * U + u] = acc;
  }
  cluster_sync_all();
  if (warp == 4) tmem_dealloc(tbase, tmem_cols);
}

template <int CELL, int BV, int U, bool WX_BF16, bool XG, bool OPTS>
int launch_bwd(const BwdParams& p, const void* cache, const float* history, const float* initial,
               const float* d_history, cudaStream_t stream) {
  using Cfg = BwdCfg<CELL, BV, U, WX_BF16>;
  using CT = typename Cfg::CT;
  const int part_bytes = p.C * BV * U * 4;
  const int part_bufs = XG ? 0 : 2;
  // the ring of TMA stages doubles as the staging area of the prologue's R load (16 rows of D bf16)
  const int ring_bytes = Cfg::NST * Cfg::STAGE_BYTES > 16 * p.D * 2 ? Cfg::NST * Cfg::STAGE_BYTES : 16 * p.D * 2;
  int smem = ((Cfg::DGBUF_BYTES + part_bufs * part_bytes + Cfg::DBUF_BYTES + 127) & ~127) + ring_bytes;
  const int MTB = (p.D + 127) / 128;
  if (MTB > kMaxTiles || ((MTB * Cfg::BT + 31) / 32 * 32) + MTB * (Cfg::ROWS / 2) > 512) return -3;
  if (smem > 227 * 1024) return -2;
  const uint64_t uD = p.D, uN = p.N, uT = p.T, uB = p.B;
  const uint32_t ub = static_cast<uint32_t>(p.box_b);
  CUtensorMap cache_map, hist_map, init_map, dhist_map;
  {
    const uint64_t dims[5] = {uD, uN, static_cast<uint64_t>(Cfg::GCL > 0 ? Cfg::GCL : 1), uT, uB};
    const uint32_t box[5] = {U, 1u, static_cast<uint32_t>(Cfg::GCL > 0 ? Cfg::GCL : 1), 1u, ub};
    // Elman has no cache: describe the history instead so that the (unused) map is valid.
    const void* base = Cfg::GCL > 0 ? static_cast<const void*>(cache) : static_cast<const void*>(history);
    if (make_tensor_map(&cache_map, base, Cfg::GCL > 0 ? CT::CES : 4, 5, dims, box) != 0) return -4;
  }
  {
    const uint64_t dims[5] = {uD, uN, uT, uB, static_cast<uint64_t>(CT::S)};
    const uint32_t box[5] = {U, 1u, 1u, ub, static_cast<uint32_t>(CT::S)};
    if (make_tensor_map(&hist_map, history, 4, 5, dims, box) != 0) return -4;
    if (make_tensor_map(&dhist_map, d_history, 4, 5, dims, box) != 0) return -4;
    const uint64_t dims1[5] = {uD, uN, 1u, uB, static_cast<uint64_t>(CT::S)};
    if (make_tensor_map(&init_map, initial, 4, 5, dims1, box) != 0) return -4;
  }
  auto kern = frnn_bwd_kernel<CELL, BV, U, WX_BF16, XG, OPTS>;
  const int fit = fit_tmem_budget(
      kern, kBwdThreads, tmem_cols_pow2(((MTB * Cfg::BT + 31) / 32 * 32) + MTB * (Cfg::ROWS / 2), 32u), &smem);
  if (fit != 0) return fit;
  cudaError_t e = cudaSuccess;
  if (p.C > 8 && !XG) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const int n_btiles = (p.B + BV - 1) / BV;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(p.N * n_btiles * p.C));
  cfg.blockDim = dim3(kBwdThreads);
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
  e = cudaLaunchKernelEx(&cfg, kern, p, cache_map, hist_map, init_map, dhist_map);
  return static_cast<int>(e);
}

template <int CELL, int BV, int U>
int launch_bwd_dt(const BwdParams& p, const void* cache, const float* history, const float* initial,
                  const float* d_history, int wx_bf16, cudaStream_t s) {
  const bool opts = p.grad_clip > 0.0f || p.cut_recurrent != 0 || p.slstm_v1 != 0;
  if (p.xg_data != nullptr) {  // groups wider than a cluster exchange through global memory
    if (opts)
      return wx_bf16 ? launch_bwd<CELL, BV, U, true, true, true>(p, cache, history, initial, d_history, s)
                     : launch_bwd<CELL, BV, U, false, true, true>(p, cache, history, initial, d_history, s);
    return wx_bf16 ? launch_bwd<CELL, BV, U, true, true, false>(p, cache, history, initial, d_history, s)
                   : launch_bwd<CELL, BV, U, false, true, false>(p, cache, history, initial, d_history, s);
  }
  if (opts)
    return wx_bf16 ? launch_bwd<CELL, BV, U, true, false, true>(p, cache, history, initial, d_history, s)
                   : launch_bwd<CELL, BV, U, false, false, true>(p, cache, history, initial, d_history, s);
  return wx_bf16 ? launch_bwd<CELL, BV, U, true, false, false>(p, cache, history, initial, d_history, s)
                 : launch_bwd<CELL, BV, U, false, false, false>(p, cache, history, initial, d_history, s);
}
template <int CELL>
int launch_bwd_cell(const BwdParams& p, const void* cache, const float* history, const float* initial,
                    const float* d_history, int wx_bf16, int bv, int unit, cudaStream_t s) {
  if (bv == 8 && unit == 32) return launch_bwd_dt<CELL, 8, 32>(p, cache, history, initial, d_history, wx_bf16, s);
  if (bv == 16 && unit == 32) return launch_bwd_dt<CELL, 16, 32>(p, cache, history, initial, d_history, wx_bf16, s);
  if (bv == 8 && unit == 16) return launch_bwd_dt<CELL, 8, 16>(p, cache, history, initial, d_history, wx_bf16, s);
  if (bv == 16 && unit == 16) return launch_bwd_dt<CELL, 16, 16>(p, cache, history, initial, d_history, wx_bf16, s);
  return -2;
}

}  // namespace

int backward_dispatch(int cell, const BwdParams& p, const void* cache, const float* history, const float* initial,
                      const float* d_history, int wx_bf16, int bv, int unit, cudaStream_t s) {
  switch (cell) {
    case kLSTM: return launch_bwd_cell<kLSTM>(p, cache, history, initial, d_history, wx_bf16, bv, unit, s);
    case kSLSTM: return launch_bwd_cell<kSLSTM>(p, cache, history, initial, d_history, wx_bf16, bv, unit, s);
    case kGRU: return launch_bwd_cell<kGRU>(p, cache, history, initial, d_history, wx_bf16, bv, unit, s);
    case kElman: return launch_bwd_cell<kElman>(p, cache, history, initial, d_history, wx_bf16, bv, unit, s);
    default: return -1;
  }
}

}  // namespace frnn
