// Persistent forward recurrence of ONE wide head whose rows of R are split over the GPUs of a node.
//
// Rank r owns the hidden units [r*Dl, (r+1)*Dl). Its CTAs form a 2-D grid: Dl/32 row tiles (32 units = GR*32
// rows of R) times KS chunks of the contraction dimension K = D. CTA (rt, ks) multiplies its [128 x Kc] block
// of R with the K-chunk of round_bf16(h_{t-1}) on tcgen05 every step. The block of R never leaves the SM
// when it fits: the first k_tmem columns sit in tensor memory (operand A from TMEM), the rest in a ring of
// 128-byte-swizzled shared-memory stages filled by TMA (operand A from shared memory); when the ring is too
// short for the rest (wide chunks on few GPUs) the TMA warp streams those stages again every step.
// The KS CTAs of a row tile are a thread-block cluster: each owns 32/KS batch rows, receives the partial
// gate sums of all KS chunks by asynchronous DSMEM stores, adds them in a fixed order, runs the cell and
// publishes round_bf16(h_t) of its rows to EVERY rank (peer stores, see recurrent_mg_common.cuh).
// The operand of a step is staged from this rank's own history buffer in sub-chunks of 512 k.
//
// Arithmetic: reference.recurrence (flashrnn/flashrnn2/reference.py:72-114); multi-GPU forward of the
// reference: flashrnn/flashrnn2/multi_gpu.py:87-297.
#include "recurrent_mg_common.cuh"

namespace frnn {

namespace {

constexpr int kEpi = 128;
constexpr int kMgThreads = 224;  // 4 epilogue warps, MMA warp, Wx TMA warp, weight-ring TMA warp

template <int CELL, int KS, bool WX_BF16>
struct MgFwdCfg {
  using CT = CellTraits<CELL>;
  static constexpr int BO = kMgBT / KS;                 // batch rows owned by one CTA of the cluster
  static constexpr int ITEMS = 32 * BO;                 // (unit, batch row) items of the owner
  static constexpr int NI = (ITEMS + kEpi - 1) / kEpi;  // items per epilogue thread
  static constexpr int ROWS = CT::GR * 32;              // accumulator rows in use
  static constexpr int WX_ES = WX_BF16 ? 2 : 4;
  static constexpr int WX_STAGE_BYTES = BO * CT::GW * 32 * WX_ES;
  static constexpr int NWX = WX_STAGE_BYTES * 4 <= 32768 ? 4 : 2;
  static constexpr int PART_FLOATS = KS * 128 * BO;     // one parity: [source][row][owned batch row]
  static constexpr int PART_BYTES = PART_FLOATS * 4;
  static constexpr int PUB_BYTES = BO * 32 * 2;         // staging of round_bf16(h_t): [batch row][unit]
  static_assert(KS == 1 || KS == 2 || KS == 4 || KS == 8 || KS == 16, "cluster width");
};

template <int CELL, int KS, bool WX_BF16>
__global__ void __launch_bounds__(kMgThreads, 1)
frnn_fwd_mg_kernel(const MgFwdParams p, const __grid_constant__ CUtensorMap wx_map,
                   const __grid_constant__ CUtensorMap r_map) {
  using Cfg = MgFwdCfg<CELL, KS, WX_BF16>;
  using CT = typename Cfg::CT;
  constexpr int BT = kMgBT, BO = Cfg::BO, NI = Cfg::NI, S = CT::S;

  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) uint64_t s_hbar[2];
  __shared__ __align__(8) uint64_t s_hfree[2];
  __shared__ __align__(8) uint64_t s_mma_bar;
  __shared__ __align__(8) uint64_t s_part_bar[2];
  __shared__ __align__(8) uint64_t s_wx_full[4];
  __shared__ __align__(8) uint64_t s_wx_empty[4];
  __shared__ __align__(8) uint64_t s_afull[kMgMaxRing];
  __shared__ __align__(8) uint64_t s_aempty[kMgMaxRing];
  __shared__ uint32_t s_tmem_base;
  __shared__ int s_ready_ok;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int D = p.D, T = p.T, B = p.B, Dl = p.Dl, ldx = p.ldx, P = p.P;
  const int per_rank = (Dl / 32) * KS;
  const int lr = static_cast<int>(blockIdx.x) / per_rank;  // rank slot inside this launch
  const int rank = p.rank0 + lr;
  const int cta = static_cast<int>(blockIdx.x) % per_rank;
  const int ks = cta % KS;                                  // == rank inside the cluster
  const int rt = cta / KS;
  const int xu = lr * p.x_rank_stride + rt * 32;            // first unit of the tile inside the local tensors
  const int ug = rank * Dl + rt * 32;                       // first unit of the tile inside the head
  const int Kc = D / KS;
  const int SCK = Kc < kMgSubK ? Kc : kMgSubK;
  const int NSC = Kc / SCK;
  const int hb_bytes = mg_operand_bytes(SCK);
  const int k_tmem = p.k_tmem, n_ring = p.n_ring, NA = p.ring_stages;
  const bool resident = p.resident != 0;
  uint8_t* const ring = smem;                               // 1024-byte aligned stages of 16 KB
  uint8_t* const hbuf = smem + NA * kMgRingBytes;
  float* const part = reinterpret_cast<float*>(hbuf + 2 * hb_bytes);
  // outgoing partial rows, two parities like `part`: [destination][row][its batch rows]. A block is written again two
  // steps later, after this CTA has used the partners' sums of the step in between, which they can only have sent
  // after taking delivery of the block's previous content.
  float* const part_out = part + 2 * Cfg::PART_FLOATS;
  __nv_bfloat16* const pub = reinterpret_cast<__nv_bfloat16*>(reinterpret_cast<uint8_t*>(part) + 4 * Cfg::PART_BYTES);
  uint8_t* const wxs = reinterpret_cast<uint8_t*>(pub) + ((Cfg::PUB_BYTES + 127) & ~127);
  const volatile int* abort_flag = p.err;
  const uint64_t limit = p.wait_limit_ns;
  const int mute_from = p.err[4] != 0 ? p.err[5] : 0x7fffffff;  // test hook: nobody publishes from this step on
  // Second test hook, race verification by delay injection (err[6] = seed, see jitter_stall). It is compiled into the
  // fp32-Wx instantiations only: the exchange code is the same for both Wx types, and even the untaken per-step test
  // costs the bf16 backward more than 1 %.
  constexpr bool kJitter = !WX_BF16;
  const uint32_t jitter = kJitter ? static_cast<uint32_t>(p.err[6]) : 0u;
  const bool zero_first = p.slstm_zero_first != 0;
  constexpr uint32_t tmem_cols = 512;
  const size_t hrow = static_cast<size_t>(T + 1) * D;       // elements per batch row of a history buffer

  // ---------------- prologue ----------------
  if (tid == 0) {
    mbar_init(smem_u32(&s_hbar[0]), kEpi);
    mbar_init(smem_u32(&s_hbar[1]), kEpi);
    mbar_init(smem_u32(&s_hfree[0]), 1);
    mbar_init(smem_u32(&s_hfree[1]), 1);
    mbar_init(smem_u32(&s_mma_bar), 1);
    mbar_init(smem_u32(&s_part_bar[0]), 1);
    mbar_init(smem_u32(&s_part_bar[1]), 1);
    for (int s = 0; s < Cfg::NWX; ++s) {
      mbar_init(smem_u32(&s_wx_full[s]), 1);
      mbar_init(smem_u32(&s_wx_empty[s]), kEpi);
    }
    for (int s = 0; s < kMgMaxRing; ++s) {
      mbar_init(smem_u32(&s_afull[s]), 1);
      mbar_init(smem_u32(&s_aempty[s]), 1);
    }
    fence_mbar_init();
    s_ready_ok = 1;
    // nothing may be stored into a peer's history buffer before the peer has filled it for this call
    if (p.ranks_here < P && !mg_handshake(p.ready, rank, P, p.epoch, cta == 0, limit, abort_flag)) {
      mg_report(p.err, kErrWaitReady, 0);
      s_ready_ok = 0;
    }
  }
  if (warp == 4) {
    tmem_alloc(smem_u32(&s_tmem_base), tmem_cols);
    tmem_relinquish_alloc();
  }
  for (int i = tid; i < 2 * hb_bytes / 16; i += kMgThreads) reinterpret_cast<uint4*>(hbuf)[i] = make_uint4(0u, 0u, 0u, 0u);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = s_tmem_base;
  const bool ready_ok = s_ready_ok != 0;

  if (warp < 4) {
    // rows (gate g, unit u) of the tile, first k_tmem columns of the K-chunk -> tensor memory
    const bool valid = tid < Cfg::ROWS;
    const int g = valid ? tid / 32 : 0, u = tid % 32;
    const __nv_bfloat16* src = p.R + (static_cast<size_t>(g) * p.ldx + xu + u) * D + static_cast<size_t>(ks) * Kc;
    for (int c0 = 0; c0 < k_tmem / 2; c0 += 8) {
      uint32_t r[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
      if (valid) {
        const uint4 lo = __ldg(reinterpret_cast<const uint4*>(src + 2 * c0));
        const uint4 hi = __ldg(reinterpret_cast<const uint4*>(src + 2 * c0 + 8));
        r[0] = lo.x; r[1] = lo.y; r[2] = lo.z; r[3] = lo.w;
        r[4] = hi.x; r[5] = hi.y; r[6] = hi.z; r[7] = hi.w;
      }
      tmem_st_x8(tmem_addr(tbase, 32 * warp, BT + c0), r);
    }
    tmem_st_wait();
  }

  // cell items of this thread: item i = tid + 128 j -> owned batch row bl = i % BO, unit u = i / BO
  float st[NI][S];
  float bias[NI][CT::GB];
  bool act[NI];
  int it_u[NI], it_b[NI];
#pragma unroll
  for (int j = 0; j < NI; ++j) {
    const int i = tid + kEpi * j;
    it_u[j] = (i / BO) % 32;
    it_b[j] = ks * BO + i % BO;
    act[j] = warp < 4 && i < Cfg::ITEMS && it_b[j] < B;
#pragma unroll
    for (int s = 0; s < S; ++s)
      st[j][s] = act[j] ? p.initial[(static_cast<size_t>(s) * B + it_b[j]) * ldx + xu + it_u[j]] : 0.0f;
#pragma unroll
    for (int g = 0; g < CT::GB; ++g) bias[j][g] = warp < 4 ? p.bias[static_cast<size_t>(g) * ldx + xu + it_u[j]] : 0.0f;
  }
  constexpr uint32_t part_tx = static_cast<uint32_t>(KS) * Cfg::ROWS * BO * 4u;
  if (warp == 4 && lane == 0) {
    mbar_arrive_expect_tx(smem_u32(&s_part_bar[0]), part_tx);
    if (T >= 2) mbar_arrive_expect_tx(smem_u32(&s_part_bar[1]), part_tx);
    tma_prefetch_desc(&wx_map);
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
      const uint32_t idesc = umma_idesc_bf16(128, BT, false, false);
      int committed = 0;
      int ring_stage = 0;        // next stage of the weight ring to consume, and the phase its barrier is in
      uint32_t ring_phase = 0;
      bool ok = true;
      const bool prof = p.err[3] != 0 && blockIdx.x == 0;  // phase timers of CTA 0 (SM clock cycles, summed over all steps)
      long long pf_h = 0, pf_a = 0, pf_tot = prof ? clock64() : 0;
      for (int t = 0; t < T && ok; ++t) {
        if (kJitter && jitter != 0u) jitter_stall(jitter, 1u, static_cast<uint32_t>(t));
        for (int sc = 0; sc < NSC && ok; ++sc) {
          const long long q = static_cast<long long>(t) * NSC + sc;
          const int buf = static_cast<int>(q & 1);
          const long long w0 = prof ? clock64() : 0;
          if (!mbar_wait_bounded<false, true>(smem_u32(&s_hbar[buf]), static_cast<uint32_t>((q >> 1) & 1), limit, abort_flag)) {
            mg_report(p.err, kErrWaitH, t);
            ok = false;
            break;
          }
          if (prof) pf_h += clock64() - w0;
          fence_proxy_async_smem();
          tc_fence_after_sync();
          // Descriptors advance by constants: 16 k = 32 B inside a 128-byte swizzled row (2 in units of 16 B), the
          // next 64-k block of the operand is 4096 B further (256); eight 32-bit columns of tensor memory.
          const uint64_t bdesc0 = umma_smem_desc_k_sw128(smem_u32(hbuf + buf * hb_bytes));
          const int k0 = sc * SCK;
          int n_ts = (k_tmem - k0) / 16;
          n_ts = n_ts < 0 ? 0 : (n_ts > SCK / 16 ? SCK / 16 : n_ts);
          uint32_t acol = tbase + BT + k0 / 2;
          int kk = 0;
#pragma unroll 4
          for (; kk < n_ts; ++kk) {
            umma_bf16_ts(tbase, acol, bdesc0 + (kk >> 2) * 256 + (kk & 3) * 2, idesc, (k0 | kk) != 0 ? 1u : 0u);
            acol += 8;
          }
          for (; kk < SCK / 16; kk += kMgRingK / 16) {
            if (!resident || t == 0) {
              const long long w1 = prof ? clock64() : 0;
              if (!mbar_wait_bounded<false, true>(smem_u32(&s_afull[ring_stage]), ring_phase, limit, abort_flag)) {
                mg_report(p.err, kErrWaitRing, t);
                ok = false;
                break;
              }
              if (prof) pf_a += clock64() - w1;
              tc_fence_after_sync();
            }
            uint64_t adesc = umma_smem_desc_k_sw128(smem_u32(ring + ring_stage * kMgRingBytes));
            uint64_t bdesc = bdesc0 + (kk >> 2) * 256;
#pragma unroll
            for (int i = 0; i < kMgRingK / 16; ++i) {
              umma_bf16_ss(tbase, adesc, bdesc, idesc, (k0 | kk | i) != 0 ? 1u : 0u);
              adesc += 2;
              bdesc += 2;
            }
            if (!resident) umma_commit(smem_u32(&s_aempty[ring_stage]));
            if (++ring_stage == NA) {
              ring_stage = 0;
              ring_phase ^= 1u;
            }
          }
          if (!ok) break;
          umma_commit(smem_u32(&s_hfree[buf]));
        }
        if (!ok) break;
        umma_commit(smem_u32(&s_mma_bar));
        ++committed;
      }
      // every issued MMA must have finished before tensor and shared memory are released; one more commit
      // covers the MMAs of a step that was cut short by a failed wait
      if (!ok) {
        umma_commit(smem_u32(&s_mma_bar));
        ++committed;
      }
      if (committed > 0) mbar_wait_bounded<false, true>(smem_u32(&s_mma_bar), (committed - 1) & 1, limit, nullptr);
      if (prof) {  // err[16]: operand wait, err[17]: weight-stage wait, err[18]: whole loop (all in units of 1024 cycles)
        p.err[16] = static_cast<int>(pf_h >> 10);
        p.err[17] = static_cast<int>(pf_a >> 10);
        p.err[18] = static_cast<int>((clock64() - pf_tot) >> 10);
      }
    }
  } else if (warp == 5) {
    if (lane == 0 && ready_ok) {
      constexpr uint32_t stage_tx = static_cast<uint32_t>(Cfg::WX_STAGE_BYTES);
      for (int t = 0; t < T; ++t) {
        const int s = t % Cfg::NWX;
        if (t >= Cfg::NWX &&
            !mbar_wait_bounded<false>(smem_u32(&s_wx_empty[s]), ((t / Cfg::NWX) - 1) & 1, limit, abort_flag)) {
          mg_report(p.err, kErrWaitEmpty, t);
          break;
        }
        if (*abort_flag != 0) break;  // stages are released early after a failed wait: do not arm a busy barrier
        mbar_arrive_expect_tx(smem_u32(&s_wx_full[s]), stage_tx);
        tma_load_5d(smem_u32(wxs + s * Cfg::WX_STAGE_BYTES), &wx_map, smem_u32(&s_wx_full[s]), xu, 0, 0, t, ks * BO);
      }
    }
  } else if (warp == 6) {
    if (lane == 0 && ready_ok && n_ring > 0) {
      // weight columns beyond the tensor-memory part: [128 rows x 64 k] stages, 128-byte swizzle
      const int k_base = ks * Kc + k_tmem;
      if (resident) {
        for (int j = 0; j < n_ring; ++j) {
          mbar_arrive_expect_tx(smem_u32(&s_afull[j]), static_cast<uint32_t>(Cfg::ROWS) * kMgRingK * 2u);
          tma_load_3d(smem_u32(ring + j * kMgRingBytes), &r_map, smem_u32(&s_afull[j]), k_base + j * kMgRingK, xu, 0);
        }
      } else {
        int stage = 0;
        uint32_t phase = 1;  // parity of the release this stage's next refill waits for (none before the first lap)
        bool first_lap = true, ok = true;
        const bool prof = p.err[3] != 0 && blockIdx.x == 0;
        long long pf_e = 0;
        for (int t = 0; t < T && ok; ++t) {
          for (int j = 0; j < n_ring; ++j) {
            const long long w0 = prof ? clock64() : 0;
            if (!first_lap && !mbar_wait_bounded<false, true>(smem_u32(&s_aempty[stage]), phase, limit, abort_flag)) {
              mg_report(p.err, kErrWaitRing, t);
              ok = false;
              break;
            }
            if (prof) pf_e += clock64() - w0;
            // (a bounded wait that returned true saw no abort; the flag itself is read only once per step)
            if (j == 0 && *abort_flag != 0) { ok = false; break; }
            mbar_arrive_expect_tx(smem_u32(&s_afull[stage]), static_cast<uint32_t>(Cfg::ROWS) * kMgRingK * 2u);
            tma_load_3d(smem_u32(ring + stage * kMgRingBytes), &r_map, smem_u32(&s_afull[stage]), k_base + j * kMgRingK, xu, 0);
            if (++stage == NA) {
              stage = 0;
              phase ^= 1u;
              first_lap = false;
            }
          }
        }
        if (prof) p.err[19] = static_cast<int>(pf_e >> 10);  // producer: waiting for released stages
      }
    }
  } else if (ready_ok) {
    const bool row_valid = tid < Cfg::ROWS;
    bool dead = false;  // after a failed wait the warp keeps walking through the loop without waiting

    // round_bf16(h) of the owned items -> slot `slot` of every rank's history buffer
    auto publish = [&](int slot, const uint32_t (&hb16)[NI], bool on) {
#pragma unroll
      for (int j = 0; j < NI; ++j) {
        const int i = tid + kEpi * j;
        if (i < Cfg::ITEMS) pub[(i % BO) * 32 + it_u[j]] = __ushort_as_bfloat16(static_cast<unsigned short>(hb16[j]));
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (on) {
        // job = (packet of 8 units of one owned batch row, destination rank)
        for (int job = tid; job < BO * 4 * P; job += kEpi) {
          const int pk = job % (BO * 4), q = job / (BO * 4);
          const int bl = pk / 4, u8 = pk % 4;
          const int b = ks * BO + bl;
          if (b < B) {
            const uint4 v = *reinterpret_cast<const uint4*>(pub + bl * 32 + u8 * 8);
            st_relaxed_sys_v4(p.hbf[q] + static_cast<size_t>(b) * hrow + static_cast<size_t>(slot) * D + ug + u8 * 8,
                              make_uint4(xg_clean(v.x), xg_clean(v.y), xg_clean(v.z), xg_clean(v.w)));
          }
        }
      }
    };
    // this CTA's K-chunk of slot `slot` -> operand buffers, one sub-chunk at a time
    const bool prof = p.err[3] != 0 && blockIdx.x == 0 && tid == 0;
    long long pf_free = 0, pf_poll = 0, pf_mma = 0, pf_part = 0, pf_scat = 0, pf_cell = 0, pf_pub = 0, pf_st = 0;
    auto fetch = [&](int slot) {
      for (int sc = 0; sc < NSC; ++sc) {
        const long long q = static_cast<long long>(slot) * NSC + sc;
        const int buf = static_cast<int>(q & 1);
        const long long f0 = prof ? clock64() : 0;
        if (q >= 2 && !dead &&
            !mbar_wait_bounded<false, true>(smem_u32(&s_hfree[buf]), static_cast<uint32_t>(((q >> 1) - 1) & 1), limit, abort_flag)) {
          mg_report(p.err, kErrWaitMma, slot);
          dead = true;
        }
        const long long f1 = prof ? clock64() : 0;
        if (prof) pf_free += f1 - f0;
        if (!dead && !mg_fetch_subchunk(p.hbf[rank] + static_cast<size_t>(slot) * D + static_cast<size_t>(ks) * Kc + sc * SCK, hrow,
                                        hbuf + buf * hb_bytes, SCK, B, warp, lane, limit, abort_flag)) {
          mg_report(p.err, kErrWaitH, slot);
          dead = true;
        }
        dead = __any_sync(0xffffffffu, dead);
        fence_proxy_async_smem();
        mbar_arrive(smem_u32(&s_hbar[buf]));
        if (prof) pf_poll += clock64() - f1;
      }
    };

    {
      uint32_t hb16[NI];
#pragma unroll
      for (int j = 0; j < NI; ++j)
        hb16[j] = act[j] ? static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(st[j][0]))) : 0u;
      publish(0, hb16, true);
      fetch(0);
    }
    const size_t sBT = static_cast<size_t>(B) * T;
    for (int t = 0; t < T; ++t) {
      if (kJitter && jitter != 0u) jitter_stall(jitter, 0u, static_cast<uint32_t>(t));
      const int s = t % Cfg::NWX, pb = t & 1;
      if (!dead && !mbar_wait_bounded<false, true>(smem_u32(&s_wx_full[s]), (t / Cfg::NWX) & 1, limit, abort_flag)) {
        mg_report(p.err, kErrWaitWx, t);
        dead = true;
      }
      float wx[NI][CT::GW];
#pragma unroll
      for (int j = 0; j < NI; ++j) {
        const int i = tid + kEpi * j;
        const int bl = i % BO;
#pragma unroll
        for (int g = 0; g < CT::GW; ++g) {
          const int e = (bl * CT::GW + g) * 32 + it_u[j];
          if (i < Cfg::ITEMS) {
            if constexpr (WX_BF16) wx[j][g] = __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(wxs + s * Cfg::WX_STAGE_BYTES)[e]);
            else wx[j][g] = reinterpret_cast<const float*>(wxs + s * Cfg::WX_STAGE_BYTES)[e];
          } else {
            wx[j][g] = 0.0f;
          }
        }
      }
      mbar_arrive(smem_u32(&s_wx_empty[s]));
      const long long e0 = prof ? clock64() : 0;
      if (!dead && !mbar_wait_bounded<false, true>(smem_u32(&s_mma_bar), t & 1, limit, abort_flag)) {
        mg_report(p.err, kErrWaitMma, t);
        dead = true;
      }
      const long long e0b = prof ? clock64() : 0;
      if (prof) pf_mma += e0b - e0;
      tc_fence_after_sync();
      // partial gates of this row: batch columns [ks'*BO, (ks'+1)*BO) go to CTA ks' of the cluster. The rows are
      // collected in shared memory as one block per destination, then ONE bulk copy per destination carries a block
      // into the owner's `part` buffer (a store per 16 bytes would make a thousand updates of the owner's barrier).
      {
        uint32_t r[4][8];
#pragma unroll
        for (int c = 0; c < 4; ++c) tmem_ld_x8(tmem_addr(tbase, 32 * warp, 8 * c), r[c]);
        tmem_ld_wait();
        tc_fence_before_sync();
        if (row_valid) {
#pragma unroll
          for (int d = 0; d < KS; ++d) {
            float* dstrow = part_out + pb * Cfg::PART_FLOATS + (d * 128 + tid) * BO;
            if constexpr (BO >= 4) {
#pragma unroll
              for (int v = 0; v < BO / 4; ++v) {
                const int c0 = d * BO + 4 * v;
                *reinterpret_cast<uint4*>(dstrow + 4 * v) =
                    make_uint4(r[c0 / 8][c0 % 8], r[c0 / 8][c0 % 8 + 1], r[c0 / 8][c0 % 8 + 2], r[c0 / 8][c0 % 8 + 3]);
              }
            } else {
              const int c0 = d * BO;
              *reinterpret_cast<uint2*>(dstrow) = make_uint2(r[c0 / 8][c0 % 8], r[c0 / 8][c0 % 8 + 1]);
            }
          }
        }
        fence_proxy_async_smem();
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (tid < KS && !dead) {
          const uint32_t off = static_cast<uint32_t>(pb) * Cfg::PART_BYTES + static_cast<uint32_t>(ks * 128 * BO) * 4u;
          bulk_copy_to_cluster(map_to_cta(smem_u32(part) + off, tid), smem_u32(part_out + pb * Cfg::PART_FLOATS + tid * 128 * BO),
                               static_cast<uint32_t>(Cfg::ROWS * BO) * 4u, map_to_cta(smem_u32(&s_part_bar[pb]), tid));
        }
      }
      const long long e1 = prof ? clock64() : 0;
      if (prof) pf_scat += e1 - e0b;
      if (!dead && !mbar_wait_bounded<true, true>(smem_u32(&s_part_bar[pb]), (t >> 1) & 1, limit, abort_flag)) {
        mg_report(p.err, kErrWaitPart, t);
        dead = true;
      }
      const long long e2 = prof ? clock64() : 0;
      if (prof) pf_part += e2 - e1;
      float ry[NI][CT::GR];
      {
        const float* pbuf = part + pb * Cfg::PART_FLOATS;
#pragma unroll
        for (int j = 0; j < NI; ++j) {
          const int i = tid + kEpi * j;
          const int bl = i % BO;
#pragma unroll
          for (int g = 0; g < CT::GR; ++g) {
            float acc = 0.0f;
            if (i < Cfg::ITEMS) {
#pragma unroll
              for (int src = 0; src < KS; ++src) acc += pbuf[(src * 128 + g * 32 + it_u[j]) * BO + bl];
            }
            ry[j][g] = acc;
          }
        }
      }
      // The buffer of this parity is free again: every thread of this CTA passes the barrier inside publish()
      // before h_t leaves, and nobody can send the sums of step t + 2 before it has seen h_{t+1}.
      if (tid == 0 && !dead && t + 2 < T) mbar_arrive_expect_tx(smem_u32(&s_part_bar[pb]), part_tx);
      float cv[NI][CT::GC];
      uint32_t hb16[NI];
      const bool take_i = CELL == kSLSTM && t == 0 && zero_first;
#pragma unroll
      for (int j = 0; j < NI; ++j) {
        cell_forward<CELL>(ry[j], wx[j], bias[j], st[j], cv[j], take_i);
        hb16[j] = act[j] ? static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(st[j][0]))) : 0u;
      }
      // slot T (h of the last step) has no reader: not the recurrence, and the dR contraction stops at slot T - 1
      const long long e3 = prof ? clock64() : 0;
      publish(t + 1, hb16, !dead && t < mute_from && t + 1 < T);
      const long long e4 = prof ? clock64() : 0;
      if (prof) { pf_cell += e3 - e2; pf_pub += e4 - e3; }
      if (t + 1 < T) fetch(t + 1);
      const long long e5 = prof ? clock64() : 0;
      // state and cache stores last: the tensor core now works on h_t and this thread would only wait for it
#pragma unroll
      for (int j = 0; j < NI; ++j) {
        if (act[j]) {
          const size_t row = static_cast<size_t>(it_b[j]) * T + t;
#pragma unroll
          for (int q = 0; q < S; ++q) p.history[(static_cast<size_t>(q) * sBT + row) * ldx + xu + it_u[j]] = st[j][q];
          if (p.cache != nullptr && CELL != kElman) {
#pragma unroll
            for (int q = 0; q < CT::GC; ++q) st_cache<CT::CES>(p.cache, (row * CT::GC + q) * ldx + xu + it_u[j], cv[j][q]);
          }
        }
      }
      if (prof) pf_st += clock64() - e5;
    }
    if (prof) {  // epilogue thread 0: err[8] buffer-free wait, [9] operand poll + copy, [10] tensor-core wait, [11] partner sums
      p.err[8] = static_cast<int>(pf_free >> 10);
      p.err[9] = static_cast<int>(pf_poll >> 10);
      p.err[10] = static_cast<int>(pf_mma >> 10);
      p.err[11] = static_cast<int>(pf_part >> 10);
      // [12] accumulator read + partial rows sent, [13] sums + cell, [14] publication of h, [15] state and cache stores
      p.err[12] = static_cast<int>(pf_scat >> 10);
      p.err[13] = static_cast<int>(pf_cell >> 10);
      p.err[14] = static_cast<int>(pf_pub >> 10);
      p.err[15] = static_cast<int>(pf_st >> 10);
    }
#pragma unroll
    for (int j = 0; j < NI; ++j) {
      if (act[j]) {
#pragma unroll
        for (int q = 0; q < S; ++q) p.carry[(static_cast<size_t>(q) * B + it_b[j]) * ldx + xu + it_u[j]] = st[j][q];
      }
    }
  }

  // ---------------- teardown ----------------
  if (*abort_flag != 0) {
    const uint64_t t0 = global_timer_ns();  // copies still in flight get time to land
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  cluster_sync_all();
  if (warp == 4) tmem_dealloc(tbase, tmem_cols);
}

template <int CELL, int KS, bool WX_BF16>
int launch_fwd_mg(const MgFwdParams& p, const void* wx, cudaStream_t stream, int* capacity_only) {
  using Cfg = MgFwdCfg<CELL, KS, WX_BF16>;
  using CT = typename Cfg::CT;
  const int Kc = p.D / KS;
  const int SCK = Kc < kMgSubK ? Kc : kMgSubK;
  int smem = p.ring_stages * kMgRingBytes + 2 * mg_operand_bytes(SCK) + 4 * Cfg::PART_BYTES + ((Cfg::PUB_BYTES + 127) & ~127) +
             Cfg::NWX * Cfg::WX_STAGE_BYTES;
  if (smem > 227 * 1024) return -2;
  CUtensorMap wx_map, r_map;
  if (capacity_only == nullptr) {
    const uint64_t dims[5] = {static_cast<uint64_t>(p.ldx), 1u, static_cast<uint64_t>(CT::GW), static_cast<uint64_t>(p.T),
                              static_cast<uint64_t>(p.B)};
    const uint32_t box[5] = {32u, 1u, static_cast<uint32_t>(CT::GW), 1u, static_cast<uint32_t>(Cfg::BO)};
    if (make_tensor_map(&wx_map, wx, Cfg::WX_ES, 5, dims, box) != 0) return -4;
    // R rows as (k, row inside a gate, gate): a box is [gate][32 units][64 k], i.e. 128 rows of 128 bytes
    const uint64_t rdims[3] = {static_cast<uint64_t>(p.D), static_cast<uint64_t>(p.ldx), static_cast<uint64_t>(CT::GR)};
    const uint32_t rbox[3] = {static_cast<uint32_t>(kMgRingK), 32u, static_cast<uint32_t>(CT::GR)};
    if (make_tensor_map(&r_map, p.R, 2, 3, rdims, rbox, true) != 0) return -4;
  }
  auto kern = frnn_fwd_mg_kernel<CELL, KS, WX_BF16>;
  const int fit = fit_tmem_budget(kern, kMgThreads, 512u, &smem);
  if (fit != 0) return fit;
  cudaError_t e = cudaSuccess;
  if (KS > 8) {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(static_cast<unsigned>(p.ranks_here * (p.Dl / 32) * KS));
  cfg.blockDim = dim3(kMgThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  // all CTAs wait on one another (through the history buffers): the whole grid must be resident
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeCooperative;
  attr[0].val.cooperative = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = KS;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  // The cluster attribute is given for a cluster of one as well: the kernel scatters with st.async into
  // shared::cluster addresses, which a launch without cluster dimensions rejects as an illegal instruction.
  cfg.numAttrs = 2;
  int capacity = 0;
  {
    int max_clusters = 0;
    e = cudaOccupancyMaxActiveClusters(&max_clusters, kern, &cfg);
    if (e != cudaSuccess) return static_cast<int>(e);
    capacity = max_clusters * KS;
  }
  if (capacity_only != nullptr) {
    *capacity_only = capacity;
    return 0;
  }
  if (capacity < static_cast<int>(cfg.gridDim.x)) return -2;
  e = cudaLaunchKernelEx(&cfg, kern, p, wx_map, r_map);
  return static_cast<int>(e);
}

template <int CELL, int KS>
int launch_fwd_mg_dt(const MgFwdParams& p, const void* wx, int wx_bf16, cudaStream_t s, int* cap) {
  return wx_bf16 ? launch_fwd_mg<CELL, KS, true>(p, wx, s, cap) : launch_fwd_mg<CELL, KS, false>(p, wx, s, cap);
}
template <int CELL>
int launch_fwd_mg_ks(const MgFwdParams& p, const void* wx, int wx_bf16, int ks, cudaStream_t s, int* cap) {
  switch (ks) {
    case 1: return launch_fwd_mg_dt<CELL, 1>(p, wx, wx_bf16, s, cap);
    case 2: return launch_fwd_mg_dt<CELL, 2>(p, wx, wx_bf16, s, cap);
    case 4: return launch_fwd_mg_dt<CELL, 4>(p, wx, wx_bf16, s, cap);
    case 8: return launch_fwd_mg_dt<CELL, 8>(p, wx, wx_bf16, s, cap);
    case 16: return launch_fwd_mg_dt<CELL, 16>(p, wx, wx_bf16, s, cap);
    default: return -2;
  }
}

}  // namespace

// Launch (or, with capacity_only, only report how many CTAs of this configuration the device holds at once).
int forward_mg_dispatch(int cell, const MgFwdParams& p, const void* wx, int wx_bf16, int ksplit, cudaStream_t s,
                        int* capacity_only) {
  switch (cell) {
    case kLSTM: return launch_fwd_mg_ks<kLSTM>(p, wx, wx_bf16, ksplit, s, capacity_only);
    case kSLSTM: return launch_fwd_mg_ks<kSLSTM>(p, wx, wx_bf16, ksplit, s, capacity_only);
    case kGRU: return launch_fwd_mg_ks<kGRU>(p, wx, wx_bf16, ksplit, s, capacity_only);
    case kElman: return launch_fwd_mg_ks<kElman>(p, wx, wx_bf16, ksplit, s, capacity_only);
    default: return -1;
  }
}

// shared-memory bytes of the forward besides the weight ring, for the plan
int forward_mg_fixed_smem(int cell, int ksplit, int D, int wx_bf16) {
  const int gw = cell == kGRU ? 3 : (cell == kElman ? 1 : 4);
  const int bo = kMgBT / ksplit;
  const int Kc = D / ksplit;
  const int SCK = Kc < kMgSubK ? Kc : kMgSubK;
  const int wx_stage = bo * gw * 32 * (wx_bf16 ? 2 : 4);
  const int nwx = wx_stage * 4 <= 32768 ? 4 : 2;
  return 2 * mg_operand_bytes(SCK) + 4 * (ksplit * 128 * bo * 4) + ((bo * 32 * 2 + 127) & ~127) + nwx * wx_stage;
}

}  // namespace frnn
