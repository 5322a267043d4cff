// Weight gradients of the recurrence:
//   dR[g,n,o,p] = sum_{b,t} dg[b,t,g,n,o] * round_bf16(h_{t-1})[b,n,p]      (tcgen05 GEMM, K = B*T)
//   db[g,n,d]   = sum over batch tiles of the per-tile sums the backward kernel produced.
// Split-K partial tiles go to caller-provided scratch and are reduced in a fixed order, so the
// result is deterministic and no atomics are used.
//
// Replaces the strided-batched cuBLAS GEMM and gradientBiasAggregationKernel of
// flashrnn/flashrnn/fused/flashrnn_fused_backward.cu:1050-1070, 627-666.
#include <mutex>

#include "frnn_common.cuh"

namespace frnn {

namespace {

constexpr int kThreads = 128;
constexpr int kKC = 64;  // (b,t) rows per shared-memory chunk

struct WgradParams {
  const __nv_bfloat16* dgr;  // [B*T][GR][N][D]
  const __nv_bfloat16* hbf;  // [B][T+1][N][D]
  float* out;                // dR, or split-K scratch [ksplit][GR*N*D*D]
  int* err;
  int B, T, N, D, GR;
  int NP;       // p columns per tile
  int ksplit;
  int chunks_per_split;
  int pack;     // heads that share one 64-wide TMA box (narrow heads, D = 16 or 32), else 1
  // Row window (TMA kernel, pack == 1): the contraction produces only the rows o in [m_off, m_off + Dm) of every
  // gate (a rank's units of a row-sharded head) and writes them as [GR][N][out_rows][D] starting at `out`.
  // Dm = out_rows = D and m_off = 0 describe the whole matrix.
  int Dm, m_off, out_rows;
};

// Both operands are MN-major (the contraction index is the slow one in memory). Un-swizzled
// canonical tiles: 8(k) x 8(mn) core matrices of 128 bytes, k-groups 128 B apart, mn-groups
// 1024 B apart.
__global__ void __launch_bounds__(kThreads, 1) wgrad_kernel(const WgradParams p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  __shared__ __align__(8) uint64_t s_bar;
  __shared__ uint32_t s_tmem_base;
  const int tid = threadIdx.x, warp = tid >> 5;
  const int D = p.D, N = p.N, T = p.T, GR = p.GR, NP = p.NP;
  const int npt = D / NP;
  const int mtile = blockIdx.x / npt, ptile = blockIdx.x % npt;
  const int n = blockIdx.y, split = blockIdx.z;
  const int m0 = mtile * 128, p0 = ptile * NP;
  const int M = GR * D;
  const long long K = static_cast<long long>(p.B) * T;
  uint8_t* const sA = smem;               // 16 mn-groups * 1024
  uint8_t* const sB = smem + 16 * 1024;   // NP/8 mn-groups * 1024
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(NP)) tmem_cols <<= 1;

  if (tid == 0) {
    mbar_init(smem_u32(&s_bar), 1);
    fence_mbar_init();
  }
  if (warp == 0) {
    tmem_alloc(smem_u32(&s_tmem_base), tmem_cols);
    tmem_relinquish_alloc();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = s_tmem_base;
  const uint32_t idesc = umma_idesc_bf16(128, NP, true, true);
  const int c_begin = split * p.chunks_per_split;
  const long long total_chunks = (K + kKC - 1) / kKC;
  int c_end = c_begin + p.chunks_per_split;
  if (c_end > total_chunks) c_end = static_cast<int>(total_chunks);
  bool ok = true;
  int issued = 0;
  for (int c = c_begin; c < c_end; ++c) {
    const long long k0 = static_cast<long long>(c) * kKC;
    // A chunk: dg^T [128 m x 64 k]
    for (int v = tid; v < kKC * 16; v += kThreads) {
      const int k = v >> 4, mg = v & 15;
      const int m = m0 + mg * 8;
      const long long kt = k0 + k;
      uint4 val = make_uint4(0u, 0u, 0u, 0u);
      if (m < M && kt < K) {
        const int g = m / D, o = m % D;
        val = __ldg(reinterpret_cast<const uint4*>(p.dgr + ((kt * GR + g) * N + n) * D + o));
      }
      *reinterpret_cast<uint4*>(sA + mg * 1024 + (k >> 3) * 128 + (k & 7) * 16) = val;
    }
    // B chunk: round_bf16(h_{t-1}) [NP p x 64 k]
    const int pgs = NP / 8;
    for (int v = tid; v < kKC * pgs; v += kThreads) {
      const int k = v / pgs, pg = v % pgs;
      const long long kt = k0 + k;
      uint4 val = make_uint4(0u, 0u, 0u, 0u);
      if (kt < K) {
        const long long b = kt / T, t = kt % T;
        val = __ldg(reinterpret_cast<const uint4*>(p.hbf + ((b * (T + 1) + t) * N + n) * D + p0 + pg * 8));
      }
      *reinterpret_cast<uint4*>(sB + pg * 1024 + (k >> 3) * 128 + (k & 7) * 16) = val;
    }
    fence_proxy_async_smem();
    __syncthreads();
    if (tid == 0) {
      tc_fence_after_sync();
      for (int kk = 0; kk < kKC / 16; ++kk) {
        const uint64_t ad = umma_smem_desc(smem_u32(sA) + kk * 256, 128, 1024);
        const uint64_t bd = umma_smem_desc(smem_u32(sB) + kk * 256, 128, 1024);
        umma_bf16_ss(tbase, ad, bd, idesc, (issued > 0 || kk > 0) ? 1u : 0u);
      }
      umma_commit(smem_u32(&s_bar));
    }
    ok = mbar_wait_bounded<false, true>(smem_u32(&s_bar), issued & 1, 2000000000ull, p.err);
    ++issued;
    if (!ok) break;
  }
  if (!ok && tid == 0) {
    atomicCAS(p.err, 0, kErrWaitMma);
    // the chunk whose commit was not seen may still be on the tensor core: wait for it once more (no abort
    // flag: the commit completes by itself) before the tensor memory is released below
    mbar_wait_bounded<false, true>(smem_u32(&s_bar), (issued - 1) & 1, 2000000000ull, nullptr);
  }
  tc_fence_after_sync();
  // epilogue: accumulator rows -> global (row = (g, o), contiguous along p)
  {
    const int m = m0 + tid;
    float* dst = nullptr;
    if (m < M) {
      const int g = m / D, o = m % D;
      dst = p.out + static_cast<size_t>(split) * GR * N * D * D + ((static_cast<size_t>(g) * N + n) * D + o) * D + p0;
    }
    for (int c8 = 0; c8 < NP; c8 += 8) {
      uint32_t r[8];
      if (issued > 0 && ok) {
        tmem_ld_x8(tmem_addr(tbase, 32 * warp, c8), r);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int q = 0; q < 8; ++q) r[q] = 0u;
      }
      if (dst != nullptr) {
        *reinterpret_cast<float4*>(dst + c8) = make_float4(__uint_as_float(r[0]), __uint_as_float(r[1]), __uint_as_float(r[2]), __uint_as_float(r[3]));
        *reinterpret_cast<float4*>(dst + c8 + 4) = make_float4(__uint_as_float(r[4]), __uint_as_float(r[5]), __uint_as_float(r[6]), __uint_as_float(r[7]));
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, tmem_cols);
}

// ---------------------------------------------------------------------------------------------
// Pipelined variant for D % 64 == 0: operands arrive by TMA (128-byte swizzle, 64 x 64 boxes)
// through a 4-stage ring; warp 0 = TMA producer, warp 1 = UMMA issuer, warps 2-5 = epilogue.
// A stage holds 64 (b,t) rows: A = dg^T [128 m x 64 k] as two boxes, B = h~ [NP p x 64 k] as
// NP/64 boxes. A chunk never straddles a batch row; rows past T read as zeros on the dg side.
// ---------------------------------------------------------------------------------------------
constexpr int kTmaThreads = 192;
constexpr int kTmaStages = 4;

__global__ void __launch_bounds__(kTmaThreads, 1)
wgrad_tma_kernel(const WgradParams p, const __grid_constant__ CUtensorMap dgr_map,
                 const __grid_constant__ CUtensorMap hbf_map) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_full[kTmaStages];
  __shared__ __align__(8) uint64_t s_empty[kTmaStages];
  __shared__ __align__(8) uint64_t s_acc;
  __shared__ uint32_t s_tmem_base;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int D = p.D, T = p.T, GR = p.GR, NP = p.NP;
  const int npt = p.pack > 1 ? 1 : D / NP;
  const int mtile = blockIdx.x / npt, ptile = blockIdx.x % npt;
  const int n = blockIdx.y, split = blockIdx.z;
  const int m0 = mtile * 128, p0 = ptile * NP;
  const int Dm = p.Dm;
  const int M = GR * Dm;
  // Narrow heads (pack > 1): one box spans `pack` neighbouring heads of one gate, so the 128 x 64
  // tile holds pack x pack head blocks per gate of which only the diagonal ones are kept;
  // blockIdx.x = gate pair, blockIdx.y = head group.
  const int pack = p.pack;
  const int cpb = (T + kKC - 1) / kKC;  // chunks per batch row
  const int total_chunks = p.B * cpb;
  const int c_begin = split * p.chunks_per_split;
  const int c_end = min(c_begin + p.chunks_per_split, total_chunks);
  const int n_chunks = max(c_end - c_begin, 0);
  const uint32_t stage_bytes = 16384u + static_cast<uint32_t>(NP) * 128u;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint32_t tmem_cols = 32;
  while (tmem_cols < static_cast<uint32_t>(NP)) tmem_cols <<= 1;
  const volatile int* abort_flag = p.err;
  constexpr uint64_t kLimit = 2000000000ull;

  if (tid == 0) {
    for (int s = 0; s < kTmaStages; ++s) {
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&s_empty[s]), 1);
    }
    mbar_init(smem_u32(&s_acc), 1);
    fence_mbar_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(&s_tmem_base), tmem_cols);
    tmem_relinquish_alloc();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = s_tmem_base;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&dgr_map);
      tma_prefetch_desc(&hbf_map);
      for (int i = 0; i < n_chunks; ++i) {
        const int s = i % kTmaStages, c = c_begin + i;
        if (i >= kTmaStages &&
            !mbar_wait_bounded<false, true>(smem_u32(&s_empty[s]), ((i / kTmaStages) - 1) & 1, kLimit, abort_flag)) {
          atomicCAS(p.err, 0, kErrWaitEmpty);
          break;
        }
        const int b = c / cpb, t0 = (c % cpb) * kKC;
        const uint32_t bar = smem_u32(&s_full[s]);
        const uint32_t sa = base + s * stage_bytes, sb = sa + 16384u;
        mbar_arrive_expect_tx(bar, stage_bytes);
        if (pack == 1) {
          for (int h = 0; h < 2; ++h) {
            const int m = m0 + 64 * h;
            tma_load_5d(sa + h * 8192u, &dgr_map, bar, p.m_off + m % Dm, n, m / Dm, t0, b);
          }
          for (int j = 0; j < NP / 64; ++j) tma_load_4d(sb + j * 8192u, &hbf_map, bar, p0 + 64 * j, n, t0, b);
        } else {
          // maps flatten (head, unit): x = 64 * head group; gates past GR read as zeros
          for (int h = 0; h < 2; ++h) tma_load_4d(sa + h * 8192u, &dgr_map, bar, 64 * n, 2 * mtile + h, t0, b);
          tma_load_3d(sb, &hbf_map, bar, 64 * n, t0, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(128, NP, true, true);
      for (int i = 0; i < n_chunks; ++i) {
        const int s = i % kTmaStages;
        if (!mbar_wait_bounded<false, true>(smem_u32(&s_full[s]), (i / kTmaStages) & 1, kLimit, abort_flag)) {
          atomicCAS(p.err, 0, kErrWaitWx);
          break;
        }
        tc_fence_after_sync();
        const uint32_t sa = base + s * stage_bytes, sb = sa + 16384u;
#pragma unroll
        for (int kk = 0; kk < kKC / 16; ++kk) {
          const uint64_t ad = umma_smem_desc_mn_sw128(sa + kk * 2048u, 8192u);
          const uint64_t bd = umma_smem_desc_mn_sw128(sb + kk * 2048u, 8192u);
          umma_bf16_ss(tbase, ad, bd, idesc, (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(smem_u32(&s_empty[s]));  // the stage is free once these MMAs have read it
      }
      // One commit covers every MMA this thread has issued, also after a failed wait. The issuing thread then
      // waits for it itself (the commit completes without any other party, hence no abort flag) so that the
      // tensor memory and the stages are never released while an MMA still runs.
      if (n_chunks > 0) {
        umma_commit(smem_u32(&s_acc));
        mbar_wait_bounded<false, true>(smem_u32(&s_acc), 0, kLimit, nullptr);
      }
    }
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    const int m = m0 + 32 * q + lane;
    bool have = n_chunks > 0;
    if (have && !mbar_wait_bounded<false, true>(smem_u32(&s_acc), 0, kLimit, abort_flag)) {
      atomicCAS(p.err, 0, kErrWaitMma);
      have = false;
    }
    tc_fence_after_sync();
    if (pack == 1) {
      float* dst = nullptr;
      if (m < M) {
        const int g = m / Dm, o = m % Dm;
        dst = p.out + static_cast<size_t>(split) * GR * p.N * p.out_rows * D +
              ((static_cast<size_t>(g) * p.N + n) * p.out_rows + o) * D + p0;
      }
      for (int c8 = 0; c8 < NP; c8 += 8) {
        uint32_t r[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
        if (have) {
          tmem_ld_x8(tmem_addr(tbase, 32 * q, c8), r);
          tmem_ld_wait();
        }
        if (dst != nullptr) {
          *reinterpret_cast<float4*>(dst + c8) = make_float4(__uint_as_float(r[0]), __uint_as_float(r[1]), __uint_as_float(r[2]), __uint_as_float(r[3]));
          *reinterpret_cast<float4*>(dst + c8 + 4) = make_float4(__uint_as_float(r[4]), __uint_as_float(r[5]), __uint_as_float(r[6]), __uint_as_float(r[7]));
        }
      }
    } else {
      // row = (gate of the pair, head of the group, unit); keep the columns of the same head
      const int row = 32 * q + lane;
      const int g = 2 * mtile + row / 64, hh = (row % 64) / D, o = row % D;
      const int head = n * pack + hh;
      float* dst = nullptr;
      if (g < GR && head < p.N)
        dst = p.out + static_cast<size_t>(split) * GR * p.N * D * D + ((static_cast<size_t>(g) * p.N + head) * D + o) * D;
      for (int h2 = 0; h2 < pack; ++h2) {      // the TMEM address of a load is warp-uniform
        for (int c8 = 0; c8 < D; c8 += 8) {
          uint32_t r[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
          if (have) {
            tmem_ld_x8(tmem_addr(tbase, 32 * q, h2 * D + c8), r);
            tmem_ld_wait();
          }
          if (dst != nullptr && h2 == hh) {
            *reinterpret_cast<float4*>(dst + c8) = make_float4(__uint_as_float(r[0]), __uint_as_float(r[1]), __uint_as_float(r[2]), __uint_as_float(r[3]));
            *reinterpret_cast<float4*>(dst + c8 + 4) = make_float4(__uint_as_float(r[4]), __uint_as_float(r[5]), __uint_as_float(r[6]), __uint_as_float(r[7]));
          }
        }
      }
    }
  }
  if (*abort_flag != 0) {
    const uint64_t t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tbase, tmem_cols);
}

__global__ void reduce_parts_kernel(const float* __restrict__ parts, float* __restrict__ out, long long n, int nparts) {
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 acc = *reinterpret_cast<const float4*>(parts + i);
  for (int s = 1; s < nparts; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(parts + static_cast<long long>(s) * n + i);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  *reinterpret_cast<float4*>(out + i) = acc;
}

// out[i] = sum over parts of parts[part * part_stride + i], i < n (n a multiple of 4)
__global__ void reduce_parts_strided_kernel(const float* __restrict__ parts, float* __restrict__ out, int n,
                                            long long part_stride, int nparts) {
  const int i = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 acc = *reinterpret_cast<const float4*>(parts + i);
  for (int s = 1; s < nparts; ++s) {
    const float4 v = *reinterpret_cast<const float4*>(parts + s * part_stride + i);
    acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
  }
  *reinterpret_cast<float4*>(out + i) = acc;
}

}  // namespace

// The TMA kernel needs whole 64-element boxes along both output dimensions; heads of 16 or 32
// units are packed 4 or 2 to a box.
static bool wgrad_uses_tma(int D, int np) { return D % 64 == 0 && np % 64 == 0; }
static int wgrad_pack(int D) { return (D == 16 || D == 32) ? 64 / D : 1; }

int wgrad_plan(int gr, int B, int T, int N, int D, int* np_out, int* ksplit_out, int* cps_out) {
  // column tiles: the fewest equal parts of D that are at most 256 wide and a multiple of 16
  if (D % 16 != 0) return -2;
  int npt = (D + 255) / 256;
  while (D % npt != 0 || (D / npt) % 16 != 0) ++npt;
  const int pack = wgrad_pack(D);
  const int np = pack > 1 ? 64 : D / npt;
  const int mtiles = pack > 1 ? (gr + 1) / 2 : (gr * D + 127) / 128;
  const long long tiles = pack > 1 ? static_cast<long long>(mtiles) * ((N + pack - 1) / pack)
                                   : static_cast<long long>(mtiles) * npt * N;
  const long long chunks = (pack > 1 || wgrad_uses_tma(D, np))
                               ? static_cast<long long>(B) * ((T + kKC - 1) / kKC)   // per batch row
                               : (static_cast<long long>(B) * T + kKC - 1) / kKC;
  long long ks = 148 / tiles;
  if (ks < 1) ks = 1;
  if (ks > 32) ks = 32;
  if (ks > chunks) ks = chunks;
  const long long cps = (chunks + ks - 1) / ks;
  ks = (chunks + cps - 1) / cps;
  *np_out = np;
  *ksplit_out = static_cast<int>(ks);
  *cps_out = static_cast<int>(cps);
  return 0;
}

int wgrad_launch(int gr, int gb, const __nv_bfloat16* dgr, const __nv_bfloat16* hbf, const float* db_part, int n_btiles,
                 float* dR, float* db, float* work, int* err, int B, int T, int N, int D, cudaStream_t s) {
  int np, ksplit, cps;
  if (wgrad_plan(gr, B, T, N, D, &np, &ksplit, &cps) != 0) return -2;
  if (ksplit > 1 && work == nullptr) return -5;
  WgradParams p{};
  p.dgr = dgr; p.hbf = hbf;
  p.out = ksplit > 1 ? work : dR;
  p.err = err;
  p.B = B; p.T = T; p.N = N; p.D = D; p.GR = gr;
  p.NP = np; p.ksplit = ksplit; p.chunks_per_split = cps;
  p.Dm = D; p.m_off = 0; p.out_rows = D;
  const int pack = wgrad_pack(D);
  p.pack = pack;
  const int mtiles = pack > 1 ? (gr + 1) / 2 : (gr * D + 127) / 128;
  dim3 grid(static_cast<unsigned>(pack > 1 ? mtiles : mtiles * (D / np)),
            static_cast<unsigned>(pack > 1 ? (N + pack - 1) / pack : N), static_cast<unsigned>(ksplit));
  cudaError_t e;
  if (pack > 1) {
    CUtensorMap dgr_map, hbf_map;
    const uint64_t ddims[4] = {static_cast<uint64_t>(N) * D, static_cast<uint64_t>(gr), static_cast<uint64_t>(T),
                               static_cast<uint64_t>(B)};
    const uint32_t dbox[4] = {64u, 1u, static_cast<uint32_t>(kKC), 1u};
    const uint64_t hdims[3] = {static_cast<uint64_t>(N) * D, static_cast<uint64_t>(T + 1), static_cast<uint64_t>(B)};
    const uint32_t hbox[3] = {64u, static_cast<uint32_t>(kKC), 1u};
    if (make_tensor_map(&dgr_map, dgr, 2, 4, ddims, dbox, true) != 0) return -4;
    if (make_tensor_map(&hbf_map, hbf, 2, 3, hdims, hbox, true) != 0) return -4;
    const int smem = kTmaStages * (16384 + 64 * 128) + 1024;
    e = cudaFuncSetAttribute(wgrad_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    wgrad_tma_kernel<<<grid, kTmaThreads, smem, s>>>(p, dgr_map, hbf_map);
  } else if (wgrad_uses_tma(D, np)) {
    CUtensorMap dgr_map, hbf_map;
    const uint64_t ddims[5] = {static_cast<uint64_t>(D), static_cast<uint64_t>(N), static_cast<uint64_t>(gr),
                               static_cast<uint64_t>(T), static_cast<uint64_t>(B)};
    const uint32_t dbox[5] = {64u, 1u, 1u, static_cast<uint32_t>(kKC), 1u};
    const uint64_t hdims[4] = {static_cast<uint64_t>(D), static_cast<uint64_t>(N), static_cast<uint64_t>(T + 1),
                               static_cast<uint64_t>(B)};
    const uint32_t hbox[4] = {64u, 1u, static_cast<uint32_t>(kKC), 1u};
    if (make_tensor_map(&dgr_map, dgr, 2, 5, ddims, dbox, true) != 0) return -4;
    if (make_tensor_map(&hbf_map, hbf, 2, 4, hdims, hbox, true) != 0) return -4;
    const int smem = kTmaStages * (16384 + np * 128) + 1024;
    e = cudaFuncSetAttribute(wgrad_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    wgrad_tma_kernel<<<grid, kTmaThreads, smem, s>>>(p, dgr_map, hbf_map);
  } else {
    const int smem = 16 * 1024 + (np / 8) * 1024;
    e = cudaFuncSetAttribute(wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    wgrad_kernel<<<grid, kThreads, smem, s>>>(p);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  const long long nR = static_cast<long long>(gr) * N * D * D;
  if (ksplit > 1) {
    reduce_parts_kernel<<<static_cast<unsigned>((nR / 4 + 255) / 256), 256, 0, s>>>(work, dR, nR, ksplit);
    e = cudaGetLastError();
    if (e != cudaSuccess) return static_cast<int>(e);
  }
  const long long nb = static_cast<long long>(gb) * N * D;
  reduce_parts_kernel<<<static_cast<unsigned>((nb / 4 + 255) / 256), 256, 0, s>>>(db_part, db, nb, n_btiles);
  return static_cast<int>(cudaGetLastError());
}

// Row-sharded wide head (one head, N = 1): dR[g, o, p] for the rows o in [m_off, m_off + Dm) only, from this
// rank's full-width histories dgr [B][T][GR][D] and hbf [B][T+1][D]; slot T of hbf is never read (the tensor map
// ends at T, reads beyond it are filled with zeros), so it need not be written. db = sum of `n_parts` partial rows
// db_part [n_parts][GB][ldb] -> db [GB][ldb] restricted to the window [x0, x0 + Dm).
int wgrad_launch_rows(int gr, int gb, const __nv_bfloat16* dgr, const __nv_bfloat16* hbf, const float* db_part, int n_parts,
                      float* dR, float* db, int* err, int B, int T, int D, int Dm, int m_off, int out_rows, int ldb, int x0,
                      cudaStream_t s) {
  if (D % 256 != 0 || Dm % 128 != 0 || m_off % 64 != 0) return -2;
  WgradParams p{};
  p.dgr = dgr; p.hbf = hbf; p.out = dR; p.err = err;
  p.B = B; p.T = T; p.N = 1; p.D = D; p.GR = gr;
  p.NP = 256; p.ksplit = 1;
  p.chunks_per_split = B * ((T + kKC - 1) / kKC);
  p.pack = 1;
  p.Dm = Dm; p.m_off = m_off; p.out_rows = out_rows;
  CUtensorMap dgr_map, hbf_map;
  const uint64_t ddims[5] = {static_cast<uint64_t>(D), 1u, static_cast<uint64_t>(gr), static_cast<uint64_t>(T),
                             static_cast<uint64_t>(B)};
  const uint32_t dbox[5] = {64u, 1u, 1u, static_cast<uint32_t>(kKC), 1u};
  const uint64_t hdims[4] = {static_cast<uint64_t>(D), 1u, static_cast<uint64_t>(T), static_cast<uint64_t>(B)};
  const uint64_t hstride[4] = {static_cast<uint64_t>(D), 1u, static_cast<uint64_t>(T + 1), static_cast<uint64_t>(B)};
  const uint32_t hbox[4] = {64u, 1u, static_cast<uint32_t>(kKC), 1u};
  if (make_tensor_map(&dgr_map, dgr, 2, 5, ddims, dbox, true) != 0) return -4;
  if (make_tensor_map(&hbf_map, hbf, 2, 4, hdims, hbox, true, hstride) != 0) return -4;
  const int smem = kTmaStages * (16384 + 256 * 128) + 1024;
  cudaError_t e = cudaFuncSetAttribute(wgrad_tma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  dim3 grid(static_cast<unsigned>((gr * Dm / 128) * (D / 256)), 1u, 1u);
  wgrad_tma_kernel<<<grid, kTmaThreads, smem, s>>>(p, dgr_map, hbf_map);
  e = cudaGetLastError();
  if (e != cudaSuccess) return static_cast<int>(e);
  // db: the window of every gate row is reduced separately (the rows are ldb apart)
  for (int g = 0; g < gb; ++g) {
    reduce_parts_strided_kernel<<<static_cast<unsigned>((Dm / 4 + 127) / 128), 128, 0, s>>>(
        db_part + static_cast<size_t>(g) * ldb + x0, db + static_cast<size_t>(g) * ldb + x0, Dm,
        static_cast<long long>(gb) * ldb, n_parts);
  }
  return static_cast<int>(cudaGetLastError());
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the weight-gradient step.
//
// Some hosts of this library must not (or cannot) create device memory at the moment they need
// dR: a plugin that runs inside another framework's steady-state loop where cudaMalloc is
// forbidden because it synchronises the device, a process that was handed a fixed memory budget
// at start-up, or code that only receives raw input/output pointers and has no allocator of its
// own to ask for the split-K partial tiles. For them the partial tiles live in a fixed array that
// is part of the library image: every GPU that loads the library reserves it until the process
// exits. All calls on a device share that one array, so two such calls that overlap on the GPU
// (different streams) corrupt each other; nothing in it has to start at zero because the kernel
// overwrites every partial tile it later reduces.
// ---------------------------------------------------------------------------------------------
constexpr size_t kStaticWorkBytes = 16u << 20;  // 16 MiB
static __device__ __align__(256) unsigned char g_static_work[kStaticWorkBytes];

namespace {
// The array's name is only a host-side handle; its device address is looked up once per device
// (with that device current) and cached.
int static_work_address(float** out) {
  static std::mutex mu;
  static float* cached[64] = {};
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  if (dev < 0 || dev >= 64) return -5;
  std::lock_guard<std::mutex> lock(mu);
  if (cached[dev] == nullptr) {
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_work);
    if (e != cudaSuccess) return static_cast<int>(e);
    cached[dev] = static_cast<float*>(ptr);
  }
  *out = cached[dev];
  return 0;
}
}  // namespace

int wgrad_launch_static(int gr, int gb, const __nv_bfloat16* dgr, const __nv_bfloat16* hbf, const float* db_part,
                        int n_btiles, float* dR, float* db, int* err, int B, int T, int N, int D, cudaStream_t s) {
  int np, ksplit, cps;
  if (wgrad_plan(gr, B, T, N, D, &np, &ksplit, &cps) != 0) return -2;
  const size_t need = ksplit > 1 ? static_cast<size_t>(ksplit) * gr * N * D * D * sizeof(float) : 0;
  if (need > kStaticWorkBytes) return -6;
  float* work = nullptr;
  const int rc = static_work_address(&work);
  if (rc != 0) return rc;
  return wgrad_launch(gr, gb, dgr, hbf, db_part, n_btiles, dR, db, work, err, B, T, N, D, s);
}

}  // namespace frnn
