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
    ok = mbar_wait_bounded<false>(smem_u32(&s_bar), issued & 1, 2000000000ull, p.err);
    ++issued;
    if (!ok) break;
  }
  if (!ok && tid == 0) atomicCAS(p.err, 0, kErrWaitMma);
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

}  // namespace

int wgrad_plan(int gr, int B, int T, int N, int D, int* np_out, int* ksplit_out, int* cps_out) {
  const int npt = (D + 255) / 256;
  if (D % (16 * npt) != 0) return -2;
  const int np = D / npt;
  const int mtiles = (gr * D + 127) / 128;
  const long long tiles = static_cast<long long>(mtiles) * npt * N;
  const long long chunks = (static_cast<long long>(B) * T + kKC - 1) / kKC;
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
  const int smem = 16 * 1024 + (np / 8) * 1024;
  cudaError_t e = cudaFuncSetAttribute(wgrad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  const int mtiles = (gr * D + 127) / 128;
  dim3 grid(static_cast<unsigned>(mtiles * (D / np)), static_cast<unsigned>(N), static_cast<unsigned>(ksplit));
  wgrad_kernel<<<grid, kThreads, smem, s>>>(p);
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
