// Shared declarations of the recurrence kernels: launch plan, kernel parameter blocks,
// small vector helpers and the host-side TMA descriptor builder.
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "cells.cuh"
#include "sm100_ptx.cuh"

namespace frnn {

// Error codes written to err[0] by a kernel whose bounded wait ran out (0 = ok).
enum : int {
  kErrWaitH = 101,      // forward: recurrent operand of a step never arrived
  kErrWaitMma = 102,    // tensor-core completion barrier
  kErrWaitWx = 103,     // TMA stage never filled
  kErrWaitEmpty = 104,  // TMA stage never released
  kErrWaitEpi = 105,    // epilogue-internal barrier
  kErrWaitPart = 106,   // partial sums of a peer CTA never arrived
  kErrWaitDg = 107,     // backward: dg operand barrier
  kErrWaitReady = 108,  // multi-GPU: a peer never announced that its exchange buffer is ready
  kErrWaitRing = 109,   // multi-GPU: a stage of the streamed weight operand never arrived / was never released
};

struct FwdParams {
  const __nv_bfloat16* R;  // [GR][N][D][D] (out, in)
  const float* bias;       // [GB][N][D]
  const float* initial;    // [S][B][1][N][D]
  float* history;          // [S][B][T][N][D]
  float* carry;            // [S][B][1][N][D]
  void* cache;             // [B][T][GC][N][D] (fp16 or fp32 elements, CellTraits::CES) or null (inference)
  __nv_bfloat16* hbf;      // [B][T+1][N][D] bf16 copy of h_{-1..T-1}, or null
  int* err;                // device int[4]
  int B, T, N, D;
  int C;
  int wx_box_b;            // batch extent of the Wx TMA box
  int slstm_zero_first;
  // Forward-only extras (prepared sequences): when non-null, the sLSTM predicate is read from this
  // device word instead of slstm_zero_first (no host read, so the call can sit in a CUDA graph);
  // output_mode 0 writes every state's history [S][B][T][N][D], 1 the hidden state only
  // [B][T][N][D], 2 only the last hidden state [B][1][N][D].
  const int* zero_first_dev;
  int output_mode;
  // A call may cover the steps [t0, t0 + T) of a longer sequence of T_total steps whose Wx and output tensors
  // are laid out for the whole sequence (chunked execution of a prepared sequence); T_total = T and t0 = 0
  // otherwise. The gate cache and the bf16 copy of h are only written by whole-sequence calls.
  int T_total, t0;
  int out_bf16;            // 1: the state history is stored as bf16 snapshots (forward-only calls)
  float fwd_clip;          // h_t is clipped to [-fwd_clip, fwd_clip]; +inf = off
  unsigned long long wait_limit_ns;
  // Exchange through global memory (groups wider than a cluster), null for cluster exchange:
  // per group four slots of the bf16 operand (the data words double as arrival flags).
  uint8_t* xg_data;
};

struct BwdParams {
  const __nv_bfloat16* R;   // [GR][N][D][D]
  const float* d_carry;     // [S][B][1][N][D]
  void* dwx;                // [B][T][GW][N][D] in the Wx dtype
  __nv_bfloat16* dgr;       // [B][T][GR][N][D] bf16 operand of the dR contraction
  float* d_initial;         // [S][B][1][N][D]
  float* db_part;           // [n_btiles][GB][N][D]
  int* err;
  int B, T, N, D;
  int C;
  int box_b;
  int slstm_zero_first;
  float grad_clip;          // > 0: the gradient carried into h_t from step t+1 is clipped to [-grad_clip, grad_clip]
  int cut_recurrent;        // 1: the R path of the hidden-state gradient is dropped
  int slstm_v1;             // 1: sLSTM gradient convention of the reference's own kernels (see cell_backward)
  unsigned long long wait_limit_ns;
  // Exchange through global memory, null for cluster exchange: per group two slots of the
  // partial-dh blocks [dest CTA][source CTA][batch][unit] (1-D backward, phase bit in every word) or
  // four slots of the bf16 dG operand (backward that owns columns of R).
  uint8_t* xg_data;
};

template <int N>
__device__ __forceinline__ void ld_f32_vec(const float* p, float* v) {
  if constexpr (N % 4 == 0) {
#pragma unroll
    for (int i = 0; i < N; i += 4) {
      const float4 t = *reinterpret_cast<const float4*>(p + i);
      v[i] = t.x; v[i + 1] = t.y; v[i + 2] = t.z; v[i + 3] = t.w;
    }
  } else if constexpr (N % 2 == 0) {
#pragma unroll
    for (int i = 0; i < N; i += 2) {
      const float2 t = *reinterpret_cast<const float2*>(p + i);
      v[i] = t.x; v[i + 1] = t.y;
    }
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) v[i] = p[i];
  }
}
template <int N>
__device__ __forceinline__ void st_f32_vec(float* p, const float* v) {
  if constexpr (N % 4 == 0) {
#pragma unroll
    for (int i = 0; i < N; i += 4)
      *reinterpret_cast<float4*>(p + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
  } else if constexpr (N % 2 == 0) {
#pragma unroll
    for (int i = 0; i < N; i += 2) *reinterpret_cast<float2*>(p + i) = make_float2(v[i], v[i + 1]);
  } else {
#pragma unroll
    for (int i = 0; i < N; ++i) p[i] = v[i];
  }
}
// Gate-cache accessors: fp32 or fp16 elements (CES = 4 / 2 bytes, see CellTraits), `off` in elements.
template <int N, int CES>
__device__ __forceinline__ void st_cache_vec(void* base, size_t off, const float* v) {
  if constexpr (CES == 4) {
    st_f32_vec<N>(static_cast<float*>(base) + off, v);
  } else {
    static_assert(N % 2 == 0, "pairs");
    __half* p = static_cast<__half*>(base) + off;
#pragma unroll
    for (int i = 0; i < N; i += 2) *reinterpret_cast<__half2*>(p + i) = __floats2half2_rn(v[i], v[i + 1]);
  }
}
template <int N, int CES>
__device__ __forceinline__ void ld_cache_vec(const void* base, size_t off, float* v) {
  if constexpr (CES == 4) {
    ld_f32_vec<N>(static_cast<const float*>(base) + off, v);
  } else {
    static_assert(N % 2 == 0, "pairs");
    const __half* p = static_cast<const __half*>(base) + off;
#pragma unroll
    for (int i = 0; i < N; i += 2) {
      const float2 t = __half22float2(*reinterpret_cast<const __half2*>(p + i));
      v[i] = t.x; v[i + 1] = t.y;
    }
  }
}
template <int CES>
__device__ __forceinline__ void st_cache(void* base, size_t off, float v) {
  if constexpr (CES == 4) static_cast<float*>(base)[off] = v;
  else static_cast<__half*>(base)[off] = __float2half_rn(v);
}
template <int CES>
__device__ __forceinline__ float ld_cache(const void* base, size_t off) {
  if constexpr (CES == 4) return static_cast<const float*>(base)[off];
  else return __half2float(static_cast<const __half*>(base)[off]);
}

// Test hook for race verification (err[6] = seed, 0 = off): in a quarter of the steps the calling warp role of this
// CTA sits out a pseudo-random time of up to 8 us, chosen from (seed, CTA, role, step) and therefore the same for all
// of the role's threads, so that CTAs and roles drift against each other at every hand-off of the exchange
// protocols. Results must not depend on it.
__device__ __forceinline__ void jitter_stall(uint32_t seed, uint32_t role, uint32_t step) {
  uint32_t h = seed ^ (blockIdx.x * 0x9E3779B1u) ^ (role * 0x85EBCA77u) ^ (step * 0xC2B2AE3Du);
  h ^= h >> 15; h *= 0x2C1B3C6Du; h ^= h >> 12; h *= 0x297A2D39u; h ^= h >> 15;
  if ((h & 3u) != 0u) return;
  const uint64_t ns = (h >> 8) & 0x1fffu, t0 = global_timer_ns();
  while (global_timer_ns() - t0 < ns) __nanosleep(200);
}

template <int N>
__device__ __forceinline__ void st_bf16_vec(__nv_bfloat16* p, const float* v) {
  static_assert(N % 2 == 0, "pairs");
#pragma unroll
  for (int i = 0; i < N; i += 2) *reinterpret_cast<__nv_bfloat162*>(p + i) = __floats2bfloat162_rn(v[i], v[i + 1]);
}
template <int N>
__device__ __forceinline__ void ld_bf16_vec(const __nv_bfloat16* p, float* v) {
  static_assert(N % 2 == 0, "pairs");
#pragma unroll
  for (int i = 0; i < N; i += 2) {
    const float2 t = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p + i));
    v[i] = t.x; v[i + 1] = t.y;
  }
}
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  const __nv_bfloat162 t = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&t);
}

// Byte offset of element (row, k) inside an un-swizzled K-major UMMA operand tile of `rows`
// rows: 8x8 core matrices, K-adjacent core matrices `rows*16` bytes apart.
__host__ __device__ __forceinline__ uint32_t kmajor_offset(int rows, int row, int k) {
  return static_cast<uint32_t>((k >> 3) * (rows * 16) + (row >> 3) * 128 + (row & 7) * 16 + (k & 7) * 2);
}

// Host: keep the CTAs that can share one SM within the SM's 512 tensor-memory columns.
// tcgen05.alloc has no time limit: a CTA whose request does not fit waits until a co-resident CTA
// frees its columns. CTAs of one launch wait on one another (cluster barriers, exchange), so a CTA
// stuck in the allocation behind a CTA of another group could keep both groups from ever finishing.
// The launchers therefore ask the occupancy calculator how many CTAs of the kernel fit one SM with
// the chosen shared-memory size and, where that many would ask for more than 512 columns together,
// enlarge the dynamic shared memory until no more than 512 / tmem_cols CTAs fit. Returns 0, a
// cudaError_t, or -3 when the budget cannot be met. Sets the kernel's dynamic shared-memory limit.
template <typename Kern>
inline int fit_tmem_budget(Kern kern, int threads, uint32_t tmem_cols, int* smem) {
  const int allowed = tmem_cols >= 512u ? 1 : static_cast<int>(512u / tmem_cols);
  for (int attempt = 0; attempt < 2; ++attempt) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, *smem);
    if (e != cudaSuccess) return static_cast<int>(e);
    int blocks = 0;
    e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&blocks, kern, threads, static_cast<size_t>(*smem));
    if (e != cudaSuccess) return static_cast<int>(e);
    if (blocks <= allowed) return 0;
    if (attempt == 1) return -3;
    int dev = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&per_sm, cudaDevAttrMaxSharedMemoryPerMultiprocessor, dev) != cudaSuccess)
      return -3;
    const int need = (per_sm / (allowed + 1) + 128) & ~127;  // allowed + 1 CTAs of this size exceed the SM
    if (need > 227 * 1024) return -3;
    if (need > *smem) *smem = need;
  }
  return -3;
}
inline uint32_t tmem_cols_pow2(int needed, uint32_t minimum) {
  uint32_t c = minimum;
  while (c < static_cast<uint32_t>(needed)) c <<= 1;
  return c;
}

// Host: build a tiled tensor map (no swizzle, no interleave). dims/box innermost first.
// `stride_dims` (optional): extents the strides are computed from when the described tensor is a window of a
// larger dense array (e.g. the first T of T + 1 time slots).
int make_tensor_map(CUtensorMap* map, const void* base, int elem_bytes, int rank, const uint64_t* dims,
                    const uint32_t* box, bool swizzle128 = false, const uint64_t* stride_dims = nullptr);

}  // namespace frnn
