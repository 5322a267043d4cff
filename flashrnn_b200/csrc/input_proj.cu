// Input projection in front of the recurrence: Wx[m, j] = sum_i x[m, i] * W[j, i] (+ bias[j]), m = (b, t),
// j = (gate, head, unit), written directly in the layout and dtype the recurrent kernels stream by TMA
// (Wx[B,T,GW,N,D] is the row-major [B*T][GW*N*D] matrix). bf16 operands, fp32 accumulation in tensor memory.
//
// Persistent kernel, one CTA per SM, each walking 128 x NP output tiles (NP = 256, 128 or 64 columns; tiles that share
// rows of x are neighbours in the walk, so x comes from HBM once and W stays in L2): warp 0 feeds a 4-stage ring of
// 128-byte-swizzled K-major stages by TMA (x rows and W rows, 64 input features per stage), warp 1 issues tcgen05.mma
// (both operands from shared memory) into one of TWO accumulators in tensor memory, warps 2-5 convert the other one
// into swizzled 32-row x 128-byte staging buffers that TMA stores write out as whole lines, so the epilogue of a tile
// runs under the contraction of the next. Rows and
// features past the matrix edges are filled with zeros by TMA.
//
// The reference leaves this GEMM to the caller (README.md:16) and times it as the "-withlinear" variant of its
// benchmark (flashrnn/speed_experiments/kernel_speed_benchmark.py:388-408, a torch.nn.Linear in front of the kernel).
#include "frnn_common.cuh"

namespace frnn {

namespace {

constexpr int kProjThreads = 192;
constexpr int kProjStages = 4;
constexpr int kProjKC = 64;  // input features per stage (128 bytes of bf16: one swizzle row)

struct ProjParams {
  void* out;          // [M][J] bf16 or fp32
  const float* bias;  // [J] or null
  int* err;
  long long M, n_tiles;
  int J, I, NP, n_jt;
  int out_bf16;
};

__global__ void __launch_bounds__(kProjThreads, 1)
input_proj_kernel(const ProjParams p, const __grid_constant__ CUtensorMap x_map, const __grid_constant__ CUtensorMap w_map,
                  const __grid_constant__ CUtensorMap out_map) {
  extern __shared__ uint8_t smem_raw[];
  __shared__ __align__(8) uint64_t s_full[kProjStages];
  __shared__ __align__(8) uint64_t s_empty[kProjStages];
  __shared__ __align__(8) uint64_t s_acc_full[2];
  __shared__ __align__(8) uint64_t s_acc_empty[2];
  __shared__ __align__(8) uint64_t s_done;
  __shared__ uint32_t s_tmem_base;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NP = p.NP;
  const int n_chunks = (p.I + kProjKC - 1) / kProjKC;
  const uint32_t stage_bytes = 16384u + static_cast<uint32_t>(NP) * 128u;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint32_t tmem_cols = 32;
  while (tmem_cols < 2u * static_cast<uint32_t>(NP)) tmem_cols <<= 1;
  const volatile int* abort_flag = p.err;
  constexpr uint64_t kLimit = 2000000000ull;

  if (tid == 0) {
    for (int s = 0; s < kProjStages; ++s) {
      mbar_init(smem_u32(&s_full[s]), 1);
      mbar_init(smem_u32(&s_empty[s]), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(smem_u32(&s_acc_full[a]), 1);
      mbar_init(smem_u32(&s_acc_empty[a]), 4);  // one arrival per epilogue warp
    }
    mbar_init(smem_u32(&s_done), 1);
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
      tma_prefetch_desc(&x_map);
      tma_prefetch_desc(&w_map);
      tma_prefetch_desc(&out_map);
      uint32_t s = 0, round = 0;  // ring stage and how often the ring has wrapped
      bool dead = false;
      for (long long tile = blockIdx.x; tile < p.n_tiles && !dead; tile += gridDim.x) {
        const int m0 = static_cast<int>(tile / p.n_jt) * 128, j0 = static_cast<int>(tile % p.n_jt) * NP;
        for (int i = 0; i < n_chunks; ++i) {
          if (round > 0 && !mbar_wait_bounded<false, true>(smem_u32(&s_empty[s]), (round - 1) & 1, kLimit, abort_flag)) {
            atomicCAS(p.err, 0, kErrWaitEmpty);
            dead = true;
            break;
          }
          const uint32_t bar = smem_u32(&s_full[s]);
          const uint32_t sa = base + s * stage_bytes, sb = sa + 16384u;
          mbar_arrive_expect_tx(bar, stage_bytes);
          tma_load_3d(sa, &x_map, bar, i * kProjKC, m0, 0);
          tma_load_3d(sb, &w_map, bar, i * kProjKC, j0, 0);
          if (++s == kProjStages) { s = 0; ++round; }
        }
      }
      if (dead) {  // give the copies in flight time to land before the CTA leaves
        const uint64_t t0 = global_timer_ns();
        while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t idesc = umma_idesc_bf16(128, NP, false, false);
      uint32_t s = 0, round = 0, li = 0;
      bool dead = false;
      for (long long tile = blockIdx.x; tile < p.n_tiles && !dead; tile += gridDim.x, ++li) {
        const uint32_t a = li & 1u;
        if (li >= 2 && !mbar_wait_bounded<false, true>(smem_u32(&s_acc_empty[a]), ((li >> 1) - 1) & 1, kLimit, abort_flag)) {
          atomicCAS(p.err, 0, kErrWaitMma);
          break;
        }
        tc_fence_after_sync();
        const uint32_t d = tbase + a * static_cast<uint32_t>(NP);
        for (int i = 0; i < n_chunks; ++i) {
          if (!mbar_wait_bounded<false, true>(smem_u32(&s_full[s]), round & 1, kLimit, abort_flag)) {
            atomicCAS(p.err, 0, kErrWaitWx);
            dead = true;
            break;
          }
          tc_fence_after_sync();
          uint64_t ad = umma_smem_desc_k_sw128(base + s * stage_bytes);
          uint64_t bd = umma_smem_desc_k_sw128(base + s * stage_bytes + 16384u);
#pragma unroll
          for (int kk = 0; kk < kProjKC / 16; ++kk) {
            umma_bf16_ss(d, ad, bd, idesc, (i > 0 || kk > 0) ? 1u : 0u);
            ad += 2;  // 16 features = 32 bytes inside the swizzled 128-byte row
            bd += 2;
          }
          umma_commit(smem_u32(&s_empty[s]));
          if (++s == kProjStages) { s = 0; ++round; }
        }
        if (!dead) umma_commit(smem_u32(&s_acc_full[a]));
      }
      // one commit covers every MMA issued so far; the issuing thread waits for it itself so that tensor and shared
      // memory are never released under a running MMA (also after a failed wait)
      umma_commit(smem_u32(&s_done));
      mbar_wait_bounded<false, true>(smem_u32(&s_done), 0, kLimit, nullptr);
    }
  } else {
    const int q = warp & 3;  // TMEM lane quarter this warp may read
    // Each warp turns its 32 rows into 128-byte row pieces (64 bf16 or 32 fp32 columns) in a swizzled staging buffer
    // of its own and lets TMA write them: whole lines per row instead of 32 scattered 16-byte stores per instruction.
    const int CW = p.out_bf16 ? 64 : 32;
    const uint32_t stg = base + kProjStages * stage_bytes + static_cast<uint32_t>(q) * 8192u;
    const uint32_t my_row = static_cast<uint32_t>(lane) * 128u, sw = static_cast<uint32_t>(lane & 7);
    uint32_t li = 0, piece = 0;
    for (long long tile = blockIdx.x; tile < p.n_tiles; tile += gridDim.x, ++li) {
      const uint32_t a = li & 1u;
      const long long mw = (tile / p.n_jt) * 128 + 32 * q;  // first row of this warp
      const int j0 = static_cast<int>(tile % p.n_jt) * NP;
      bool have = mbar_wait_bounded<false, true>(smem_u32(&s_acc_full[a]), (li >> 1) & 1, kLimit, abort_flag);
      have = __all_sync(0xffffffffu, have);
      if (!have) {
        if (lane == 0) atomicCAS(p.err, 0, kErrWaitMma);
        break;
      }
      tc_fence_after_sync();
      for (int c0 = 0; c0 < NP; c0 += CW, ++piece) {
        uint32_t r0[32], r1[32];
        tmem_ld_x32(tmem_addr(tbase, 32 * q, a * NP + c0), r0);
        if (p.out_bf16) tmem_ld_x32(tmem_addr(tbase, 32 * q, a * NP + c0 + 32), r1);
        tmem_ld_wait();
        if (c0 + CW >= NP) {  // the accumulator is in registers: hand it back to the MMA warp
          tc_fence_before_sync();
          __syncwarp();
          if (lane == 0) mbar_arrive(smem_u32(&s_acc_empty[a]));
        }
        if (mw >= p.M) continue;  // warp-uniform: all 32 rows lie past the matrix
        const uint32_t buf = stg + (piece & 1u) * 4096u;
        if (lane == 0) tma_store_wait_read<1>();  // the store that read this buffer two pieces ago is done with it
        __syncwarp();
        if (p.bias != nullptr) {
#pragma unroll
          for (int k = 0; k < 32; k += 4) {
            const float4 bv = __ldg(reinterpret_cast<const float4*>(p.bias + j0 + c0 + k));
            r0[k] = __float_as_uint(__uint_as_float(r0[k]) + bv.x);
            r0[k + 1] = __float_as_uint(__uint_as_float(r0[k + 1]) + bv.y);
            r0[k + 2] = __float_as_uint(__uint_as_float(r0[k + 2]) + bv.z);
            r0[k + 3] = __float_as_uint(__uint_as_float(r0[k + 3]) + bv.w);
          }
          if (p.out_bf16) {
#pragma unroll
            for (int k = 0; k < 32; k += 4) {
              const float4 bv = __ldg(reinterpret_cast<const float4*>(p.bias + j0 + c0 + 32 + k));
              r1[k] = __float_as_uint(__uint_as_float(r1[k]) + bv.x);
              r1[k + 1] = __float_as_uint(__uint_as_float(r1[k + 1]) + bv.y);
              r1[k + 2] = __float_as_uint(__uint_as_float(r1[k + 2]) + bv.z);
              r1[k + 3] = __float_as_uint(__uint_as_float(r1[k + 3]) + bv.w);
            }
          }
        }
        auto put = [&](uint32_t k16, uint32_t w0, uint32_t w1, uint32_t w2, uint32_t w3) {
          asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};"
                       :: "r"(buf + my_row + ((k16 ^ sw) << 4)), "r"(w0), "r"(w1), "r"(w2), "r"(w3) : "memory");
        };
        if (p.out_bf16) {
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            put(k, pack_bf16x2(__uint_as_float(r0[8 * k]), __uint_as_float(r0[8 * k + 1])),
                pack_bf16x2(__uint_as_float(r0[8 * k + 2]), __uint_as_float(r0[8 * k + 3])),
                pack_bf16x2(__uint_as_float(r0[8 * k + 4]), __uint_as_float(r0[8 * k + 5])),
                pack_bf16x2(__uint_as_float(r0[8 * k + 6]), __uint_as_float(r0[8 * k + 7])));
            put(4 + k, pack_bf16x2(__uint_as_float(r1[8 * k]), __uint_as_float(r1[8 * k + 1])),
                pack_bf16x2(__uint_as_float(r1[8 * k + 2]), __uint_as_float(r1[8 * k + 3])),
                pack_bf16x2(__uint_as_float(r1[8 * k + 4]), __uint_as_float(r1[8 * k + 5])),
                pack_bf16x2(__uint_as_float(r1[8 * k + 6]), __uint_as_float(r1[8 * k + 7])));
          }
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) put(k, r0[4 * k], r0[4 * k + 1], r0[4 * k + 2], r0[4 * k + 3]);
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          tma_store_2d(&out_map, buf, j0 + c0, static_cast<int>(mw));
          tma_store_commit();
        }
      }
    }
    if (lane == 0) tma_store_wait<0>();  // every store has left shared memory and reached global memory
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) tmem_dealloc(tbase, tmem_cols);
}

}  // namespace

// x [M][I] bf16, W [J][I] bf16, bias [J] fp32 or null -> out [M][J] (bf16 or fp32). I % 8 == 0, J % 64 == 0.
int input_proj_launch(const void* x, const void* w, const float* bias, void* out, int out_bf16, long long M, int J, int I,
                      int* err, cudaStream_t s) {
  if (M < 1 || J < 64 || J % 64 != 0 || I < 8 || I % 8 != 0) return -2;
  if (((reinterpret_cast<uintptr_t>(out) | reinterpret_cast<uintptr_t>(bias)) & 15u) != 0) return -2;  // vector access
  const int np = J % 256 == 0 ? 256 : (J % 128 == 0 ? 128 : 64);
  ProjParams p{};
  p.out = out; p.bias = bias; p.err = err;
  p.M = M; p.J = J; p.I = I; p.NP = np; p.out_bf16 = out_bf16;
  const long long mt = (M + 127) / 128;
  if (mt > 0x7fffffffLL) return -2;
  p.n_jt = J / np;
  p.n_tiles = mt * p.n_jt;
  CUtensorMap x_map, w_map, out_map;
  const uint64_t xdims[3] = {static_cast<uint64_t>(I), static_cast<uint64_t>(M), 1u};
  const uint32_t xbox[3] = {static_cast<uint32_t>(kProjKC), 128u, 1u};
  const uint64_t wdims[3] = {static_cast<uint64_t>(I), static_cast<uint64_t>(J), 1u};
  const uint32_t wbox[3] = {static_cast<uint32_t>(kProjKC), static_cast<uint32_t>(np), 1u};
  if (make_tensor_map(&x_map, x, 2, 3, xdims, xbox, true) != 0) return -4;
  if (make_tensor_map(&w_map, w, 2, 3, wdims, wbox, true) != 0) return -4;
  // the output as [M][J]; one store = 32 rows x 128 bytes out of a swizzled staging buffer
  const uint64_t odims[2] = {static_cast<uint64_t>(J), static_cast<uint64_t>(M)};
  const uint32_t obox[2] = {out_bf16 ? 64u : 32u, 32u};
  if (make_tensor_map(&out_map, out, out_bf16 ? 2 : 4, 2, odims, obox, true) != 0) return -4;
  const int smem = kProjStages * (16384 + np * 128) + 4 * 8192 + 1024;  // ring + two staging buffers per epilogue warp
  cudaError_t e = cudaFuncSetAttribute(input_proj_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return static_cast<int>(e);
  int dev = 0, sms = 0;
  e = cudaGetDevice(&dev);
  if (e == cudaSuccess) e = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  if (e != cudaSuccess) return static_cast<int>(e);
  const unsigned grid = static_cast<unsigned>(p.n_tiles < sms ? p.n_tiles : sms);  // persistent: one CTA per SM
  input_proj_kernel<<<grid, kProjThreads, smem, s>>>(p, x_map, w_map, out_map);
  return static_cast<int>(cudaGetLastError());
}

}  // namespace frnn
