// Shared declarations of the row-sharded wide-head kernels: ONE head whose recurrent matrix is split over
// the GPUs of a node (rank r owns output rows [r*Dl, (r+1)*Dl) of every gate in the forward pass and the
// same units' columns in the backward pass), with the per-step operand exchanged by peer stores.
//
// Exchange protocol (forward: round_bf16(h_t); backward: round_bf16(dG_t)):
//   * every rank holds a full-width history buffer of the operand (forward: [B][T+1][D] bf16, slot 0 =
//     round(h_init), slot t+1 = round(h_t); backward: [B][T][GR*D] bf16). It doubles as an operand of the
//     dR contraction afterwards, so nothing extra is stored.
//   * the call fills the buffer with all-ones bytes; an owner stores each 16-byte packet (eight units of
//     one batch row) into the buffer of EVERY rank (its own included) with system-scope stores; a consumer
//     polls its OWN buffer until no 32-bit word of the packet shows the fill pattern (a pair of all-ones
//     NaNs never comes out of the rounding, see xg_clean). Every slot is written once per call, so there
//     is no slot reuse, no refill and no fence on the critical path.
//   * before its first remote store a kernel waits until every peer has announced (ready flag = epoch of
//     the call, written by the peer's kernel when it starts, i.e. after the peer's fill in stream order)
//     that the peer's buffer has been filled. Epochs must grow from call to call.
//   * every wait is bounded (wait_limit_ns); a wait that runs out sets err[0..2] on the local rank and the
//     kernel leaves in an orderly way. Peers then run into their own limits.
//
// With ranks_here == P all ranks run as ONE cooperative launch on one GPU over slices of full-width
// tensors (x offset rank * Dl): the form in which the multi-rank index arithmetic is tested on a single
// GPU, since separately launched kernels that wait on one another must never share a device.
//
// Reference counterparts: flashrnn/flashrnn2/multi_gpu.py:87-297 (forward, peer stores + counters
// :224-238, bounded spin :30-32,62-73), flashrnn/flashrnn2/hybrid_bw2d.cu:507-552,645-661 (backward).
#pragma once

#include "frnn_common.cuh"

namespace frnn {

constexpr int kMgMaxRanks = 8;
constexpr int kMgBT = 32;          // UMMA N: one batch tile of up to 32 rows per launch
constexpr int kMgSubK = 512;       // contraction sub-chunk staged in shared memory at a time
constexpr int kMgRingK = 64;       // k per stage of the shared-memory ring of the weight operand
constexpr int kMgRingBytes = 128 * kMgRingK * 2;
constexpr int kMgMaxRing = 12;
constexpr int kMgMaxKtmem = 960;   // 32 accumulator columns + k_tmem / 2 weight columns <= 512

struct MgFwdParams {
  const __nv_bfloat16* R;   // rows of R owned here: [GR][ldr][D] (ldr = rows per gate in the buffer)
  const float* bias;        // [GB][ldx]
  const float* initial;     // [S][B][ldx]
  float* history;           // [S][B][T][ldx]
  float* carry;             // [S][B][ldx]
  void* cache;              // [B][T][GC][ldx] (fp16 or fp32 elements, CellTraits::CES) or null (inference)
  __nv_bfloat16* hbf[kMgMaxRanks];  // every rank's [B][T+1][D] history of round_bf16(h)
  int* ready[kMgMaxRanks];          // every rank's int[kMgMaxRanks] ready flags
  int* err;
  int B, T, D, Dl, ldx;     // ldx: row length of the local tensors (Dl, or D when all ranks share one launch)
  int P, rank0, ranks_here, x_rank_stride;
  int k_tmem, n_ring, ring_stages, resident;
  int epoch;
  int slstm_zero_first;
  unsigned long long wait_limit_ns;
};

struct MgBwdParams {
  const __nv_bfloat16* Rc;  // columns of R owned here: [GR][D][ldx]
  const void* cache;        // [B][T][GC][ldx] (fp16 or fp32 elements, CellTraits::CES)
  const float* history;     // [S][B][T][ldx]
  const float* initial;     // [S][B][ldx]
  const float* d_history;   // [S][B][T][ldx]
  const float* d_carry;     // [S][B][ldx]
  void* dwx;                // [B][T][GW][ldx] in the Wx dtype
  float* d_initial;         // [S][B][ldx]
  float* db_part;           // [KS][GB][ldx]
  __nv_bfloat16* dgr[kMgMaxRanks];  // every rank's [B][T][GR][D] history of round_bf16(dG)
  int* ready[kMgMaxRanks];
  int* err;
  int B, T, D, Dl, ldx;
  int P, rank0, ranks_here, x_rank_stride;
  int k_tmem, n_ring, ring_stages, resident;
  int epoch;
  int slstm_zero_first;
  unsigned long long wait_limit_ns;
};

__device__ __forceinline__ void mg_report(int* err, int code, int detail) {
  if (atomicCAS(err, 0, code) == 0) {
    err[1] = detail;
    err[2] = static_cast<int>(blockIdx.x);
  }
  __threadfence();
}

// Announce that this rank's exchange buffer has been filled (the kernel runs after the fill in stream
// order) and wait until every peer has announced the same for the call `epoch`. One thread per CTA.
__device__ __forceinline__ bool mg_handshake(int* const* ready, int rank, int P, int epoch, bool announce,
                                             unsigned long long limit_ns, const volatile int* abort_flag) {
  if (announce) {
    for (int q = 0; q < P; ++q) st_release_sys_s32(ready[q] + rank, epoch);
  }
  const uint64_t t0 = global_timer_ns();
  for (int q = 0; q < P; ++q) {
    uint32_t spins = 0;
    while (ld_acquire_sys_s32(ready[rank] + q) < epoch) {
      if ((++spins & 63u) == 0u) {
        if (*abort_flag != 0 || global_timer_ns() - t0 > limit_ns) return false;
      }
    }
  }
  return true;
}

// Shared-memory bytes of one staged sub-chunk of the exchanged operand: blocks of [32 batch rows x 64 k] bf16,
// every row 128 bytes, K-major with the 128-byte swizzle (the layout TMA would write and tcgen05 reads).
__host__ __device__ inline int mg_operand_bytes(int sub_k) { return ((sub_k + 63) / 64) * 4096; }

// Copy `sub_k` (<= 512) consecutive k of the operand of up to 32 batch rows from this rank's history buffer into a
// staged sub-chunk, waiting for every 16-byte packet to arrive (no word shows the fill pattern). `src` points at
// (batch row 0, first k of the sub-chunk), rows are `row_stride` elements apart. Eight neighbouring lanes read one
// 128-byte piece of a row (coalesced) and store it with the swizzle (no bank conflicts). Called by the 128 epilogue
// threads; returns false if the bounded wait ran out (the caller reports it).
__device__ __forceinline__ bool mg_fetch_subchunk(const __nv_bfloat16* src, size_t row_stride, uint8_t* dst, int sub_k,
                                                  int B, int warp, int lane, unsigned long long limit_ns,
                                                  const volatile int* abort_flag) {
  constexpr int NPK = 2 * (kMgSubK / 64);  // packets per thread: two rows of every 64-k block
  const int chunk = lane & 7, r4 = lane >> 3;
  const int n_blocks = (sub_k + 63) / 64;
  uint32_t pend = 0;
#pragma unroll
  for (int j = 0; j < NPK; ++j) {
    const int blk = j >> 1, row = 4 * (warp + 4 * (j & 1)) + r4;
    if (blk < n_blocks && blk * 64 + chunk * 8 < sub_k && row < B) pend |= 1u << j;
  }
  uint64_t t0 = 0;
  uint32_t rounds = 0;
  bool ok = true;
  while (pend != 0u) {
    uint4 v[NPK];
#pragma unroll
    for (int j = 0; j < NPK; ++j) {
      if ((pend >> j) & 1u) {
        const int blk = j >> 1, row = 4 * (warp + 4 * (j & 1)) + r4;
        v[j] = ld_relaxed_sys_v4(src + static_cast<size_t>(row) * row_stride + blk * 64 + chunk * 8);
      }
    }
#pragma unroll
    for (int j = 0; j < NPK; ++j) {
      if (((pend >> j) & 1u) && xg_arrived(v[j])) {
        const int blk = j >> 1, row = 4 * (warp + 4 * (j & 1)) + r4;
        *reinterpret_cast<uint4*>(dst + blk * 4096 + row * 128 + ((chunk ^ (row & 7)) << 4)) = v[j];
        pend &= ~(1u << j);
      }
    }
    if (pend != 0u && (++rounds & 15u) == 0u) {  // the global timer is slow to read
      const uint64_t now = global_timer_ns();
      if (t0 == 0) t0 = now;
      if (*abort_flag != 0 || now - t0 > limit_ns) {
        ok = false;
        break;
      }
    }
  }
  return ok;
}

}  // namespace frnn
