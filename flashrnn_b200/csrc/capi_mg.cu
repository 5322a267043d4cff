// extern "C" boundary of the row-sharded wide-head path: plan, forward, column gather, backward, dR/db, and the
// helpers that make a device buffer reachable from the other processes of the node (CUDA IPC).
#include "../../include/flashrnn_b200.h"

#include <cstring>

#include "recurrent_mg_common.cuh"

namespace frnn {

int forward_mg_dispatch(int cell, const MgFwdParams& p, const void* wx, int wx_bf16, int ksplit, cudaStream_t s,
                        int* capacity_only);
int forward_mg_fixed_smem(int cell, int ksplit, int D, int wx_bf16);
int backward_mg_dispatch(int cell, const MgBwdParams& p, int wx_bf16, int ksplit, cudaStream_t s, int* capacity_only);
int backward_mg_fixed_smem(int cell, int ksplit, int D, int wx_bf16);
int gather_columns_launch(const void* const* rows, void* cols, int gr, int D, int Dl, int P, int rank0, int ranks_here,
                          cudaStream_t s);
int wgrad_launch_rows(int gr, int gb, const __nv_bfloat16* dgr, const __nv_bfloat16* hbf, const float* db_part, int n_parts,
                      float* dR, float* db, int* err, int B, int T, int D, int Dm, int m_off, int out_rows, int ldb, int x0,
                      cudaStream_t s);

namespace {

struct Counts { int gr, gw, gb, s, gc; };
bool counts(int cell, Counts* c) {
  switch (cell) {
    case kLSTM: *c = {4, 4, 4, 2, 4}; return true;
    case kSLSTM: *c = {4, 4, 4, 4, 4}; return true;
    case kGRU: *c = {3, 3, 4, 1, 4}; return true;
    case kElman: *c = {1, 1, 1, 1, 0}; return true;
    default: return false;
  }
}

int device_sms() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      n <= 0) {
    cudaGetLastError();
    return 148;
  }
  return n;
}

// How a [128 x Kc] block of the weight operand is kept on the SM: k_tmem columns in tensor memory, n_ring stages of
// 64 columns in shared memory, resident when they all fit beside the kernel's other shared memory.
struct Residency { int k_tmem, n_ring, stages, resident, ok; };
Residency residency(int Kc, int fixed_smem, int k_tmem_max, int ring_stages_max) {
  Residency r{};
  const int sub = Kc < kMgSubK ? Kc : kMgSubK;
  if (Kc % 16 != 0 || Kc % sub != 0) return r;
  int cap = k_tmem_max > 0 && k_tmem_max < kMgMaxKtmem ? k_tmem_max / 64 * 64 : kMgMaxKtmem;
  if (Kc <= cap) {
    r.k_tmem = Kc;
  } else {
    if (Kc % kMgRingK != 0) return r;
    r.k_tmem = cap / kMgRingK * kMgRingK;
  }
  r.n_ring = (Kc - r.k_tmem) / kMgRingK;
  int room = (227 * 1024 - fixed_smem) / kMgRingBytes;
  if (room > kMgMaxRing) room = kMgMaxRing;
  if (ring_stages_max > 0 && room > ring_stages_max) room = ring_stages_max;
  if (r.n_ring == 0) {
    r.stages = 0; r.resident = 1; r.ok = fixed_smem <= 227 * 1024;
    return r;
  }
  if (r.n_ring <= room) {
    r.stages = r.n_ring; r.resident = 1; r.ok = 1;
    return r;
  }
  r.stages = room; r.resident = 0; r.ok = room >= 2;
  return r;
}

int capacity_fwd(int cell, int ks, int D, int Dl, int wx_bf16, const Residency& r) {
  MgFwdParams p{};
  p.D = D; p.Dl = Dl; p.ldx = Dl; p.B = 1; p.T = 1; p.P = 1; p.ranks_here = 1;
  p.k_tmem = r.k_tmem; p.n_ring = r.n_ring; p.ring_stages = r.stages; p.resident = r.resident;
  int cap = 0;
  if (forward_mg_dispatch(cell, p, nullptr, wx_bf16, ks, nullptr, &cap) != 0 || cap <= 0) {
    cudaGetLastError();
    cap = device_sms() / ks * ks;  // no device visible: assume every SM can take part
  }
  return cap;
}
int capacity_bwd(int cell, int ks, int D, int Dl, int wx_bf16, const Residency& r) {
  MgBwdParams p{};
  p.D = D; p.Dl = Dl; p.ldx = Dl; p.B = 1; p.T = 1; p.P = 1; p.ranks_here = 1;
  p.k_tmem = r.k_tmem; p.n_ring = r.n_ring; p.ring_stages = r.stages; p.resident = r.resident;
  int cap = 0;
  if (backward_mg_dispatch(cell, p, wx_bf16, ks, nullptr, &cap) != 0 || cap <= 0) {
    cudaGetLastError();
    cap = device_sms() / ks * ks;
  }
  return cap;
}

bool shard_ok(const frnn_b200_mg_shard_t* sh, int D) {
  return sh != nullptr && sh->P >= 1 && sh->P <= kMgMaxRanks && D % sh->P == 0 && (sh->ranks_here == 1 || sh->ranks_here == sh->P) &&
         sh->rank >= 0 && sh->rank + sh->ranks_here <= sh->P;
}

}  // namespace

}  // namespace frnn

using namespace frnn;

extern "C" int frnn_b200_mg_plan(int cell, int B, int T, int D, int wx_bf16, const frnn_b200_mg_shard_t* sh,
                                 frnn_b200_mg_plan_t* out) {
  if (out == nullptr) return -5;
  Counts c;
  if (!counts(cell, &c)) return -1;
  if (B < 1 || T < 1 || D < 1 || !shard_ok(sh, D)) return -5;
  *out = frnn_b200_mg_plan_t{};
  const int P = sh->P, Dl = D / P, here = sh->ranks_here;
  out->local_width = Dl;
  out->hbf_bytes = static_cast<int64_t>(B) * (T + 1) * D * 2;
  out->dgr_bytes = static_cast<int64_t>(B) * T * c.gr * D * 2;
  const int64_t lw = here == P ? D : Dl;  // row length of the local tensors of one launch
  out->cache_bytes = static_cast<int64_t>(B) * T * c.gc * lw * ((cell == kLSTM || cell == kGRU) ? 2 : 4);  // CellTraits::CES
  out->r_cols_bytes = static_cast<int64_t>(c.gr) * D * lw * 2;
  if (B > kMgBT || D % 256 != 0 || Dl % 128 != 0) return 0;  // supported stays 0
  // forward: the widest split of the contraction whose CTAs are all resident (shortest tensor-core chain per step)
  for (int ks = 16; ks >= 1 && out->fwd_ksplit == 0; ks /= 2) {
    if (D % ks != 0) continue;
    const Residency r = residency(D / ks, forward_mg_fixed_smem(cell, ks, D, wx_bf16), sh->k_tmem_max, sh->ring_stages_max);
    if (!r.ok) continue;
    const int ctas = here * (Dl / 32) * ks;
    if (ctas > capacity_fwd(cell, ks, D, Dl, wx_bf16, r)) continue;
    out->fwd_ksplit = ks; out->fwd_ctas = ctas;
    out->fwd_k_tmem = r.k_tmem; out->fwd_ring_chunks = r.n_ring; out->fwd_ring_stages = r.stages; out->fwd_resident = r.resident;
  }
  const int K = c.gr * D;
  for (int ks = 16; ks >= 4 && out->bwd_ksplit == 0; ks /= 2) {
    if (K % ks != 0) continue;
    const Residency r = residency(K / ks, backward_mg_fixed_smem(cell, ks, D, wx_bf16), sh->k_tmem_max, sh->ring_stages_max);
    if (!r.ok) continue;
    const int ctas = here * (Dl / 128) * ks;
    if (ctas > capacity_bwd(cell, ks, D, Dl, wx_bf16, r)) continue;
    out->bwd_ksplit = ks; out->bwd_ctas = ctas;
    out->bwd_k_tmem = r.k_tmem; out->bwd_ring_chunks = r.n_ring; out->bwd_ring_stages = r.stages; out->bwd_resident = r.resident;
  }
  out->dbpart_bytes = static_cast<int64_t>(out->bwd_ksplit) * c.gb * lw * 4;
  out->supported = out->fwd_ksplit > 0 && out->bwd_ksplit > 0;
  return 0;
}

extern "C" int frnn_b200_mg_capacity(int cell, int forward, int ksplit, int D, int P, int wx_bf16) {
  Counts c;
  if (!counts(cell, &c) || P < 1 || D % P != 0) return -5;
  const int Kc = (forward ? D : c.gr * D) / ksplit;
  const Residency r = residency(Kc, forward ? forward_mg_fixed_smem(cell, ksplit, D, wx_bf16) : backward_mg_fixed_smem(cell, ksplit, D, wx_bf16), 0, 0);
  if (!r.ok) return 0;
  return forward ? capacity_fwd(cell, ksplit, D, D / P, wx_bf16, r) : capacity_bwd(cell, ksplit, D, D / P, wx_bf16, r);
}

extern "C" int frnn_b200_mg_forward(int cell, const void* wx, int wx_bf16, const void* r_rows, const float* bias,
                                    const float* initial, float* history, float* carry, void* cache,
                                    const frnn_b200_mg_shard_t* sh, int B, int T, int D, int slstm_zero_first,
                                    int wait_limit_ms, int* err, void* stream) {
  frnn_b200_mg_plan_t plan;
  const int rc = frnn_b200_mg_plan(cell, B, T, D, wx_bf16, sh, &plan);
  if (rc != 0) return rc;
  if (plan.fwd_ksplit == 0) return -2;
  if (!wx || !r_rows || !bias || !initial || !history || !carry || !err) return -5;
  const int P = sh->P, Dl = D / P, here = sh->ranks_here;
  MgFwdParams p{};
  p.R = static_cast<const __nv_bfloat16*>(r_rows);
  p.bias = bias; p.initial = initial; p.history = history; p.carry = carry; p.cache = cache;
  for (int q = 0; q < P; ++q) {
    if (sh->buffers[q] == nullptr || (here < P && sh->ready[q] == nullptr)) return -5;
    p.hbf[q] = static_cast<__nv_bfloat16*>(sh->buffers[q]);
    p.ready[q] = sh->ready[q];
  }
  p.err = err;
  p.B = B; p.T = T; p.D = D; p.Dl = Dl;
  p.ldx = here == P ? D : Dl;
  p.P = P; p.rank0 = sh->rank; p.ranks_here = here; p.x_rank_stride = here == P && P > 1 ? Dl : 0;
  p.k_tmem = plan.fwd_k_tmem; p.n_ring = plan.fwd_ring_chunks; p.ring_stages = plan.fwd_ring_stages; p.resident = plan.fwd_resident;
  p.epoch = sh->epoch;
  p.slstm_zero_first = slstm_zero_first;
  p.wait_limit_ns = (wait_limit_ms > 0 ? static_cast<unsigned long long>(wait_limit_ms) : 10000ull) * 1000000ull;
  // every word of the history buffers owned by this launch starts as "not yet written"
  for (int q = sh->rank; q < sh->rank + here; ++q) {
    const cudaError_t me = cudaMemsetAsync(sh->buffers[q], 0xff, static_cast<size_t>(plan.hbf_bytes), static_cast<cudaStream_t>(stream));
    if (me != cudaSuccess) return static_cast<int>(me);
  }
  return forward_mg_dispatch(cell, p, wx, wx_bf16, plan.fwd_ksplit, static_cast<cudaStream_t>(stream), nullptr);
}

extern "C" int frnn_b200_mg_gather_columns(int cell, const void* const* r_rows_all, void* r_cols,
                                           const frnn_b200_mg_shard_t* sh, int D, void* stream) {
  Counts c;
  if (!counts(cell, &c)) return -1;
  if (!shard_ok(sh, D) || !r_rows_all || !r_cols) return -5;
  for (int q = 0; q < sh->P; ++q)
    if (r_rows_all[q] == nullptr) return -5;
  if ((D / sh->P) % 8 != 0) return -2;
  return gather_columns_launch(r_rows_all, r_cols, c.gr, D, D / sh->P, sh->P, sh->rank, sh->ranks_here,
                               static_cast<cudaStream_t>(stream));
}

extern "C" int frnn_b200_mg_backward(int cell, const void* cache, const float* history, const float* initial,
                                     const void* r_cols, const float* d_history, const float* d_carry, void* dwx,
                                     int wx_bf16, float* d_initial, float* db_part, const frnn_b200_mg_shard_t* sh, int B,
                                     int T, int D, int slstm_zero_first, int wait_limit_ms, int* err, void* stream) {
  frnn_b200_mg_plan_t plan;
  const int rc = frnn_b200_mg_plan(cell, B, T, D, wx_bf16, sh, &plan);
  if (rc != 0) return rc;
  if (plan.bwd_ksplit == 0) return -2;
  Counts c;
  counts(cell, &c);
  if ((!cache && c.gc > 0) || !history || !initial || !r_cols || !d_history || !d_carry || !dwx || !d_initial || !db_part || !err)
    return -5;
  const int P = sh->P, Dl = D / P, here = sh->ranks_here;
  MgBwdParams p{};
  p.Rc = static_cast<const __nv_bfloat16*>(r_cols);
  p.cache = cache; p.history = history; p.initial = initial; p.d_history = d_history; p.d_carry = d_carry;
  p.dwx = dwx; p.d_initial = d_initial; p.db_part = db_part;
  for (int q = 0; q < P; ++q) {
    if (sh->buffers[q] == nullptr || (here < P && sh->ready[q] == nullptr)) return -5;
    p.dgr[q] = static_cast<__nv_bfloat16*>(sh->buffers[q]);
    p.ready[q] = sh->ready[q];
  }
  p.err = err;
  p.B = B; p.T = T; p.D = D; p.Dl = Dl;
  p.ldx = here == P ? D : Dl;
  p.P = P; p.rank0 = sh->rank; p.ranks_here = here; p.x_rank_stride = here == P && P > 1 ? Dl : 0;
  p.k_tmem = plan.bwd_k_tmem; p.n_ring = plan.bwd_ring_chunks; p.ring_stages = plan.bwd_ring_stages; p.resident = plan.bwd_resident;
  p.epoch = sh->epoch;
  p.slstm_zero_first = slstm_zero_first;
  p.wait_limit_ns = (wait_limit_ms > 0 ? static_cast<unsigned long long>(wait_limit_ms) : 10000ull) * 1000000ull;
  for (int q = sh->rank; q < sh->rank + here; ++q) {
    const cudaError_t me = cudaMemsetAsync(sh->buffers[q], 0xff, static_cast<size_t>(plan.dgr_bytes), static_cast<cudaStream_t>(stream));
    if (me != cudaSuccess) return static_cast<int>(me);
  }
  return backward_mg_dispatch(cell, p, wx_bf16, plan.bwd_ksplit, static_cast<cudaStream_t>(stream), nullptr);
}

extern "C" int frnn_b200_mg_wgrad(int cell, const void* dgr_all, const void* hbf_all, const float* db_part, float* dR_rows,
                                  float* db, const frnn_b200_mg_shard_t* sh, int B, int T, int D, int bwd_ksplit, int* err,
                                  void* stream) {
  Counts c;
  if (!counts(cell, &c)) return -1;
  if (!shard_ok(sh, D) || !dgr_all || !hbf_all || !db_part || !dR_rows || !db || !err || bwd_ksplit < 1) return -5;
  const int P = sh->P, Dl = D / P, here = sh->ranks_here;
  const bool together = here == P && P > 1;
  for (int lr = 0; lr < here; ++lr) {
    const int rank = sh->rank + lr;
    // one launch per rank slot: rows [rank*Dl, (rank+1)*Dl) of every gate. With all ranks in one process the outputs
    // are the full-width dR [GR][D][D] and db [GB][D]; otherwise this rank's [GR][Dl][D] and [GB][Dl].
    float* out = dR_rows + (together ? static_cast<size_t>(rank) * Dl * D : 0);
    const int rc = wgrad_launch_rows(c.gr, c.gb, static_cast<const __nv_bfloat16*>(dgr_all), static_cast<const __nv_bfloat16*>(hbf_all),
                                     db_part, bwd_ksplit, out, db, err, B, T, D, Dl, rank * Dl, together ? D : Dl,
                                     together ? D : Dl, together ? rank * Dl : 0, static_cast<cudaStream_t>(stream));
    if (rc != 0) return rc;
  }
  return 0;
}

// ---- buffers that the other processes of the node can store into (CUDA IPC) ----

extern "C" int frnn_b200_peer_alloc(size_t bytes, void** ptr) {
  if (ptr == nullptr || bytes == 0) return -5;
  return static_cast<int>(cudaMalloc(ptr, bytes));
}
extern "C" int frnn_b200_peer_free(void* ptr) { return static_cast<int>(cudaFree(ptr)); }
extern "C" int frnn_b200_peer_export(void* ptr, unsigned char handle[64]) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "handle size");
  if (ptr == nullptr || handle == nullptr) return -5;
  cudaIpcMemHandle_t h;
  const cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
  if (e != cudaSuccess) return static_cast<int>(e);
  memcpy(handle, &h, 64);
  return 0;
}
extern "C" int frnn_b200_peer_open(const unsigned char handle[64], void** ptr) {
  if (ptr == nullptr || handle == nullptr) return -5;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, 64);
  return static_cast<int>(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
}
extern "C" int frnn_b200_peer_close(void* ptr) { return static_cast<int>(cudaIpcCloseMemHandle(ptr)); }
