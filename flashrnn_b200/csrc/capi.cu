// extern "C" boundary of the library: shape planning, argument checks, kernel dispatch.
#include "../../include/flashrnn_b200.h"

#include <mutex>

#include "frnn_common.cuh"

namespace frnn {

int forward_dispatch(int cell, const FwdParams& p, const void* wx, int wx_bf16, int bv, int unit, cudaStream_t s);
int forward_ksplit_dispatch(int cell, const FwdParams& p, const void* wx, int wx_bf16, int bv, int ksplit, cudaStream_t s,
                            int* capacity_only);
int forward_ksplit_capacity(int cell, int bv, int ksplit, int D);
int backward_ksplit_width(int gates_r, int D);
bool backward_ksplit_valid(int cell, int gates_r, int D, int ks);
int backward_ksplit_dispatch(int cell, const BwdParams& p, const void* cache, const float* history, const float* initial,
                             const float* d_history, int wx_bf16, int bv, int ksplit, cudaStream_t s, int* capacity_only);
int backward_ksplit_capacity(int cell, int bv, int ksplit, int D);
int backward_dispatch(int cell, const BwdParams& p, const void* cache, const float* history, const float* initial,
                      const float* d_history, int wx_bf16, int bv, int unit, cudaStream_t s);
int wgrad_plan(int gr, int B, int T, int N, int D, int* np_out, int* ksplit_out, int* cps_out);
int wgrad_launch(int gr, int gb, const __nv_bfloat16* dgr, const __nv_bfloat16* hbf, const float* db_part, int n_btiles,
                 float* dR, float* db, float* work, int* err, int B, int T, int N, int D, cudaStream_t s);

int input_proj_launch(const void* x, const void* w, const float* bias, void* out, int out_bf16, long long M, int J, int I,
                      int* err, cudaStream_t s);

int wgrad_launch_static(int gr, int gb, const __nv_bfloat16* dgr, const __nv_bfloat16* hbf, const float* db_part,
                        int n_btiles, float* dR, float* db, int* err, int B, int T, int N, int D, cudaStream_t s);

namespace {

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(sym);
  });
  return fn;
}

// SMs of the current device (148 on a B200; also the answer when no device is visible).
int sm_count() {
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      n <= 0) {
    cudaGetLastError();
    return 148;
  }
  return n;
}

// CTAs of the clustered backward launch that the device can hold at once, remembered per shape
// class (the query is a driver call and the plan is computed on every call).
int ksplit_capacity_cached(bool forward, int cell, int bv, int ks, int D) {
  struct Entry { int fwd, cell, bv, ks, D, cap; };
  static std::mutex mu;
  static Entry table[64];
  static int used = 0;
  std::lock_guard<std::mutex> lock(mu);
  for (int i = 0; i < used; ++i)
    if (table[i].fwd == static_cast<int>(forward) && table[i].cell == cell && table[i].bv == bv && table[i].ks == ks &&
        table[i].D == D)
      return table[i].cap;
  int cap = forward ? forward_ksplit_capacity(cell, bv, ks, D) : backward_ksplit_capacity(cell, bv, ks, D);
  if (cap <= 0) {
    cudaGetLastError();
    cap = sm_count() / ks * ks;  // no device visible: assume every SM can take part
  }
  if (used < 64) table[used++] = Entry{static_cast<int>(forward), cell, bv, ks, D, cap};
  return cap;
}
int bwd_ksplit_capacity_cached(int cell, int bv, int ks, int D) { return ksplit_capacity_cached(false, cell, bv, ks, D); }

struct CellCounts {
  int gr, gw, gb, s, gc;
};
bool cell_counts(int cell, CellCounts* c) {
  switch (cell) {
    case kLSTM: *c = {4, 4, 4, 2, 4}; return true;
    case kSLSTM: *c = {4, 4, 4, 4, 4}; return true;
    case kGRU: *c = {3, 3, 4, 1, 4}; return true;
    case kElman: *c = {1, 1, 1, 1, 0}; return true;
    default: return false;
  }
}

}  // namespace

int make_tensor_map(CUtensorMap* map, const void* base, int elem_bytes, int rank, const uint64_t* dims,
                    const uint32_t* box, bool swizzle128, const uint64_t* stride_dims) {
  EncodeTiledFn fn = encode_tiled_fn();
  if (fn == nullptr) return -4;
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5], estr[5];
  uint64_t stride = static_cast<uint64_t>(elem_bytes);
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    stride *= stride_dims != nullptr ? stride_dims[i] : dims[i];
    if (i < rank - 1) gstrides[i] = stride;
  }
  const CUtensorMapDataType dt = elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const CUresult r = fn(map, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdims, gstrides, gbox, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? 0 : -4;
}

}  // namespace frnn

using namespace frnn;

extern "C" int frnn_b200_version(void) { return 1000; }

extern "C" int frnn_b200_plan(int cell, int B, int T, int N, int D, frnn_b200_plan_t* out) {
  if (out == nullptr) return -5;
  CellCounts c;
  if (!cell_counts(cell, &c)) return -1;
  if (B < 1 || T < 1 || N < 1 || D < 1) return -5;
  *out = frnn_b200_plan_t{};
  out->gates_r = c.gr; out->gates_w = c.gw; out->gates_b = c.gb; out->states = c.s; out->cache_gates = c.gc;
  out->unit = (D % 32 == 0) ? 32 : 16;
  out->cluster = D / out->unit;
  // Batch tile: a step costs the same tensor-core time for 8 or 16 rows but twice the epilogue and
  // exchange work, so 8-row tiles (more, independent groups) win as long as every group still
  // gets its own SMs; beyond that 16-row tiles halve the number of groups.
  out->batch_tile = 8;
  if (B > 8 && static_cast<long long>(N) * ((B + 7) / 8) * out->cluster > sm_count()) out->batch_tile = 16;
  out->n_btiles = (B + out->batch_tile - 1) / out->batch_tile;
  out->grid_ctas = N * out->n_btiles * out->cluster;
  const int bt = 16;  // UMMA N: batch tile padded to 16 columns
  int rows = c.gr * out->unit;
  const int mt = (rows + 127) / 128;
  const int fwd_cols = ((mt * bt + 31) / 32 * 32) + mt * (D / 2);
  const int mtb = (D + 127) / 128;
  int bwd_cols = ((mtb * bt + 31) / 32 * 32) + mtb * (rows / 2);
  // exchange 0: one thread-block cluster per group; 1: groups wider than a cluster exchange through
  // global memory; 2: heads whose rows of R do not fit one CTA's tensor memory: the forward splits
  // the contraction over two CTAs per row tile, the backward runs with 16-unit slices.
  out->exchange = out->cluster > 16 ? 1 : 0;
  out->supported = (D % 16 == 0) && fwd_cols <= 512 && bwd_cols <= 512 && (out->exchange == 0 || out->unit == 32);
  const int bks_width = out->exchange || !out->supported ? backward_ksplit_width(c.gr, D) : 0;
  bool slices16_fit = true;  // can the 1-D backward hold its slice of R in tensor memory
  if (!out->supported && D % 64 == 0 && D / 2 <= 896) {
    out->exchange = 2;
    out->unit = 16;
    out->cluster = D / 16;  // CTAs per group, forward (D/32 row tiles x 2) and 1-D backward alike
    rows = c.gr * 16;
    bwd_cols = ((mtb * bt + 31) / 32 * 32) + mtb * (rows / 2);
    slices16_fit = bwd_cols <= 512;
    out->supported = slices16_fit || bks_width > 0;
  }
  out->fwd_ctas = out->grid_ctas;
  out->fwd_batch_tile = out->batch_tile;
  if (out->exchange && out->supported) {
    // All CTAs of such a launch wait on one another: they must be resident together. Forward and
    // backward are separate launches and choose their decomposition and batch tile independently.
    const int slice_ctas = out->cluster;
    const int sms = sm_count();
    // Forward, best first: contraction of a 32-unit row tile split over 4 or 2 CTAs (shorter tensor-core
    // chain per step) with 8-row batch tiles, then the same with 16-row tiles (about a quarter more
    // time per step), last one CTA per 32 units (only while its rows of R fit tensor memory).
    bool fwd_ok = false;
    for (int tile = 8; tile <= 16 && !fwd_ok; tile += 8) {
      if (tile == 16 && B <= 8) break;
      const int groups = N * ((B + tile - 1) / tile);
      for (int ks = 4; ks >= 2 && !fwd_ok; ks /= 2) {
        if (D % 32 != 0 || D % ks != 0 || (D / ks) % 16 != 0 || D / ks > 896) continue;
        if (groups * (D / 32) * ks > ksplit_capacity_cached(true, cell, tile, ks, D)) continue;
        out->fwd_ksplit = ks;
        out->fwd_batch_tile = tile;
        out->fwd_ctas = groups * (D / 32) * ks;
        fwd_ok = true;
      }
    }
    for (int tile = 8; tile <= 16 && !fwd_ok && out->exchange == 1; tile += 8) {
      const int groups = N * ((B + tile - 1) / tile);
      if (groups * (D / 32) > sms) continue;
      out->fwd_ksplit = 0;
      out->fwd_batch_tile = tile;
      out->fwd_ctas = groups * (D / 32);
      fwd_ok = true;
    }
    // Backward, best first: columns of R in 128-unit tiles with the gate rows split over 8, 4 or 2 CTAs
    // (the widest split that fits: shortest tensor-core chain per step), first with 8-row batch tiles,
    // then with 16-row tiles; last the 1-D backward (32- or 16-unit slices of rows of R).
    bool bwd_ok = false;
    for (int tile = 8; tile <= 16 && !bwd_ok && bks_width > 0; tile += 8) {
      if (tile == 16 && B <= 8) break;
      const int groups = N * ((B + tile - 1) / tile);
      for (int ks = 8; ks >= 2 && !bwd_ok; ks /= 2) {
        if (!backward_ksplit_valid(cell, c.gr, D, ks)) continue;
        if (groups * (D / 128) * ks > bwd_ksplit_capacity_cached(cell, tile, ks, D)) continue;
        out->bwd_ksplit = ks;
        out->batch_tile = tile;
        out->cluster = (D / 128) * ks;
        bwd_ok = true;
      }
    }
    for (int tile = 8; tile <= 16 && !bwd_ok && slices16_fit; tile += 8) {
      const int groups = N * ((B + tile - 1) / tile);
      if (groups * slice_ctas > sms) continue;
      out->bwd_ksplit = 0;
      out->batch_tile = tile;
      out->cluster = slice_ctas;
      bwd_ok = true;
    }
    out->n_btiles = (B + out->batch_tile - 1) / out->batch_tile;
    out->grid_ctas = N * out->n_btiles * out->cluster;
    out->supported = fwd_ok && bwd_ok;
    const int64_t fwd_groups = static_cast<int64_t>(N) * ((B + out->fwd_batch_tile - 1) / out->fwd_batch_tile);
    const int64_t bwd_groups = static_cast<int64_t>(N) * out->n_btiles;
    const int64_t fwd_b = 4ll * bt * D * 2;  // four operand slots
    const int64_t bwd_b = out->bwd_ksplit ? 4ll * bt * c.gr * D * 2                                        // four slots of dG
                                          : 2ll * out->cluster * out->cluster * out->unit * out->batch_tile * 4;  // two slots of partial dh
    out->xchg_bytes = fwd_groups * fwd_b > bwd_groups * bwd_b ? fwd_groups * fwd_b : bwd_groups * bwd_b;
  }
  const int64_t btnd = static_cast<int64_t>(B) * T * N * D;
  out->cache_bytes = btnd * c.gc * ((cell == kLSTM || cell == kGRU) ? 2 : 4);  // CellTraits::CES
  out->hbf_bytes = static_cast<int64_t>(B) * (T + 1) * N * D * 2;
  out->dgr_bytes = btnd * c.gr * 2;
  out->dbpart_bytes = static_cast<int64_t>(out->n_btiles) * c.gb * N * D * 4;
  int np = 0, ksplit = 1, cps = 0;
  if (D % 16 == 0 && wgrad_plan(c.gr, B, T, N, D, &np, &ksplit, &cps) == 0) {
    out->wgrad_ksplit = ksplit;
    out->wgrad_work_bytes = ksplit > 1 ? static_cast<int64_t>(ksplit) * c.gr * N * D * D * 4 : 0;
  } else {
    out->supported = 0;
  }
  return 0;
}

namespace {

int forward_common(int cell, const void* wx, int wx_bf16, const void* r_bf16, const float* bias, const float* initial,
                   float* history, float* carry, void* cache, void* hbf, void* xchg, int B, int T, int N, int D,
                   int slstm_zero_first, const int* zero_first_dev, int output_mode, int wait_limit_ms, int* err,
                   void* stream, int T_total = 0, int t0 = 0, int out_bf16 = 0, const frnn_b200_options_t* opt = nullptr) {
  frnn_b200_plan_t plan;
  const int rc = frnn_b200_plan(cell, B, T, N, D, &plan);
  if (rc != 0) return rc;
  if (!plan.supported) return -2;
  if (!wx || !r_bf16 || !bias || !initial || !history || !carry || !err) return -5;
  FwdParams p{};
  p.R = static_cast<const __nv_bfloat16*>(r_bf16);
  p.bias = bias;
  p.initial = initial;
  p.history = history;
  p.carry = carry;
  p.cache = cache;
  p.hbf = static_cast<__nv_bfloat16*>(hbf);
  p.err = err;
  p.B = B; p.T = T; p.N = N; p.D = D;
  p.C = plan.exchange ? D / 32 : plan.cluster;  // CTAs per group of the 1-D forward
  p.wx_box_b = plan.fwd_batch_tile;  // rows past B are filled with zeros by TMA
  p.slstm_zero_first = slstm_zero_first;
  p.zero_first_dev = zero_first_dev;
  p.output_mode = output_mode;
  p.T_total = T_total > 0 ? T_total : T;
  p.t0 = t0;
  p.out_bf16 = out_bf16;
  p.fwd_clip = opt != nullptr && opt->forward_clipval > 0.0f ? opt->forward_clipval : INFINITY;  // branch-free in the kernels
  if (t0 < 0 || t0 + T > p.T_total) return -5;
  if ((cache != nullptr || hbf != nullptr) && (t0 != 0 || p.T_total != T || out_bf16)) return -5;
  p.wait_limit_ns = (wait_limit_ms > 0 ? static_cast<unsigned long long>(wait_limit_ms) : 2000ull) * 1000000ull;
  if (plan.exchange) {
    if (!xchg) return -5;
    // every exchange word starts as "not yet written" (all ones)
    const cudaError_t me = cudaMemsetAsync(xchg, 0xff, static_cast<size_t>(plan.xchg_bytes), static_cast<cudaStream_t>(stream));
    if (me != cudaSuccess) return static_cast<int>(me);
    p.xg_data = static_cast<uint8_t*>(xchg);
  }
  if (plan.fwd_ksplit)
    return forward_ksplit_dispatch(cell, p, wx, wx_bf16, plan.fwd_batch_tile, plan.fwd_ksplit, static_cast<cudaStream_t>(stream),
                                   nullptr);
  return forward_dispatch(cell, p, wx, wx_bf16, plan.fwd_batch_tile, plan.exchange ? 32 : plan.unit, static_cast<cudaStream_t>(stream));
}

}  // namespace

extern "C" int frnn_b200_forward(int cell, const void* wx, int wx_bf16, const void* r_bf16, const float* bias,
                                 const float* initial, float* history, float* carry, void* cache, void* hbf,
                                 void* xchg, int B, int T, int N, int D, int slstm_zero_first, int wait_limit_ms,
                                 int* err, void* stream) {
  return forward_common(cell, wx, wx_bf16, r_bf16, bias, initial, history, carry, cache, hbf, xchg, B, T, N, D,
                        slstm_zero_first, nullptr, 0, wait_limit_ms, err, stream);
}

extern "C" int frnn_b200_forward_ex(int cell, const void* wx, int wx_bf16, const void* r_bf16, const float* bias,
                                    const float* initial, float* history, float* carry, void* cache, void* hbf,
                                    void* xchg, int B, int T, int N, int D, int slstm_zero_first, int wait_limit_ms,
                                    int* err, void* stream, const frnn_b200_options_t* options) {
  return forward_common(cell, wx, wx_bf16, r_bf16, bias, initial, history, carry, cache, hbf, xchg, B, T, N, D,
                        slstm_zero_first, nullptr, 0, wait_limit_ms, err, stream, 0, 0, 0, options);
}

extern "C" int frnn_b200_forward_prepared(int cell, const void* wx, int wx_bf16, const void* r_bf16, const float* bias,
                                          const float* initial, void* output, float* carry, void* xchg, int B, int T,
                                          int N, int D, int output_mode, const int* slstm_zero_first_dev,
                                          int wait_limit_ms, int* err, void* stream) {
  return frnn_b200_forward_chunk(cell, wx, wx_bf16, r_bf16, bias, initial, output, 0, carry, xchg, B, T, 0, T, N, D,
                                 output_mode, slstm_zero_first_dev, wait_limit_ms, err, stream);
}

extern "C" int frnn_b200_forward_chunk(int cell, const void* wx, int wx_bf16, const void* r_bf16, const float* bias,
                                       const float* initial, void* output, int output_bf16, float* carry, void* xchg, int B,
                                       int T_total, int t_start, int steps, int N, int D, int output_mode,
                                       const int* slstm_zero_first_dev, int wait_limit_ms, int* err, void* stream) {
  if (output_mode < 0 || output_mode > 2 || steps < 1) return -5;
  if (cell == kSLSTM && slstm_zero_first_dev == nullptr) return -5;
  return forward_common(cell, wx, wx_bf16, r_bf16, bias, initial, static_cast<float*>(output), carry, nullptr, nullptr, xchg, B,
                        steps, N, D, 0, cell == kSLSTM ? slstm_zero_first_dev : nullptr, output_mode, wait_limit_ms, err,
                        stream, T_total, t_start, output_bf16 != 0);
}

extern "C" int frnn_b200_backward(int cell, const void* cache, const float* history, const float* initial,
                                  const void* r_bf16, const float* d_history, const float* d_carry, void* dwx,
                                  int wx_bf16, void* dgr, float* d_initial, float* db_part, void* xchg, int B, int T,
                                  int N, int D, int slstm_zero_first, int wait_limit_ms, int* err, void* stream) {
  return frnn_b200_backward_ex(cell, cache, history, initial, r_bf16, d_history, d_carry, dwx, wx_bf16, dgr, d_initial,
                               db_part, xchg, B, T, N, D, slstm_zero_first, wait_limit_ms, err, stream, nullptr);
}

extern "C" int frnn_b200_backward_ex(int cell, const void* cache, const float* history, const float* initial,
                                     const void* r_bf16, const float* d_history, const float* d_carry, void* dwx,
                                     int wx_bf16, void* dgr, float* d_initial, float* db_part, void* xchg, int B, int T,
                                     int N, int D, int slstm_zero_first, int wait_limit_ms, int* err, void* stream,
                                     const frnn_b200_options_t* options) {
  frnn_b200_plan_t plan;
  const int rc = frnn_b200_plan(cell, B, T, N, D, &plan);
  if (rc != 0) return rc;
  if (!plan.supported) return -2;
  if ((!cache && plan.cache_gates > 0) || !history || !initial || !r_bf16 || !d_history || !d_carry || !dwx || !dgr ||
      !d_initial || !db_part || !err)
    return -5;
  BwdParams p{};
  p.R = static_cast<const __nv_bfloat16*>(r_bf16);
  p.d_carry = d_carry;
  p.dwx = dwx;
  p.dgr = static_cast<__nv_bfloat16*>(dgr);
  p.d_initial = d_initial;
  p.db_part = db_part;
  p.err = err;
  p.B = B; p.T = T; p.N = N; p.D = D;
  p.C = plan.cluster;
  p.box_b = plan.batch_tile;  // rows past B are filled with zeros by TMA
  p.slstm_zero_first = slstm_zero_first;
  if (options != nullptr) {
    p.grad_clip = options->gradient_recurrent_clipval;
    p.cut_recurrent = options->gradient_recurrent_cut != 0;
    p.slstm_v1 = options->slstm_v1_gradient != 0;
  }
  p.wait_limit_ns = (wait_limit_ms > 0 ? static_cast<unsigned long long>(wait_limit_ms) : 2000ull) * 1000000ull;
  if (plan.exchange) {
    if (!xchg) return -5;
    const cudaError_t me = cudaMemsetAsync(xchg, 0xff, static_cast<size_t>(plan.xchg_bytes), static_cast<cudaStream_t>(stream));
    if (me != cudaSuccess) return static_cast<int>(me);
    p.xg_data = static_cast<uint8_t*>(xchg);
  }
  if (plan.bwd_ksplit)
    return backward_ksplit_dispatch(cell, p, cache, history, initial, d_history, wx_bf16, plan.batch_tile,
                                    plan.bwd_ksplit, static_cast<cudaStream_t>(stream), nullptr);
  return backward_dispatch(cell, p, cache, history, initial, d_history, wx_bf16, plan.batch_tile, plan.unit,
                           static_cast<cudaStream_t>(stream));
}

extern "C" int frnn_b200_wgrad(int cell, const void* dgr, const void* hbf, const float* db_part, float* dR, float* db,
                               float* work, int B, int T, int N, int D, int* err, void* stream) {
  frnn_b200_plan_t plan;
  const int rc = frnn_b200_plan(cell, B, T, N, D, &plan);
  if (rc != 0) return rc;
  if (!plan.supported) return -2;
  if (!dgr || !hbf || !db_part || !dR || !db || !err) return -5;
  if (plan.wgrad_work_bytes > 0 && !work) return -5;
  return wgrad_launch(plan.gates_r, plan.gates_b, static_cast<const __nv_bfloat16*>(dgr),
                      static_cast<const __nv_bfloat16*>(hbf), db_part, plan.n_btiles, dR, db, work, err, B, T, N, D,
                      static_cast<cudaStream_t>(stream));
}

extern "C" int frnn_b200_wgrad_noalloc(int cell, const void* dgr, const void* hbf, const float* db_part, float* dR,
                                       float* db, int B, int T, int N, int D, int* err, void* stream) {
  frnn_b200_plan_t plan;
  const int rc = frnn_b200_plan(cell, B, T, N, D, &plan);
  if (rc != 0) return rc;
  if (!plan.supported) return -2;
  if (!dgr || !hbf || !db_part || !dR || !db || !err) return -5;
  return wgrad_launch_static(plan.gates_r, plan.gates_b, static_cast<const __nv_bfloat16*>(dgr),
                             static_cast<const __nv_bfloat16*>(hbf), db_part, plan.n_btiles, dR, db, err, B, T, N, D,
                             static_cast<cudaStream_t>(stream));
}

extern "C" int frnn_b200_input_projection(const void* x_bf16, const void* w_bf16, const float* bias, void* wx, int wx_bf16,
                                          int B, int T, int gates_times_width, int inputs, int* err, void* stream) {
  if (!x_bf16 || !w_bf16 || !wx || !err || B < 1 || T < 1) return -5;
  return input_proj_launch(x_bf16, w_bf16, bias, wx, wx_bf16 != 0, static_cast<long long>(B) * T, gates_times_width, inputs, err,
                           static_cast<cudaStream_t>(stream));
}
