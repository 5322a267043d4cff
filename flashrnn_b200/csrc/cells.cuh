// Per-cell pointwise arithmetic of the recurrence, forward and backward, in fp32.
//
// The formulas restate the step of `recurrence()` in the reference
// (flashrnn/flashrnn2/reference.py:72-114) and the derivative torch autograd forms for it.
// Gate order is (i, f, z, o) for lstm/slstm; gru uses W-gates (reset, update, candidate-input),
// R-gates (candidate-recurrent, reset, update) and four biases (reference.py:84-89).
#pragma once

#include <cuda_runtime.h>

namespace frnn {

enum : int { kLSTM = 0, kSLSTM = 1, kGRU = 2, kElman = 3 };

// GR: gates fed by R*h, GW: gates in Wx, GB: bias gates, S: states, GC: values cached per
// (batch, step, unit) by a training forward for the backward pass.
template <int CELL> struct CellTraits;
// CES: bytes per cached value. LSTM and GRU cache activations in [-1, 1] (and the GRU's O(1) candidate pre-activation):
// fp16 keeps 11 significant bits of them, which moves no gradient by more than a few 1e-4 of its scale (the bf16
// tensor-core operands cost ten times that) and halves the largest stream of a training step. The sLSTM caches raw
// pre-activations that go through exp(): fp32.
template <> struct CellTraits<kLSTM>  { static constexpr int GR = 4, GW = 4, GB = 4, S = 2, GC = 4, CES = 2; };
template <> struct CellTraits<kSLSTM> { static constexpr int GR = 4, GW = 4, GB = 4, S = 4, GC = 4, CES = 4; };
template <> struct CellTraits<kGRU>   { static constexpr int GR = 3, GW = 3, GB = 4, S = 1, GC = 4, CES = 2; };
template <> struct CellTraits<kElman> { static constexpr int GR = 1, GW = 1, GB = 1, S = 1, GC = 1, CES = 4; };

// MUFU-based primitives: ex2.approx / rcp.approx are accurate to about 2 ulp, far inside the
// tolerance of a bf16-operand recurrence, and take one instruction each where the IEEE-rounded
// reciprocal takes a dozen.
__device__ __forceinline__ float rcp_fast(float x) {
  float r;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float exp2_fast(float x) {
  float r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
// Two-instruction forms (ex2 + rcp, about 2 ulp).
__device__ __forceinline__ float sigmoid_p(float x) { return rcp_fast(1.0f + exp2_fast(-1.4426950408889634f * x)); }
__device__ __forceinline__ float tanh_p(float x) {
  // 1 - 2/(1+e^{2x}); saturates correctly at +-1 when e^{2x} over/underflows.
  return 1.0f - 2.0f * rcp_fast(1.0f + exp2_fast(2.885390081777927f * x));
}
#ifndef FRNN_PRECISE_ACTIVATIONS
// One MUFU instruction per activation (tanh.approx.f32, relative error about 2^-11) for the LSTM,
// GRU and Elman cells: against the oracle the error of every output is unchanged (it is set by the
// bf16 rounding of the recurrent operands), and the forward step gets about 100 cycles shorter.
// The sLSTM keeps the two-instruction forms: its normaliser clamp makes gradients discontinuous,
// so it gets the most accurate forward values that cost nothing on its critical path.
// Compile with -DFRNN_PRECISE_ACTIVATIONS for the two-instruction forms everywhere.
__device__ __forceinline__ float tanh_f(float x) {
  float r;
  asm("tanh.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
  return r;
}
__device__ __forceinline__ float sigmoid_f(float x) { return fmaf(0.5f, tanh_f(0.5f * x), 0.5f); }
#else
__device__ __forceinline__ float sigmoid_f(float x) { return sigmoid_p(x); }
__device__ __forceinline__ float tanh_f(float x) { return tanh_p(x); }
#endif
__device__ __forceinline__ float logsigmoid_f(float x) {
  return fminf(x, 0.0f) - __logf(1.0f + __expf(-fabsf(x)));
}

// ---------------------------------------------------------------------------------------------
// forward: st holds the previous state on entry and the new state on return.
// ry = R*round_bf16(h_prev) for the GR recurrent gates, wx = this step's input gates.
// cache receives what cell_backward needs (nothing useful for Elman).
// ---------------------------------------------------------------------------------------------
template <int CELL>
__device__ __forceinline__ void cell_forward(const float* ry, const float* wx, const float* b,
                                             float* st, float* cache, bool slstm_take_i) {
  if constexpr (CELL == kLSTM) {
    const float si = sigmoid_f((wx[0] + ry[0]) + b[0]);
    const float sf = sigmoid_f((wx[1] + ry[1]) + b[1]);
    const float tz = tanh_f((wx[2] + ry[2]) + b[2]);
    const float so = sigmoid_f((wx[3] + ry[3]) + b[3]);
    const float c = sf * st[1] + si * tz;
    st[0] = so * tanh_f(c);
    st[1] = c;
    cache[0] = si; cache[1] = sf; cache[2] = tz; cache[3] = so;
  } else if constexpr (CELL == kSLSTM) {
    const float i = (wx[0] + ry[0]) + b[0];
    const float f = (wx[1] + ry[1]) + b[1];
    const float z = (wx[2] + ry[2]) + b[2];
    const float o = (wx[3] + ry[3]) + b[3];
    const float logf = logsigmoid_f(f) + st[3];
    const float m = slstm_take_i ? i : fmaxf(i, logf);
    const float ig = __expf(i - m);
    const float fg = __expf(logf - m);
    const float c = fg * st[1] + ig * tanh_p(z);
    const float n = fmaxf(fg * st[2] + ig, 1.0f);
    st[0] = sigmoid_p(o) * c * rcp_fast(n);  // rcp.approx: 1 ulp, against a dozen instructions for the IEEE quotient
    st[1] = c; st[2] = n; st[3] = m;
    cache[0] = i; cache[1] = f; cache[2] = z; cache[3] = o;
  } else if constexpr (CELL == kGRU) {
    const float cand = ry[0] + b[0];
    const float r = sigmoid_f((wx[0] + ry[1]) + b[1]);
    const float u = sigmoid_f((wx[1] + ry[2]) + b[2]);
    const float v = tanh_f((wx[2] + b[3]) + r * cand);
    st[0] = u * st[0] + (1.0f - u) * v;
    // the cache holds fp16 values: keep an (absurdly) large candidate finite there
    cache[0] = fminf(fmaxf(cand, -60000.0f), 60000.0f); cache[1] = r; cache[2] = u; cache[3] = v;
  } else {
    st[0] = tanh_f((wx[0] + ry[0]) + b[0]);
    cache[0] = 0.0f;
  }
}

// ---------------------------------------------------------------------------------------------
// backward of one step for one (batch, unit).
//   ds    in : total gradient w.r.t. the NEW state (history gradient + everything carried back,
//              including the R path into h);
//         out: gradient w.r.t. the PREVIOUS state through the pointwise path only (the R path
//              dgr * R is added by the caller).
//   dgr / dgw / dgb: gradients of the recurrent pre-activations, the Wx gates and the biases.
// slstm: follows autograd exactly, i.e. the stabiliser m carries a gradient and max(., 1) /
// max(i, logf) split a tie 0.5 / 0.5 as torch.maximum does.
// ---------------------------------------------------------------------------------------------
// slstm_v1 selects the gradient convention of the reference's own kernels instead (flashrnn/flashrnn2/
// grad_reference.py:1-13, flashrnn/flashrnn/vanilla_fwbw/bw.py:147-190): m carries no gradient (neither m_t nor the
// m_{t-1} inside log f, so d(initial m) = 0) and the clamp n = max(., 1) passes its gradient straight through.
template <int CELL>
__device__ __forceinline__ void cell_backward(const float* cache, const float* sp, const float* sn,
                                              float* ds, float* dgr, float* dgw, float* dgb,
                                              bool slstm_take_i, bool slstm_v1 = false) {
  if constexpr (CELL == kLSTM) {
    const float si = cache[0], sf = cache[1], tz = cache[2], so = cache[3];
    const float tc = tanh_f(sn[1]);
    const float dh = ds[0];
    const float dc = ds[1] + dh * so * (1.0f - tc * tc);
    const float d_o = dh * tc * so * (1.0f - so);
    const float d_f = dc * sp[1] * sf * (1.0f - sf);
    const float d_i = dc * tz * si * (1.0f - si);
    const float d_z = dc * si * (1.0f - tz * tz);
    ds[0] = 0.0f;
    ds[1] = dc * sf;
    dgr[0] = d_i; dgr[1] = d_f; dgr[2] = d_z; dgr[3] = d_o;
    dgw[0] = d_i; dgw[1] = d_f; dgw[2] = d_z; dgw[3] = d_o;
    dgb[0] = d_i; dgb[1] = d_f; dgb[2] = d_z; dgb[3] = d_o;
  } else if constexpr (CELL == kSLSTM) {
    const float i = cache[0], f = cache[1], z = cache[2], o = cache[3];
    const float c_p = sp[1], n_p = sp[2], m_p = sp[3];
    const float c_n = sn[1], n_n = sn[2], m_n = sn[3];
    const float so = sigmoid_p(o);
    const float tz = tanh_p(z);
    const float sgf = sigmoid_p(f);
    const float logf = logsigmoid_f(f) + m_p;
    const float ig = __expf(i - m_n);
    const float fg = __expf(logf - m_n);
    const float dh = ds[0];
    const float inv_n = rcp_fast(n_n);
    const float dc = ds[1] + dh * so * inv_n;
    const float dn = ds[2] - dh * so * c_n * inv_n * inv_n;
    const float d_o = dh * (c_n * inv_n) * so * (1.0f - so);
    const float pre_n = fg * n_p + ig;
    const float mask = slstm_v1 ? 1.0f : (pre_n > 1.0f ? 1.0f : (pre_n == 1.0f ? 0.5f : 0.0f));
    const float dpre = dn * mask;
    const float d_ig = dc * tz + dpre;
    const float d_fg = dc * c_p + dpre * n_p;
    const float d_z = dc * ig * (1.0f - tz * tz);
    float d_i = d_ig * ig;
    float d_logf = d_fg * fg;
    const float dm = slstm_v1 ? 0.0f : ds[3] - d_i - d_logf;
    if (slstm_take_i) {
      d_i += dm;
    } else if (i > logf) {
      d_i += dm;
    } else if (i < logf) {
      d_logf += dm;
    } else {
      d_i += 0.5f * dm;
      d_logf += 0.5f * dm;
    }
    const float d_f = d_logf * (1.0f - sgf);
    ds[0] = 0.0f;
    ds[1] = dc * fg;
    ds[2] = dpre * fg;
    ds[3] = slstm_v1 ? 0.0f : d_logf;
    dgr[0] = d_i; dgr[1] = d_f; dgr[2] = d_z; dgr[3] = d_o;
    dgw[0] = d_i; dgw[1] = d_f; dgw[2] = d_z; dgw[3] = d_o;
    dgb[0] = d_i; dgb[1] = d_f; dgb[2] = d_z; dgb[3] = d_o;
  } else if constexpr (CELL == kGRU) {
    const float cand = cache[0], r = cache[1], u = cache[2], v = cache[3];
    const float dh = ds[0];
    const float d_u = dh * (sp[0] - v) * u * (1.0f - u);
    const float d_v = dh * (1.0f - u) * (1.0f - v * v);
    const float d_r = d_v * cand * r * (1.0f - r);
    const float d_cand = d_v * r;
    ds[0] = dh * u;
    dgr[0] = d_cand; dgr[1] = d_r; dgr[2] = d_u;
    dgw[0] = d_r; dgw[1] = d_u; dgw[2] = d_v;
    dgb[0] = d_cand; dgb[1] = d_r; dgb[2] = d_u; dgb[3] = d_v;
  } else {
    const float h = sn[0];
    const float d = ds[0] * (1.0f - h * h);
    ds[0] = 0.0f;
    dgr[0] = d; dgw[0] = d; dgb[0] = d;
  }
}

// Options of the reference's v1 configuration (flashrnn/flashrnn/flashrnn.py:128-133), applied as its fused kernels
// apply them (flashrnn/flashrnn/fused/lstm_fused_pointwise.cuh:76-81,116-122): the new hidden state is clipped to
// [-forward_clipval, forward_clipval] before it is stored and fed back (the backward pass treats the clip as the
// identity); the gradient that reaches h_t from step t+1 (the R path plus the cell's direct h term) is clipped to
// [-gradient_recurrent_clipval, ...] before the external gradient of h_t is added; with gradient_recurrent_cut the R
// path contributes nothing at all (flashrnn/flashrnn/fused/flashrnn_fused_backward_cut.cu:90). Values <= 0 switch a
// clip off.
__device__ __forceinline__ float clip_sym(float x, float c) { return c > 0.0f ? fminf(fmaxf(x, -c), c) : x; }

}  // namespace frnn
