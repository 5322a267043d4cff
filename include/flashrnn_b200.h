/*
 * flashrnn_b200 — C ABI of the sm_100a fused recurrence (forward, BPTT backward, dR/db).
 *
 * All pointers are DEVICE pointers owned by the caller; the library never allocates, frees or
 * synchronises, and every launch goes to the CUDA stream passed as `stream` (a cudaStream_t).
 * Tensors are dense and use the public layouts of the reference:
 *   Wx[B,T,GW,N,D]  R[GR,N,D,D] (gate, head, out, in)  b[GB,N,D]  states[S,B,T|1,N,D].
 * Return value: 0 on success, a positive cudaError_t, or a negative library code
 *   -1 unknown cell, -2 shape not supported by this kernel family (see frnn_b200_plan),
 *   -3 tensor-memory budget exceeded, -4 TMA descriptor could not be built, -5 bad argument,
 *   -6 problem too large for the built-in scratch of frnn_b200_wgrad_noalloc.
 * Device-side problems (a bounded wait that ran out) are reported through the caller-owned
 * `err` array (int[32], zeroed by the caller): err[0] = code (101..107), err[1] = step,
 * err[2] = CTA. The kernels then leave in an orderly way; the context stays usable.
 * In-kernel phase timers (the counterpart of the reference's %globaltimer phase probes,
 * flashrnn/flashrnn2/hybrid_fw2d.cu:85-89,366-373): if the caller sets err[3] = 1, CTA 0 adds up
 * SM clock cycles per phase over all steps into err[8..12] (epilogue warp: input wait, operand /
 * tensor-core wait, accumulator read, epilogue sync, cell + stores + exchange) and err[16..17]
 * (MMA warp: operand wait, issue).
 * Test hook for the failure path: with err[4] = 1 the CTAs stop publishing their per-step exchange
 * data from step err[5] on, so the next bounded wait (limit = wait_limit_ms) runs out and the call
 * reports err[0] = 101 (forward) / 106 or 107 (backward) and returns normally.
 *
 * Counterparts in the reference (0z5a/flashrnn):
 *   flashrnn/flashrnn/fused/flashrnn.cc:56-347      pybind class FlashRNNFuncFused
 *   flashrnn/flashrnn2/hybrid_fw2d.cu:404-419       extern "C" frnn_hybrid_fw2d (ctypes ABI model)
 *   flashrnn/flashrnn2/hybrid_bw2d.cu:664-678       extern "C" frnn_hybrid_bw2d
 */
#ifndef FLASHRNN_B200_H_
#define FLASHRNN_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { FRNN_CELL_LSTM = 0, FRNN_CELL_SLSTM = 1, FRNN_CELL_GRU = 2, FRNN_CELL_ELMAN = 3 };

/* Gate / state counts of a cell, as rnn_function_registry (flashrnn/flashrnn/flashrnn.py:46-68)
 * and SIZES (flashrnn/flashrnn2/reference.py:16-21) define them. */
typedef struct frnn_b200_plan {
  int gates_r, gates_w, gates_b, states, cache_gates;
  int unit;        /* hidden units owned by one CTA                              */
  int cluster;     /* CTAs per (head, batch tile) group = D / unit               */
  int batch_tile;  /* batch rows per group                                        */
  int n_btiles;    /* ceil(B / batch_tile)                                        */
  int grid_ctas;   /* N * n_btiles * cluster                                      */
  int supported;   /* 1 if the shape runs on this kernel family                   */
  int64_t cache_bytes;   /* [B,T,cache_gates,N,D] forward -> backward: fp16 (lstm, gru) or fp32 (slstm) */
  int64_t hbf_bytes;     /* bf16   [B,T+1,N,D]             forward -> wgrad        */
  int64_t dgr_bytes;     /* bf16   [B,T,gates_r,N,D]       backward -> wgrad       */
  int64_t dbpart_bytes;  /* float  [n_btiles,gates_b,N,D]  backward -> wgrad       */
  int64_t wgrad_work_bytes; /* float [wgrad_ksplit, gates_r,N,D,D] split-K partials, 0 if none */
  int wgrad_ksplit;
  int exchange;          /* 0: CTAs of a group exchange through cluster shared memory;
                            1: group wider than a cluster (D > 512): through global memory;
                            2: as 1, with 16-unit slices in the backward (768 < D)           */
  int64_t xchg_bytes;    /* scratch for exchange >= 1 (forward and backward), else 0      */
  int fwd_ksplit;        /* 0, or 2/4: the forward splits the contraction of a 32-unit row
                            tile over this many CTAs (a cluster) and exchanges h through
                            global memory                                                  */
  int fwd_ctas;          /* CTAs of the forward launch                                     */
  int bwd_ksplit;        /* 0, or 2/4/8: the backward owns columns of R in tiles of 128 units
                            and splits the gates_r * D gate rows over this many CTAs (a
                            cluster); cluster / grid_ctas then describe that launch        */
  int fwd_batch_tile;    /* batch rows per group in the forward (batch_tile, n_btiles, cluster
                            and grid_ctas describe the backward; the two launches choose
                            independently when exchange >= 1)                               */
} frnn_b200_plan_t;

/* Library / ABI version (major*1000 + minor). */
int frnn_b200_version(void);

/* Describe how (cell, B, T, N, D) is executed and how much scratch the caller must provide.
 * Replaces the per-shape constraint solving + JIT of the reference
 * (flashrnn/flashrnn/flashrnn.py:383-677, cuda_init_parametric.py). D must be a multiple of 16. */
int frnn_b200_plan(int cell, int B, int T, int N, int D, frnn_b200_plan_t* out);

/* Forward recurrence over T steps (flashrnn/flashrnn/fused/flashrnn.cc:69-145 forward();
 * arithmetic of flashrnn/flashrnn2/reference.py:72-114 with fp32 state and bf16 R / h operands).
 *   wx        : Wx, fp32 (wx_bf16 = 0) or bf16 (wx_bf16 = 1)
 *   r_bf16    : R rounded to bf16
 *   bias, initial : fp32
 *   history   : out fp32 [S,B,T,N,D];  carry: out fp32 [S,B,1,N,D]
 *   cache, hbf: scratch written for the backward pass, or NULL for inference
 *   xchg      : scratch of plan.xchg_bytes when plan.exchange >= 1 (initialised by the call), else NULL;
 *               such shapes are launched cooperatively: N * n_btiles * cluster CTAs must be
 *               resident at once (one per SM), otherwise the launch returns a CUDA error
 *   slstm_zero_first: 1 if every element of initial n is zero (reference.py:99)
 *   wait_limit_ms: bound for every in-kernel wait (0 = default 2000 ms)              */
int frnn_b200_forward(int cell, const void* wx, int wx_bf16, const void* r_bf16, const float* bias,
                      const float* initial, float* history, float* carry, void* cache, void* hbf,
                      void* xchg, int B, int T, int N, int D, int slstm_zero_first, int wait_limit_ms,
                      int* err, void* stream);

/* Options of the reference's v1 configuration (flashrnn/flashrnn/flashrnn.py:128-133), applied the way its fused
 * kernels apply them (flashrnn/flashrnn/fused/lstm_fused_pointwise.cuh:76-81,116-122,
 * flashrnn/flashrnn/fused/flashrnn_fused_backward_cut.cu:90), and the choice of the sLSTM gradient convention
 * (flashrnn/flashrnn2/grad_reference.py:1-13). A NULL pointer or an all-zero struct means "none": the behaviour of
 * frnn_b200_forward / frnn_b200_backward. */
typedef struct frnn_b200_options {
  float forward_clipval;             /* > 0: h_t is clipped to [-v, v] before it is stored and fed back; the
                                        backward pass treats the clip as the identity                              */
  float gradient_recurrent_clipval;  /* > 0: the gradient that reaches h_t from step t+1 is clipped to [-v, v]
                                        before the external gradient of h_t is added                               */
  int gradient_recurrent_cut;        /* 1: the R path contributes nothing to the hidden-state gradient              */
  int slstm_v1_gradient;             /* 1: sLSTM stabiliser m carries no gradient, the normaliser clamp passes its
                                        gradient straight through (0: exactly what autograd gives)                  */
} frnn_b200_options_t;

/* frnn_b200_forward / frnn_b200_backward with options. */
int frnn_b200_forward_ex(int cell, const void* wx, int wx_bf16, const void* r_bf16, const float* bias,
                         const float* initial, float* history, float* carry, void* cache, void* hbf, void* xchg,
                         int B, int T, int N, int D, int slstm_zero_first, int wait_limit_ms, int* err, void* stream,
                         const frnn_b200_options_t* options);
int frnn_b200_backward_ex(int cell, const void* cache, const float* history, const float* initial,
                          const void* r_bf16, const float* d_history, const float* d_carry, void* dwx, int wx_bf16,
                          void* dgr, float* d_initial, float* db_part, void* xchg, int B, int T, int N, int D,
                          int slstm_zero_first, int wait_limit_ms, int* err, void* stream,
                          const frnn_b200_options_t* options);

/* Forward-only variant for preallocated, replayable sequences (the reference's PreparedSequence,
 * flashrnn/flashrnn2/prepared.py:18-192, and the output modes of hybrid_fw2d.cu:52-66): no gate
 * cache and no bf16 copy of h are written.
 *   output_mode 0: output = every state's history, fp32 [S,B,T,N,D]
 *               1: output = the hidden state only, fp32 [B,T,N,D]
 *               2: output = the last hidden state only, fp32 [B,1,N,D]
 *   slstm_zero_first_dev : device word read by the kernel (non-zero: the normaliser of the whole
 *               logical call starts at zero); required for the sLSTM cell, ignored otherwise. No
 *               host read is involved, so the call can be captured in a CUDA graph.
 * Everything else as frnn_b200_forward. */
int frnn_b200_forward_prepared(int cell, const void* wx, int wx_bf16, const void* r_bf16, const float* bias,
                               const float* initial, void* output, float* carry, void* xchg, int B, int T, int N,
                               int D, int output_mode, const int* slstm_zero_first_dev, int wait_limit_ms, int* err,
                               void* stream);

/* One chunk [t_start, t_start + steps) of a prepared sequence of T_total steps (the chunked execution with
 * alternating carries of flashrnn/flashrnn2/prepared.py:61-63,120-159): wx and output are the tensors of the WHOLE
 * sequence, `initial` is the carry of the previous chunk (the sequence's initial state for the first one), `carry`
 * receives this chunk's final state. With output_bf16 = 1 the state snapshots are stored as bf16 (prepared.py:21,
 * 58-60 snapshot_dtype); carries stay fp32. The sLSTM word must hold the predicate of the sequence's initial state;
 * it only takes effect in the chunk that contains step 0. output_mode 2 ("last") writes h of the chunk's last step. */
int frnn_b200_forward_chunk(int cell, const void* wx, int wx_bf16, const void* r_bf16, const float* bias,
                            const float* initial, void* output, int output_bf16, float* carry, void* xchg, int B,
                            int T_total, int t_start, int steps, int N, int D, int output_mode,
                            const int* slstm_zero_first_dev, int wait_limit_ms, int* err, void* stream);

/* Reverse-time recurrence (flashrnn/flashrnn/fused/flashrnn.cc:147-247 backward();
 * gradient structure of flashrnn/flashrnn/vanilla_fwbw/bw.py:20-98).
 *   cache, history, initial : as written / passed in the forward call
 *   d_history [S,B,T,N,D], d_carry [S,B,1,N,D] : incoming gradients, fp32
 *   dwx  : out, [B,T,GW,N,D] in the Wx dtype
 *   dgr  : out scratch, bf16 [B,T,GR,N,D] (operand of frnn_b200_wgrad). With bf16 Wx and a cell whose Wx gates
 *          are its recurrent gates (lstm, slstm, elman) dwx and dgr hold the same values in the same layout: the
 *          caller may pass the SAME buffer for both, which is then written once (saves the second copy's traffic)
 *   d_initial : out fp32 [S,B,1,N,D];  db_part: out scratch fp32 [n_btiles,GB,N,D]    */
int frnn_b200_backward(int cell, const void* cache, const float* history, const float* initial,
                       const void* r_bf16, const float* d_history, const float* d_carry, void* dwx,
                       int wx_bf16, void* dgr, float* d_initial, float* db_part, void* xchg, int B,
                       int T, int N, int D, int slstm_zero_first, int wait_limit_ms, int* err,
                       void* stream);

/* dR[g,n,o,p] = sum_{b,t} dgr[b,t,g,n,o] * hbf[b,t,n,p] and db = sum over batch tiles of
 * db_part (the cuBLAS GEMM + gradientBiasAggregationKernel of
 * flashrnn/flashrnn/fused/flashrnn_fused_backward.cu:1050-1070, 627-666). Outputs fp32,
 * overwritten (not accumulated). `work`: split-K scratch of plan.wgrad_work_bytes (may be
 * NULL when that is 0).                                                               */
int frnn_b200_wgrad(int cell, const void* dgr, const void* hbf, const float* db_part, float* dR,
                    float* db, float* work, int B, int T, int N, int D, int* err, void* stream);

/* Same result as frnn_b200_wgrad, for callers that cannot hand over scratch memory: hosts that
 * must not call cudaMalloc once they are running (it synchronises the device), processes with a
 * memory budget fixed at start-up, or thin plugins that only ever see input and output pointers.
 * This entry point has no counterpart in the reference. The split-K partial tiles go to a fixed
 * 16 MiB array inside the library image (each GPU that loads the library holds it until the
 * process exits); the call returns -6 when plan.wgrad_work_bytes exceeds that. It allocates
 * nothing. The first call on a device looks up the array's device address (a one-time set-up
 * that should happen before any stream capture starts). All calls on a device share the array:
 * calls that overlap on the GPU race with each other; consecutive calls on one stream are safe,
 * and no clearing is needed because every partial tile is rewritten before it is reduced. */
int frnn_b200_wgrad_noalloc(int cell, const void* dgr, const void* hbf, const float* db_part,
                            float* dR, float* db, int B, int T, int N, int D, int* err,
                            void* stream);

/* Input projection in front of the recurrence: wx[b,t,j] = sum_i x[b,t,i] * w[j,i] (+ bias[j]), j = (gate, head,
 * unit), i.e. Wx[B,T,GW,N,D] in the layout frnn_b200_forward streams, as bf16 (wx_bf16 = 1) or fp32. x [B,T,inputs] and
 * w [GW*N*D, inputs] are bf16, bias fp32 [GW*N*D] or NULL; inputs % 8 == 0, gates_times_width % 64 == 0, wx and bias
 * 16-byte aligned (else -2).
 * The reference leaves this GEMM to the caller (README.md:16) and times it as the "-withlinear" variant of its
 * benchmark: a torch.nn.Linear in front of the kernel (flashrnn/speed_experiments/kernel_speed_benchmark.py:388-408). */
int frnn_b200_input_projection(const void* x_bf16, const void* w_bf16, const float* bias, void* wx, int wx_bf16, int B,
                               int T, int gates_times_width, int inputs, int* err, void* stream);

/* ------------------------------------------------------------------------------------------------
 * One WIDE head (N = 1, D a multiple of 256) whose recurrent matrix is split over P GPUs of a node:
 * rank r owns the hidden units [r*Dl, (r+1)*Dl), Dl = D/P (a multiple of 128): the rows R[g, o in slice, :] in the
 * forward pass and the columns R[g, :, p in slice] in the backward pass; the per-step operand (round_bf16(h_t),
 * round_bf16(dG_t)) is exchanged by peer stores issued inside the kernels, receivers poll their own memory.
 * Counterparts in the reference: flashrnn/flashrnn2/multi_gpu.py:87-297 (forward; peer stores and counters
 * :224-238, bounded waits :30-32,62-73, address tables before the first launch :429) and the `_mg` entry point
 * flashrnn/flashrnn2/hybrid_bw2d.cu:645-661 (backward with peer tables, rank, np).
 *
 * Local tensors of a rank are dense with row length Dl: Wx[B,T,GW,Dl], R rows [GR,Dl,D], R columns [GR,D,Dl],
 * b[GB,Dl], states [S,B,T|1,Dl], dR rows [GR,Dl,D]. With ranks_here == P all ranks run as ONE launch on one GPU
 * (how the multi-rank arithmetic is tested on a single device): the local tensors then are the full-width ones
 * (row length D) and rank r works on the columns [r*Dl, (r+1)*Dl) of them.
 * At most 32 batch rows per call. Every wait inside the kernels is bounded by wait_limit_ms (0 = 10 s: ranks
 * start their kernels at different times); a wait that runs out is reported through err[0..2] of that rank
 * (108: a peer never became ready, 109: weight stage) and the kernel returns. */
typedef struct frnn_b200_mg_shard {
  int P;               /* ranks the head is split over, 1..8                                              */
  int rank;            /* this rank (the first rank of the launch)                                        */
  int ranks_here;      /* 1: one rank per launch (one process per GPU); P: all ranks in one launch        */
  int epoch;           /* identical on all ranks, larger in every later call that uses the same `ready`   */
  int k_tmem_max;      /* 0 = default; caps the weight columns kept in tensor memory (tuning / tests)     */
  int ring_stages_max; /* 0 = default; caps the shared-memory stages of the weight operand                */
  void* buffers[8];    /* every rank's exchange buffer of this call, as addresses valid on THIS device:
                          forward  bf16 [B][T+1][D]   (plan.hbf_bytes), afterwards operand of the dR contraction
                          backward bf16 [B][T][GR][D] (plan.dgr_bytes), likewise. The call fills the buffers of
                          its own rank(s) with 0xFF bytes before the launch.                             */
  int* ready[8];       /* every rank's int[8] flag array (zeroed once when allocated); unused when
                          ranks_here == P                                                                 */
} frnn_b200_mg_shard_t;

typedef struct frnn_b200_mg_plan {
  int supported;
  int local_width;                 /* Dl */
  int fwd_ksplit, fwd_ctas;        /* CTAs per row tile (cluster width) and per launch                     */
  int fwd_k_tmem, fwd_ring_chunks, fwd_ring_stages, fwd_resident;
  int bwd_ksplit, bwd_ctas;
  int bwd_k_tmem, bwd_ring_chunks, bwd_ring_stages, bwd_resident;
  int64_t hbf_bytes, dgr_bytes;    /* one rank's exchange buffers                                          */
  int64_t cache_bytes;             /* [B][T][GC][row length], fp16 (lstm, gru) or fp32 (slstm)             */
  int64_t r_cols_bytes;            /* bf16 [GR][D][row length]                                             */
  int64_t dbpart_bytes;            /* fp32 [bwd_ksplit][GB][row length]                                    */
} frnn_b200_mg_plan_t;

int frnn_b200_mg_plan(int cell, int B, int T, int D, int wx_bf16, const frnn_b200_mg_shard_t* shard,
                      frnn_b200_mg_plan_t* out);

/* How many CTAs of the forward (forward != 0) or backward launch with `ksplit` CTAs per tile the current device
 * holds at once (thread-block clusters are placed inside one GPC, so this can be less than the SM count); the
 * counterpart of the reference's frnn_hybrid_fw2d_ctas() query (flashrnn/flashrnn2/hybrid_fw2d.cu:404-419). */
int frnn_b200_mg_capacity(int cell, int forward, int ksplit, int D, int P, int wx_bf16);

/* Forward (multi_gpu.py:87-297). sh->buffers = the ranks' h histories. Outputs: history [S,B,T,Dl], carry [S,B,1,Dl],
 * cache (NULL for inference). The h history of this rank holds round_bf16(h) of ALL units afterwards (slots 0..T-1). */
int frnn_b200_mg_forward(int cell, const void* wx, int wx_bf16, const void* r_rows, const float* bias,
                         const float* initial, float* history, float* carry, void* cache,
                         const frnn_b200_mg_shard_t* shard, int B, int T, int D, int slstm_zero_first,
                         int wait_limit_ms, int* err, void* stream);

/* r_cols[g, o, pl] = R[g, o, rank*Dl + pl] from the ranks' row slices (r_rows_all[q] = rank q's [GR,Dl,D], addresses
 * valid on this device; plain peer loads). Once per call of the backward (hybrid_bw2d.cu:645-661 takes the
 * column slice as an input). */
int frnn_b200_mg_gather_columns(int cell, const void* const* r_rows_all, void* r_cols,
                                const frnn_b200_mg_shard_t* shard, int D, void* stream);

/* Backward (hybrid_bw2d.cu:507-552,645-661). sh->buffers = the ranks' dG histories. Outputs: dwx [B,T,GW,Dl] in the
 * Wx dtype, d_initial [S,B,1,Dl], db_part [plan.bwd_ksplit][GB][Dl]. */
int frnn_b200_mg_backward(int cell, const void* cache, const float* history, const float* initial,
                          const void* r_cols, const float* d_history, const float* d_carry, void* dwx, int wx_bf16,
                          float* d_initial, float* db_part, const frnn_b200_mg_shard_t* shard, int B, int T, int D,
                          int slstm_zero_first, int wait_limit_ms, int* err, void* stream);

/* dR rows [GR,Dl,D] of this rank's units and db [GB,Dl] from this rank's two histories: disjoint slices, no
 * reduction over ranks (the reference gathers dG on rank 0 instead, flashrnn/flashrnn2/hybrid_bw.py:280-286). */
int frnn_b200_mg_wgrad(int cell, const void* dgr_all, const void* hbf_all, const float* db_part, float* dR_rows,
                       float* db, const frnn_b200_mg_shard_t* shard, int B, int T, int D, int bwd_ksplit, int* err,
                       void* stream);

/* Buffers that other processes of the node can address (cudaMalloc + CUDA IPC; no multicast object is created).
 * Set-up calls, never used on the hot path: alloc / free in the owning process, export there, open / close in
 * the peers (open enables peer access). The reference builds its peer address tables the same way before the
 * first launch (flashrnn/flashrnn2/multi_gpu.py:313-335,429). */
int frnn_b200_peer_alloc(size_t bytes, void** ptr);
int frnn_b200_peer_free(void* ptr);
int frnn_b200_peer_export(void* ptr, unsigned char handle[64]);
int frnn_b200_peer_open(const unsigned char handle[64], void** ptr);
int frnn_b200_peer_close(void* ptr);

#ifdef __cplusplus
}
#endif

#endif /* FLASHRNN_B200_H_ */
