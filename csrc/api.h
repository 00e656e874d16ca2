// Raw-pointer launch API of the native library.  Everything here is torch-free; the tensor
// glue in bindings.cpp fills these structs from torch tensors.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace rt {

// ------------------------------------------------------------------ gemm/gemm_tcgen05.cu
enum EpiMode : int {
  EPI_NONE = 0,       // C = alpha*acc (+bias)
  EPI_GELU_DUAL = 1,  // aux = alpha*acc+bias ; C = gelu(aux)
  EPI_DGELU = 2,      // C = alpha*acc * gelu'(aux)
  EPI_RESIDUAL = 3,   // C = alpha*acc + bias + aux
};

struct GemmArgs {
  const void* a;  // K-major: [batch][M][K] ; MN-major: [batch][K][M]  (bf16)
  bool a_mn;
  long long lda, a_batch_stride;  // in elements
  const void* b;  // K-major: [batch][N][K] ; MN-major: [batch][K][N]  (bf16)
  bool b_mn;
  long long ldb, b_batch_stride;
  void* c;  // [batch][M][N] bf16 or fp32
  long long ldc, c_batch_stride;
  bool out_fp32;
  const void* bias;  // bf16 [N] or null
  void* aux;         // bf16, geometry of C, or null
  long long ld_aux, aux_batch_stride;
  int M, N, K, batch;
  int epi_mode;
  float alpha;
  bool accumulate;  // fp32 C only: C += result with float atomics
  int split_k;
  int block_n;  // 0 = auto, 128 or 256
  bool ab_fp16 = false;  // A/B hold fp16 (C must be fp32, no fused epilogue)
  const float* alpha_dev = nullptr;  // optional fp32 device scalar: the result is scaled by alpha * (*alpha_dev)
};
void gemm_bf16(const GemmArgs& g, cudaStream_t stream);

// ------------------------------------------------------- attention/flash_{fwd,bwd}.cu
// q: [B][Tq][H][D], k/v: [B][Tk][Hkv][D] as strided views (strides in elements, D contiguous).
struct AttnArgs {
  const void *q, *k, *v;
  long long q_sb, q_st, q_sh, k_sb, k_st, k_sh, v_sb, v_st, v_sh;
  void* o;  // bf16, [B][Tq][H][D] strided
  long long o_sb, o_st, o_sh;
  float* lse;  // [B][H][Tq] natural-log sum-exp of the scaled scores
  int B, H, Hkv, Tq, Tk, D;
  int causal;
  float scale;
  int io_fp16 = 0;  // forward only: q / k / v / o are fp16 instead of bf16
  // backward only
  const void* d_o;  // same strides as o
  float* delta;     // [B][H][Tq] scratch: rowsum(o * do)
  float* dq_acc = nullptr;  // optional fp32 scratch [B][Tq][H][D]: enables the single-kernel backward for D == 64
  void *dq, *dk, *dv;  // bf16, strides below
  long long dq_sb, dq_st, dq_sh, dk_sb, dk_st, dk_sh, dv_sb, dv_st, dv_sh;
};
void attn_fwd(const AttnArgs& a, cudaStream_t stream);
void attn_bwd(const AttnArgs& a, cudaStream_t stream);

// ----------------------------------------------------------------------- norm/norm.cu
struct NormArgs {
  const void* x;      // bf16 [rows][C]
  const void* gamma;  // bf16 [C]
  const void* beta;   // bf16 [C] or null (ignored for RMSNorm)
  void* y;            // bf16 [rows][C]               (forward)
  float* mean;        // fp32 [rows] (LayerNorm only; may be null for RMSNorm)
  float* rstd;        // fp32 [rows]
  long long rows;
  int C;
  float eps;
  bool rms;
  // backward
  const void* dy;    // bf16 [rows][C]
  const void* dres;  // bf16 [rows][C] or null: added to dx
  void* dx;          // bf16 [rows][C]
  float* dgamma;     // fp32 [C], accumulated into (may be null)
  float* dbeta;      // fp32 [C], accumulated into (may be null)
  float* partial;    // backward scratch: fp32 [2][n_partial][C] per-CTA partial sums
  int n_partial;     // = norm_bwd_num_partials(rows, sm_count)
};
void norm_fwd(const NormArgs& a, cudaStream_t stream);
void norm_bwd(const NormArgs& a, cudaStream_t stream);
// The two stages separately: stage 1 writes dx and the partial sums (and runs stage 2 itself when `reduce_stream` is
// null); norm_bwd_reduce folds the partial sums into dgamma / dbeta.
void norm_bwd_stage1(const NormArgs& a, cudaStream_t stream, const cudaStream_t* reduce_stream);
void norm_bwd_reduce(const NormArgs& a, cudaStream_t stream);
// Number of CTAs (and therefore partial-sum rows) the backward kernel uses for `rows` rows.
int norm_bwd_num_partials(long long rows, int sm_count);

// ------------------------------------------------------------------ norm/batchnorm.cu
// Channels-last matrix x[M][C]; gamma/beta/statistics fp32; scratch fp32 [2][C].
struct BatchNormArgs {
  int dtype;             // DType of x / y / residual / dy / dx
  const void* x;
  const void* residual;  // added before the ReLU, or null
  void* y;
  const float *gamma, *beta;                // may be null (affine = false)
  float *running_mean, *running_var;        // updated in training when non-null; read in inference
  float *save_mean, *save_rstd;             // [C], written in training, read by backward
  float* scratch;
  long long M;
  int C;
  float eps, momentum;
  int relu, training;
  // backward
  const void* dy;
  const void* y_relu;  // forward output when ReLU was fused (masks dy), else null
  void* dx;
  void* dres;          // gradient of the residual branch (= masked dy), or null
};
void batchnorm_fwd(const BatchNormArgs& a, cudaStream_t s);
void batchnorm_bwd(const BatchNormArgs& a, cudaStream_t s);

// ------------------------------------------------------------------ norm/groupnorm.cu
// Contiguous x[N][C][HW]; G groups (G == C: InstanceNorm); gamma/beta/statistics fp32; mean/rstd [N*G].
struct GroupNormArgs {
  int dtype;
  const void* x;
  void* y;
  const float *gamma, *beta;  // may be null
  float *mean, *rstd;         // written by forward, read by backward
  long long N;
  int C, G;
  long long HW;
  float eps;
  // backward
  const void* dy;
  void* dx;
  float *dgamma, *dbeta;      // fp32 [C], accumulated into (caller zeroes), may be null
};
void groupnorm_fwd(const GroupNormArgs& a, cudaStream_t s);
void groupnorm_bwd(const GroupNormArgs& a, cudaStream_t s);

// ------------------------------------------------------------------- nn/embedding.cu
void embedding_fwd(const long long* idx, const void* wte, const void* wpe, void* out,
                   long long rows, int T, int C, int vocab, cudaStream_t stream);
void embedding_bwd(const long long* idx, const void* dout, float* dwte, float* dwpe,
                   long long rows, int T, int C, int vocab, cudaStream_t stream);

// ------------------------------------------------------------- loss/cross_entropy.cu
// logits: bf16 [rows][ld] (ld >= vocab, ld % 8 == 0), overwritten with the gradient.
void cross_entropy_fwd_bwd(void* logits, const long long* targets, float* loss, long long rows,
                           int vocab, int ld, float grad_scale, long long ignore_index,
                           cudaStream_t stream);

// ------------------------------------------------------------------ reduce/reduce.cu
void colsum_accum(const void* x_bf16, float* out, long long M, int N, long long ld,
                  cudaStream_t stream);
// dtype: 0 fp32, 1 bf16.  mode: 0 sum, 1 sum of squares, 2 max, 3 min.  *out pre-initialised.
void reduce_all(const void* x, int dtype, int mode, float* out, long long n, cudaStream_t stream);

// --------------------------------------------------------------- optim/fused_optim.cu
enum OptimMode : int { OPT_ADAMW = 0, OPT_ADAM = 1, OPT_SGD = 2 };
struct OptimArgs {
  float* master;   // fp32 parameters [n]
  float* grad;     // fp32 gradients  [n]
  float* m;        // first moment / momentum buffer (null for plain SGD)
  float* v;        // second moment (null for SGD)
  void* param_lp;  // bf16 copy of the parameters to refresh, or null
  long long n;
  float lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, grad_scale;
  int mode;
  int zero_grad;
  int nesterov;
  int first_step;
};
void fused_optim_step(const OptimArgs& a, cudaStream_t stream);

// ---------------------------------------------------------- quant/gemm_i8_tcgen05.cu
// acc = A_s8[M][K] . B_s8[N][K]^T on the integer tensor cores.  Output either the raw int32 accumulator or
// fp32 acc * row_scale * col_scale + bias (scales per tensor or per row / column).
struct GemmI8Args {
  const void* a;   // s8 [M][K], row stride lda (elements = bytes, multiple of 16)
  const void* b;   // s8 [N][K], row stride ldb
  long long lda, ldb;
  int M, N, K;     // K a multiple of 16
  int32_t* c_i32 = nullptr;
  float* c_f32 = nullptr;
  long long ldc = 0;
  const float* row_scale = nullptr;  // fp32 output: [M] when row_scale_per_row, else one value
  const float* col_scale = nullptr;  // fp32 output: [N] when col_scale_per_col, else one value
  const float* bias = nullptr;       // fp32 [N] or null
  bool row_scale_per_row = false, col_scale_per_col = false;
};
void gemm_i8(const GemmI8Args& g, cudaStream_t stream);

// ------------------------------------------------------- optim/multi_tensor_optim.cu
enum MultiTensorMode : int {
  MT_ADAM = 0, MT_ADAMW, MT_SGD, MT_NADAM, MT_RADAM, MT_ADAMAX, MT_RMSPROP, MT_ADAGRAD, MT_ADABOUND, MT_LAMB_STAGE1, MT_LAMB_STAGE2
};
constexpr int MT_MAX_TENSORS = 32;
struct MultiTensorArgs {
  void* param[MT_MAX_TENSORS];        // fp32 or bf16 (param_bf16)
  const void* grad[MT_MAX_TENSORS];   // fp32 or bf16 (grad_bf16)
  float* state0[MT_MAX_TENSORS];      // first moment / momentum buffer, or null
  float* state1[MT_MAX_TENSORS];      // second moment / infinity norm / square average / sum of squares, or null
  float* state2[MT_MAX_TENSORS];      // centered RMSprop: gradient average, else null
  long long numel[MT_MAX_TENSORS];
  int chunk_start[MT_MAX_TENSORS + 1];  // filled by the launcher
  int n_tensors;
  int mode;                           // MultiTensorMode
  int param_bf16, grad_bf16;
  int decoupled, maximize;
  float lr, beta1, beta2, eps, weight_decay, grad_scale;
  float c0, c1, c2;                   // per-step scalars of the rule (see multi_tensor_optim.cu)
  float* norms;                       // LAMB: fp32 [2 * total tensors] (|w|^2, |update|^2), zeroed before stage 1
  int tensor_base;                    // index of param[0] in the norm table
};
void multi_tensor_optim_step(MultiTensorArgs& a, cudaStream_t stream);

// ------------------------------------------------------------ collective/ddp_fused.cu
constexpr int RT_MAX_PEERS = 8;
struct DdpBucketArgs {
  float* grad[RT_MAX_PEERS];  // every rank's flat fp32 gradient buffer (peer pointers)
  void* lp[RT_MAX_PEERS];     // every rank's flat bf16 parameter buffer (peer pointers)
  int* flags[RT_MAX_PEERS];   // every rank's flag array (peer pointers)
  float* mc_grad = nullptr;   // multicast (NVLS) mapping of the gradient buffers, or null: plain peer loads / stores
  void* mc_lp = nullptr;      // multicast mapping of the bf16 parameter buffers (needed together with mc_grad)
  float* master;              // local flat fp32 master weights / moments (indexed like grad)
  float* m;                   // first moment / momentum buffer (null for SGD without momentum)
  float* v;                   // second moment (null for SGD)
  unsigned* done_counter;     // local, zero-initialised
  long long bucket_start;     // flat index of the bucket
  long long chunk_len;        // elements owned by each rank inside the bucket (multiple of 4)
  int world, rank;
  int epoch;                  // strictly increasing per step
  int start_slot, end_slot;   // offsets into the flag arrays (slot * world)
  unsigned long long timeout_ns;
  int opt_mode = 0;           // OptimMode: OPT_ADAMW, OPT_ADAM or OPT_SGD (beta1 = momentum, beta2 = dampening)
  int nesterov = 0, first_step = 0;
  float lr, beta1, beta2, eps, weight_decay, bias_corr1, bias_corr2, grad_scale;
  int* status;
};
void ddp_bucket_step(const DdpBucketArgs& a, int n_ctas, cudaStream_t stream);  // n_ctas <= 0: two per SM
void ddp_wait_end(const int* flags, int n_slots, int world, int rank, int epoch,
                  unsigned long long timeout_ns, int* status, cudaStream_t stream);

// ------------------------------------------------------------------ conv/conv2d_igemm.cu
// Channels-last bf16 tensors: x [N][H][W][Cin], w [Cout][KH][KW][Cin], out / dy [N][OH][OW][Cout]; dw fp32 like w.
struct Conv2dArgs {
  int N, H, W, Cin, Cout, KH, KW, stride, pad;  // pad: both directions unless pad_h >= 0 (then pad is along W only)
  int pad_h = -1;
  const void* x;
  const void* w;
  void* out;
  const void* bias;  // bf16 [Cout] or null (forward)
  const void* dy;    // wgrad
  float* dw;         // wgrad: accumulated into (zero it first)
  // forward only: explicit output extent and element strides of the output view (0 = derive / contiguous NHWC).
  // Used by the strided input gradient, which writes every stride-th pixel of dx from a stride-1 convolution of dy.
  int out_h = 0, out_w = 0;
  long long out_sn = 0, out_sh = 0, out_sw = 0;
};
bool conv2d_igemm_supported(int Cin, int Cout, int KH, int KW, int stride);
void conv2d_fwd(const Conv2dArgs& a, cudaStream_t stream);
void conv2d_wgrad(const Conv2dArgs& a, cudaStream_t stream);

// ------------------------------------------------------- elementwise/elementwise.cu, softmax.cu
enum DType : int { DT_F32 = 0, DT_BF16 = 1, DT_F16 = 2 };
enum BinaryOp : int { EW_ADD = 0, EW_SUB, EW_MUL, EW_DIV, EW_MAX, EW_MIN, EW_POW };
enum UnaryOp : int {
  ACT_RELU = 0, ACT_SIGMOID, ACT_TANH, ACT_GELU_TANH, ACT_GELU_ERF, ACT_SILU, ACT_ELU, ACT_LEAKY_RELU, ACT_SELU,
  ACT_MISH, ACT_SOFTPLUS, ACT_HARDTANH, ACT_RELU6, ACT_HARDSIGMOID, ACT_HARDSWISH, ACT_EXP, ACT_LOG, ACT_SQRT,
  ACT_RSQRT, ACT_NEG, ACT_ABS, ACT_SQUARE, ACT_SIN, ACT_COS, ACT_SCALE_SHIFT, ACT_RECIPROCAL
};
// mode 0: out = op(a, b) ; 1: out = op(a, scalar) ; 2: out = op(scalar, a).  ADD/SUB use a +- alpha * b.
void elementwise_binary(int op, int dtype, const void* a, const void* b, void* out, long long n, float scalar,
                        float alpha, int mode, cudaStream_t s);
// forward: out = f(x; p0, p1) ; backward: out = dy * f'(x; p0, p1)
void elementwise_unary(int op, int dtype, const void* x, const void* dy, void* out, long long n, float p0, float p1,
                       bool backward, cudaStream_t s);
// rows x C (contiguous rows, stride ld).  log_mode: 0 softmax, 1 log_softmax.
void softmax_rows_fwd(int dtype, const void* x, void* y, long long rows, int C, long long ld, int log_mode, cudaStream_t s);
// dx = y * (dy - sum(dy * y))  (softmax) ; dx = dy - exp(y) * sum(dy)  (log_softmax); y is the forward OUTPUT.
void softmax_rows_bwd(int dtype, const void* y, const void* dy, void* dx, long long rows, int C, long long ld, int log_mode,
                      cudaStream_t s);
// Row reductions over the last dim: mode 0 sum, 1 mean, 2 max, 3 min, 4 variance (unbiased = p0 != 0), out fp32 [rows].
void reduce_rows(int dtype, const void* x, float* out, long long rows, int C, long long ld, int mode, float p0, cudaStream_t s);

// ------------------------------------------------------ collective/p2p_collectives.cu
enum P2PMode : int { P2P_ALL_REDUCE_ONE_SHOT = 0, P2P_ALL_REDUCE_TWO_SHOT = 1, P2P_ALL_GATHER = 2, P2P_REDUCE_SCATTER = 3, P2P_BROADCAST = 4 };
struct P2PCollArgs {
  int mode, dtype, world, rank, root;
  long long numel;               // elements of one rank's input (all-gather: per-rank count; others: full length)
  const void* in[RT_MAX_PEERS];  // every rank's input buffer (symmetric)
  void* result[RT_MAX_PEERS];    // two-shot all-reduce: every rank's result buffer (symmetric), else unused
  void* out;                     // local output
  int* flags[RT_MAX_PEERS];      // symmetric int32[3 * world], zero-initialised once
  int* epoch_dev;                // local int32, zero-initialised once; the kernel advances it
  unsigned* grid_counter;        // local uint32[2], zero-initialised once
  unsigned long long timeout_ns;
  int* status;
};
void p2p_collective(const P2PCollArgs& a, cudaStream_t stream);

// conv/im2col.cu: patch matrix [N*OH*OW][k_pad] of a channels-last bf16 image (rows zero-padded to k_pad)
void im2col_nhwc(const void* x, void* col, int N, int H, int W, int C, int OH, int OW, int KH, int KW, int stride, int pad, int k_pad,
                 cudaStream_t s);
// conv/unfold_nd.cu: patch gather / scatter for 1-3 D convolutions with stride, padding, dilation and groups on
// channels-last bf16 tensors; col is [groups][N*OD*OH*OW][k_pad] with k_pad >= KD*KH*KW*(C/groups), a multiple of 8.
struct UnfoldArgs {
  const void* x_in = nullptr;  // unused alias kept zero; x below is read by unfold_nd and written by fold_nd
  void* x;
  void* col;
  int N, D, H, W, C;
  int OD, OH, OW;
  int KD, KH, KW;
  int stride[3], pad[3], dilation[3];
  int groups;
  int k_pad;
};
void unfold_nd(const UnfoldArgs& a, cudaStream_t s);
void fold_nd(const UnfoldArgs& a, cudaStream_t s);
// ------------------------------------------------------------ nn/pool_dropout.cu
// Channels-last pooling.  Forward: x [N][H][W][C] -> y [N][OH][OW][C] (+ idx for max).  Backward: y holds dy, x receives dx.
struct Pool2dArgs {
  int dtype;
  bool max, backward;
  void* x;              // forward: input (read); backward: dx (written)
  void* y;              // forward: output (written); backward: dy (read)
  unsigned char* idx;   // max pooling: window position of the maximum per output element
  int N, H, W, C, OH, OW, kh, kw, sh, sw, ph, pw;
};
void pool2d(const Pool2dArgs& a, cudaStream_t stream);
void dropout(int dtype, const void* x, void* y, long long n, float p, unsigned long long seed, unsigned long long offset,
             cudaStream_t stream);
// ------------------------------------------------------------ nn/llama_ops.cu (bf16)
// forward: packed [rows][(H + 2 Hkv) D] -> q, k (rotated), v; backward: (dq, dk, dv) -> packed gradient (inverse rotation).
void rope_split(void* packed, void* q, void* k, void* v, const float* cos_t, const float* sin_t, long long rows, int T, int H, int Hkv,
                int D, bool backward, cudaStream_t s);
// forward: out[rows][F] = silu(gu[:, :F]) * gu[:, F:]; backward: out[rows][2F] = d(gate) | d(up) from dact.
void swiglu(const void* gu, const void* dact, void* out, long long rows, int F, bool backward, cudaStream_t s);
// ------------------------------------------------------------ nn/rnn_amp_sparse.cu
void lstm_gates_fwd(int dtype, void* gates, const void* c, void* h_out, void* c_out, int B, int H, cudaStream_t s);
void lstm_gates_bwd(int dtype, const void* act, const void* c, const void* c_new, const void* dh, const void* dc_new, void* dgates,
                    void* dc, int B, int H, cudaStream_t s);
void gru_gates_fwd(int dtype, const void* gi, const void* gh, const void* h, void* h_out, void* save, int B, int H, cudaStream_t s);
void gru_gates_bwd(int dtype, const void* save, const void* h, const void* dh_new, void* dgi, void* dgh, void* dh, int B, int H,
                   cudaStream_t s);
void amp_unscale(int dtype, void* grads, long long n, float inv_scale, float* found_inf, cudaStream_t s);
void csr_spmm(const long long* row_ptr, const long long* col, const float* val, const float* x, float* y, long long rows, int n_dense,
              cudaStream_t s);

// ------------------------------------------------------ collective/ar_residual_norm.cu
// x[rows][d] += sum over ranks of partial[rows][d]; h = rmsnorm(x) * w (h may be null).  fp16 / bf16.
struct ArNormArgs {
  int dtype, world, rank;
  int rows, d;
  float eps;
  void* bufs[RT_MAX_PEERS];   // symmetric receive buffers [3][world][cap_numel], every 16-bit lane pre-set to 0x8000
  long long cap_numel;        // elements per (slot, source) region
  const void* partial;        // this rank's partial sums
  void* x;                    // residual stream, updated in place
  const void* w;              // norm weight [d] or null
  void* h;                    // normalised output or null
  int* state;                 // local int32[8], zero-initialised once
  unsigned long long timeout_ns;
  int* status;
};
void ar_residual_norm(const ArNormArgs& a, cudaStream_t stream);

// ------------------------------------------------------------ collective/tp_gemm.cu
// mode 0: y[W*rows][N] = all_gather(x_shards)[.][K] . B^T (+bias)      (x_shards, flags: symmetric peer pointers)
// mode 1: out[rows][N] = reduce_scatter(x[W*rows][K] . B^T) (+bias) (+residual)   (stage, flags: symmetric)
struct TpGemmArgs {
  int mode;
  int world, rank, epoch;      // epoch: 1, 2, 3, ... per call on the same buffers
  int rows_per_rank, N, K;     // rows_per_rank multiple of 128
  const void* b;               // weights: [N][K] (b_mn = false) or [K][N] (b_mn = true), bf16
  bool b_mn;
  long long ldb;
  void* out;
  long long ld_out;
  const void* bias;            // bf16 [N] or null
  const void* residual;        // mode 1: bf16 [rows][ld_res] or null
  long long ld_res;
  unsigned long long timeout_ns;
  int* flags[RT_MAX_PEERS];    // int32[2*world + (rows_per_rank/128)*world] per rank, zero-initialised once
  // mode 0
  const void* x_shards[RT_MAX_PEERS];  // every rank's [rows_per_rank][K] shard
  void* gather;                        // local [W*rows_per_rank][K]
  int* mb_ready;                       // local int32[W*rows_per_rank/128], zero-initialised once
  unsigned* comm_done;                 // local, zero-initialised once
  int n_comm;                          // copy CTAs (0 = default 8)
  // mode 1
  const void* x;                       // local [W*rows_per_rank][ld_x]
  long long ld_x;
  void* stage[RT_MAX_PEERS];           // every rank's staging: bf16 [2][W][rows_per_rank][N]
};
void tp_gemm(const TpGemmArgs& a, cudaStream_t stream);

// ------------------------------------------------------------------ quant/q_gemv.cu
struct QGemvArgs {
  const void* qs;      // repacked quantised weights (layout in q_gemv.cu)
  const void* scales;  // fp16 [N][K/32]
  const void* x;       // fp16 [M][ldx]
  long long ldx;
  void* y;             // fp16 [M][ldy]
  long long ldy;
  const void* bias;      // fp16 [N] or null
  const void* residual;  // fp16 [M][ldr] or null (added to the result)
  long long ldr;
  int M, N, K;
  bool q8;  // false: Q4_0, true: Q8_0
  int path = 0;  // 0: pick by shape, 1: register-fed kernel, 2: TMA-ring kernel (tests and comparisons)
};
void q_gemv(const QGemvArgs& a, cudaStream_t stream);
// quant/q_gemv_bulk.cu: bulk-copy (TMA engine) fed variant; q_gemv() uses it when the shape allows (K % 256 == 0).
bool q_gemv_bulk_supported(const QGemvArgs& a);
bool q_gemv_bulk_preferred(const QGemvArgs& a);  // shape heuristic from measurements
void q_gemv_bulk(const QGemvArgs& a, cudaStream_t stream);
// quant/q_gemv_fused.cu: decode projection in one kernel: optional RMSNorm of x, GEMV, residual or SwiGLU epilogue.
struct QGemvFusedArgs {
  const void* qs;
  const void* scales;
  const void* x;       // fp16 [M][ldx]
  long long ldx;
  const void* norm_w;  // fp16 [K] RMSNorm weight applied to x first, or null
  float eps;
  void* y;             // fp16 [M][ldy]; swiglu: N / 2 columns
  long long ldy;
  const void* residual;  // fp16 [M][ldr] or null
  long long ldr;
  int M, N, K;         // N weight rows (swiglu: gate rows then up rows)
  bool q8;
  bool swiglu;
  // two byte ranges (the next projection's nibbles and scales) to pull towards L2 meanwhile, or null
  const void* prefetch0 = nullptr;
  long long prefetch0_bytes = 0;
  const void* prefetch1 = nullptr;
  long long prefetch1_bytes = 0;
  // rotary + KV-cache epilogue over [q; k; v] rows (interleaved pairs), when rope_pos is set
  const int* rope_pos = nullptr;  // [M] positions
  const int* rope_seq = nullptr;  // [M] sequence numbers
  void* cache_k = nullptr;        // fp16 [n_seq][Hkv][T_max][D]
  void* cache_v = nullptr;
  int rope_H = 0, rope_Hkv = 0, rope_D = 0, rope_T_max = 0, rope_n_seq = 0;
  float rope_theta = 10000.f;
};
bool q_gemv_fused_supported(int M, int N, int K, bool swiglu);
void q_gemv_fused(const QGemvFusedArgs& a, cudaStream_t stream);
// quant/q_gemm_tc.cu: dequant-fused tcgen05 GEMM for 1 <= M <= 256 rows (weights read once whatever M is).
bool q_gemm_tc_supported(int M, int N, int K);
void q_gemm_tc_scratch(int M, int N, int K, bool q8, int sms, long long* partial_floats, int* counters, int* splits_out);
void q_gemm_tc(const QGemvArgs& a, void* partial, int* counters, cudaStream_t stream);
// quant/q_gemm_ts.cu: same product with the expanded weights held in tensor memory (tcgen05.st + A-from-TMEM MMA).
void q_gemm_ts(const QGemvArgs& a, void* partial, int* counters, cudaStream_t stream);
void dequant_f16(const void* qs, const void* scales, void* out, long long n_blocks, bool q8, cudaStream_t s);
void repack_q4_0(const void* blocks, void* qs, void* scales, long long n_blocks, cudaStream_t s);
void repack_q8_0(const void* blocks, void* qs, void* scales, long long n_blocks, cudaStream_t s);

// ------------------------------------------------------------- llm/decode_kernels.cu
void rmsnorm_f16(const void* x, const void* w, void* y, long long rows, int C, float eps, cudaStream_t s);
struct RopeKvArgs {
  void *q, *k;          // fp16, rotated in place; [n_tok][H][D] / [n_tok][Hkv][D] with token strides
  const void* v;
  long long q_st, k_st, v_st;
  void *cache_k, *cache_v;  // fp16 [B][Hkv][T_max][D]
  const int* pos;           // [n_tok] position of each token in its sequence
  const int* seq;           // [n_tok] sequence (batch) index of each token
  int n_tok, H, Hkv, D, T_max;
  int n_seq;  // sequences in the cache (B): seq[t] is checked against it on the device
  float theta;
  int interleaved;  // 1: pairs (2i, 2i+1) (GGUF llama), 0: pairs (i, i + D/2)
};
void rope_kv_f16(const RopeKvArgs& a, cudaStream_t s);
struct AttnCacheArgs {
  const void* q;  // fp16 [n_tok][H][D]
  long long q_st;
  const void *cache_k, *cache_v;
  void* out;  // fp16 [n_tok][H][D]
  long long o_st;
  const int* kv_len;  // [n_tok] number of cached positions visible to the token
  const int* seq;
  int n_tok, H, Hkv, D, T_max, max_kv_len;
  int n_seq = 0;  // sequences in the cache (B)
  float scale;
  // split-KV path only: fp32 scratch [n_tok][H][n_split][D + 2] (unused when n_split == 1)
  float* partial = nullptr;
  int* counters = nullptr;  // [n_tok * Hkv] zeros (n_split > 1); every call leaves them zero
  int n_split = 1;
};
void attn_cache_f16(const AttnCacheArgs& a, cudaStream_t s);
// llm/attn_decode_split.cu: split-KV variant (D in {64,128,256}, H/Hkv in {1,2,4,8})
bool attn_decode_split_supported(int D, int H, int Hkv);
int attn_decode_num_splits(int n_tok, int Hkv, int max_kv_len, int sm_count);
void attn_decode_split(const AttnCacheArgs& a, cudaStream_t s);
void silu_mul_f16(const void* gate, const void* up, void* out, long long rows, int cols, long long g_ld,
                  long long u_ld, long long o_ld, cudaStream_t s);

}  // namespace rt
