// Bindings for the ops added after the core training path (elementwise family, quantised
// GEMV, collectives).  Kept separate so touching one group does not recompile the other.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <map>
#include <mutex>

#include <cstring>

#include "api.h"
#include "common/launch.h"

namespace {

using at::Tensor;

cudaStream_t cur_stream(int device) { return at::cuda::getCurrentCUDAStream(device).stream(); }
void check_f32_cuda_extra(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kFloat, name, ": fp32 CUDA tensor required");
}

// Peer pointers arrive as Python ints (they come from symmetric-memory rendezvous).
void ddp_bucket_step(const std::vector<int64_t>& grad_ptrs, const std::vector<int64_t>& lp_ptrs,
                     const std::vector<int64_t>& flag_ptrs, Tensor& master, const c10::optional<Tensor>& m_opt,
                     const c10::optional<Tensor>& v_opt, Tensor& done_counter, int64_t bucket_start, int64_t chunk_len,
                     int64_t rank, int64_t epoch, int64_t start_slot, int64_t end_slot, double timeout_s, double lr,
                     double beta1, double beta2, double eps, double weight_decay, double bias_corr1,
                     double bias_corr2, double grad_scale, int64_t n_ctas, int64_t opt_mode, bool nesterov,
                     bool first_step, int64_t mc_grad_ptr, int64_t mc_lp_ptr) {
  const int world = int(grad_ptrs.size());
  TORCH_CHECK(world >= 1 && world <= rt::RT_MAX_PEERS, "ddp: world size must be in [1, 8]");
  TORCH_CHECK(int(lp_ptrs.size()) == world && int(flag_ptrs.size()) == world, "ddp: pointer lists differ");
  TORCH_CHECK(master.is_cuda() && master.scalar_type() == at::kFloat && master.is_contiguous(),
              "ddp: master must be a flat fp32 CUDA buffer");
  auto state_ptr = [&](const c10::optional<Tensor>& t) -> float* {
    if (!t.has_value() || !t->defined()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == master.numel(),
                "ddp: optimizer state must be a flat fp32 CUDA buffer as long as master");
    return t->data_ptr<float>();
  };
  TORCH_CHECK(bucket_start >= 0 && bucket_start + chunk_len * world <= master.numel(),
              "ddp: bucket outside the flat buffer");
  c10::cuda::CUDAGuard guard(master.device());
  rt::DdpBucketArgs a{};
  for (int p = 0; p < world; ++p) {
    a.grad[p] = reinterpret_cast<float*>(grad_ptrs[p]);
    a.lp[p] = reinterpret_cast<void*>(lp_ptrs[p]);
    a.flags[p] = reinterpret_cast<int*>(flag_ptrs[p]);
  }
  a.master = master.data_ptr<float>();
  a.m = state_ptr(m_opt);
  a.v = state_ptr(v_opt);
  a.mc_grad = reinterpret_cast<float*>(mc_grad_ptr);
  a.mc_lp = reinterpret_cast<void*>(mc_lp_ptr);
  a.opt_mode = int(opt_mode);
  a.nesterov = nesterov ? 1 : 0;
  a.first_step = first_step ? 1 : 0;
  a.done_counter = reinterpret_cast<unsigned*>(done_counter.data_ptr<int32_t>());
  a.bucket_start = bucket_start;
  a.chunk_len = chunk_len;
  a.world = world;
  a.rank = int(rank);
  a.epoch = int(epoch);
  a.start_slot = int(start_slot);
  a.end_slot = int(end_slot);
  a.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  a.lr = float(lr);
  a.beta1 = float(beta1);
  a.beta2 = float(beta2);
  a.eps = float(eps);
  a.weight_decay = float(weight_decay);
  a.bias_corr1 = float(bias_corr1);
  a.bias_corr2 = float(bias_corr2);
  a.grad_scale = float(grad_scale);
  a.status = rt::status_word(master.device().index());
  rt::ddp_bucket_step(a, int(n_ctas), cur_stream(master.device().index()));
}

// x: channels-last bf16 [N, D, H, W, C] (contiguous), col: bf16 [groups, N*OD*OH*OW, k_pad].  fold = false gathers patches
// from x into col; fold = true sums col back into x.
void unfold_nd(Tensor& x, Tensor& col, std::vector<int64_t> out_size, std::vector<int64_t> kernel, std::vector<int64_t> stride,
               std::vector<int64_t> pad, std::vector<int64_t> dilation, int64_t groups, bool fold) {
  TORCH_CHECK(x.is_cuda() && col.is_cuda() && x.scalar_type() == at::kBFloat16 && col.scalar_type() == at::kBFloat16,
              "unfold_nd: bf16 CUDA tensors required");
  TORCH_CHECK(x.dim() == 5 && x.is_contiguous() && col.dim() == 3 && col.is_contiguous(), "unfold_nd: x [N, D, H, W, C], col [G, M, k_pad]");
  TORCH_CHECK(out_size.size() == 3 && kernel.size() == 3 && stride.size() == 3 && pad.size() == 3 && dilation.size() == 3,
              "unfold_nd: three values per geometry list");
  rt::UnfoldArgs a{};
  a.x = x.data_ptr();
  a.col = col.data_ptr();
  a.N = int(x.size(0)); a.D = int(x.size(1)); a.H = int(x.size(2)); a.W = int(x.size(3)); a.C = int(x.size(4));
  a.OD = int(out_size[0]); a.OH = int(out_size[1]); a.OW = int(out_size[2]);
  a.KD = int(kernel[0]); a.KH = int(kernel[1]); a.KW = int(kernel[2]);
  for (int i = 0; i < 3; ++i) { a.stride[i] = int(stride[i]); a.pad[i] = int(pad[i]); a.dilation[i] = int(dilation[i]); }
  a.groups = int(groups);
  a.k_pad = int(col.size(2));
  TORCH_CHECK(col.size(0) == groups && col.size(1) == int64_t(a.N) * a.OD * a.OH * a.OW, "unfold_nd: col must be [groups, N*OD*OH*OW, k_pad]");
  c10::cuda::CUDAGuard guard(x.device());
  if (fold) rt::fold_nd(a, cur_stream(x.device().index()));
  else rt::unfold_nd(a, cur_stream(x.device().index()));
}

// int8 GEMM: a [M, K] s8, b [N, K] s8 -> out int32 [M, N] (no scales) or fp32 [M, N] (scales given).
void gemm_i8(const Tensor& a, const Tensor& b, Tensor& out, const c10::optional<Tensor>& row_scale,
             const c10::optional<Tensor>& col_scale, const c10::optional<Tensor>& bias) {
  TORCH_CHECK(a.is_cuda() && b.is_cuda() && out.is_cuda(), "gemm_i8: CUDA tensors required");
  TORCH_CHECK(a.scalar_type() == at::kChar && b.scalar_type() == at::kChar, "gemm_i8: int8 operands required");
  TORCH_CHECK(a.dim() == 2 && b.dim() == 2 && out.dim() == 2 && a.stride(1) == 1 && b.stride(1) == 1 && out.stride(1) == 1,
              "gemm_i8: rank-2 operands with contiguous rows");
  TORCH_CHECK(a.size(1) == b.size(1) && out.size(0) == a.size(0) && out.size(1) == b.size(0), "gemm_i8: a [M, K], b [N, K], out [M, N]");
  c10::cuda::CUDAGuard guard(a.device());
  rt::GemmI8Args g{};
  g.a = a.data_ptr();
  g.b = b.data_ptr();
  g.lda = a.stride(0);
  g.ldb = b.stride(0);
  g.M = int(a.size(0));
  g.N = int(b.size(0));
  g.K = int(a.size(1));
  g.ldc = out.stride(0);
  if (out.scalar_type() == at::kInt) {
    g.c_i32 = out.data_ptr<int32_t>();
  } else {
    TORCH_CHECK(out.scalar_type() == at::kFloat, "gemm_i8: out must be int32 or fp32");
    TORCH_CHECK(row_scale.has_value() && col_scale.has_value(), "gemm_i8: an fp32 output needs row_scale and col_scale");
    check_f32_cuda_extra(*row_scale, "gemm_i8 row_scale");
    check_f32_cuda_extra(*col_scale, "gemm_i8 col_scale");
    TORCH_CHECK(row_scale->is_contiguous() && (row_scale->numel() == 1 || row_scale->numel() == g.M), "gemm_i8: row_scale has 1 or M values");
    TORCH_CHECK(col_scale->is_contiguous() && (col_scale->numel() == 1 || col_scale->numel() == g.N), "gemm_i8: col_scale has 1 or N values");
    g.c_f32 = out.data_ptr<float>();
    g.row_scale = row_scale->data_ptr<float>();
    g.col_scale = col_scale->data_ptr<float>();
    g.row_scale_per_row = row_scale->numel() == g.M && g.M > 1;
    g.col_scale_per_col = col_scale->numel() == g.N && g.N > 1;
    if (bias.has_value() && bias->defined()) {
      check_f32_cuda_extra(*bias, "gemm_i8 bias");
      TORCH_CHECK(bias->is_contiguous() && bias->numel() == g.N, "gemm_i8: bias has N values");
      g.bias = bias->data_ptr<float>();
    }
  }
  rt::gemm_i8(g, cur_stream(a.device().index()));
}

// One rule applied to a list of tensors; lists longer than 32 are cut into several launches.
void multi_tensor_optim(int64_t mode, const std::vector<Tensor>& params, const std::vector<Tensor>& grads,
                        const std::vector<c10::optional<Tensor>>& s0, const std::vector<c10::optional<Tensor>>& s1,
                        const std::vector<c10::optional<Tensor>>& s2, double lr, double beta1, double beta2, double eps,
                        double weight_decay, double c0, double c1, double c2, double grad_scale, bool decoupled,
                        bool maximize, const c10::optional<Tensor>& norms, int64_t tensor_base) {
  const size_t n = params.size();
  TORCH_CHECK(grads.size() == n && s0.size() == n && s1.size() == n && s2.size() == n, "multi_tensor_optim: list lengths differ");
  if (n == 0) return;
  const auto pd = params[0].scalar_type(), gd = grads[0].scalar_type();
  TORCH_CHECK(pd == at::kFloat || pd == at::kBFloat16, "multi_tensor_optim: parameters must be fp32 or bf16");
  TORCH_CHECK(gd == at::kFloat || gd == at::kBFloat16, "multi_tensor_optim: gradients must be fp32 or bf16");
  c10::cuda::CUDAGuard guard(params[0].device());
  auto state_ptr = [&](const c10::optional<Tensor>& t, const Tensor& p) -> float* {
    if (!t.has_value() || !t->defined()) return nullptr;
    TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == p.numel(),
                "multi_tensor_optim: state tensors must be contiguous fp32 CUDA tensors shaped like their parameter");
    return t->data_ptr<float>();
  };
  float* norm_ptr = nullptr;
  if (norms.has_value() && norms->defined()) {
    TORCH_CHECK(norms->is_cuda() && norms->scalar_type() == at::kFloat && norms->is_contiguous() &&
                    norms->numel() >= 2 * (tensor_base + int64_t(n)), "multi_tensor_optim: norm table too small");
    norm_ptr = norms->data_ptr<float>();
  }
  for (size_t base = 0; base < n; base += rt::MT_MAX_TENSORS) {
    rt::MultiTensorArgs a{};
    const size_t cnt = std::min<size_t>(rt::MT_MAX_TENSORS, n - base);
    for (size_t k = 0; k < cnt; ++k) {
      const Tensor& p = params[base + k];
      const Tensor& g = grads[base + k];
      TORCH_CHECK(p.is_cuda() && g.is_cuda() && p.is_contiguous() && g.is_contiguous() && p.numel() == g.numel() &&
                      p.scalar_type() == pd && g.scalar_type() == gd && p.device() == params[0].device(),
                  "multi_tensor_optim: parameters / gradients must be contiguous CUDA tensors of one dtype on one device");
      a.param[k] = p.data_ptr();
      a.grad[k] = g.data_ptr();
      a.state0[k] = state_ptr(s0[base + k], p);
      a.state1[k] = state_ptr(s1[base + k], p);
      a.state2[k] = state_ptr(s2[base + k], p);
      a.numel[k] = p.numel();
    }
    a.n_tensors = int(cnt);
    a.mode = int(mode);
    a.param_bf16 = pd == at::kBFloat16;
    a.grad_bf16 = gd == at::kBFloat16;
    a.decoupled = decoupled ? 1 : 0;
    a.maximize = maximize ? 1 : 0;
    a.lr = float(lr); a.beta1 = float(beta1); a.beta2 = float(beta2); a.eps = float(eps);
    a.weight_decay = float(weight_decay); a.grad_scale = float(grad_scale);
    a.c0 = float(c0); a.c1 = float(c1); a.c2 = float(c2);
    a.norms = norm_ptr;
    a.tensor_base = int(tensor_base + int64_t(base));
    rt::multi_tensor_optim_step(a, cur_stream(params[0].device().index()));
  }
}

void ddp_wait_end(int64_t flags_ptr, int64_t n_slots, int64_t world, int64_t rank, int64_t epoch,
                  double timeout_s, int64_t device) {
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
  rt::ddp_wait_end(reinterpret_cast<const int*>(flags_ptr), int(n_slots), int(world), int(rank),
                   int(epoch), (unsigned long long)(timeout_s * 1e9), rt::status_word(int(device)),
                   cur_stream(int(device)));
}

void check_f16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kHalf, name, ": fp16 CUDA tensor required");
}

// y[M, N] = dequant(W)[N, K] @ x[M, K]^T (+bias) (+residual); qs / scales are the repacked device layout.
static rt::QGemvArgs make_qargs(const Tensor& qs, const Tensor& scales, const Tensor& x, Tensor& y, const c10::optional<Tensor>& bias,
                                const c10::optional<Tensor>& residual, bool q8, int64_t path) {
  check_f16(scales, "q_gemv scales");
  check_f16(x, "q_gemv x");
  check_f16(y, "q_gemv y");
  TORCH_CHECK(qs.is_cuda() && qs.is_contiguous() && scales.is_contiguous(), "q_gemv: contiguous CUDA weights required");
  TORCH_CHECK(x.dim() == 2 && y.dim() == 2 && x.stride(1) == 1 && y.stride(1) == 1, "q_gemv: x [M, K], y [M, N]");
  rt::QGemvArgs a{};
  a.N = int(scales.size(0));
  a.K = int(scales.size(1)) * 32;
  a.M = int(x.size(0));
  TORCH_CHECK(x.size(1) == a.K && y.size(0) == a.M && y.size(1) == a.N, "q_gemv: shape mismatch");
  TORCH_CHECK(qs.numel() * qs.element_size() == (int64_t)a.N * (a.K / 32) * (q8 ? 32 : 16), "q_gemv: qs size mismatch");
  a.qs = qs.data_ptr();
  a.scales = scales.data_ptr();
  a.x = x.data_ptr();
  a.ldx = x.stride(0);
  a.y = y.data_ptr();
  a.ldy = y.stride(0);
  if (bias.has_value() && bias->defined()) {
    check_f16(*bias, "q_gemv bias");
    a.bias = bias->data_ptr();
  }
  if (residual.has_value() && residual->defined()) {
    check_f16(*residual, "q_gemv residual");
    TORCH_CHECK(residual->size(0) == a.M && residual->size(1) == a.N && residual->stride(1) == 1, "q_gemv: bad residual");
    a.residual = residual->data_ptr();
    a.ldr = residual->stride(0);
  }
  a.q8 = q8;
  a.path = int(path);
  return a;
}

void q_gemv(const Tensor& qs, const Tensor& scales, const Tensor& x, Tensor& y, const c10::optional<Tensor>& bias,
            const c10::optional<Tensor>& residual, bool q8, int64_t path) {
  c10::cuda::CUDAGuard guard(x.device());
  const rt::QGemvArgs a = make_qargs(qs, scales, x, y, bias, residual, q8, path);
  rt::q_gemv(a, cur_stream(x.device().index()));
}

// y = epilogue(dequant(W) @ rmsnorm(x)); norm_w / residual optional; swiglu: W = [gate; up], y has N / 2 columns.
void q_gemv_fused(const Tensor& qs, const Tensor& scales, const Tensor& x, Tensor& y, const c10::optional<Tensor>& norm_w, double eps,
                  const c10::optional<Tensor>& residual, bool q8, bool swiglu, const c10::optional<Tensor>& prefetch_qs,
                  const c10::optional<Tensor>& prefetch_scales, const c10::optional<Tensor>& rope_pos,
                  const c10::optional<Tensor>& rope_seq, const c10::optional<Tensor>& cache_k, const c10::optional<Tensor>& cache_v,
                  int64_t n_head, double rope_theta) {
  check_f16(scales, "q_gemv_fused scales");
  check_f16(x, "q_gemv_fused x");
  check_f16(y, "q_gemv_fused y");
  TORCH_CHECK(qs.is_cuda() && qs.is_contiguous() && scales.is_contiguous() && scales.dim() == 2, "q_gemv_fused: contiguous CUDA weights required");
  TORCH_CHECK(x.dim() == 2 && y.dim() == 2 && x.stride(1) == 1 && y.stride(1) == 1, "q_gemv_fused: x [M, K], y [M, N]");
  rt::QGemvFusedArgs a{};
  a.M = int(x.size(0));
  a.K = int(x.size(1));
  a.N = int(scales.size(0));
  a.q8 = q8;
  a.swiglu = swiglu;
  TORCH_CHECK(scales.size(1) * 32 == a.K, "q_gemv_fused: scales do not match K");
  TORCH_CHECK(y.size(0) == a.M && y.size(1) == (swiglu ? a.N / 2 : a.N), "q_gemv_fused: bad output shape");
  TORCH_CHECK(qs.numel() * qs.element_size() == (int64_t)a.N * (a.K / 32) * (q8 ? 32 : 16), "q_gemv_fused: qs size mismatch");
  TORCH_CHECK(rt::q_gemv_fused_supported(a.M, a.N, a.K, swiglu), "q_gemv_fused: unsupported shape");
  a.qs = qs.data_ptr();
  a.scales = scales.data_ptr();
  a.x = x.data_ptr();
  a.ldx = x.stride(0);
  a.y = y.data_ptr();
  a.ldy = y.stride(0);
  a.eps = float(eps);
  if (norm_w.has_value()) {
    check_f16(*norm_w, "q_gemv_fused norm weight");
    TORCH_CHECK(norm_w->is_contiguous() && norm_w->numel() == a.K, "q_gemv_fused: norm weight must be [K]");
    a.norm_w = norm_w->data_ptr();
  }
  if (residual.has_value()) {
    check_f16(*residual, "q_gemv_fused residual");
    TORCH_CHECK(residual->dim() == 2 && residual->size(0) == a.M && residual->size(1) == a.N && residual->stride(1) == 1, "q_gemv_fused: bad residual");
    a.residual = residual->data_ptr();
    a.ldr = residual->stride(0);
  }
  if (prefetch_qs.has_value() && prefetch_qs->is_cuda() && prefetch_qs->is_contiguous()) {
    a.prefetch0 = prefetch_qs->data_ptr();
    a.prefetch0_bytes = prefetch_qs->numel() * prefetch_qs->element_size();
  }
  if (prefetch_scales.has_value() && prefetch_scales->is_cuda() && prefetch_scales->is_contiguous()) {
    a.prefetch1 = prefetch_scales->data_ptr();
    a.prefetch1_bytes = prefetch_scales->numel() * prefetch_scales->element_size();
  }
  if (rope_pos.has_value()) {
    TORCH_CHECK(rope_seq.has_value() && cache_k.has_value() && cache_v.has_value(), "q_gemv_fused: rotary epilogue needs seq and both caches");
    TORCH_CHECK(rope_pos->scalar_type() == at::kInt && rope_seq->scalar_type() == at::kInt && rope_pos->is_cuda() && rope_seq->is_cuda() &&
                    rope_pos->numel() == a.M && rope_seq->numel() == a.M, "q_gemv_fused: int32 CUDA pos / seq, one per row");
    check_f16(*cache_k, "q_gemv_fused cache_k");
    check_f16(*cache_v, "q_gemv_fused cache_v");
    TORCH_CHECK(cache_k->dim() == 4 && cache_k->is_contiguous() && cache_v->is_contiguous() && cache_v->sizes() == cache_k->sizes(),
                "q_gemv_fused: caches [n_seq, Hkv, T_max, D], contiguous");
    a.rope_pos = rope_pos->data_ptr<int>();
    a.rope_seq = rope_seq->data_ptr<int>();
    a.cache_k = cache_k->data_ptr();
    a.cache_v = cache_v->data_ptr();
    a.rope_H = int(n_head);
    a.rope_Hkv = int(cache_k->size(1));
    a.rope_T_max = int(cache_k->size(2));
    a.rope_D = int(cache_k->size(3));
    a.rope_n_seq = int(cache_k->size(0));
    a.rope_theta = float(rope_theta);
  }
  c10::cuda::CUDAGuard guard(x.device());
  rt::q_gemv_fused(a, cur_stream(x.device().index()));
}

// (fp32 words of split-K scratch, counters, splits) for a shape on the current device
std::vector<int64_t> q_gemm_tc_scratch(int64_t M, int64_t N, int64_t K, bool q8) {
  long long pf; int nc, sp;
  rt::q_gemm_tc_scratch(int(M), int(N), int(K), q8, rt::sm_count(rt::current_device()), &pf, &nc, &sp);
  return {pf, nc, sp};
}

// partial: fp32 scratch (>= q_gemm_tc_scratch()[0] words); counters: int32 zeros, one per 128 output columns.
void q_gemm_tc(const Tensor& qs, const Tensor& scales, const Tensor& x, Tensor& y, const c10::optional<Tensor>& bias,
               const c10::optional<Tensor>& residual, bool q8, const c10::optional<Tensor>& partial, const c10::optional<Tensor>& counters,
               int64_t path) {
  c10::cuda::CUDAGuard guard(x.device());
  const rt::QGemvArgs a = make_qargs(qs, scales, x, y, bias, residual, q8, 0);
  long long pf; int nc, sp;
  rt::q_gemm_tc_scratch(a.M, a.N, a.K, q8, rt::sm_count(rt::current_device()), &pf, &nc, &sp);
  void* pp = nullptr;
  int* cc = nullptr;
  if (sp > 1) {
    TORCH_CHECK(partial.has_value() && partial->is_cuda() && partial->scalar_type() == at::kFloat && partial->numel() >= pf &&
                    counters.has_value() && counters->is_cuda() && counters->scalar_type() == at::kInt && counters->numel() >= nc,
                "q_gemm_tc: split-K scratch too small (need ", pf, " floats, ", nc, " counters)");
    pp = partial->data_ptr();
    cc = counters->data_ptr<int>();
  }
  // path 0 / 2: operand A in tensor memory; 1: operand A staged in shared memory
  if (path == 1) rt::q_gemm_tc(a, pp, cc, cur_stream(x.device().index()));
  else rt::q_gemm_ts(a, pp, cc, cur_stream(x.device().index()));
}

// GGUF block stream (uint8 [n_blocks, 18 | 34]) -> (qs, scales) device layout.
// out[N, K] fp16 = dequant(qs, scales): feeds the tensor-core GEMM on the prefill / large-batch path.
void dequant_f16(const Tensor& qs, const Tensor& scales, Tensor& out, bool q8) {
  check_f16(scales, "dequant scales");
  check_f16(out, "dequant out");
  TORCH_CHECK(qs.is_cuda() && qs.is_contiguous() && scales.is_contiguous() && out.is_contiguous(), "dequant: contiguous CUDA tensors");
  const int64_t n_blocks = scales.numel();
  TORCH_CHECK(out.numel() == n_blocks * 32 && qs.numel() * qs.element_size() == n_blocks * (q8 ? 32 : 16), "dequant: size mismatch");
  c10::cuda::CUDAGuard guard(qs.device());
  rt::dequant_f16(qs.data_ptr(), scales.data_ptr(), out.data_ptr(), n_blocks, q8, cur_stream(qs.device().index()));
}

void repack_quant(const Tensor& blocks, Tensor& qs, Tensor& scales, bool q8) {
  TORCH_CHECK(blocks.is_cuda() && blocks.scalar_type() == at::kByte && blocks.is_contiguous(), "repack: uint8 CUDA blocks");
  check_f16(scales, "repack scales");
  const int64_t bb = q8 ? 34 : 18;
  const int64_t n_blocks = blocks.numel() / bb;
  TORCH_CHECK(scales.numel() == n_blocks && qs.numel() * qs.element_size() == n_blocks * (q8 ? 32 : 16), "repack: size mismatch");
  c10::cuda::CUDAGuard guard(blocks.device());
  if (q8) rt::repack_q8_0(blocks.data_ptr(), qs.data_ptr(), scales.data_ptr(), n_blocks, cur_stream(blocks.device().index()));
  else rt::repack_q4_0(blocks.data_ptr(), qs.data_ptr(), scales.data_ptr(), n_blocks, cur_stream(blocks.device().index()));
}

void rmsnorm_f16(const Tensor& x, const Tensor& w, Tensor& y, double eps) {
  check_f16(x, "rmsnorm x");
  check_f16(w, "rmsnorm w");
  check_f16(y, "rmsnorm y");
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous(), "rmsnorm: contiguous");
  c10::cuda::CUDAGuard guard(x.device());
  const int C = int(w.numel());
  rt::rmsnorm_f16(x.data_ptr(), w.data_ptr(), y.data_ptr(), x.numel() / C, C, float(eps), cur_stream(x.device().index()));
}

void rope_kv(Tensor& q, Tensor& k, const Tensor& v, Tensor& cache_k, Tensor& cache_v, const Tensor& pos,
             const Tensor& seq, double theta, bool interleaved) {
  check_f16(q, "rope q");
  check_f16(k, "rope k");
  check_f16(v, "rope v");
  check_f16(cache_k, "rope cache_k");
  TORCH_CHECK(q.dim() == 3 && k.dim() == 3 && v.dim() == 3 && q.stride(2) == 1 && k.stride(2) == 1 && v.stride(2) == 1 &&
                  q.stride(1) == q.size(2) && k.stride(1) == k.size(2) && v.stride(1) == v.size(2),
              "rope: q/k/v must be [n_tok, heads, D] with packed heads");
  TORCH_CHECK(cache_k.dim() == 4 && cache_k.is_contiguous() && cache_v.is_contiguous(), "rope: cache [B, Hkv, T, D]");
  TORCH_CHECK(pos.scalar_type() == at::kInt && seq.scalar_type() == at::kInt && pos.is_cuda(), "rope: int32 CUDA pos/seq");
  c10::cuda::CUDAGuard guard(q.device());
  rt::RopeKvArgs a{};
  a.q = q.data_ptr(); a.k = k.data_ptr(); a.v = v.data_ptr();
  a.q_st = q.stride(0); a.k_st = k.stride(0); a.v_st = v.stride(0);
  a.cache_k = cache_k.data_ptr(); a.cache_v = cache_v.data_ptr();
  a.pos = pos.data_ptr<int>(); a.seq = seq.data_ptr<int>();
  a.n_tok = int(q.size(0)); a.H = int(q.size(1)); a.Hkv = int(k.size(1)); a.D = int(q.size(2));
  a.T_max = int(cache_k.size(2));
  a.n_seq = int(cache_k.size(0));
  a.theta = float(theta);
  a.interleaved = interleaved ? 1 : 0;
  rt::rope_kv_f16(a, cur_stream(q.device().index()));
}

void attn_cache(const Tensor& q, const Tensor& cache_k, const Tensor& cache_v, Tensor& out, const Tensor& kv_len,
                const Tensor& seq, int64_t max_kv_len, double scale) {
  check_f16(q, "attn_cache q");
  check_f16(out, "attn_cache out");
  TORCH_CHECK(q.dim() == 3 && out.dim() == 3 && q.stride(2) == 1 && out.stride(2) == 1 && q.stride(1) == q.size(2) &&
                  out.stride(1) == out.size(2), "attn_cache: q/out [n_tok, H, D] with packed heads");
  c10::cuda::CUDAGuard guard(q.device());
  rt::AttnCacheArgs a{};
  a.q = q.data_ptr(); a.q_st = q.stride(0);
  a.cache_k = cache_k.data_ptr(); a.cache_v = cache_v.data_ptr();
  a.out = out.data_ptr(); a.o_st = out.stride(0);
  a.kv_len = kv_len.data_ptr<int>(); a.seq = seq.data_ptr<int>();
  a.n_tok = int(q.size(0)); a.H = int(q.size(1)); a.Hkv = int(cache_k.size(1)); a.D = int(q.size(2));
  a.T_max = int(cache_k.size(2)); a.max_kv_len = int(max_kv_len);
  a.n_seq = int(cache_k.size(0));
  a.scale = float(scale);
  if (rt::attn_decode_split_supported(a.D, a.H, a.Hkv) && q.stride(0) % 8 == 0 &&
      (reinterpret_cast<uintptr_t>(a.q) & 15) == 0) {
    a.n_split = rt::attn_decode_num_splits(a.n_tok, a.Hkv, a.max_kv_len, rt::sm_count(q.device().index()));
    Tensor part;
    if (a.n_split > 1) {
      part = at::empty({int64_t(a.n_tok) * a.H * a.n_split * (a.D + 2)}, q.options().dtype(at::kFloat));
      a.partial = part.data_ptr<float>();
      // arrival counters of the in-kernel merge: one zeroed buffer per device, re-armed by the kernel itself
      static std::mutex mu;
      // (outgrown buffers stay alive: a captured CUDA graph may still point at them)
      static std::map<int, std::vector<Tensor>> counters;
      std::lock_guard<std::mutex> lock(mu);
      std::vector<Tensor>& cs = counters[q.device().index()];
      const int64_t need = int64_t(a.n_tok) * a.Hkv;
      if (cs.empty() || cs.back().numel() < need) cs.push_back(at::zeros({std::max<int64_t>(need, 4096)}, q.options().dtype(at::kInt)));
      a.counters = cs.back().data_ptr<int>();
    }
    rt::attn_decode_split(a, cur_stream(q.device().index()));
    return;
  }
  rt::attn_cache_f16(a, cur_stream(q.device().index()));
}

void silu_mul(const Tensor& gate, const Tensor& up, Tensor& out) {
  check_f16(gate, "silu_mul gate");
  check_f16(up, "silu_mul up");
  check_f16(out, "silu_mul out");
  TORCH_CHECK(gate.dim() == 2 && gate.stride(1) == 1 && up.stride(1) == 1 && out.stride(1) == 1, "silu_mul: 2-D rows");
  c10::cuda::CUDAGuard guard(gate.device());
  rt::silu_mul_f16(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.size(0), int(gate.size(1)), gate.stride(0),
                   up.stride(0), out.stride(0), cur_stream(gate.device().index()));
}

// CRC-64 (reflected polynomial 0xC96C5795D7870F42, init and final XOR all-ones): the checksum of the
// RusTorch binary container (reference: src/serialization/core.rs:255-269), slicing-by-8.
uint64_t crc64_bytes(const pybind11::bytes& data) {
  static uint64_t table[8][256];
  static bool ready = false;
  if (!ready) {
    for (int b = 0; b < 256; ++b) {
      uint64_t c = uint64_t(b);
      for (int k = 0; k < 8; ++k) c = (c & 1) ? (c >> 1) ^ 0xC96C5795D7870F42ull : (c >> 1);
      table[0][b] = c;
    }
    for (int b = 0; b < 256; ++b)
      for (int t = 1; t < 8; ++t) table[t][b] = table[0][table[t - 1][b] & 0xFF] ^ (table[t - 1][b] >> 8);
    ready = true;
  }
  char* buf = nullptr;
  Py_ssize_t n = 0;
  if (PyBytes_AsStringAndSize(data.ptr(), &buf, &n) != 0) throw pybind11::error_already_set();
  const unsigned char* p = reinterpret_cast<const unsigned char*>(buf);
  uint64_t crc = ~0ull;
  pybind11::gil_scoped_release release;
  while (n >= 8) {
    uint64_t w;
    memcpy(&w, p, 8);
    crc ^= w;
    crc = table[7][crc & 0xFF] ^ table[6][(crc >> 8) & 0xFF] ^ table[5][(crc >> 16) & 0xFF] ^
          table[4][(crc >> 24) & 0xFF] ^ table[3][(crc >> 32) & 0xFF] ^ table[2][(crc >> 40) & 0xFF] ^
          table[1][(crc >> 48) & 0xFF] ^ table[0][crc >> 56];
    p += 8;
    n -= 8;
  }
  while (n-- > 0) crc = table[0][(crc ^ *p++) & 0xFF] ^ (crc >> 8);
  return ~crc;
}

}  // namespace

void check_bf16(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.scalar_type() == at::kBFloat16, name, ": bf16 CUDA tensor required");
}

// all-gather -> GEMM.  x_ptrs / flag_ptrs: peer pointers of the symmetric shard [rows, K] and flag buffers.
void tp_ag_gemm(const std::vector<int64_t>& x_ptrs, const std::vector<int64_t>& flag_ptrs, Tensor& gather, Tensor& mb_ready,
                Tensor& comm_done, const Tensor& weight, bool b_mn, Tensor& out, const c10::optional<Tensor>& bias, int64_t rank,
                int64_t epoch, int64_t rows_per_rank, double timeout_s, int64_t n_comm) {
  const int world = int(x_ptrs.size());
  check_bf16(gather, "tp_ag_gemm gather");
  check_bf16(weight, "tp_ag_gemm weight");
  check_bf16(out, "tp_ag_gemm out");
  TORCH_CHECK(int(flag_ptrs.size()) == world && weight.dim() == 2 && weight.stride(1) == 1 && out.dim() == 2 && out.stride(1) == 1 &&
                  gather.is_contiguous() && gather.dim() == 2, "tp_ag_gemm: bad operands");
  rt::TpGemmArgs a{};
  a.mode = 0;
  a.world = world; a.rank = int(rank); a.epoch = int(epoch); a.rows_per_rank = int(rows_per_rank);
  a.K = int(gather.size(1));
  a.N = int(b_mn ? weight.size(1) : weight.size(0));
  TORCH_CHECK((b_mn ? weight.size(0) : weight.size(1)) == a.K, "tp_ag_gemm: weight K mismatch");
  TORCH_CHECK(gather.size(0) == rows_per_rank * world && out.size(0) == gather.size(0) && out.size(1) == a.N, "tp_ag_gemm: shape mismatch");
  TORCH_CHECK(mb_ready.scalar_type() == at::kInt && mb_ready.numel() >= gather.size(0) / 128 && comm_done.scalar_type() == at::kInt,
              "tp_ag_gemm: int32 mb_ready / comm_done");
  a.b = weight.data_ptr(); a.b_mn = b_mn; a.ldb = weight.stride(0);
  a.out = out.data_ptr(); a.ld_out = out.stride(0);
  if (bias.has_value() && bias->defined()) { check_bf16(*bias, "tp bias"); a.bias = bias->data_ptr(); }
  a.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  for (int r = 0; r < world; ++r) {
    a.x_shards[r] = reinterpret_cast<const void*>(x_ptrs[r]);
    a.flags[r] = reinterpret_cast<int*>(flag_ptrs[r]);
  }
  a.gather = gather.data_ptr();
  a.mb_ready = mb_ready.data_ptr<int>();
  a.comm_done = reinterpret_cast<unsigned*>(comm_done.data_ptr<int>());
  a.n_comm = int(n_comm);
  c10::cuda::CUDAGuard guard(gather.device());
  rt::tp_gemm(a, cur_stream(gather.device().index()));
}

// GEMM -> reduce-scatter.  stage_ptrs / flag_ptrs: peer pointers of the symmetric staging and flag buffers.
void tp_gemm_rs(const Tensor& x, const Tensor& weight, bool b_mn, const std::vector<int64_t>& stage_ptrs,
                const std::vector<int64_t>& flag_ptrs, Tensor& out, const c10::optional<Tensor>& bias,
                const c10::optional<Tensor>& residual, int64_t rank, int64_t epoch, double timeout_s) {
  const int world = int(stage_ptrs.size());
  check_bf16(x, "tp_gemm_rs x");
  check_bf16(weight, "tp_gemm_rs weight");
  check_bf16(out, "tp_gemm_rs out");
  TORCH_CHECK(int(flag_ptrs.size()) == world && x.dim() == 2 && x.stride(1) == 1 && weight.dim() == 2 && weight.stride(1) == 1 &&
                  out.dim() == 2 && out.stride(1) == 1, "tp_gemm_rs: bad operands");
  rt::TpGemmArgs a{};
  a.mode = 1;
  a.world = world; a.rank = int(rank); a.epoch = int(epoch);
  TORCH_CHECK(x.size(0) % world == 0, "tp_gemm_rs: rows must divide by the world size");
  a.rows_per_rank = int(x.size(0) / world);
  a.K = int(x.size(1));
  a.N = int(b_mn ? weight.size(1) : weight.size(0));
  TORCH_CHECK((b_mn ? weight.size(0) : weight.size(1)) == a.K, "tp_gemm_rs: weight K mismatch");
  TORCH_CHECK(out.size(0) == a.rows_per_rank && out.size(1) == a.N, "tp_gemm_rs: out must be [rows / world, N]");
  a.b = weight.data_ptr(); a.b_mn = b_mn; a.ldb = weight.stride(0);
  a.x = x.data_ptr(); a.ld_x = x.stride(0);
  a.out = out.data_ptr(); a.ld_out = out.stride(0);
  if (bias.has_value() && bias->defined()) { check_bf16(*bias, "tp bias"); a.bias = bias->data_ptr(); }
  if (residual.has_value() && residual->defined()) {
    check_bf16(*residual, "tp residual");
    TORCH_CHECK(residual->dim() == 2 && residual->stride(1) == 1 && residual->size(0) == a.rows_per_rank && residual->size(1) == a.N,
                "tp_gemm_rs: residual must match out");
    a.residual = residual->data_ptr(); a.ld_res = residual->stride(0);
  }
  a.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  for (int r = 0; r < world; ++r) {
    a.stage[r] = reinterpret_cast<void*>(stage_ptrs[r]);
    a.flags[r] = reinterpret_cast<int*>(flag_ptrs[r]);
  }
  c10::cuda::CUDAGuard guard(x.device());
  rt::tp_gemm(a, cur_stream(x.device().index()));
}

// x [N,H,W,Cin], w [Cout,KH,KW,Cin], out [N,OH,OW,Cout]: contiguous bf16 (channels-last views of NCHW tensors).
void conv2d_fwd(const Tensor& x, const Tensor& w, Tensor& out, const c10::optional<Tensor>& bias, int64_t stride, int64_t pad,
                int64_t pad_h) {
  check_bf16(x, "conv2d x");
  check_bf16(w, "conv2d w");
  check_bf16(out, "conv2d out");
  TORCH_CHECK(x.dim() == 4 && w.dim() == 4 && out.dim() == 4 && x.is_contiguous() && w.is_contiguous() && out.is_contiguous(),
              "conv2d: contiguous NHWC / OHWI tensors required");
  rt::Conv2dArgs a{};
  a.N = int(x.size(0)); a.H = int(x.size(1)); a.W = int(x.size(2)); a.Cin = int(x.size(3));
  a.Cout = int(w.size(0)); a.KH = int(w.size(1)); a.KW = int(w.size(2));
  TORCH_CHECK(w.size(3) == a.Cin, "conv2d: weight / input channel mismatch");
  a.stride = int(stride); a.pad = int(pad); a.pad_h = int(pad_h);
  const int64_t ph = pad_h >= 0 ? pad_h : pad;
  const int64_t OH = (a.H + 2 * ph - a.KH) / a.stride + 1, OW = (a.W + 2 * a.pad - a.KW) / a.stride + 1;
  TORCH_CHECK(out.size(0) == a.N && out.size(1) == OH && out.size(2) == OW && out.size(3) == a.Cout, "conv2d: bad output shape");
  a.x = x.data_ptr(); a.w = w.data_ptr(); a.out = out.data_ptr();
  if (bias.has_value() && bias->defined()) { check_bf16(*bias, "conv2d bias"); a.bias = bias->data_ptr(); }
  c10::cuda::CUDAGuard guard(x.device());
  rt::conv2d_fwd(a, cur_stream(x.device().index()));
}

// Stride-1 convolution of x [N,H,W,Cin] (zero outside the image, first tap at input offset -pad) whose out_h x out_w
// results go to every step-th pixel of the contiguous NHWC tensor `out`, starting at pixel (off_h, off_w): one parity
// class of a strided input gradient.
void conv2d_fwd_scatter(const Tensor& x, const Tensor& w, Tensor& out, int64_t pad, int64_t out_h, int64_t out_w, int64_t step,
                        int64_t off_h, int64_t off_w, int64_t pad_h) {
  check_bf16(x, "conv2d x");
  check_bf16(w, "conv2d w");
  check_bf16(out, "conv2d out");
  TORCH_CHECK(x.dim() == 4 && w.dim() == 4 && out.dim() == 4 && x.is_contiguous() && w.is_contiguous() && out.is_contiguous(),
              "conv2d: contiguous NHWC / OHWI tensors required");
  rt::Conv2dArgs a{};
  a.N = int(x.size(0)); a.H = int(x.size(1)); a.W = int(x.size(2)); a.Cin = int(x.size(3));
  a.Cout = int(w.size(0)); a.KH = int(w.size(1)); a.KW = int(w.size(2));
  TORCH_CHECK(w.size(3) == a.Cin && out.size(0) == a.N && out.size(3) == a.Cout, "conv2d_fwd_scatter: channel / batch mismatch");
  TORCH_CHECK(pad >= 0 && step >= 1 && out_h >= 1 && out_w >= 1 && off_h >= 0 && off_w >= 0 &&
                  off_h + (out_h - 1) * step < out.size(1) && off_w + (out_w - 1) * step < out.size(2),
              "conv2d_fwd_scatter: the scattered results must lie inside the output tensor");
  a.stride = 1; a.pad = int(pad); a.pad_h = int(pad_h);
  a.out_h = int(out_h); a.out_w = int(out_w);
  const int64_t H = out.size(1), W = out.size(2), C = out.size(3);
  a.out_sn = H * W * C; a.out_sh = step * W * C; a.out_sw = step * C;
  a.x = x.data_ptr(); a.w = w.data_ptr();
  a.out = static_cast<at::BFloat16*>(out.data_ptr()) + (off_h * W + off_w) * C;
  c10::cuda::CUDAGuard guard(x.device());
  rt::conv2d_fwd(a, cur_stream(x.device().index()));
}

// dw [Cout,KH,KW,Cin] fp32 += dy^T (*) x
void conv2d_wgrad(const Tensor& x, const Tensor& dy, Tensor& dw, int64_t stride, int64_t pad, int64_t pad_h) {
  check_bf16(x, "conv2d_wgrad x");
  check_bf16(dy, "conv2d_wgrad dy");
  TORCH_CHECK(dw.is_cuda() && dw.scalar_type() == at::kFloat && dw.is_contiguous() && dw.dim() == 4 && x.is_contiguous() &&
                  dy.is_contiguous() && x.dim() == 4 && dy.dim() == 4, "conv2d_wgrad: contiguous NHWC tensors and fp32 dw");
  rt::Conv2dArgs a{};
  a.N = int(x.size(0)); a.H = int(x.size(1)); a.W = int(x.size(2)); a.Cin = int(x.size(3));
  a.Cout = int(dw.size(0)); a.KH = int(dw.size(1)); a.KW = int(dw.size(2));
  a.stride = int(stride); a.pad = int(pad); a.pad_h = int(pad_h);
  const int64_t ph = pad_h >= 0 ? pad_h : pad;
  const int64_t OH = (a.H + 2 * ph - a.KH) / a.stride + 1, OW = (a.W + 2 * a.pad - a.KW) / a.stride + 1;
  TORCH_CHECK(dw.size(3) == a.Cin && dy.size(0) == a.N && dy.size(1) == OH && dy.size(2) == OW && dy.size(3) == a.Cout,
              "conv2d_wgrad: shape mismatch");
  a.x = x.data_ptr(); a.dy = dy.data_ptr(); a.dw = dw.data_ptr<float>();
  c10::cuda::CUDAGuard guard(x.device());
  rt::conv2d_wgrad(a, cur_stream(x.device().index()));
}

int dtype_code(const Tensor& t, const char* name);

// in_ptrs / result_ptrs / flag_ptrs: peer pointers of symmetric buffers.  out: local tensor.
void p2p_collective(int64_t mode, const std::vector<int64_t>& in_ptrs, const std::vector<int64_t>& result_ptrs,
                    const std::vector<int64_t>& flag_ptrs, Tensor& out, int64_t numel, Tensor& epoch_dev, Tensor& barrier_state,
                    int64_t rank, int64_t root, double timeout_s) {
  const int world = int(in_ptrs.size());
  rt::P2PCollArgs a{};
  a.mode = int(mode);
  a.dtype = dtype_code(out, "p2p_collective out");
  a.world = world; a.rank = int(rank); a.root = int(root); a.numel = numel;
  TORCH_CHECK(int(flag_ptrs.size()) == world && out.is_contiguous(), "p2p_collective: bad operands");
  TORCH_CHECK(epoch_dev.scalar_type() == at::kInt && barrier_state.scalar_type() == at::kInt && barrier_state.numel() >= 2 &&
                  epoch_dev.is_cuda() && barrier_state.is_cuda(), "p2p_collective: int32 CUDA epoch / barrier words");
  for (int r = 0; r < world; ++r) {
    a.in[r] = reinterpret_cast<const void*>(in_ptrs[r]);
    a.result[r] = r < int(result_ptrs.size()) ? reinterpret_cast<void*>(result_ptrs[r]) : nullptr;
    a.flags[r] = reinterpret_cast<int*>(flag_ptrs[r]);
  }
  a.out = out.data_ptr();
  a.epoch_dev = epoch_dev.data_ptr<int>();
  a.grid_counter = reinterpret_cast<unsigned*>(barrier_state.data_ptr<int>());
  a.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  c10::cuda::CUDAGuard guard(out.device());
  rt::p2p_collective(a, cur_stream(out.device().index()));
}

// partial, x: [rows, d]; buf_ptrs: peer pointers of the receive buffers; state: int32[8].
void ar_residual_norm(const std::vector<int64_t>& buf_ptrs, int64_t cap_numel, const Tensor& partial, Tensor& x,
                      const c10::optional<Tensor>& w, const c10::optional<Tensor>& h, Tensor& state, int64_t rank, double eps,
                      double timeout_s) {
  rt::ArNormArgs a{};
  a.dtype = dtype_code(x, "ar_residual_norm x");
  a.world = int(buf_ptrs.size()); a.rank = int(rank);
  TORCH_CHECK(x.dim() == 2 && x.is_contiguous() && partial.is_contiguous() && partial.sizes() == x.sizes() &&
                  partial.scalar_type() == x.scalar_type() && partial.is_cuda(), "ar_residual_norm: partial and x must be matching [rows, d]");
  TORCH_CHECK(state.scalar_type() == at::kInt && state.is_cuda() && state.numel() >= 8, "ar_residual_norm: int32[8] CUDA state");
  a.rows = int(x.size(0)); a.d = int(x.size(1)); a.eps = float(eps);
  for (int r = 0; r < a.world; ++r) a.bufs[r] = reinterpret_cast<void*>(buf_ptrs[r]);
  a.cap_numel = cap_numel;
  a.partial = partial.data_ptr(); a.x = x.data_ptr();
  if (h.has_value()) {
    TORCH_CHECK(w.has_value() && w->is_cuda() && w->is_contiguous() && w->numel() == x.size(1) && w->scalar_type() == x.scalar_type() &&
                    h->is_contiguous() && h->sizes() == x.sizes() && h->scalar_type() == x.scalar_type() && h->is_cuda(),
                "ar_residual_norm: norm weight [d] and output [rows, d] of the activation dtype");
    a.w = w->data_ptr(); a.h = h->data_ptr();
  }
  a.state = state.data_ptr<int>();
  a.timeout_ns = (unsigned long long)(timeout_s * 1e9);
  c10::cuda::CUDAGuard guard(x.device());
  rt::ar_residual_norm(a, cur_stream(x.device().index()));
}

int dtype_code(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, ": CUDA tensor required");
  switch (t.scalar_type()) {
    case at::kFloat: return rt::DT_F32;
    case at::kBFloat16: return rt::DT_BF16;
    case at::kHalf: return rt::DT_F16;
    default: TORCH_CHECK(false, name, ": dtype must be fp32, bf16 or fp16, got ", t.scalar_type());
  }
  return -1;
}

// mode 0: out = op(a, b) (same shape); 1: op(a, scalar); 2: op(scalar, a)
void ew_binary(int64_t op, const Tensor& a, const c10::optional<Tensor>& b, Tensor& out, double scalar, double alpha,
               int64_t mode) {
  const int dt = dtype_code(a, "elementwise a");
  TORCH_CHECK(a.is_contiguous() && out.is_contiguous() && out.numel() == a.numel() && out.scalar_type() == a.scalar_type(),
              "elementwise: contiguous operands of one dtype and size");
  const void* pb = nullptr;
  if (mode == 0) {
    TORCH_CHECK(b.has_value() && b->is_contiguous() && b->numel() == a.numel() && b->scalar_type() == a.scalar_type() &&
                    b->is_cuda(), "elementwise: b must match a");
    pb = b->data_ptr();
  }
  c10::cuda::CUDAGuard guard(a.device());
  rt::elementwise_binary(int(op), dt, a.data_ptr(), pb, out.data_ptr(), a.numel(), float(scalar), float(alpha), int(mode),
                         cur_stream(a.device().index()));
}

void ew_unary(int64_t op, const Tensor& x, const c10::optional<Tensor>& dy, Tensor& out, double p0, double p1) {
  const int dt = dtype_code(x, "elementwise x");
  TORCH_CHECK(x.is_contiguous() && out.is_contiguous() && out.numel() == x.numel() && out.scalar_type() == x.scalar_type(),
              "elementwise: contiguous operands of one dtype and size");
  const void* pg = nullptr;
  if (dy.has_value() && dy->defined()) {
    TORCH_CHECK(dy->is_contiguous() && dy->numel() == x.numel() && dy->scalar_type() == x.scalar_type() && dy->is_cuda(),
                "elementwise: dy must match x");
    pg = dy->data_ptr();
  }
  c10::cuda::CUDAGuard guard(x.device());
  rt::elementwise_unary(int(op), dt, x.data_ptr(), pg, out.data_ptr(), x.numel(), float(p0), float(p1), pg != nullptr,
                        cur_stream(x.device().index()));
}

void softmax_rows(const Tensor& x, const c10::optional<Tensor>& dy, Tensor& out, bool log_mode) {
  const int dt = dtype_code(x, "softmax x");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && out.dim() == 2 && out.stride(1) == 1 && out.stride(0) == x.stride(0) &&
                  out.scalar_type() == x.scalar_type() && out.sizes() == x.sizes(), "softmax: 2-D rows, equal strides");
  c10::cuda::CUDAGuard guard(x.device());
  auto st = cur_stream(x.device().index());
  if (dy.has_value() && dy->defined()) {
    TORCH_CHECK(dy->sizes() == x.sizes() && dy->stride(1) == 1 && dy->stride(0) == x.stride(0) &&
                    dy->scalar_type() == x.scalar_type(), "softmax: dy must match y");
    rt::softmax_rows_bwd(dt, x.data_ptr(), dy->data_ptr(), out.data_ptr(), x.size(0), int(x.size(1)), x.stride(0), log_mode, st);
  } else {
    rt::softmax_rows_fwd(dt, x.data_ptr(), out.data_ptr(), x.size(0), int(x.size(1)), x.stride(0), log_mode, st);
  }
}

void reduce_rows(const Tensor& x, Tensor& out, int64_t mode, double p0) {
  const int dt = dtype_code(x, "reduce_rows x");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && out.scalar_type() == at::kFloat && out.is_contiguous() &&
                  out.numel() == x.size(0) && out.is_cuda(), "reduce_rows: x [rows, C], out fp32 [rows]");
  c10::cuda::CUDAGuard guard(x.device());
  rt::reduce_rows(dt, x.data_ptr(), out.data_ptr<float>(), x.size(0), int(x.size(1)), x.stride(0), int(mode), float(p0),
                  cur_stream(x.device().index()));
}

const float* opt_f32(const c10::optional<Tensor>& t, int64_t n, const char* name) {
  if (!t.has_value() || !t->defined()) return nullptr;
  TORCH_CHECK(t->is_cuda() && t->scalar_type() == at::kFloat && t->is_contiguous() && t->numel() == n, name,
              ": fp32 CUDA tensor with one value per channel required");
  return t->data_ptr<float>();
}

// x2 / y2: [M, C] contiguous (channels last).  scratch fp32 [2, C].
void batchnorm_fwd(const Tensor& x2, const c10::optional<Tensor>& residual, Tensor& y2, const c10::optional<Tensor>& gamma,
                   const c10::optional<Tensor>& beta, const c10::optional<Tensor>& running_mean,
                   const c10::optional<Tensor>& running_var, const c10::optional<Tensor>& save_mean,
                   const c10::optional<Tensor>& save_rstd, Tensor& scratch, double eps, double momentum, bool relu, bool training) {
  rt::BatchNormArgs a{};
  a.dtype = dtype_code(x2, "batchnorm x");
  TORCH_CHECK(x2.dim() == 2 && x2.is_contiguous() && y2.is_contiguous() && y2.sizes() == x2.sizes() &&
                  y2.scalar_type() == x2.scalar_type(), "batchnorm: x, y [M, C] contiguous");
  a.M = x2.size(0);
  a.C = int(x2.size(1));
  a.x = x2.data_ptr();
  a.y = y2.data_ptr();
  if (residual.has_value() && residual->defined()) {
    TORCH_CHECK(residual->is_contiguous() && residual->sizes() == x2.sizes() && residual->scalar_type() == x2.scalar_type(),
                "batchnorm: residual must match x");
    a.residual = residual->data_ptr();
  }
  a.gamma = opt_f32(gamma, a.C, "batchnorm gamma");
  a.beta = opt_f32(beta, a.C, "batchnorm beta");
  a.running_mean = const_cast<float*>(opt_f32(running_mean, a.C, "batchnorm running_mean"));
  a.running_var = const_cast<float*>(opt_f32(running_var, a.C, "batchnorm running_var"));
  a.save_mean = const_cast<float*>(opt_f32(save_mean, a.C, "batchnorm save_mean"));
  a.save_rstd = const_cast<float*>(opt_f32(save_rstd, a.C, "batchnorm save_rstd"));
  TORCH_CHECK(training || (a.running_mean && a.running_var), "batchnorm: inference needs running statistics");
  a.scratch = const_cast<float*>(opt_f32(scratch, 2 * int64_t(a.C), "batchnorm scratch"));
  a.eps = float(eps);
  a.momentum = float(momentum);
  a.relu = relu;
  a.training = training;
  c10::cuda::CUDAGuard guard(x2.device());
  rt::batchnorm_fwd(a, cur_stream(x2.device().index()));
}

// scratch returns [dbeta, dgamma] (fp32 [2, C]).
void batchnorm_bwd(const Tensor& x2, const Tensor& dy2, const c10::optional<Tensor>& y_relu, Tensor& dx2,
                   const c10::optional<Tensor>& dres, const c10::optional<Tensor>& gamma, const Tensor& save_mean,
                   const Tensor& save_rstd, Tensor& scratch) {
  rt::BatchNormArgs a{};
  a.dtype = dtype_code(x2, "batchnorm x");
  TORCH_CHECK(x2.dim() == 2 && x2.is_contiguous() && dy2.is_contiguous() && dx2.is_contiguous() && dy2.sizes() == x2.sizes() &&
                  dx2.sizes() == x2.sizes() && dy2.scalar_type() == x2.scalar_type() && dx2.scalar_type() == x2.scalar_type(),
              "batchnorm_bwd: x, dy, dx [M, C] contiguous of one dtype");
  a.M = x2.size(0);
  a.C = int(x2.size(1));
  a.x = x2.data_ptr();
  a.dy = dy2.data_ptr();
  a.dx = dx2.data_ptr();
  if (y_relu.has_value() && y_relu->defined()) {
    TORCH_CHECK(y_relu->is_contiguous() && y_relu->sizes() == x2.sizes() && y_relu->scalar_type() == x2.scalar_type(),
                "batchnorm_bwd: y must match x");
    a.y_relu = y_relu->data_ptr();
  }
  if (dres.has_value() && dres->defined()) {
    TORCH_CHECK(dres->is_contiguous() && dres->sizes() == x2.sizes() && dres->scalar_type() == x2.scalar_type(),
                "batchnorm_bwd: dres must match x");
    a.dres = dres->data_ptr();
  }
  a.gamma = opt_f32(gamma, a.C, "batchnorm gamma");
  a.save_mean = const_cast<float*>(opt_f32(save_mean, a.C, "batchnorm save_mean"));
  a.save_rstd = const_cast<float*>(opt_f32(save_rstd, a.C, "batchnorm save_rstd"));
  a.scratch = const_cast<float*>(opt_f32(scratch, 2 * int64_t(a.C), "batchnorm scratch"));
  c10::cuda::CUDAGuard guard(x2.device());
  rt::batchnorm_bwd(a, cur_stream(x2.device().index()));
}


// x, y (and dy, dx): contiguous [N, C, *]; mean / rstd fp32 [N * groups]; gamma / beta / dgamma / dbeta fp32 [C] or none.
void groupnorm(const Tensor& x, Tensor& out, const c10::optional<Tensor>& dy, const c10::optional<Tensor>& gamma,
               const c10::optional<Tensor>& beta, Tensor& mean, Tensor& rstd, const c10::optional<Tensor>& dgamma,
               const c10::optional<Tensor>& dbeta, int64_t groups, double eps) {
  rt::GroupNormArgs a{};
  a.dtype = dtype_code(x, "groupnorm x");
  TORCH_CHECK(x.dim() >= 2 && x.is_contiguous() && out.is_contiguous() && out.sizes() == x.sizes() &&
                  out.scalar_type() == x.scalar_type(), "groupnorm: x and out must be contiguous [N, C, ...] of one dtype");
  a.N = x.size(0);
  a.C = int(x.size(1));
  a.G = int(groups);
  TORCH_CHECK(a.N > 0 && a.C > 0 && a.G > 0 && a.C % a.G == 0 && x.numel() > 0, "groupnorm: bad shape");
  a.HW = x.numel() / (a.N * a.C);
  a.eps = float(eps);
  a.x = x.data_ptr();
  a.gamma = opt_f32(gamma, a.C, "groupnorm gamma");
  a.beta = opt_f32(beta, a.C, "groupnorm beta");
  a.mean = const_cast<float*>(opt_f32(mean, a.N * a.G, "groupnorm mean"));
  a.rstd = const_cast<float*>(opt_f32(rstd, a.N * a.G, "groupnorm rstd"));
  c10::cuda::CUDAGuard guard(x.device());
  if (dy.has_value() && dy->defined()) {
    TORCH_CHECK(dy->is_contiguous() && dy->sizes() == x.sizes() && dy->scalar_type() == x.scalar_type(), "groupnorm: dy must match x");
    a.dy = dy->data_ptr();
    a.dx = out.data_ptr();
    a.dgamma = const_cast<float*>(opt_f32(dgamma, a.C, "groupnorm dgamma"));
    a.dbeta = const_cast<float*>(opt_f32(dbeta, a.C, "groupnorm dbeta"));
    rt::groupnorm_bwd(a, cur_stream(x.device().index()));
  } else {
    a.y = out.data_ptr();
    rt::groupnorm_fwd(a, cur_stream(x.device().index()));
  }
}

// x: channels-last storage viewed as [N, H, W, C] (contiguous); y likewise [N, OH, OW, C].
void pool2d(Tensor& x, Tensor& y, const c10::optional<Tensor>& idx, bool is_max, bool backward, int64_t kh, int64_t kw, int64_t sh,
            int64_t sw, int64_t ph, int64_t pw) {
  rt::Pool2dArgs a{};
  a.dtype = dtype_code(x, "pool2d x");
  TORCH_CHECK(x.dim() == 4 && y.dim() == 4 && x.is_contiguous() && y.is_contiguous() && y.scalar_type() == x.scalar_type() &&
                  y.is_cuda() && y.size(0) == x.size(0) && y.size(3) == x.size(3), "pool2d: contiguous [N, H, W, C] tensors of one dtype");
  a.max = is_max; a.backward = backward;
  a.x = x.data_ptr(); a.y = y.data_ptr();
  if (idx.has_value() && idx->defined()) {
    TORCH_CHECK(idx->scalar_type() == at::kByte && idx->is_cuda() && idx->is_contiguous() && idx->numel() == y.numel(),
                "pool2d: idx must be a uint8 tensor shaped like the output");
    a.idx = idx->data_ptr<uint8_t>();
  }
  a.N = int(x.size(0)); a.H = int(x.size(1)); a.W = int(x.size(2)); a.C = int(x.size(3));
  a.OH = int(y.size(1)); a.OW = int(y.size(2));
  a.kh = int(kh); a.kw = int(kw); a.sh = int(sh); a.sw = int(sw); a.ph = int(ph); a.pw = int(pw);
  c10::cuda::CUDAGuard guard(x.device());
  rt::pool2d(a, cur_stream(x.device().index()));
}

void dropout(const Tensor& x, Tensor& y, double p, int64_t seed, int64_t offset) {
  const int dt = dtype_code(x, "dropout x");
  TORCH_CHECK(x.is_non_overlapping_and_dense() && y.strides() == x.strides() && y.is_cuda() && y.scalar_type() == x.scalar_type() &&
                  y.numel() == x.numel(), "dropout: dense tensors of one dtype, size and memory layout");
  c10::cuda::CUDAGuard guard(x.device());
  rt::dropout(dt, x.data_ptr(), y.data_ptr(), x.numel(), float(p), (unsigned long long)seed, (unsigned long long)offset,
              cur_stream(x.device().index()));
}

static void check_bh(const Tensor& t, int64_t B, int64_t cols, at::ScalarType st, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == st && t.dim() == 2 && t.size(0) == B && t.size(1) == cols, name,
              ": expected a contiguous CUDA [", B, ", ", cols, "] tensor");
}

void lstm_gates_fwd(Tensor& gates, const Tensor& c, Tensor& h_out, Tensor& c_out) {
  const int dt = dtype_code(gates, "lstm gates");
  const int64_t B = c.size(0), H = c.size(1);
  check_bh(gates, B, 4 * H, gates.scalar_type(), "lstm gates");
  check_bh(c, B, H, gates.scalar_type(), "lstm c"); check_bh(h_out, B, H, gates.scalar_type(), "lstm h_out");
  check_bh(c_out, B, H, gates.scalar_type(), "lstm c_out");
  c10::cuda::CUDAGuard guard(gates.device());
  rt::lstm_gates_fwd(dt, gates.data_ptr(), c.data_ptr(), h_out.data_ptr(), c_out.data_ptr(), int(B), int(H), cur_stream(gates.device().index()));
}

void lstm_gates_bwd(const Tensor& act, const Tensor& c, const Tensor& c_new, const c10::optional<Tensor>& dh,
                    const c10::optional<Tensor>& dc_new, Tensor& dgates, Tensor& dc) {
  const int dt = dtype_code(act, "lstm act");
  const int64_t B = c.size(0), H = c.size(1);
  const auto st = act.scalar_type();
  check_bh(act, B, 4 * H, st, "lstm act"); check_bh(dgates, B, 4 * H, st, "lstm dgates");
  check_bh(c, B, H, st, "lstm c"); check_bh(c_new, B, H, st, "lstm c_new"); check_bh(dc, B, H, st, "lstm dc");
  const void *pdh = nullptr, *pdc = nullptr;
  if (dh.has_value() && dh->defined()) { check_bh(*dh, B, H, st, "lstm dh"); pdh = dh->data_ptr(); }
  if (dc_new.has_value() && dc_new->defined()) { check_bh(*dc_new, B, H, st, "lstm dc_new"); pdc = dc_new->data_ptr(); }
  c10::cuda::CUDAGuard guard(act.device());
  rt::lstm_gates_bwd(dt, act.data_ptr(), c.data_ptr(), c_new.data_ptr(), pdh, pdc, dgates.data_ptr(), dc.data_ptr(), int(B), int(H),
                     cur_stream(act.device().index()));
}

void gru_gates_fwd(const Tensor& gi, const Tensor& gh, const Tensor& h, Tensor& h_out, Tensor& save) {
  const int dt = dtype_code(gi, "gru gi");
  const int64_t B = h.size(0), H = h.size(1);
  const auto st = gi.scalar_type();
  check_bh(gi, B, 3 * H, st, "gru gi"); check_bh(gh, B, 3 * H, st, "gru gh"); check_bh(h, B, H, st, "gru h");
  check_bh(h_out, B, H, st, "gru h_out"); check_bh(save, B, 4 * H, st, "gru save");
  c10::cuda::CUDAGuard guard(gi.device());
  rt::gru_gates_fwd(dt, gi.data_ptr(), gh.data_ptr(), h.data_ptr(), h_out.data_ptr(), save.data_ptr(), int(B), int(H),
                    cur_stream(gi.device().index()));
}

void gru_gates_bwd(const Tensor& save, const Tensor& h, const Tensor& dh_new, Tensor& dgi, Tensor& dgh, Tensor& dh) {
  const int dt = dtype_code(save, "gru save");
  const int64_t B = h.size(0), H = h.size(1);
  const auto st = save.scalar_type();
  check_bh(save, B, 4 * H, st, "gru save"); check_bh(h, B, H, st, "gru h"); check_bh(dh_new, B, H, st, "gru dh_new");
  check_bh(dgi, B, 3 * H, st, "gru dgi"); check_bh(dgh, B, 3 * H, st, "gru dgh"); check_bh(dh, B, H, st, "gru dh");
  c10::cuda::CUDAGuard guard(save.device());
  rt::gru_gates_bwd(dt, save.data_ptr(), h.data_ptr(), dh_new.data_ptr(), dgi.data_ptr(), dgh.data_ptr(), dh.data_ptr(), int(B), int(H),
                    cur_stream(save.device().index()));
}

void amp_unscale(Tensor& grads, double inv_scale, Tensor& found_inf) {
  const int dt = dtype_code(grads, "amp_unscale grads");
  TORCH_CHECK(grads.is_contiguous() && found_inf.is_cuda() && found_inf.scalar_type() == at::kFloat && found_inf.numel() >= 1,
              "amp_unscale: contiguous gradients and a float CUDA flag");
  c10::cuda::CUDAGuard guard(grads.device());
  rt::amp_unscale(dt, grads.data_ptr(), grads.numel(), float(inv_scale), found_inf.data_ptr<float>(), cur_stream(grads.device().index()));
}

void csr_spmm(const Tensor& row_ptr, const Tensor& col, const Tensor& val, const Tensor& x, Tensor& y) {
  TORCH_CHECK(row_ptr.is_cuda() && col.is_cuda() && val.is_cuda() && x.is_cuda() && y.is_cuda(), "csr_spmm: CUDA tensors");
  TORCH_CHECK(row_ptr.scalar_type() == at::kLong && col.scalar_type() == at::kLong && val.scalar_type() == at::kFloat &&
                  x.scalar_type() == at::kFloat && y.scalar_type() == at::kFloat, "csr_spmm: int64 indices, fp32 values");
  TORCH_CHECK(row_ptr.is_contiguous() && col.is_contiguous() && val.is_contiguous() && x.is_contiguous() && y.is_contiguous() &&
                  x.dim() == 2 && y.dim() == 2 && y.size(0) == row_ptr.numel() - 1 && y.size(1) == x.size(1) && col.numel() == val.numel(),
              "csr_spmm: x [cols, n], y [rows, n]");
  c10::cuda::CUDAGuard guard(x.device());
  rt::csr_spmm(reinterpret_cast<const long long*>(row_ptr.data_ptr<int64_t>()), reinterpret_cast<const long long*>(col.data_ptr<int64_t>()), val.data_ptr<float>(), x.data_ptr<float>(), y.data_ptr<float>(),
               y.size(0), int(x.size(1)), cur_stream(x.device().index()));
}


static void check_bf16c(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda() && t.is_contiguous() && t.scalar_type() == at::kBFloat16, name, ": contiguous CUDA bf16 tensor required");
}

// packed [rows, (H + 2 Hkv) * D]; q [rows, H, D]; k, v [rows, Hkv, D]; cos / sin [T, D / 2] fp32; rows = B * T.
void rope_split(Tensor& packed, Tensor& q, Tensor& k, Tensor& v, const Tensor& cos_t, const Tensor& sin_t, int64_t T, bool backward) {
  check_bf16c(packed, "rope_split packed"); check_bf16c(q, "rope_split q"); check_bf16c(k, "rope_split k"); check_bf16c(v, "rope_split v");
  const int64_t D = q.size(-1), H = q.size(-2), Hkv = k.size(-2);
  const int64_t rows = q.numel() / (H * D);
  TORCH_CHECK(k.numel() == rows * Hkv * D && v.numel() == k.numel() && packed.numel() == rows * (H + 2 * Hkv) * D && rows % T == 0,
              "rope_split: shape mismatch");
  TORCH_CHECK(cos_t.is_cuda() && sin_t.is_cuda() && cos_t.scalar_type() == at::kFloat && sin_t.scalar_type() == at::kFloat &&
                  cos_t.is_contiguous() && sin_t.is_contiguous() && cos_t.size(-1) == D / 2 && sin_t.size(-1) == D / 2 &&
                  cos_t.size(0) >= T && sin_t.size(0) >= T, "rope_split: cos / sin tables must be fp32 [>= T, D / 2]");
  c10::cuda::CUDAGuard guard(packed.device());
  rt::rope_split(packed.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), cos_t.data_ptr<float>(), sin_t.data_ptr<float>(), rows,
                 int(T), int(H), int(Hkv), int(D), backward, cur_stream(packed.device().index()));
}

void swiglu(const Tensor& gu, const c10::optional<Tensor>& dact, Tensor& out, bool backward) {
  check_bf16c(gu, "swiglu gu"); check_bf16c(out, "swiglu out");
  TORCH_CHECK(gu.dim() == 2 && gu.size(1) % 2 == 0, "swiglu: gu must be [rows, 2 F]");
  const int64_t rows = gu.size(0), F = gu.size(1) / 2;
  const void* pd = nullptr;
  if (backward) {
    TORCH_CHECK(dact.has_value() && dact->numel() == rows * F && out.numel() == rows * 2 * F, "swiglu backward: shape mismatch");
    check_bf16c(*dact, "swiglu dact");
    pd = dact->data_ptr();
  } else {
    TORCH_CHECK(out.numel() == rows * F, "swiglu: out must be [rows, F]");
  }
  c10::cuda::CUDAGuard guard(gu.device());
  rt::swiglu(gu.data_ptr(), pd, out.data_ptr(), rows, int(F), backward, cur_stream(gu.device().index()));
}

// x: [N, H, W, C] contiguous bf16; col: [N * OH * OW, k_pad] bf16.
void im2col_nhwc(const Tensor& x, Tensor& col, int64_t KH, int64_t KW, int64_t stride, int64_t pad) {
  check_bf16c(x, "im2col x"); check_bf16c(col, "im2col col");
  TORCH_CHECK(x.dim() == 4 && col.dim() == 2, "im2col: x [N, H, W, C], col [N * OH * OW, k_pad]");
  const int64_t N = x.size(0), H = x.size(1), W = x.size(2), C = x.size(3);
  const int64_t OH = (H + 2 * pad - KH) / stride + 1, OW = (W + 2 * pad - KW) / stride + 1;
  TORCH_CHECK(col.size(0) == N * OH * OW, "im2col: col has ", col.size(0), " rows, expected ", N * OH * OW);
  c10::cuda::CUDAGuard guard(x.device());
  rt::im2col_nhwc(x.data_ptr(), col.data_ptr(), int(N), int(H), int(W), int(C), int(OH), int(OW), int(KH), int(KW), int(stride), int(pad),
                  int(col.size(1)), cur_stream(x.device().index()));
}

void register_extra_ops(pybind11::module_& m) {
  m.def("im2col_nhwc", &im2col_nhwc, "patch matrix of a channels-last bf16 image (few input channels)");
  m.def("p2p_collective", &p2p_collective, "all-reduce / all-gather / reduce-scatter / broadcast over symmetric peer memory");
  m.def("rope_split", &rope_split, "rotary embedding fused with the q / k / v split (bf16), forward or backward");
  m.def("swiglu", &swiglu, "silu(gate) * up over a [rows, 2F] gate|up matrix (bf16), forward or backward");
  m.def("pool2d", &pool2d, "channels-last max / average pooling, forward or backward");
  m.def("dropout", &dropout, "Philox dropout (the backward pass is the same call on dy)");
  m.def("lstm_gates_fwd", &lstm_gates_fwd);
  m.def("lstm_gates_bwd", &lstm_gates_bwd);
  m.def("gru_gates_fwd", &gru_gates_fwd);
  m.def("gru_gates_bwd", &gru_gates_bwd);
  m.def("amp_unscale", &amp_unscale, "grads *= inv_scale, found_inf = 1 on any non-finite value");
  m.def("csr_spmm", &csr_spmm, "CSR sparse x dense product (fp32)");
  m.def("ar_residual_norm", &ar_residual_norm, "all-reduce over peer memory + residual add + RMSNorm in one kernel");
  m.def("conv2d_fwd_scatter", &conv2d_fwd_scatter, "stride-1 convolution written to every step-th output pixel", py::arg("x"),
        py::arg("w"), py::arg("out"), py::arg("pad"), py::arg("out_h"), py::arg("out_w"), py::arg("step"), py::arg("off_h"),
        py::arg("off_w"), py::arg("pad_h") = -1);
  m.def("conv2d_fwd", &conv2d_fwd, "implicit-GEMM conv2d forward (channels-last bf16); pad_h >= 0: pad is along W only", py::arg("x"),
        py::arg("w"), py::arg("out"), py::arg("bias"), py::arg("stride"), py::arg("pad"), py::arg("pad_h") = -1);
  m.def("conv2d_wgrad", &conv2d_wgrad, "implicit-GEMM conv2d weight gradient (fp32 accumulate)", py::arg("x"), py::arg("dy"),
        py::arg("dw"), py::arg("stride"), py::arg("pad"), py::arg("pad_h") = -1);
  m.def("conv2d_igemm_supported", &rt::conv2d_igemm_supported);
  m.def("tp_ag_gemm", &tp_ag_gemm, "fused all-gather -> GEMM over symmetric peer memory");
  m.def("tp_gemm_rs", &tp_gemm_rs, "fused GEMM -> reduce-scatter over symmetric peer memory");
  m.def("groupnorm", &groupnorm, "GroupNorm / InstanceNorm forward (dy absent) or backward (out = dx) over contiguous [N, C, ...]");
  m.def("batchnorm_fwd", &batchnorm_fwd, "BatchNorm forward over a channels-last matrix (+residual, +ReLU)");
  m.def("batchnorm_bwd", &batchnorm_bwd, "BatchNorm backward; scratch returns [dbeta, dgamma]");
  m.def("ew_binary", &ew_binary, "elementwise binary op (add/sub/mul/div/max/min/pow)");
  m.def("ew_unary", &ew_unary, "elementwise unary op / activation, forward or backward");
  m.def("softmax_rows", &softmax_rows, "row softmax / log-softmax forward (dy absent) or backward");
  m.def("reduce_rows", &reduce_rows, "row reduction over the last dim (sum/mean/max/min/var)");
  m.def("crc64", &crc64_bytes, "CRC-64/XZ of a bytes object");
  m.def("dequant_f16", &dequant_f16, "expand repacked Q4_0 / Q8_0 weights to dense fp16");
  m.def("q_gemv", &q_gemv, "dequant-fused Q4_0 / Q8_0 matrix-vector product", pybind11::arg("qs"), pybind11::arg("scales"),
        pybind11::arg("x"), pybind11::arg("y"), pybind11::arg("bias"), pybind11::arg("residual"), pybind11::arg("q8"),
        pybind11::arg("path") = 0);
  m.def("q_gemv_fused", &q_gemv_fused, "decode projection: RMSNorm prologue + dequant-fused GEMV + residual / SwiGLU epilogue",
        pybind11::arg("qs"), pybind11::arg("scales"), pybind11::arg("x"), pybind11::arg("y"), pybind11::arg("norm_w"), pybind11::arg("eps"),
        pybind11::arg("residual"), pybind11::arg("q8"), pybind11::arg("swiglu") = false, pybind11::arg("prefetch_qs") = pybind11::none(),
        pybind11::arg("prefetch_scales") = pybind11::none(), pybind11::arg("rope_pos") = pybind11::none(),
        pybind11::arg("rope_seq") = pybind11::none(), pybind11::arg("cache_k") = pybind11::none(), pybind11::arg("cache_v") = pybind11::none(),
        pybind11::arg("n_head") = 0, pybind11::arg("rope_theta") = 10000.0);
  m.def("q_gemm_tc", &q_gemm_tc, "dequant-fused Q4_0 / Q8_0 tcgen05 GEMM for up to 256 activation rows", pybind11::arg("qs"),
        pybind11::arg("scales"), pybind11::arg("x"), pybind11::arg("y"), pybind11::arg("bias"), pybind11::arg("residual"),
        pybind11::arg("q8"), pybind11::arg("partial"), pybind11::arg("counters"), pybind11::arg("path") = 0);
  m.def("q_gemm_tc_scratch", &q_gemm_tc_scratch);
  m.def("bounds_check_build", []() { return rt::bounds_check_build(); }, "true when the extension was compiled with -DRT_BOUNDS_CHECK");
  m.def("repack_quant", &repack_quant);
  m.def("rmsnorm_f16", &rmsnorm_f16);
  m.def("rope_kv", &rope_kv);
  m.def("attn_cache", &attn_cache);
  m.def("silu_mul", &silu_mul);
  m.def("ddp_bucket_step", &ddp_bucket_step,
        "fused reduce-scatter + scale + AdamW / Adam / SGD + all-gather of one gradient bucket over peer memory "
        "(plain peer loads / stores, or NVLS multimem when the multicast pointers are non-zero)");
  m.def("ddp_wait_end", &ddp_wait_end);
  m.def("unfold_nd", &unfold_nd, "patch gather (fold = false) / scatter-sum (fold = true) for 1-3 D convolutions with groups and dilation");
  m.def("gemm_i8", &gemm_i8, "int8 x int8 -> int32 tcgen05 GEMM, optional fused dequantisation to fp32", py::arg("a"), py::arg("b"),
        py::arg("out"), py::arg("row_scale") = py::none(), py::arg("col_scale") = py::none(), py::arg("bias") = py::none());
  m.def("multi_tensor_optim", &multi_tensor_optim,
        "one launch per 32 tensors: Adam / AdamW / SGD / NAdam / RAdam / Adamax / RMSprop / AdaGrad / AdaBound / LAMB update");
}
