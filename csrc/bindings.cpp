// Tensor-facing glue: validates torch tensors, fills the raw launch structs of api.h and
// launches on torch's current CUDA stream.  All math lives in the .cu files.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDACachingAllocator.h>
#include <c10/cuda/CUDAGuard.h>
#include <c10/cuda/CUDAStream.h>
#include <torch/extension.h>

#include "api.h"
#include "common/launch.h"

namespace {

using at::Tensor;
using OptTensor = c10::optional<at::Tensor>;

cudaStream_t stream_of(const Tensor& t) {
  return at::cuda::getCurrentCUDAStream(t.device().index()).stream();
}

void check_bf16_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, ": CUDA tensor required");
  TORCH_CHECK(t.scalar_type() == at::kBFloat16, name, ": bf16 required, got ", t.scalar_type());
}
void check_f32_cuda(const Tensor& t, const char* name) {
  TORCH_CHECK(t.is_cuda(), name, ": CUDA tensor required");
  TORCH_CHECK(t.scalar_type() == at::kFloat, name, ": fp32 required, got ", t.scalar_type());
}

void gemm(const Tensor& a, bool a_mn, const Tensor& b, bool b_mn, Tensor& c, const OptTensor& bias,
          const OptTensor& aux, int64_t epi_mode, double alpha, bool accumulate, int64_t split_k,
          int64_t block_n, const OptTensor& alpha_dev) {
  const bool ab_fp16 = a.scalar_type() == at::kHalf;
  if (ab_fp16) {
    TORCH_CHECK(a.is_cuda() && b.is_cuda() && b.scalar_type() == at::kHalf, "gemm: fp16 A needs a CUDA fp16 B");
  } else {
    check_bf16_cuda(a, "gemm a");
    check_bf16_cuda(b, "gemm b");
  }
  TORCH_CHECK(c.is_cuda(), "gemm c: CUDA tensor required");
  TORCH_CHECK(a.dim() == b.dim() && a.dim() == c.dim() && (a.dim() == 2 || a.dim() == 3),
              "gemm: all operands rank 2 or all rank 3");
  TORCH_CHECK(a.stride(-1) == 1 && b.stride(-1) == 1 && c.stride(-1) == 1,
              "gemm: last dim must be contiguous");
  c10::cuda::CUDAGuard guard(a.device());
  const bool batched = a.dim() == 3;
  rt::GemmArgs g{};
  g.ab_fp16 = ab_fp16;
  g.batch = batched ? int(a.size(0)) : 1;
  g.M = int(a_mn ? a.size(-1) : a.size(-2));
  g.K = int(a_mn ? a.size(-2) : a.size(-1));
  g.N = int(b_mn ? b.size(-1) : b.size(-2));
  const int64_t Kb = b_mn ? b.size(-2) : b.size(-1);
  TORCH_CHECK(g.K == Kb, "gemm: reduction dims differ: ", g.K, " vs ", Kb);
  TORCH_CHECK(c.size(-2) == g.M && c.size(-1) == g.N, "gemm: output shape must be [M, N] = [", g.M,
              ", ", g.N, "]");
  if (batched) TORCH_CHECK(b.size(0) == g.batch && c.size(0) == g.batch, "gemm: batch mismatch");
  g.out_fp32 = c.scalar_type() == at::kFloat;
  TORCH_CHECK(g.out_fp32 || c.scalar_type() == at::kBFloat16, "gemm: C must be bf16 or fp32");
  g.a = a.data_ptr();
  g.a_mn = a_mn;
  g.lda = a.stride(-2);
  g.a_batch_stride = batched ? a.stride(0) : 0;
  g.b = b.data_ptr();
  g.b_mn = b_mn;
  g.ldb = b.stride(-2);
  g.b_batch_stride = batched ? b.stride(0) : 0;
  g.c = c.data_ptr();
  g.ldc = c.stride(-2);
  g.c_batch_stride = batched ? c.stride(0) : 0;
  if (bias.has_value() && bias->defined()) {
    check_bf16_cuda(*bias, "gemm bias");
    TORCH_CHECK(bias->numel() == g.N && bias->is_contiguous(), "gemm: bias must be contiguous [N]");
    g.bias = bias->data_ptr();
  }
  if (aux.has_value() && aux->defined()) {
    check_bf16_cuda(*aux, "gemm aux");
    TORCH_CHECK(aux->dim() == c.dim() && aux->size(-2) == g.M && aux->size(-1) == g.N &&
                    aux->stride(-1) == 1,
                "gemm: aux must have the shape of C");
    g.aux = aux->data_ptr();
    g.ld_aux = aux->stride(-2);
    g.aux_batch_stride = batched ? aux->stride(0) : 0;
  }
  g.epi_mode = int(epi_mode);
  g.alpha = float(alpha);
  g.accumulate = accumulate;
  g.split_k = int(split_k);
  g.block_n = int(block_n);
  if (alpha_dev.has_value() && alpha_dev->defined()) {
    check_f32_cuda(*alpha_dev, "gemm alpha_dev");
    TORCH_CHECK(alpha_dev->numel() == 1, "gemm: alpha_dev must hold one fp32 value");
    g.alpha_dev = alpha_dev->data_ptr<float>();
  }
  rt::gemm_bf16(g, stream_of(a));
}

rt::AttnArgs make_attn_args(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o,
                            const Tensor& lse, bool causal, double scale, bool allow_f16 = false) {
  const bool f16 = allow_f16 && q.scalar_type() == at::kHalf;
  if (f16) {
    TORCH_CHECK(q.is_cuda() && k.is_cuda() && v.is_cuda() && o.is_cuda() && k.scalar_type() == at::kHalf &&
                    v.scalar_type() == at::kHalf && o.scalar_type() == at::kHalf, "attention: q, k, v, o must all be fp16 CUDA tensors");
  } else {
    check_bf16_cuda(q, "attention q");
    check_bf16_cuda(k, "attention k");
    check_bf16_cuda(v, "attention v");
    check_bf16_cuda(o, "attention o");
  }
  check_f32_cuda(lse, "attention lse");
  TORCH_CHECK(q.dim() == 4 && k.dim() == 4 && v.dim() == 4 && o.dim() == 4,
              "attention: tensors must be [B, T, H, D]");
  TORCH_CHECK(q.stride(3) == 1 && k.stride(3) == 1 && v.stride(3) == 1 && o.stride(3) == 1,
              "attention: head dim must be contiguous");
  rt::AttnArgs a{};
  a.B = int(q.size(0));
  a.Tq = int(q.size(1));
  a.H = int(q.size(2));
  a.D = int(q.size(3));
  a.Tk = int(k.size(1));
  a.Hkv = int(k.size(2));
  TORCH_CHECK(k.size(0) == a.B && v.size(0) == a.B && k.size(3) == a.D && v.size(3) == a.D &&
                  v.size(1) == a.Tk && v.size(2) == a.Hkv,
              "attention: k/v shape mismatch");
  TORCH_CHECK(o.sizes() == q.sizes(), "attention: o must have the shape of q");
  TORCH_CHECK(lse.is_contiguous() && lse.numel() == int64_t(a.B) * a.H * a.Tq,
              "attention: lse must be contiguous [B, H, Tq]");
  a.q = q.data_ptr();
  a.k = k.data_ptr();
  a.v = v.data_ptr();
  a.o = o.data_ptr();
  a.q_sb = q.stride(0); a.q_st = q.stride(1); a.q_sh = q.stride(2);
  a.k_sb = k.stride(0); a.k_st = k.stride(1); a.k_sh = k.stride(2);
  a.v_sb = v.stride(0); a.v_st = v.stride(1); a.v_sh = v.stride(2);
  a.o_sb = o.stride(0); a.o_st = o.stride(1); a.o_sh = o.stride(2);
  a.lse = lse.data_ptr<float>();
  a.causal = causal ? 1 : 0;
  a.scale = float(scale);
  a.io_fp16 = f16 ? 1 : 0;
  return a;
}

void attn_fwd(const Tensor& q, const Tensor& k, const Tensor& v, Tensor& o, Tensor& lse,
              bool causal, double scale) {
  c10::cuda::CUDAGuard guard(q.device());
  rt::AttnArgs a = make_attn_args(q, k, v, o, lse, causal, scale, /*allow_f16=*/true);
  rt::attn_fwd(a, stream_of(q));
}

void attn_bwd(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor& o, const Tensor& d_o,
              const Tensor& lse, Tensor& delta, Tensor& dq, Tensor& dk, Tensor& dv, bool causal,
              double scale, const OptTensor& dq_acc) {
  c10::cuda::CUDAGuard guard(q.device());
  rt::AttnArgs a = make_attn_args(q, k, v, o, lse, causal, scale);
  check_bf16_cuda(d_o, "attention do");
  check_f32_cuda(delta, "attention delta");
  check_bf16_cuda(dq, "attention dq");
  check_bf16_cuda(dk, "attention dk");
  check_bf16_cuda(dv, "attention dv");
  TORCH_CHECK(d_o.sizes() == o.sizes() && d_o.strides() == o.strides(),
              "attention: do must have the shape and strides of o");
  TORCH_CHECK(delta.is_contiguous() && delta.numel() == lse.numel(), "attention: bad delta");
  TORCH_CHECK(dq.sizes() == q.sizes() && dk.sizes() == k.sizes() && dv.sizes() == v.sizes(),
              "attention: gradient shapes must match inputs");
  TORCH_CHECK(dq.stride(3) == 1 && dk.stride(3) == 1 && dv.stride(3) == 1,
              "attention: gradient head dim must be contiguous");
  a.d_o = d_o.data_ptr();
  a.delta = delta.data_ptr<float>();
  a.dq = dq.data_ptr();
  a.dk = dk.data_ptr();
  a.dv = dv.data_ptr();
  a.dq_sb = dq.stride(0); a.dq_st = dq.stride(1); a.dq_sh = dq.stride(2);
  a.dk_sb = dk.stride(0); a.dk_st = dk.stride(1); a.dk_sh = dk.stride(2);
  a.dv_sb = dv.stride(0); a.dv_st = dv.stride(1); a.dv_sh = dv.stride(2);
  for (int64_t s : {a.dq_sb, a.dq_st, a.dq_sh, a.dk_sb, a.dk_st, a.dk_sh, a.dv_sb, a.dv_st, a.dv_sh})
    TORCH_CHECK(s % 8 == 0, "attention: gradient strides must be multiples of 8 elements");
  if (dq_acc.has_value() && dq_acc->defined()) {
    check_f32_cuda(*dq_acc, "attention dq_acc");
    TORCH_CHECK(dq_acc->is_contiguous() && dq_acc->numel() == q.numel(), "attention: dq_acc must be a contiguous fp32 tensor shaped like q");
    a.dq_acc = dq_acc->data_ptr<float>();
  }
  rt::attn_bwd(a, stream_of(q));
}

void norm_fwd(const Tensor& x, const Tensor& gamma, const OptTensor& beta, Tensor& y,
              const OptTensor& mean, Tensor& rstd, double eps, bool rms) {
  check_bf16_cuda(x, "norm x");
  check_bf16_cuda(gamma, "norm gamma");
  check_bf16_cuda(y, "norm y");
  check_f32_cuda(rstd, "norm rstd");
  TORCH_CHECK(x.is_contiguous() && y.is_contiguous() && gamma.is_contiguous(), "norm: contiguous");
  c10::cuda::CUDAGuard guard(x.device());
  rt::NormArgs a{};
  a.C = int(gamma.numel());
  a.rows = x.numel() / a.C;
  a.x = x.data_ptr();
  a.gamma = gamma.data_ptr();
  a.beta = (beta.has_value() && beta->defined()) ? beta->data_ptr() : nullptr;
  a.y = y.data_ptr();
  a.mean = (mean.has_value() && mean->defined()) ? mean->data_ptr<float>() : nullptr;
  a.rstd = rstd.data_ptr<float>();
  TORCH_CHECK(rms || a.mean != nullptr, "layer norm needs a mean buffer");
  a.eps = float(eps);
  a.rms = rms;
  rt::norm_fwd(a, stream_of(x));
}

OptTensor norm_bwd(const Tensor& dy, const Tensor& x, const Tensor& gamma, const OptTensor& mean,
              const Tensor& rstd, const OptTensor& dres, Tensor& dx, const OptTensor& dgamma,
              const OptTensor& dbeta, bool rms, int64_t reduce_stream) {
  check_bf16_cuda(dy, "norm dy");
  check_bf16_cuda(x, "norm x");
  check_bf16_cuda(dx, "norm dx");
  TORCH_CHECK(dy.is_contiguous() && x.is_contiguous() && dx.is_contiguous(), "norm: contiguous");
  c10::cuda::CUDAGuard guard(x.device());
  rt::NormArgs a{};
  a.C = int(gamma.numel());
  a.rows = x.numel() / a.C;
  a.dy = dy.data_ptr();
  a.x = x.data_ptr();
  a.gamma = gamma.data_ptr();
  a.mean = (mean.has_value() && mean->defined()) ? mean->data_ptr<float>() : nullptr;
  a.rstd = rstd.data_ptr<float>();
  if (dres.has_value() && dres->defined()) {
    check_bf16_cuda(*dres, "norm dres");
    TORCH_CHECK(dres->is_contiguous() && dres->numel() == x.numel(), "norm: bad dres");
    a.dres = dres->data_ptr();
  }
  a.dx = dx.data_ptr();
  if (dgamma.has_value() && dgamma->defined()) {
    check_f32_cuda(*dgamma, "norm dgamma");
    a.dgamma = dgamma->data_ptr<float>();
  }
  if (dbeta.has_value() && dbeta->defined()) {
    check_f32_cuda(*dbeta, "norm dbeta");
    a.dbeta = dbeta->data_ptr<float>();
  }
  a.rms = rms;
  // scratch for the two-stage gamma/beta reduction
  a.n_partial = rt::norm_bwd_num_partials(a.rows, rt::sm_count(x.device().index()));
  at::Tensor partial = at::empty({2, a.n_partial, a.C}, x.options().dtype(at::kFloat));
  a.partial = partial.data_ptr<float>();
  if (reduce_stream == 0) {
    rt::norm_bwd(a, stream_of(x));
    return c10::nullopt;
  }
  // dgamma / dbeta have no consumer before the optimizer: their reduction goes to the caller's side stream, ordered
  // after stage 1 by an event; the partial sums go back to the caller, who keeps them alive for it
  cudaStream_t main_s = stream_of(x), side = reinterpret_cast<cudaStream_t>(reduce_stream);
  rt::norm_bwd_stage1(a, main_s, &side);
  static thread_local cudaEvent_t ev[64] = {nullptr};
  const int dev = x.device().index();
  if (ev[dev] == nullptr) C10_CUDA_CHECK(cudaEventCreateWithFlags(&ev[dev], cudaEventDisableTiming));
  C10_CUDA_CHECK(cudaEventRecord(ev[dev], main_s));
  C10_CUDA_CHECK(cudaStreamWaitEvent(side, ev[dev], 0));
  rt::norm_bwd_reduce(a, side);
  return partial;  // the caller holds it until its main stream has waited for the side stream
}

void embedding_fwd(const Tensor& idx, const Tensor& wte, const OptTensor& wpe, Tensor& out,
                   int64_t T) {
  TORCH_CHECK(idx.is_cuda() && idx.scalar_type() == at::kLong && idx.is_contiguous(),
              "embedding: idx must be a contiguous CUDA int64 tensor");
  check_bf16_cuda(wte, "embedding wte");
  check_bf16_cuda(out, "embedding out");
  c10::cuda::CUDAGuard guard(idx.device());
  const int C = int(wte.size(1));
  const void* pe = nullptr;
  if (wpe.has_value() && wpe->defined()) {
    check_bf16_cuda(*wpe, "embedding wpe");
    TORCH_CHECK(wpe->size(1) == C && wpe->size(0) >= T, "embedding: wpe too small");
    pe = wpe->data_ptr();
  }
  rt::embedding_fwd(idx.data_ptr<int64_t>() ? reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()) : nullptr,
                    wte.data_ptr(), pe, out.data_ptr(), idx.numel(), int(T), C, int(wte.size(0)),
                    stream_of(idx));
}

void embedding_bwd(const Tensor& idx, const Tensor& dout, const OptTensor& dwte,
                   const OptTensor& dwpe, int64_t T, int64_t vocab) {
  check_bf16_cuda(dout, "embedding dout");
  TORCH_CHECK(dout.is_contiguous(), "embedding: dout must be contiguous");
  c10::cuda::CUDAGuard guard(idx.device());
  const int C = int(dout.size(-1));
  float* pw = nullptr;
  float* pp = nullptr;
  if (dwte.has_value() && dwte->defined()) {
    check_f32_cuda(*dwte, "embedding dwte");
    pw = dwte->data_ptr<float>();
  }
  if (dwpe.has_value() && dwpe->defined()) {
    check_f32_cuda(*dwpe, "embedding dwpe");
    pp = dwpe->data_ptr<float>();
  }
  rt::embedding_bwd(reinterpret_cast<const long long*>(idx.data_ptr<int64_t>()), dout.data_ptr(), pw,
                    pp, idx.numel(), int(T), C, int(vocab), stream_of(idx));
}

void cross_entropy(Tensor& logits, const Tensor& targets, Tensor& loss, int64_t vocab,
                   double grad_scale, int64_t ignore_index) {
  check_bf16_cuda(logits, "cross_entropy logits");
  check_f32_cuda(loss, "cross_entropy loss");
  TORCH_CHECK(logits.dim() == 2 && logits.stride(1) == 1, "cross_entropy: logits must be 2-D");
  TORCH_CHECK(targets.is_cuda() && targets.scalar_type() == at::kLong && targets.is_contiguous() &&
                  targets.numel() == logits.size(0),
              "cross_entropy: targets must be int64 [rows]");
  TORCH_CHECK(loss.numel() == logits.size(0) && loss.is_contiguous(), "cross_entropy: bad loss");
  TORCH_CHECK(vocab <= logits.size(1), "cross_entropy: vocab exceeds row length");
  c10::cuda::CUDAGuard guard(logits.device());
  rt::cross_entropy_fwd_bwd(logits.data_ptr(),
                            reinterpret_cast<const long long*>(targets.data_ptr<int64_t>()),
                            loss.data_ptr<float>(), logits.size(0), int(vocab),
                            int(logits.stride(0)), float(grad_scale), ignore_index,
                            stream_of(logits));
}

void colsum_accum(const Tensor& x, Tensor& out) {
  check_bf16_cuda(x, "colsum x");
  check_f32_cuda(out, "colsum out");
  TORCH_CHECK(x.dim() == 2 && x.stride(1) == 1 && out.numel() == x.size(1) && out.is_contiguous(),
              "colsum: x [M, N], out [N]");
  c10::cuda::CUDAGuard guard(x.device());
  rt::colsum_accum(x.data_ptr(), out.data_ptr<float>(), x.size(0), int(x.size(1)), x.stride(0),
                   stream_of(x));
}

void reduce_all(const Tensor& x, int64_t mode, Tensor& out) {
  TORCH_CHECK(x.is_cuda() && x.is_contiguous(), "reduce_all: contiguous CUDA tensor required");
  check_f32_cuda(out, "reduce_all out");
  int dtype;
  if (x.scalar_type() == at::kFloat) dtype = 0;
  else if (x.scalar_type() == at::kBFloat16) dtype = 1;
  else TORCH_CHECK(false, "reduce_all: fp32 or bf16 input required");
  c10::cuda::CUDAGuard guard(x.device());
  rt::reduce_all(x.data_ptr(), dtype, int(mode), out.data_ptr<float>(), x.numel(), stream_of(x));
}

void fused_optim_step(Tensor& master, Tensor& grad, const OptTensor& m, const OptTensor& v,
                      const OptTensor& param_lp, int64_t mode, double lr, double beta1, double beta2,
                      double eps, double weight_decay, double bias_corr1, double bias_corr2,
                      double grad_scale, bool zero_grad, bool nesterov, bool first_step) {
  check_f32_cuda(master, "optim master");
  check_f32_cuda(grad, "optim grad");
  TORCH_CHECK(master.is_contiguous() && grad.is_contiguous() && grad.numel() == master.numel(),
              "optim: flat contiguous buffers of equal length required");
  c10::cuda::CUDAGuard guard(master.device());
  rt::OptimArgs a{};
  a.master = master.data_ptr<float>();
  a.grad = grad.data_ptr<float>();
  if (m.has_value() && m->defined()) {
    check_f32_cuda(*m, "optim m");
    TORCH_CHECK(m->numel() == master.numel() && m->is_contiguous(), "optim: bad m");
    a.m = m->data_ptr<float>();
  }
  if (v.has_value() && v->defined()) {
    check_f32_cuda(*v, "optim v");
    TORCH_CHECK(v->numel() == master.numel() && v->is_contiguous(), "optim: bad v");
    a.v = v->data_ptr<float>();
  }
  if (param_lp.has_value() && param_lp->defined()) {
    check_bf16_cuda(*param_lp, "optim param_lp");
    TORCH_CHECK(param_lp->numel() == master.numel() && param_lp->is_contiguous(), "optim: bad lp");
    a.param_lp = param_lp->data_ptr();
  }
  TORCH_CHECK(mode == rt::OPT_SGD || (a.m && a.v), "optim: Adam modes need m and v");
  a.n = master.numel();
  a.lr = float(lr);
  a.beta1 = float(beta1);
  a.beta2 = float(beta2);
  a.eps = float(eps);
  a.weight_decay = float(weight_decay);
  a.bias_corr1 = float(bias_corr1);
  a.bias_corr2 = float(bias_corr2);
  a.grad_scale = float(grad_scale);
  a.mode = int(mode);
  a.zero_grad = zero_grad;
  a.nesterov = nesterov;
  a.first_step = first_step;
  rt::fused_optim_step(a, stream_of(master));
}

}  // namespace

void register_extra_ops(pybind11::module_& m);  // bindings_extra.cpp

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "rustorch_b200 native sm_100a kernels";
  m.def("gemm", &gemm, "bf16 tcgen05 GEMM with fused epilogues", pybind11::arg("a"), pybind11::arg("a_mn"), pybind11::arg("b"),
        pybind11::arg("b_mn"), pybind11::arg("c"), pybind11::arg("bias"), pybind11::arg("aux"), pybind11::arg("epi_mode"),
        pybind11::arg("alpha"), pybind11::arg("accumulate"), pybind11::arg("split_k"), pybind11::arg("block_n"),
        pybind11::arg("alpha_dev") = pybind11::none());
  m.def("attn_fwd", &attn_fwd);
  m.def("attn_bwd", &attn_bwd, pybind11::arg("q"), pybind11::arg("k"), pybind11::arg("v"), pybind11::arg("o"), pybind11::arg("d_o"),
        pybind11::arg("lse"), pybind11::arg("delta"), pybind11::arg("dq"), pybind11::arg("dk"), pybind11::arg("dv"), pybind11::arg("causal"),
        pybind11::arg("scale"), pybind11::arg("dq_acc") = pybind11::none());
  m.def("norm_fwd", &norm_fwd);
  m.def("norm_bwd", &norm_bwd, pybind11::arg("dy"), pybind11::arg("x"), pybind11::arg("gamma"), pybind11::arg("mean"), pybind11::arg("rstd"), pybind11::arg("dres"), pybind11::arg("dx"),
        pybind11::arg("dgamma"), pybind11::arg("dbeta"), pybind11::arg("rms"), pybind11::arg("reduce_stream") = 0);
  m.def("embedding_fwd", &embedding_fwd);
  m.def("embedding_bwd", &embedding_bwd);
  m.def("cross_entropy", &cross_entropy);
  m.def("colsum_accum", &colsum_accum);
  m.def("reduce_all", &reduce_all);
  m.def("fused_optim_step", &fused_optim_step);
  m.def("launch_count", []() { return rt::launch_count(); });
  m.def("read_status", [](int64_t device) { return rt::read_status(int(device)); });
  register_extra_ops(m);
}
