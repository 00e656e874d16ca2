// Bindings for the ops added after the core training path (elementwise family, quantised
// GEMV, collectives).  Kept separate so touching one group does not recompile the other.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <cstring>

#include "api.h"
#include "common/launch.h"

namespace {

using at::Tensor;

cudaStream_t cur_stream(int device) { return at::cuda::getCurrentCUDAStream(device).stream(); }

// Peer pointers arrive as Python ints (they come from symmetric-memory rendezvous).
void ddp_bucket_adamw(const std::vector<int64_t>& grad_ptrs, const std::vector<int64_t>& lp_ptrs,
                      const std::vector<int64_t>& flag_ptrs, Tensor& master, Tensor& m, Tensor& v,
                      Tensor& done_counter, int64_t bucket_start, int64_t chunk_len, int64_t rank,
                      int64_t epoch, int64_t start_slot, int64_t end_slot, double timeout_s, double lr,
                      double beta1, double beta2, double eps, double weight_decay, double bias_corr1,
                      double bias_corr2, double grad_scale, int64_t n_ctas) {
  const int world = int(grad_ptrs.size());
  TORCH_CHECK(world >= 1 && world <= rt::RT_MAX_PEERS, "ddp: world size must be in [1, 8]");
  TORCH_CHECK(int(lp_ptrs.size()) == world && int(flag_ptrs.size()) == world, "ddp: pointer lists differ");
  TORCH_CHECK(master.is_cuda() && master.scalar_type() == at::kFloat && master.is_contiguous() &&
                  m.scalar_type() == at::kFloat && v.scalar_type() == at::kFloat &&
                  m.numel() == master.numel() && v.numel() == master.numel(),
              "ddp: master/m/v must be flat fp32 CUDA buffers of equal length");
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
  a.m = m.data_ptr<float>();
  a.v = v.data_ptr<float>();
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
  rt::ddp_bucket_adamw(a, int(n_ctas), cur_stream(master.device().index()));
}

void ddp_wait_end(int64_t flags_ptr, int64_t n_slots, int64_t world, int64_t rank, int64_t epoch,
                  double timeout_s, int64_t device) {
  c10::cuda::CUDAGuard guard(static_cast<c10::DeviceIndex>(device));
  rt::ddp_wait_end(reinterpret_cast<const int*>(flags_ptr), int(n_slots), int(world), int(rank),
                   int(epoch), (unsigned long long)(timeout_s * 1e9), rt::status_word(int(device)),
                   cur_stream(int(device)));
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

void register_extra_ops(pybind11::module_& m) {
  m.def("crc64", &crc64_bytes, "CRC-64/XZ of a bytes object");
  m.def("ddp_bucket_adamw", &ddp_bucket_adamw,
        "fused reduce-scatter + scale + AdamW + all-gather of one gradient bucket over peer memory");
  m.def("ddp_wait_end", &ddp_wait_end);
}
