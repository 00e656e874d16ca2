// Python module `_host`: the torch-free, CUDA-free part of the native runtime (arena allocator, CRC-64,
// plan scheduler).  It loads on machines without a GPU, so the host-side logic is tested there.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstdint>
#include <string>

#include "arena.h"
#include "cpu_optim.h"
#include "plan.h"
#include "protocol_sim.h"

namespace py = pybind11;

namespace {

// CRC-64/XZ (reflected polynomial 0xC96C5795D7870F42, init and final XOR all-ones), slicing-by-8: the
// checksum of the RusTorch binary container (reference: src/serialization/core.rs:255-269).
uint64_t crc64(py::bytes data, uint64_t crc) {
  static uint64_t table[8][256];
  static bool ready = false;
  if (!ready) {
    for (int i = 0; i < 256; ++i) {
      uint64_t c = (uint64_t)i;
      for (int k = 0; k < 8; ++k) c = (c & 1) ? (c >> 1) ^ 0xC96C5795D7870F42ull : c >> 1;
      table[0][i] = c;
    }
    for (int i = 0; i < 256; ++i)
      for (int t = 1; t < 8; ++t) table[t][i] = (table[t - 1][i] >> 8) ^ table[0][table[t - 1][i] & 0xFF];
    ready = true;
  }
  char* buf;
  py::ssize_t len;
  if (PyBytes_AsStringAndSize(data.ptr(), &buf, &len)) throw py::error_already_set();
  const unsigned char* p = reinterpret_cast<const unsigned char*>(buf);
  uint64_t c = ~crc;
  size_t n = (size_t)len;
  while (n >= 8) {
    uint64_t w;
    memcpy(&w, p, 8);
    c ^= w;
    c = table[7][c & 0xFF] ^ table[6][(c >> 8) & 0xFF] ^ table[5][(c >> 16) & 0xFF] ^ table[4][(c >> 24) & 0xFF] ^
        table[3][(c >> 32) & 0xFF] ^ table[2][(c >> 40) & 0xFF] ^ table[1][(c >> 48) & 0xFF] ^ table[0][c >> 56];
    p += 8;
    n -= 8;
  }
  while (n--) c = table[0][(c ^ *p++) & 0xFF] ^ (c >> 8);
  return ~c;
}

}  // namespace

PYBIND11_MODULE(_host, m) {
  m.doc() = "host-side native runtime (no CUDA, no torch)";
  m.def("crc64", &crc64, py::arg("data"), py::arg("crc") = 0);
  // optimizer updates on host buffers given by address (torch tensors' data_ptr(); the module itself is torch-free)
  m.def("cpu_adam_family_step",
        [](int kind, uintptr_t p, uintptr_t g, uintptr_t mm, uintptr_t v, int64_t n, double lr, double b1, double b2, double eps,
           double wd, int64_t step, double momentum_decay, double mu_product) {
          rt::cpu_adam_family_step(kind, reinterpret_cast<float*>(p), reinterpret_cast<const float*>(g), reinterpret_cast<float*>(mm),
                                   reinterpret_cast<float*>(v), n, lr, b1, b2, eps, wd, step, momentum_decay, &mu_product);
          return mu_product;
        });
  m.def("cpu_lbfgs_step", [](uintptr_t p, uintptr_t g, uintptr_t pp, uintptr_t pg, uintptr_t S, uintptr_t Y, uintptr_t rho,
                             uintptr_t scratch, int64_t n, int64_t hist, int64_t count, int64_t head, int64_t has_prev, double lr) {
    return rt::cpu_lbfgs_step(reinterpret_cast<float*>(p), reinterpret_cast<const float*>(g), reinterpret_cast<float*>(pp),
                              reinterpret_cast<float*>(pg), reinterpret_cast<float*>(S), reinterpret_cast<float*>(Y),
                              reinterpret_cast<float*>(rho), reinterpret_cast<float*>(scratch), n, hist, count, head, has_prev, lr);
  });

  // host emulation of the peer-memory kernels' synchronisation protocols, one thread per rank (GIL released)
  auto sim_dict = [](const rt_host::SimResult& r) {
    py::dict d;
    d["mismatches"] = r.mismatches;
    d["timeouts"] = r.timeouts;
    d["checked"] = r.checked;
    return d;
  };
  m.def("sim_lamport_allreduce",
        [sim_dict](int world, long long calls, int words, int slots, int slow_rank, int slow_us, unsigned seed) {
          rt_host::SimResult r;
          {
            py::gil_scoped_release nogil;
            r = rt_host::sim_lamport_allreduce(world, calls, words, slots, slow_rank, slow_us, seed);
          }
          return sim_dict(r);
        },
        py::arg("world"), py::arg("calls"), py::arg("words") = 64, py::arg("slots") = 3, py::arg("slow_rank") = -1,
        py::arg("slow_us") = 0, py::arg("seed") = 1);
  m.def("sim_epoch_counters",
        [sim_dict](int world, long long calls, int blocks, int tiles, int parities, int slow_rank, int slow_us, unsigned seed) {
          rt_host::SimResult r;
          {
            py::gil_scoped_release nogil;
            r = rt_host::sim_epoch_counters(world, calls, blocks, tiles, parities, slow_rank, slow_us, seed);
          }
          return sim_dict(r);
        },
        py::arg("world"), py::arg("calls"), py::arg("blocks") = 4, py::arg("tiles") = 8, py::arg("parities") = 2,
        py::arg("slow_rank") = -1, py::arg("slow_us") = 0, py::arg("seed") = 1);

  py::class_<rt::Arena>(m, "Arena")
      .def(py::init<uint64_t, uint64_t>(), py::arg("capacity"), py::arg("alignment") = 256)
      .def("allocate", &rt::Arena::allocate)
      .def("release", &rt::Arena::release)
      .def("reset", &rt::Arena::reset)
      .def("size_of", &rt::Arena::size_of)
      .def("stats", [](const rt::Arena& a) {
        const rt::ArenaStats s = a.stats();
        py::dict d;
        d["capacity"] = s.capacity;
        d["in_use"] = s.in_use;
        d["peak"] = s.peak;
        d["n_alloc"] = s.n_alloc;
        d["n_free"] = s.n_free;
        d["n_fail"] = s.n_fail;
        d["live_blocks"] = s.live_blocks;
        d["free_ranges"] = s.free_ranges;
        d["largest_free"] = s.largest_free;
        d["fragmentation"] = s.fragmentation;
        return d;
      });

  py::class_<rt::PlanNode>(m, "PlanNode")
      .def_readonly("id", &rt::PlanNode::id)
      .def_readonly("op", &rt::PlanNode::op)
      .def_readonly("inputs", &rt::PlanNode::inputs)
      .def_readonly("out_bytes", &rt::PlanNode::out_bytes);

  py::class_<rt::ExecutionPlan>(m, "ExecutionPlan")
      .def(py::init<>())
      .def("add_node", &rt::ExecutionPlan::add_node, py::arg("op"), py::arg("inputs"), py::arg("out_bytes") = 0)
      .def("mark_output", &rt::ExecutionPlan::mark_output)
      .def("num_nodes", &rt::ExecutionPlan::num_nodes)
      .def("node", &rt::ExecutionPlan::node, py::return_value_policy::reference_internal)
      .def("topo_order", &rt::ExecutionPlan::topo_order)
      .def("levels", &rt::ExecutionPlan::levels)
      .def("eliminate_dead", &rt::ExecutionPlan::eliminate_dead)
      .def("memory_plan", &rt::ExecutionPlan::memory_plan, py::arg("alignment") = 256)
      .def("fusible_chains", &rt::ExecutionPlan::fusible_chains);
}
