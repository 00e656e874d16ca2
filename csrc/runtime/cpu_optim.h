// Single-tensor optimizer updates on host memory (fp32), for the small-tensor regime where interpreter overhead, not
// arithmetic, sets the step rate (the reference publishes 15-34 K steps/s on a 1000-element parameter,
// docs/guides/performance.md:15-18; its updates are src/optim/adamax.rs, nadam.rs:135-156, radam.rs:187-205,
// lbfgs.rs:192-203).  Same update formulas as torch.optim, so the two paths are interchangeable.
#pragma once
#include <cstdint>

namespace rt {

enum CpuOptKind : int { OPT_CPU_ADAM = 0, OPT_CPU_ADAMW = 1, OPT_CPU_ADAMAX = 2, OPT_CPU_NADAM = 3, OPT_CPU_RADAM = 4 };

// p, g, m, v: n floats each.  `step` counts from 1.  mu_product: NAdam's running product (in / out), else unused.
void cpu_adam_family_step(int kind, float* p, const float* g, float* m, float* v, int64_t n, double lr, double beta1, double beta2,
                          double eps, double weight_decay, int64_t step, double momentum_decay, double* mu_product);

// One L-BFGS iteration from an explicit gradient: d = -H g by the two-loop recursion over the `count` newest (s, y)
// pairs of the ring buffers S, Y [hist][n] (newest at index (head + hist - 1) % hist), p += lr * d; then the pair for
// the next call is started (prev_p, prev_g).  Returns the new (count, head) packed as count * 65536 + head.
int64_t cpu_lbfgs_step(float* p, const float* g, float* prev_p, float* prev_g, float* S, float* Y, float* rho, float* scratch,
                       int64_t n, int64_t hist, int64_t count, int64_t head, int64_t has_prev, double lr);

}  // namespace rt
