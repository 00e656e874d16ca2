#include "cpu_optim.h"

#include <algorithm>
#include <cmath>

namespace rt {

void cpu_adam_family_step(int kind, float* p, const float* g, float* m, float* v, int64_t n, double lr, double beta1, double beta2,
                          double eps, double weight_decay, int64_t step, double momentum_decay, double* mu_product) {
  const float b1 = (float)beta1, b2 = (float)beta2, e = (float)eps, wd = (float)weight_decay;
  const double bc1 = 1.0 - std::pow(beta1, (double)step), bc2 = 1.0 - std::pow(beta2, (double)step);
  if (kind == OPT_CPU_ADAMW && wd != 0.f) {
    const float k = 1.f - (float)lr * wd;
    for (int64_t i = 0; i < n; ++i) p[i] *= k;
  }
  const bool l2 = wd != 0.f && kind != OPT_CPU_ADAMW;
  if (kind == OPT_CPU_ADAM || kind == OPT_CPU_ADAMW) {
    const float step_size = (float)(lr / bc1), inv_sqrt_bc2 = (float)(1.0 / std::sqrt(bc2));
    for (int64_t i = 0; i < n; ++i) {
      const float gi = l2 ? g[i] + wd * p[i] : g[i];
      m[i] = b1 * m[i] + (1.f - b1) * gi;
      v[i] = b2 * v[i] + (1.f - b2) * gi * gi;
      p[i] -= step_size * m[i] / (std::sqrt(v[i]) * inv_sqrt_bc2 + e);
    }
  } else if (kind == OPT_CPU_ADAMAX) {
    const float clr = (float)(lr / bc1);
    for (int64_t i = 0; i < n; ++i) {
      const float gi = l2 ? g[i] + wd * p[i] : g[i];
      m[i] = b1 * m[i] + (1.f - b1) * gi;
      v[i] = std::max(b2 * v[i], std::fabs(gi) + e);        // v holds the exponentially weighted infinity norm
      p[i] -= clr * m[i] / v[i];
    }
  } else if (kind == OPT_CPU_NADAM) {
    const double mu = beta1 * (1.0 - 0.5 * std::pow(0.96, (double)step * momentum_decay));
    const double mu_next = beta1 * (1.0 - 0.5 * std::pow(0.96, (double)(step + 1) * momentum_decay));
    *mu_product *= mu;
    const float cg = (float)(lr * (1.0 - mu) / (1.0 - *mu_product));
    const float cm = (float)(lr * mu_next / (1.0 - *mu_product * mu_next));
    const float inv_sqrt_bc2 = (float)(1.0 / std::sqrt(bc2));
    for (int64_t i = 0; i < n; ++i) {
      const float gi = l2 ? g[i] + wd * p[i] : g[i];
      m[i] = b1 * m[i] + (1.f - b1) * gi;
      v[i] = b2 * v[i] + (1.f - b2) * gi * gi;
      const float denom = std::sqrt(v[i]) * inv_sqrt_bc2 + e;
      p[i] -= cg * gi / denom + cm * m[i] / denom;
    }
  } else {  // RAdam
    const double rho_inf = 2.0 / (1.0 - beta2) - 1.0;
    const double rho_t = rho_inf - 2.0 * (double)step * std::pow(beta2, (double)step) / bc2;
    const bool rectify = rho_t > 5.0;
    const float rect = rectify ? (float)std::sqrt((rho_t - 4.0) * (rho_t - 2.0) * rho_inf / ((rho_inf - 4.0) * (rho_inf - 2.0) * rho_t)) : 0.f;
    const float c1 = (float)(lr / bc1), sqrt_bc2 = (float)std::sqrt(bc2);
    for (int64_t i = 0; i < n; ++i) {
      const float gi = l2 ? g[i] + wd * p[i] : g[i];
      m[i] = b1 * m[i] + (1.f - b1) * gi;
      v[i] = b2 * v[i] + (1.f - b2) * gi * gi;
      p[i] -= rectify ? c1 * m[i] * rect * sqrt_bc2 / (std::sqrt(v[i]) + e) : c1 * m[i];
    }
  }
}

static inline double dot(const float* a, const float* b, int64_t n) {
  double s = 0.0;
  for (int64_t i = 0; i < n; ++i) s += (double)a[i] * b[i];
  return s;
}

int64_t cpu_lbfgs_step(float* p, const float* g, float* prev_p, float* prev_g, float* S, float* Y, float* rho, float* scratch,
                       int64_t n, int64_t hist, int64_t count, int64_t head, int64_t has_prev, double lr) {
  // close the pair opened by the previous call: s = p - prev_p, y = g - prev_g
  if (has_prev) {
    float* s = S + head * n;
    float* y = Y + head * n;
    for (int64_t i = 0; i < n; ++i) {
      s[i] = p[i] - prev_p[i];
      y[i] = g[i] - prev_g[i];
    }
    const double ys = dot(y, s, n);
    if (ys > 1e-10) {
      rho[head] = (float)(1.0 / ys);
      head = (head + 1) % hist;
      count = std::min(count + 1, hist);
    }
  }
  // two-loop recursion, newest pair first
  float* q = scratch;               // n floats
  float* alpha = scratch + n;       // hist floats
  for (int64_t i = 0; i < n; ++i) q[i] = g[i];
  for (int64_t k = 0; k < count; ++k) {
    const int64_t j = (head + hist - 1 - k) % hist;
    const double a = rho[j] * dot(S + j * n, q, n);
    alpha[k] = (float)a;
    const float* y = Y + j * n;
    for (int64_t i = 0; i < n; ++i) q[i] -= (float)a * y[i];
  }
  if (count > 0) {
    const int64_t j = (head + hist - 1) % hist;
    const double gamma = dot(S + j * n, Y + j * n, n) / dot(Y + j * n, Y + j * n, n);
    for (int64_t i = 0; i < n; ++i) q[i] *= (float)gamma;
  }
  for (int64_t k = count - 1; k >= 0; --k) {
    const int64_t j = (head + hist - 1 - k) % hist;
    const double b = rho[j] * dot(Y + j * n, q, n);
    const float* s = S + j * n;
    const float c = alpha[k] - (float)b;
    for (int64_t i = 0; i < n; ++i) q[i] += c * s[i];
  }
  for (int64_t i = 0; i < n; ++i) {
    prev_p[i] = p[i];
    prev_g[i] = g[i];
    p[i] -= (float)lr * q[i];
  }
  return count * 65536 + head;
}

}  // namespace rt
