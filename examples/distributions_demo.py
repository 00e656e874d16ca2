"""Probability distributions: sampling, log-densities, CDF / inverse CDF, entropy, reparameterised gradients."""
import _path  # noqa: F401

import torch

from rustorch_b200 import distributions as D

torch.manual_seed(0)
n = D.Normal(1.0, 2.0)
s = n.sample((50000,))
print("Normal(1, 2): sample mean %.3f std %.3f; log_prob(1) %.4f; cdf(1) %.2f; icdf(0.975) %.3f; entropy %.4f"
      % (float(s.mean()), float(s.std()), float(n.log_prob(torch.tensor(1.0))), float(n.cdf(torch.tensor(1.0))),
         float(n.icdf(torch.tensor(0.975))), float(n.entropy())))
for name, dist in (("Uniform(0, 4)", D.Uniform(0.0, 4.0)), ("Exponential(2)", D.Exponential(2.0)), ("Gamma(3, 2)", D.Gamma(3.0, 2.0)),
                   ("Beta(2, 5)", D.Beta(2.0, 5.0))):
    x = dist.sample((50000,))
    print(f"{name:<15} mean {float(dist.mean):.3f} (sampled {float(x.mean()):.3f})  variance {float(dist.variance):.3f} (sampled {float(x.var()):.3f})")
b = D.Bernoulli(probs=torch.tensor(0.3))
c = D.Categorical(probs=torch.tensor([0.1, 0.2, 0.7]))
print("Bernoulli(0.3) frequency %.3f; Categorical counts" % float(b.sample((20000,)).mean()),
      torch.bincount(c.sample((10000,)), minlength=3).tolist(), " entropy %.4f" % float(c.entropy()))
mu = torch.tensor(0.0, requires_grad=True)
(D.Normal(mu, 1.0).rsample((4096,)) ** 2).mean().backward()
print("d/dmu E[x^2] at mu = 0 by reparameterisation: %.3f (exact 0)" % float(mu.grad))
print("registered:", sorted(D.available_distributions()))
