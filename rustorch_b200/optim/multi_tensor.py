"""Native multi-tensor step for the per-tensor optimizers (``csrc/optim/multi_tensor_optim.cu``).

``try_step(opt, kind)`` updates every parameter of a ``torch.optim``-style optimizer with ONE kernel launch per 32
tensors when all parameters that have gradients are dense contiguous fp32 / bf16 CUDA tensors and no exotic flag
(amsgrad, capturable, differentiable, sparse gradients) is set; otherwise it returns ``False`` and the caller falls
back to the stock per-tensor arithmetic.  The optimizer state keeps torch's key names (``step``, ``exp_avg``,
``exp_avg_sq``, ``exp_inf``, ``mu_product``, ``square_avg``, ``momentum_buffer``, ``grad_avg``, ``sum``), so
``state_dict`` round trips and a later fallback step continue from the same state.  State tensors are fp32 even for
bf16 parameters.

Step-count dependent scalars are evaluated here once per step and group (the reference evaluates them per tensor on
the host: src/optim/nadam.rs:13-182, radam.rs:13-239, adamax.rs:13-178, adabound.rs:19-78, lamb.rs:19-82,
mod.rs:408-755).
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

from .. import _native

ADAM, ADAMW, SGD, NADAM, RADAM, ADAMAX, RMSPROP, ADAGRAD, ADABOUND, LAMB1, LAMB2 = range(11)
_BAD_FLAGS = ("amsgrad", "capturable", "differentiable", "fused")
launches = 0          # native launches issued so far (tests read it to see which path ran)


def _eligible(opt) -> Optional[List[dict]]:
    """Per group: the parameters that have a gradient, or None when any of them rules the native path out."""
    plan = []
    any_param = False
    for g in opt.param_groups:
        if any(g.get(f) for f in _BAD_FLAGS):
            return None
        ps = [p for p in g["params"] if p.grad is not None]
        for p in ps:
            gr = p.grad
            if (not p.is_cuda or not gr.is_cuda or gr.is_sparse or not p.is_contiguous() or not gr.is_contiguous()
                    or p.dtype not in (torch.float32, torch.bfloat16) or gr.dtype not in (torch.float32, torch.bfloat16)):
                return None
        any_param = any_param or bool(ps)
        plan.append({"group": g, "params": ps})
    return plan if any_param else None


def _state_f32(st: dict, key: str, p: torch.Tensor, fill: float = 0.0) -> torch.Tensor:
    t = st.get(key)
    if t is None or t.dtype != torch.float32 or not t.is_contiguous():
        base = torch.full_like(p, fill, dtype=torch.float32, memory_format=torch.contiguous_format) if t is None else t.float().contiguous()
        st[key] = t = base
    return t


def _step_of(st: dict) -> float:
    s = st.get("step", 0)
    return float(s.item()) if torch.is_tensor(s) else float(s)


def _bump_step(st: dict, as_tensor: bool = True) -> int:
    t = int(_step_of(st)) + 1
    st["step"] = torch.tensor(float(t)) if as_tensor else t
    return t


def _launch(C, mode, ps, grads, s0, s1, s2, *, lr, b1=0.0, b2=0.0, eps=0.0, wd=0.0, c0=0.0, c1=0.0, c2=0.0, decoupled=False,
            maximize=False, norms=None, base=0):
    global launches
    # one dtype combination per call
    combos: Dict[tuple, List[int]] = {}
    for i, (p, g) in enumerate(zip(ps, grads)):
        combos.setdefault((p.dtype, g.dtype), []).append(i)
    for idx in combos.values():
        pick = lambda xs: [xs[i] for i in idx]  # noqa: E731
        if norms is not None and len(combos) > 1:
            raise RuntimeError("LAMB: mixed parameter dtypes in one group are not supported by the native step")
        C.multi_tensor_optim(mode, pick(ps), pick(grads), pick(s0), pick(s1), pick(s2), lr, b1, b2, eps, wd, c0, c1, c2, 1.0,
                             decoupled, maximize, norms, base)
        launches += -(-len(idx) // 32)


def try_step(opt, kind: int) -> bool:
    C = _native.load(required=False)
    if C is None or not torch.cuda.is_available():
        return False
    plan = _eligible(opt)
    if plan is None:
        return False
    for item in plan:
        g, ps = item["group"], item["params"]
        if not ps:
            continue
        grads = [p.grad for p in ps]
        sts = [opt.state[p] for p in ps]
        none = [None] * len(ps)
        lr, wd = float(g["lr"]), float(g.get("weight_decay", 0.0))
        mx = bool(g.get("maximize", False))
        # parameters of one group normally share the step count; bucket them in case they do not
        buckets: Dict[float, List[int]] = {}
        for i, st in enumerate(sts):
            key = _step_of(st) if kind != SGD else (0.0 if st.get("momentum_buffer") is None else 1.0)
            if kind == NADAM:
                mp = st.get("mu_product", 1.0)
                key = (key, float(mp.item()) if torch.is_tensor(mp) else float(mp))
            buckets.setdefault(key, []).append(i)
        for idx in buckets.values():
            P = [ps[i] for i in idx]
            G = [grads[i] for i in idx]
            ST = [sts[i] for i in idx]
            N = [None] * len(idx)
            if kind in (ADAM, ADAMW, RADAM, ADABOUND, LAMB1):
                b1, b2 = g["betas"]
                t = [_bump_step(st, as_tensor=kind in (ADAM, ADAMW, RADAM)) for st in ST][0]
                m = [_state_f32(st, "exp_avg", p) for st, p in zip(ST, P)]
                v = [_state_f32(st, "exp_avg_sq", p) for st, p in zip(ST, P)]
                bc1, bc2 = 1.0 - b1 ** t, 1.0 - b2 ** t
                if kind in (ADAM, ADAMW):
                    _launch(C, kind, P, G, m, v, N, lr=lr, b1=b1, b2=b2, eps=g["eps"], wd=wd, c0=bc1, c1=bc2, maximize=mx)
                elif kind == RADAM:
                    rho_inf = 2.0 / (1.0 - b2) - 1.0
                    rho_t = rho_inf - 2.0 * t * (b2 ** t) / bc2
                    rect = math.sqrt((rho_t - 4) * (rho_t - 2) * rho_inf / ((rho_inf - 4) * (rho_inf - 2) * rho_t)) if rho_t > 5.0 else 0.0
                    _launch(C, RADAM, P, G, m, v, N, lr=lr, b1=b1, b2=b2, eps=g["eps"], wd=wd, c0=bc1, c1=rect, c2=math.sqrt(bc2),
                            decoupled=bool(g.get("decoupled_weight_decay", False)), maximize=mx)
                elif kind == ADABOUND:
                    final_lr = g["final_lr"] * lr / g["base_lr"]
                    lower = final_lr * (1.0 - 1.0 / (g["gamma"] * t + 1.0))
                    upper = final_lr * (1.0 + 1.0 / (g["gamma"] * t))
                    _launch(C, ADABOUND, P, G, m, v, N, lr=lr, b1=b1, b2=b2, eps=g["eps"], wd=wd, c0=lr * math.sqrt(bc2) / bc1,
                            c1=lower, c2=upper)
                else:  # LAMB: moments + norms, then the trust-ratio update
                    if not g.get("bias_correction", True):
                        bc1 = bc2 = 1.0
                    norms = torch.zeros(2 * len(P), dtype=torch.float32, device=P[0].device)
                    kw = dict(lr=lr, b1=b1, b2=b2, eps=g["eps"], wd=wd, c0=bc1, c1=bc2, norms=norms)
                    _launch(C, LAMB1, P, G, m, v, N, **kw)
                    _launch(C, LAMB2, P, G, m, v, N, **kw)
            elif kind == NADAM:
                b1, b2 = g["betas"]
                t = [_bump_step(st) for st in ST][0]
                m = [_state_f32(st, "exp_avg", p) for st, p in zip(ST, P)]
                v = [_state_f32(st, "exp_avg_sq", p) for st, p in zip(ST, P)]
                md = g["momentum_decay"]
                mu = b1 * (1.0 - 0.5 * (0.96 ** (t * md)))
                mu_next = b1 * (1.0 - 0.5 * (0.96 ** ((t + 1) * md)))
                mp0 = ST[0].get("mu_product", 1.0)
                mu_prod = (float(mp0.item()) if torch.is_tensor(mp0) else float(mp0)) * mu
                for st in ST:
                    st["mu_product"] = torch.tensor(mu_prod)
                _launch(C, NADAM, P, G, m, v, N, lr=lr, b1=b1, b2=b2, eps=g["eps"], wd=wd, c0=lr * (1.0 - mu) / (1.0 - mu_prod),
                        c1=lr * mu_next / (1.0 - mu_prod * mu_next), c2=1.0 - b2 ** t,
                        decoupled=bool(g.get("decoupled_weight_decay", False)), maximize=mx)
            elif kind == ADAMAX:
                b1, b2 = g["betas"]
                t = [_bump_step(st) for st in ST][0]
                m = [_state_f32(st, "exp_avg", p) for st, p in zip(ST, P)]
                u = [_state_f32(st, "exp_inf", p) for st, p in zip(ST, P)]
                _launch(C, ADAMAX, P, G, m, u, N, lr=lr, b1=b1, b2=b2, eps=g["eps"], wd=wd, c0=1.0 - b1 ** t, maximize=mx)
            elif kind == RMSPROP:
                [_bump_step(st) for st in ST]
                sq = [_state_f32(st, "square_avg", p) for st, p in zip(ST, P)]
                mom = [_state_f32(st, "momentum_buffer", p) for st, p in zip(ST, P)] if g["momentum"] > 0 else N
                ga = [_state_f32(st, "grad_avg", p) for st, p in zip(ST, P)] if g["centered"] else N
                _launch(C, RMSPROP, P, G, mom, sq, ga, lr=lr, b1=g["momentum"], b2=g["alpha"], eps=g["eps"], wd=wd,
                        c0=1.0 if g["centered"] else 0.0, maximize=mx)
            elif kind == ADAGRAD:
                t = [_bump_step(st) for st in ST][0]
                acc = [_state_f32(st, "sum", p, g.get("initial_accumulator_value", 0.0)) for st, p in zip(ST, P)]
                _launch(C, ADAGRAD, P, G, N, acc, N, lr=lr, eps=g["eps"], wd=wd, c0=lr / (1.0 + (t - 1) * g["lr_decay"]), maximize=mx)
            elif kind == SGD:
                mom = g["momentum"]
                first = ST[0].get("momentum_buffer") is None
                bufs = [_state_f32(st, "momentum_buffer", p) for st, p in zip(ST, P)] if mom != 0 else N
                _launch(C, SGD, P, G, bufs, N, N, lr=lr, b1=mom, b2=g["dampening"], wd=wd, c0=1.0 if first else 0.0,
                        c1=1.0 if g["nesterov"] else 0.0, maximize=mx)
            else:
                raise ValueError(f"unknown optimizer kind {kind}")
    return True
