"""Lets the wrapper classes ``Tensor`` (tensor.py) and ``Variable`` (autograd.py) go wherever a ``torch.Tensor``
goes.  The reference's Python layers take and return its own ``Variable`` / ``Tensor`` objects
(python/src/lib.rs:377-452, src/python/nn.rs), so code written for that wheel calls ``model(rustorch.tensor(...))``;
here the layers are ``torch.nn.Module``s, and two mechanisms make that call work:

* both wrappers implement ``__torch_function__``: any ``torch`` / ``torch.nn.functional`` call that receives one is
  re-issued on the wrapped tensors and its tensor results come back wrapped;
* ``accept_wrappers(namespace)`` decorates the ``forward`` of this package's own layers, whose native paths reach
  the CUDA kernels through ``autograd.Function.apply`` (which the protocol above does not cover).

A result is a ``Variable`` if any argument was one, else a ``Tensor``.  Plain ``torch.Tensor`` calls pay one
``isinstance`` test per positional argument.
"""
from __future__ import annotations

import functools

import torch



# The reference has two surfaces for the same accessors: methods in Rust (``t.shape()``, ``v.requires_grad()``,
# ``opt.learning_rate()``) and properties in its Python wheel (``t.shape``, ``v.requires_grad``, ``opt.learning_rate``;
# python/src/lib.rs:77-92, 248-270, 502-505).  The accessors return values that are also callable and return themselves,
# so both spellings work.
class ShapeValue(tuple):
    """A shape: a tuple that also compares equal to the same list (the wheel returns lists) and can be called."""

    def __call__(self):
        return tuple(self)

    def __eq__(self, other):
        return tuple(self) == tuple(other) if isinstance(other, (list, tuple)) else NotImplemented

    def __ne__(self, other):
        r = self.__eq__(other)
        return r if r is NotImplemented else not r

    __hash__ = tuple.__hash__


class IntValue(int):
    def __call__(self):
        return int(self)


class FloatValue(float):
    def __call__(self):
        return float(self)


class StrValue(str):
    def __call__(self):
        return str(self)


class ListValue(list):
    def __call__(self):
        return list(self)


class DictValue(dict):
    def __call__(self):
        return dict(self)


class FlagValue(int):
    """A boolean (``bool`` cannot be subclassed)."""

    def __call__(self):
        return bool(self)

    def __repr__(self):
        return repr(bool(self))

    __str__ = __repr__


_classes = None


def _wrappers():
    global _classes
    if _classes is None:
        from .autograd import Variable
        from .tensor import Tensor
        _classes = (Tensor, Variable)
    return _classes


def _strip(x, seen):
    """``x`` with wrappers replaced by their tensors; ``seen[0]`` / ``seen[1]`` record a Tensor / a Variable."""
    T, V = _wrappers()
    if isinstance(x, V):
        seen[1] = True
        return x.tensor
    if isinstance(x, T):
        seen[0] = True
        return x.data
    if isinstance(x, (list, tuple)):
        items = [_strip(v, seen) for v in x]
        return type(x)(items) if type(x) in (list, tuple) else type(x)(*items)
    if isinstance(x, dict):
        return {k: _strip(v, seen) for k, v in x.items()}
    return x


def _dress(x, cls):
    if isinstance(x, torch.Tensor):
        return cls(x)
    if type(x) in (list, tuple):
        return type(x)(_dress(v, cls) for v in x)
    return x


def call_unwrapped(func, args, kwargs):
    seen = [False, False]
    a, k = _strip(tuple(args), seen), _strip(dict(kwargs or {}), seen)
    out = func(*a, **k)
    if not (seen[0] or seen[1]):
        return out
    T, V = _wrappers()
    return _dress(out, V if seen[1] else T)


def torch_function(cls, func, types, args=(), kwargs=None):
    """Shared body of the wrappers' ``__torch_function__``."""
    return call_unwrapped(func, args, kwargs)


def _decorate(forward):
    @functools.wraps(forward)
    def wrapped(self, *args, **kwargs):
        T, V = _wrappers()
        for a in args:
            if isinstance(a, (T, V)) or type(a) in (list, tuple):
                break
        else:
            if not kwargs:
                return forward(self, *args)
        return call_unwrapped(functools.partial(forward, self), args, kwargs)
    wrapped._accepts_wrappers = True
    return wrapped


def accept_wrappers(namespace: dict) -> None:
    """Decorates ``forward`` of every ``torch.nn.Module`` subclass defined in ``namespace`` (a module's globals)."""
    mod = namespace.get("__name__")
    for obj in list(namespace.values()):
        if isinstance(obj, type) and issubclass(obj, torch.nn.Module) and obj.__module__ == mod:
            f = obj.__dict__.get("forward")
            if f is not None and not getattr(f, "_accepts_wrappers", False):
                obj.forward = _decorate(f)
