"""Host-language callbacks and result values of the binding layer (python/tests/test_advanced.py:9-150 and
python/tests/test_direct.py:16-30 exercise them: a registry of named Python callables that framework code calls back
into, a ``Result`` value with ``ok`` / ``err`` / ``unwrap`` / ``unwrap_or``, and ``try_catch``).

The reference crosses a language boundary here; in this package both sides are Python, so the registry is a dictionary
with the same method names and the "call from the framework" entry points simply look the callable up.  The training
loop reports through the same registry: ``Trainer(config, callbacks=registry)`` calls its ``"progress"``, ``"log"`` and
``"completed"`` entries (``training.RegistryCallback``).
"""
from __future__ import annotations

from typing import Any, Callable, Dict, List, Optional

from .error import RusTorchError

__all__ = ["CallbackRegistry", "Result", "init_callback_system", "call_python_from_rust", "progress_callback_example",
           "try_catch", "get_version", "hello_from_rust", "add_numbers", "sum_list"]


class CallbackRegistry:
    def __init__(self):
        self._callbacks: Dict[str, Callable[..., Any]] = {}

    def register_callback(self, name: str, function: Callable[..., Any]) -> None:
        if not callable(function):
            raise RusTorchError(f"callback '{name}' is not callable", 2001)
        self._callbacks[str(name)] = function

    def unregister_callback(self, name: str) -> bool:
        return self._callbacks.pop(name, None) is not None

    def has_callback(self, name: str) -> bool:
        return name in self._callbacks

    def list_callbacks(self) -> List[str]:
        return sorted(self._callbacks)

    def call(self, name: str, *args: Any) -> Any:
        try:
            fn = self._callbacks[name]
        except KeyError:
            raise RusTorchError(f"no callback named '{name}' (registered: {self.list_callbacks()})", 2002) from None
        return fn(*args)

    def call_if_registered(self, name: str, *args: Any) -> Optional[Any]:
        return self._callbacks[name](*args) if name in self._callbacks else None

    def __len__(self) -> int:
        return len(self._callbacks)

    def __contains__(self, name: str) -> bool:
        return name in self._callbacks


def init_callback_system() -> CallbackRegistry:
    return CallbackRegistry()


def call_python_from_rust(registry: CallbackRegistry, name: str, *args: Any) -> Any:
    """The framework-to-host call: looks ``name`` up in ``registry`` and calls it with ``args``."""
    return registry.call(name, *args)


def progress_callback_example(registry: CallbackRegistry, steps: int) -> List[Any]:
    """Calls ``"progress"(step, total, percent)`` once per step and ``"completed"(total)`` at the end, returning what
    the callbacks returned (entries that are not registered are skipped)."""
    out = []
    for step in range(1, int(steps) + 1):
        r = registry.call_if_registered("progress", step, int(steps), 100.0 * step / steps)
        if r is not None:
            out.append(r)
    r = registry.call_if_registered("completed", int(steps))
    if r is not None:
        out.append(r)
    return out


class Result:
    """``Result.ok(v)`` / ``Result.err(e)``; ``is_ok`` and ``is_err`` are attributes."""

    __slots__ = ("_value", "_error", "is_ok")

    def __init__(self, value: Any = None, error: Any = None, is_ok: bool = True):
        self._value, self._error, self.is_ok = value, error, bool(is_ok)

    @classmethod
    def ok(cls, value: Any) -> "Result":
        return cls(value, None, True)

    @classmethod
    def err(cls, error: Any) -> "Result":
        return cls(None, error, False)

    @property
    def is_err(self) -> bool:
        return not self.is_ok

    def unwrap(self) -> Any:
        if self.is_ok:
            return self._value
        if isinstance(self._error, BaseException):
            raise self._error
        raise RusTorchError(f"called unwrap on an error result: {self._error}", 1002)

    def unwrap_or(self, default: Any) -> Any:
        return self._value if self.is_ok else default

    def unwrap_err(self) -> Any:
        if self.is_ok:
            raise RusTorchError(f"called unwrap_err on an ok result: {self._value!r}", 1003)
        return self._error

    def map(self, fn: Callable[[Any], Any]) -> "Result":
        return Result.ok(fn(self._value)) if self.is_ok else self

    def __bool__(self) -> bool:
        return self.is_ok

    def __repr__(self) -> str:
        return f"Ok({self._value!r})" if self.is_ok else f"Err({self._error!r})"


def try_catch(operation: Callable[[], Any], error_handler: Optional[Callable[[BaseException], Any]] = None) -> Any:
    """Runs ``operation()``; on an exception returns ``error_handler(exception)``, or re-raises without a handler."""
    try:
        return operation()
    except Exception as e:  # noqa: BLE001  (the handler decides)
        if error_handler is None:
            raise
        return error_handler(e)


def get_version() -> str:
    from . import __version__
    return __version__


def hello_from_rust() -> str:
    return "Hello from RusTorch (B200-native build)!"


def add_numbers(a: float, b: float) -> float:
    return float(a) + float(b)


def sum_list(values) -> float:
    return float(sum(float(v) for v in values))
