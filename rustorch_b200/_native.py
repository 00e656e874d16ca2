"""Loader for the in-tree native library ``_C`` (hand-written sm_100a kernels).

The shared object is built by :mod:`rustorch_b200._build` and lives next to this file so
that it travels with the source tree.  On a machine with a GPU a missing library is an error:
the CUDA path must never silently degrade to eager PyTorch.
"""
from __future__ import annotations

import importlib.util
import os
import sysconfig
from pathlib import Path

import torch

_HERE = Path(__file__).resolve().parent
_SO = _HERE / f"_C{sysconfig.get_config_var('EXT_SUFFIX') or '.so'}"
_mod = None
_err: Exception | None = None


def so_path() -> Path:
    return _SO


def load(required: bool | None = None):
    """Return the native module, or None when it is absent and not required.

    ``required`` defaults to ``torch.cuda.is_available()``: on a GPU box the extension must
    load; on a CPU-only box callers may run the pure-PyTorch reference paths instead.
    """
    global _mod, _err
    if _mod is not None:
        return _mod
    if required is None:
        required = torch.cuda.is_available()
    if _err is None:
        try:
            if not _SO.exists():
                if os.environ.get("RUSTORCH_B200_AUTOBUILD", "0") == "1":
                    from . import _build

                    _build.build()
                else:
                    raise FileNotFoundError(
                        f"{_SO} is missing: run `python -m rustorch_b200._build` "
                        "(or __graft_entry__.build()) first")
            spec = importlib.util.spec_from_file_location("rustorch_b200._C", str(_SO))
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            _mod = mod
            return _mod
        except Exception as e:  # noqa: BLE001
            _err = e
    if required:
        raise RuntimeError(f"rustorch_b200 native kernels could not be loaded: {_err}") from _err
    return None


def available() -> bool:
    return load(required=False) is not None


def launch_count() -> int:
    m = load(required=False)
    return int(m.launch_count()) if m is not None else 0


def check_status(device: int | None = None) -> None:
    """Synchronise and raise if any kernel reported a bounded-wait timeout (:class:`rustorch_b200.error.KernelTimeout`)
    or a bounds error.  Reading the status clears it, so the device stays usable afterwards."""
    m = load(required=False)
    if m is None or not torch.cuda.is_available():
        return
    dev = torch.cuda.current_device() if device is None else device
    code = int(m.read_status(dev))
    if code != 0:
        names = {101: "TMA producer wait timed out", 102: "MMA issuer wait timed out",
                 103: "epilogue wait timed out", 104: "peer wait timed out",
                 105: "softmax wait timed out", 201: "index or alignment check failed"}
        from .error import check_status_to_error
        raise check_status_to_error(code, f"rustorch_b200 kernel status {code}: {names.get(code, 'unknown')}")


_HOST_SO = _HERE / f"_host{sysconfig.get_config_var('EXT_SUFFIX') or '.so'}"
_host_mod = None


def host():
    """The host-only native runtime (arena allocator, CRC-64, execution planner): no CUDA, no torch, so it loads on
    every machine once built."""
    global _host_mod
    if _host_mod is None:
        if not _HOST_SO.exists():
            from . import _build
            _build.build_host()
        spec = importlib.util.spec_from_file_location("rustorch_b200._host", str(_HOST_SO))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _host_mod = mod
    return _host_mod
