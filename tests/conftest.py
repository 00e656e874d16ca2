import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); skipped elsewhere")
    config.addinivalue_line("markers", "multigpu: needs at least 2 CUDA devices")


def pytest_collection_modifyitems(config, items):
    have_gpu = torch.cuda.is_available()
    n_gpu = torch.cuda.device_count() if have_gpu else 0
    for item in items:
        if "gpu" in item.keywords and not have_gpu:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))
        if "multigpu" in item.keywords and n_gpu < 2:
            item.add_marker(pytest.mark.skip(reason="needs >= 2 CUDA devices"))


@pytest.fixture(autouse=True)
def _kernel_status_guard(request):
    """After every GPU test, fail if a kernel recorded a bounded-wait timeout / bounds error."""
    yield
    if "gpu" in request.keywords and torch.cuda.is_available():
        from rustorch_b200 import _native

        _native.check_status()


def rel_err(out: torch.Tensor, ref: torch.Tensor) -> float:
    out, ref = out.float(), ref.float()
    return float((out - ref).abs().max() / ref.abs().max().clamp_min(1e-6))


def assert_close(out: torch.Tensor, ref: torch.Tensor, rtol: float = 2e-2, atol_frac: float = 4e-3, what: str = "") -> None:
    """Per-element check ``|out - ref| <= atol + rtol * |ref|`` with ``atol = atol_frac * max|ref|``.

    Unlike a max-error-over-max-value ratio this fails on a wrong tile of small-magnitude outputs or a wrong ragged
    tail: the absolute allowance is a few bf16 ulps of the largest value, everything above it must agree relatively.
    """
    out, ref = out.float(), ref.float()
    assert out.shape == ref.shape, f"{what}: shape {tuple(out.shape)} vs {tuple(ref.shape)}"
    atol = atol_frac * float(ref.abs().max().clamp_min(1e-12))
    bad = (out - ref).abs() > (atol + rtol * ref.abs())
    n_bad = int(bad.sum())
    if n_bad:
        idx = bad.nonzero()[0].tolist()
        raise AssertionError(
            f"{what}: {n_bad} of {out.numel()} elements differ; first at {idx}: got {float(out[tuple(idx)])}, "
            f"want {float(ref[tuple(idx)])} (atol {atol:.3e}, rtol {rtol})")
