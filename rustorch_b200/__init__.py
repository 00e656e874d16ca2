"""rustorch_b200: a Blackwell-native (sm_100a) deep-learning framework with the API surface of
RusTorch.  PyTorch is the tensor/autograd substrate; hot paths are hand-written CUDA kernels
(tcgen05 / TMEM / TMA) loaded from the in-tree ``_C`` extension.
"""
from . import _native  # noqa: F401

__version__ = "0.1.0"


def native_available() -> bool:
    """True when the compiled sm_100a kernel library is importable."""
    return _native.available()
