"""``import rustorch``: the reference's package name, resolving to :mod:`rustorch_b200` (same objects)."""
import sys

import rustorch_b200 as _impl

sys.modules[__name__] = _impl
