"""The allocation-free C entry point ``rt_norm_bwd_noalloc`` against the normal norm backward.

Some users of the library cannot allocate device memory when they need this kernel (in
allocator callbacks, in serving loops that forbid allocation after warm-up, in C hosts without
torch's caching allocator), so the
library exports one C symbol whose scratch lives in a fixed device array.  The test calls the
symbol through ctypes with raw pointers, twice in a row (the second call sees the first
call's leftovers in the shared array), and compares with the tensor path.  The file name makes
pytest collect it last.
"""
import ctypes

import pytest
import torch

from conftest import rel_err

pytestmark = pytest.mark.gpu

MAX_C = 8192
ERR_SIZE = -1


def _lib():
    from rustorch_b200 import _native
    _native.load(required=True)
    lib = ctypes.CDLL(str(_native.so_path()))
    fn = lib.rt_norm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 9 + [ctypes.c_longlong, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.rt_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None else ctypes.c_void_p(0)


def _bf(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randn(shape, device="cuda", generator=g).to(torch.bfloat16)


@pytest.mark.parametrize("rms", [False, True])
def test_noalloc_matches_tensor_path_twice(rms):
    from rustorch_b200.ops import kernels as K
    lib = _lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (rows, C) in enumerate([(3000, 768), (517, 4096)]):
        x, w, b = _bf((rows, C), 10 + call), _bf((C,), 20 + call), _bf((C,), 30 + call)
        dy, dres = _bf((rows, C), 40 + call), _bf((rows, C), 50 + call)
        if rms:
            _, rstd = K.rms_norm_fwd(x, w, 1e-5)
            mean = None
            dg_ref = torch.zeros(C, device="cuda")
            dx_ref = K.rms_norm_bwd(dy, x, w, rstd, dg_ref, dres=dres)
            db_ref = None
        else:
            _, mean, rstd = K.layer_norm_fwd(x, w, b, 1e-5)
            dg_ref, db_ref = torch.zeros(C, device="cuda"), torch.zeros(C, device="cuda")
            dx_ref = K.layer_norm_bwd(dy, x, w, mean, rstd, dg_ref, db_ref, dres=dres)
        dx = torch.empty_like(x)
        dg = torch.zeros(C, device="cuda")
        db = torch.zeros(C, device="cuda")
        rc = lib.rt_norm_bwd_noalloc(_ptr(dy), _ptr(x), _ptr(w), _ptr(mean), _ptr(rstd), _ptr(dres),
                                     _ptr(dx), _ptr(dg), _ptr(db), rows, C, int(rms), stream)
        assert rc == 0, lib.rt_noalloc_last_error()
        torch.cuda.synchronize()
        assert rel_err(dx, dx_ref) < 1e-3
        assert rel_err(dg, dg_ref) < 1e-3
        if not rms:
            assert rel_err(db, db_ref) < 1e-3
        # independent oracle: the same backward in fp32 torch math on the same bf16 inputs
        xf = x.float().requires_grad_(True)
        wf = w.float().requires_grad_(True)
        bf = b.float().requires_grad_(True)
        if rms:
            yf = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf
        else:
            yf = torch.nn.functional.layer_norm(xf, (C,), wf, bf, 1e-5)
        yf.backward(dy.float())
        assert rel_err(dx, xf.grad + dres.float()) < 2e-2
        assert rel_err(dg, wf.grad) < 2e-2
        if not rms:
            assert rel_err(db, bf.grad) < 2e-2


def test_noalloc_rejects_oversize():
    lib = _lib()
    C = MAX_C + 8
    t = torch.zeros(8, C, dtype=torch.bfloat16, device="cuda")
    f = torch.zeros(C, device="cuda")
    rc = lib.rt_norm_bwd_noalloc(_ptr(t), _ptr(t), _ptr(t), _ptr(f), _ptr(f), None, _ptr(t), _ptr(f),
                                 _ptr(f), 8, C, 0, None)
    assert rc == ERR_SIZE
    assert b"not supported" in lib.rt_noalloc_last_error()
