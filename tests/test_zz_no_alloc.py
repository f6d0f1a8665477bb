"""The allocation-free C entry point `mk_lp_norms_noalloc` against the regular (tensor-allocating) Lp-norm op.

Some hosts that embed the library own every byte of device memory themselves (a serving process with its own
pools, a C/Fortran forecast driver) and cannot let a library call cudaMalloc; they use this entry point, which
keeps its scratch in a fixed device array inside the library.  The test calls it the way such a host would:
through the exported C symbol, with raw device pointers, twice in a row (the scratch array is shared and keeps
the previous call's contents), and checks both results against the regular op.  It runs last so that a
failure here cannot hide other failures in a run that stops at the first one."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from makani_b200.ops import _ext
    _ext.require()                      # loads libtorch / the extension into the process first
    lib = ctypes.CDLL(_ext.SO_PATH)
    lib.mk_lp_norms_noalloc.restype = ctypes.c_int
    lib.mk_lp_norms_noalloc.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p,
                                        ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.mk_noalloc_last_error.restype = ctypes.c_char_p
    return lib


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_no_alloc_entry_matches_regular_op_twice(dtype):
    assert torch.cuda.is_available()
    from makani_b200.ops.loss import weighted_lp_norms
    dev = torch.device("cuda", 0)
    lib = _lib()
    torch.manual_seed(0)
    B, C, H, W = 2, 5, 181, 360
    q = (torch.rand(H, device=dev) / (H * W)).contiguous()
    stream = torch.cuda.current_stream(dev)
    for call in range(2):
        for P in (2, 1):
            pred = torch.randn(B, C, H, W, device=dev).to(dtype).contiguous()
            tgt = torch.randn(B, C, H, W, device=dev).to(dtype).contiguous()
            out = torch.empty(B * C, 2, dtype=torch.float32, device=dev)
            rc = lib.mk_lp_norms_noalloc(pred.data_ptr(), tgt.data_ptr(), int(dtype == torch.float32), q.data_ptr(),
                                         out.data_ptr(), B * C, H, W, P, ctypes.c_void_p(stream.cuda_stream))
            assert rc == 0, lib.mk_noalloc_last_error().decode()
            ref = weighted_lp_norms(pred, tgt, q, P).reshape(B * C, 2)
            torch.cuda.synchronize()
            assert torch.allclose(out, ref, rtol=1e-4, atol=1e-7), (call, P, (out - ref).abs().max().item())


def test_no_alloc_entry_rejects_oversized_problems():
    dev = torch.device("cuda", 0)
    lib = _lib()
    x = torch.zeros(8, device=dev)
    # 5000 planes of 4096x4096 would need far more scratch than the built-in array: refused before any launch
    rc = lib.mk_lp_norms_noalloc(x.data_ptr(), x.data_ptr(), 1, x.data_ptr(), x.data_ptr(), 5000, 4096, 4096, 2, None)
    assert rc == -2
    assert b"scratch" in lib.mk_noalloc_last_error()
    rc = lib.mk_lp_norms_noalloc(x.data_ptr(), x.data_ptr(), 1, x.data_ptr(), x.data_ptr(), 1, 4, 4, 3, None)
    assert rc == -1
