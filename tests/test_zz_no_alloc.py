"""The allocation-free RMSNorm backward, called through its exported C symbol.

Some users of the library may not allocate device memory at all (a serving loop with a
frozen memory budget, a plugin inside a process that owns the GPU heap).  For them the
library exports ``agb_rms_norm_bwd_noalloc``, which keeps its scratch in a fixed array
inside the library.  This test calls that symbol with ctypes on caller-provided buffers,
twice in a row (the scratch keeps the first call's contents), and compares against the
regular entry point.  It lives in the last-collected file so that a failure here cannot
hide failures elsewhere in a run that stops at the first error.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    from agentgarten_b200.ops import native

    ext = native.require()
    lib = ctypes.CDLL(ext.__file__)
    fn = lib.agb_rms_norm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_int64, ctypes.c_int, ctypes.c_void_p]
    lib.agb_noalloc_last_error.restype = ctypes.c_char_p
    return ext, lib, fn


def test_no_alloc_rms_norm_bwd_matches_regular_entry_point():
    ext, lib, fn = _library()
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    stream = torch.cuda.current_stream().cuda_stream
    for call, (rows, width, seed) in enumerate([(1000, 4096, 0), (333, 512, 1)]):
        g = torch.Generator(device=device).manual_seed(seed)
        x = torch.randn(rows, width, device=device, dtype=torch.bfloat16, generator=g)
        grad = torch.randn(rows, width, device=device, dtype=torch.bfloat16, generator=g)
        w = (1 + 0.1 * torch.randn(width, device=device, generator=g)).to(torch.bfloat16)
        _, rstd = ext.rms_norm_fwd(x, w, 1e-6)
        dx_ref, dw_ref = ext.rms_norm_bwd(grad, x, w, rstd)
        dx = torch.empty_like(x)
        dw = torch.empty(width, device=device, dtype=torch.float32)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        # The driver's own count of free device memory sees what torch's allocator cannot
        # (a cudaMalloc inside the library); compared from the second call on, after the
        # first has loaded the module's code and its static scratch.
        free_before = torch.cuda.mem_get_info(device)[0]
        code = fn(grad.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(),
                  dw.data_ptr(), rows, width, stream)
        torch.cuda.synchronize()
        assert code == 0, lib.agb_noalloc_last_error().decode()
        assert torch.cuda.memory_allocated() == before
        if call > 0:
            assert torch.cuda.mem_get_info(device)[0] >= free_before
        assert torch.equal(dx, dx_ref), call
        assert torch.allclose(dw, dw_ref, rtol=1e-5, atol=1e-5), call


def test_no_alloc_rejects_oversized_request():
    _, lib, fn = _library()
    dummy = torch.zeros(8, device="cuda", dtype=torch.float32)
    p = dummy.data_ptr()
    code = fn(p, p, p, p, p, p, 1 << 22, 8192, None)
    assert code < 0
    assert b"scratch" in lib.agb_noalloc_last_error()
    assert fn(p, p, p, p, p, p, 16, 12, None) < 0
    assert b"width" in lib.agb_noalloc_last_error()
    assert fn(p, p, p, p, p, p, -1, 64, None) < 0
    assert b"rows" in lib.agb_noalloc_last_error()
