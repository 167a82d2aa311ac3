"""The allocation-free RMSNorm backward, called through its exported C symbol the way a host program without a tensor
allocator would call it (raw device pointers, raw stream), must agree with the regular entry point.

The scratch of this variant lives inside the library, is shared by all calls and keeps stale contents, so the check is
made on two consecutive calls with different shapes and data. The file name sorts last on purpose: a run that stops
at the first failure has then already executed every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _library():
    from lm_engine.ops.build import load_extension, shared_object_path

    load_extension()  # the object (and the libtorch symbols it needs) is now mapped into this process
    lib = ctypes.CDLL(str(shared_object_path()))
    fn = lib.b200_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 7 + [ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int]
    return fn


def _call(fn, dy, h, w, rstd, dres, dh, dw, accumulate):
    message = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    code = fn(dy.data_ptr(), h.data_ptr(), w.data_ptr(), rstd.data_ptr(), 0 if dres is None else dres.data_ptr(),
              dh.data_ptr(), dw.data_ptr(), int(accumulate), h.shape[0], h.shape[1], stream, message, 256)
    return code, message.value.decode()


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


def test_no_alloc_rmsnorm_bwd_matches_regular_entry_point_twice():
    from lm_engine.ops.build import load_extension

    C = load_extension()
    fn = _library()
    torch.manual_seed(0)
    for T, H, use_dres in [(777, 4096, True), (33, 2560, False)]:
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        w = (1 + 0.1 * torch.randn(H, device="cuda")).to(torch.bfloat16)
        dy = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        dres = torch.randn(T, H, device="cuda", dtype=torch.bfloat16) if use_dres else None
        _, rstd = C.rmsnorm_fwd(x, None, w, 1e-5, False)

        dw_ref = torch.zeros(H, device="cuda")
        dh_ref = C.rmsnorm_bwd(dy, x, w, rstd, dres, dw_ref, False)

        dh = torch.empty_like(x)
        dw = torch.full((H,), 123.0, device="cuda")
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]  # the driver's view: catches allocations that bypass torch's allocator
        allocated_before = torch.cuda.memory_allocated()
        code, message = _call(fn, dy, x, w, rstd, dres, dh, dw, False)
        assert code == 0, message
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated() == allocated_before
        if (T, H) != (777, 4096):  # the very first call may still load the kernels' code onto the device
            assert torch.cuda.mem_get_info()[0] >= free_before - 2**20
        assert _rel(dh, dh_ref) < 1e-3
        assert _rel(dw, dw_ref) < 1e-4

        # accumulate on top of the previous result
        code, message = _call(fn, dy, x, w, rstd, dres, dh, dw, True)
        assert code == 0, message
        torch.cuda.synchronize()
        assert _rel(dw, 2 * dw_ref) < 1e-4


def test_no_alloc_rejects_oversized_rows():
    fn = _library()
    H = 16384
    x = torch.zeros(2, H, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(2, device="cuda")
    dw = torch.zeros(H, device="cuda")
    code, message = _call(fn, x, x, w, rstd, None, torch.empty_like(x), dw, False)
    assert code == 2 and "MAX_H" in message


def test_no_alloc_rejects_missing_and_misaligned_pointers():
    # checked on the host before any launch: nothing reaches the GPU
    fn = _library()
    T, H = 4, 256
    x = torch.zeros(T, H + 8, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(T, device="cuda")
    dw = torch.zeros(H, device="cuda")
    good = x[:, :H].contiguous()
    message = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    code = fn(good.data_ptr(), good.data_ptr(), w.data_ptr(), 0, 0, good.data_ptr(), dw.data_ptr(), 0, T, H, stream, message, 256)
    assert code == 6 and "NULL" in message.value.decode()
    code = fn(good.data_ptr() + 2, good.data_ptr(), w.data_ptr(), rstd.data_ptr(), 0, good.data_ptr(), dw.data_ptr(), 0, T, H, stream, message, 256)
    assert code == 7 and "aligned" in message.value.decode()
