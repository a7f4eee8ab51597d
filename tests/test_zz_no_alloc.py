# SPDX-License-Identifier: Apache-2.0
"""The allocation-free RMSNorm backward (`atb_rmsnorm_bwd_noalloc`, an exported C symbol) must agree with the
tensor-based operator.

Some hosts of this library may not allocate on the device while they run (all memory belongs to one pool, or an
allocation's implicit synchronisation is unaffordable, or there is no tensor framework to allocate through), so
this variant keeps its scratch in a fixed array inside the library.  The test calls it the way such a host would:
through ctypes, with raw device pointers and a raw stream handle, twice in a row on different data (the scratch
array is shared between calls and keeps old contents, which must not leak into the second result), and checks
the size limit.  This file sorts last on purpose so that a run stopping at the first failure has already run
every other test.
"""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_HIDDEN = 8192


@pytest.fixture(scope="module")
def lib():
    from arctictraining_b200.ops import _ext

    _ext.require()
    handle = ctypes.CDLL(str(_ext.lib_path()))
    fn = handle.atb_rmsnorm_bwd_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_longlong, ctypes.c_int, ctypes.c_void_p, ctypes.c_char_p, ctypes.c_ulong]
    # One call before any measurement: the CUDA runtime loads a kernel's code when it is first launched, which takes
    # device memory once per process and has nothing to do with the entry point's own behaviour.
    x = torch.randn(8, 1024, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(1024, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(8, device="cuda")
    dx, dw = torch.empty_like(x), torch.empty(1024, device="cuda")
    err = ctypes.create_string_buffer(256)
    rc = fn(x.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), 8, 1024,
            ctypes.c_void_p(torch.cuda.current_stream().cuda_stream), err, 256)
    assert rc == 0, err.value.decode()
    torch.cuda.synchronize()
    return fn


def call(fn, dy, x, w, rstd, dx, dw):
    err = ctypes.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    rc = fn(dy.data_ptr(), x.data_ptr(), w.data_ptr(), rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), x.shape[0], x.shape[1],
            ctypes.c_void_p(stream), err, 256)
    return rc, err.value.decode()


def rel(a, b):
    return float((a.float() - b.float()).norm() / (b.float().norm() + 1e-12))


@pytest.mark.parametrize("shapes", [[(513, 4096), (77, 1024)], [(4000, 8192), (4000, 8192)]])
def test_matches_tensor_operator_on_two_calls_in_a_row(lib, shapes):
    torch.manual_seed(0)
    k = torch.ops.atb200
    for T, H in shapes:  # consecutive calls share the built-in scratch array
        x = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        w = (1 + 0.1 * torch.randn(H, device="cuda")).bfloat16()
        dy = torch.randn(T, H, device="cuda", dtype=torch.bfloat16)
        _, rstd = k.rmsnorm_fwd(x, w, 1e-5)
        dx_ref, dw_ref = k.rmsnorm_bwd(dy, x, w, rstd)
        dx = torch.empty_like(x)
        dw = torch.full((H,), float("nan"), device="cuda")
        # unmeasured first call for this width: every kernel variant is loaded by the runtime at its first launch
        rc, msg = call(lib, dy, x, w, rstd, torch.empty_like(x), torch.empty(H, device="cuda"))
        assert rc == 0, msg
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        free_before, _ = torch.cuda.mem_get_info()  # sees allocations made behind the framework's back as well
        rc, msg = call(lib, dy, x, w, rstd, dx, dw)
        assert rc == 0, msg
        torch.cuda.synchronize()
        free_after, _ = torch.cuda.mem_get_info()
        # "<=": the framework may hand a block that an earlier operator released on its own schedule back to its pool
        # meanwhile; what matters is that nothing new was taken, from the pool or (next line) from the device
        assert torch.cuda.memory_allocated() <= before
        assert free_before - free_after < (1 << 20), "device memory was allocated during the call"
        # the same operation in plain fp32 PyTorch (after the memory checks: autograd's worker thread releases its
        # temporaries on its own schedule, which would move the framework's allocation counter)
        xf = x.float().requires_grad_(True)
        wf = w.float().requires_grad_(True)
        (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5) * wf).backward(dy.float())
        assert rel(dx, dx_ref) < 1e-2 and rel(dw, dw_ref) < 1e-2      # the tensor-based entry point
        assert rel(dx, xf.grad) < 2e-2 and rel(dw, wf.grad) < 2e-2      # the fp32 reference


def test_sizes_beyond_the_limit_are_refused_with_a_message(lib):
    H = MAX_HIDDEN + 8
    x = torch.zeros(4, H, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(4, device="cuda")
    dx, dw = torch.empty_like(x), torch.empty(H, device="cuda")
    rc, msg = call(lib, x, x, w, rstd, dx, dw)
    assert rc == 1 and "limit" in msg and str(MAX_HIDDEN) in msg
    rc, msg = call(lib, x[:, :12], x[:, :12], w, rstd, dx, dw)  # hidden = 12 is not a multiple of 8
    assert rc == 1 and "multiple of 8" in msg


def test_operands_outside_the_current_device_are_refused(lib):
    H = 1024
    x = torch.zeros(4, H, device="cuda", dtype=torch.bfloat16)
    w = torch.ones(H, device="cuda", dtype=torch.bfloat16)
    rstd = torch.ones(4, device="cuda")
    dx, dw = torch.empty_like(x), torch.empty(H, device="cuda")
    host = torch.zeros(4, H, dtype=torch.bfloat16).pin_memory()  # reachable from the GPU, but not device memory
    rc, msg = call(lib, host, x, w, rstd, dx, dw)
    assert rc == 1 and "device memory of the current device" in msg
