"""The allocation-free sweep entry point, checked against the ordinary one through the C ABI.

``g2d_sweep_fused_static`` serves callers that have no way to allocate device memory (a plugin inside an application
that owns the whole device, or a running low-latency service that must not trigger cudaMalloc's device-wide
synchronisation): they pass inputs and outputs only and the scratch planes come from a fixed array inside the
library.  The entry point always takes the tile schedule, so the comparison call asks for that schedule too.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

STATIC_BYTES = 32 * 1024 * 1024  # G2D_STATIC_SCRATCH_BYTES of include/gptq2d_b200.h


def _problem(m, n, batch, dtype, seed):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    x = 4 * torch.randn(batch, m, n, generator=gen, device="cuda", dtype=dtype)
    l = torch.tril(torch.randn(m, m, generator=gen, device="cuda", dtype=dtype) * (0.3 / m ** .5), -1)
    u = torch.triu(torch.randn(n, n, generator=gen, device="cuda", dtype=dtype) * (0.3 / n ** .5), 1)
    scale = 0.5 + torch.rand(m, n, generator=gen, device="cuda", dtype=dtype)
    zero = torch.round(torch.randn(m, n, generator=gen, device="cuda", dtype=dtype))
    return x, l, u, scale, zero


def _descriptor(_abi, y, l, u, scale, zero):
    batch, m, n = y.shape
    desc = _abi.SweepDesc()
    desc.dtype, desc.quant_kind = _abi.dtype_code(y.dtype), _abi.Q_AFFINE
    desc.batch, desc.m, desc.n = batch, m, n
    desc.y, desc.l, desc.u = y.data_ptr(), l.data_ptr(), u.data_ptr()
    desc.scale, desc.zero = scale.data_ptr(), zero.data_ptr()
    desc.scale_row_stride, desc.scale_col_stride = scale.stride()
    desc.zero_row_stride, desc.zero_col_stride = zero.stride()
    desc.qmin, desc.qmax = -8.0, 7.0
    return desc


def test_static_scratch_sweep_matches_workspace_sweep():
    import _abi

    lib = _abi.library()
    stream = torch.cuda.current_stream().cuda_stream
    # the first call on a device does the one-time set-up (the driver may load the library's module, and with it
    # the fixed array, only now); do it before watching the memory counters
    x, l, u, scale, zero = _problem(8, 8, 1, torch.float32, 0)
    _abi.check(lib.g2d_sweep_fused_static(ctypes.byref(_descriptor(_abi, x, l, u, scale, zero)), stream), "g2d_sweep_fused_static")
    # two calls in a row on different problems: the second finds the first one's leftovers in the shared array
    # the last case is the most common caller shape (one float32 matrix, sides multiples of 4) at exactly the size limit
    for m, n, batch, dtype, seed in ((300, 500, 2, torch.float32, 1), (130, 97, 3, torch.float64, 2), (300, 500, 2, torch.float32, 3),
                                     (2048, 2048, 1, torch.float32, 4)):
        x, l, u, scale, zero = _problem(m, n, batch, dtype, seed)

        expected = x.clone()
        desc = _descriptor(_abi, expected, l, u, scale, zero)
        desc.reserved = 1  # the tile schedule, which the allocation-free entry point always takes
        size = ctypes.c_size_t()
        _abi.check(lib.g2d_sweep_workspace_bytes(ctypes.byref(desc), ctypes.byref(size)), "g2d_sweep_workspace_bytes")
        assert size.value <= STATIC_BYTES
        if (m, n, batch) == (2048, 2048, 1):
            assert size.value == STATIC_BYTES
        workspace = torch.empty(size.value, dtype=torch.uint8, device="cuda")
        desc.workspace, desc.workspace_bytes = workspace.data_ptr(), size.value
        _abi.check(lib.g2d_sweep_fused(ctypes.byref(desc), stream), "g2d_sweep_fused")

        actual = x.clone()
        desc = _descriptor(_abi, actual, l, u, scale, zero)  # no workspace: inputs and outputs only
        torch.cuda.synchronize()
        free_before, reserved_before = torch.cuda.mem_get_info()[0], torch.cuda.memory_reserved()
        _abi.check(lib.g2d_sweep_fused_static(ctypes.byref(desc), stream), "g2d_sweep_fused_static")
        torch.cuda.synchronize()
        # nothing was allocated: not through torch, and not behind its back either (the device-wide figure may move by
        # what other processes on the same GPU do, so it only has to stay within a small margin)
        assert torch.cuda.memory_reserved() == reserved_before
        assert torch.cuda.mem_get_info()[0] >= free_before - (8 << 20)
        assert torch.equal(actual, expected)  # same kernels, same schedule: identical bits
        assert not torch.equal(actual, x)


def test_static_scratch_refuses_oversized_problems():
    import _abi

    lib = _abi.library()
    m = n = 2049  # 2 planes x 2049^2 x 4 B > 32 MiB
    x, l, u, scale, zero = _problem(8, 8, 1, torch.float32, 0)
    desc = _descriptor(_abi, x, l, u, scale, zero)
    desc.m, desc.n = m, n  # rejected from the sizes alone, before any buffer is touched
    status = lib.g2d_sweep_fused_static(ctypes.byref(desc), torch.cuda.current_stream().cuda_stream)
    assert status == -5
    assert lib.g2d_status_string(status) == b"size exceeds a fixed maximum"
