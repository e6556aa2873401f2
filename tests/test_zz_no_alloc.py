"""The allocation-free adaLN + quantize entry point (llnv_adaln_quantize_nvfp4_static).

It exists for hosts that cannot allocate device memory at the call site (all memory owned by
their own arena, or no tolerance for cudaMalloc's device-wide synchronisation): its scratch is a
fixed array inside the library instead of a caller-provided one.  The test drives it through the
C ABI with ctypes and requires bit-identical codes, scales, amax and modulated activations to
the regular entry point - twice in a row with different shapes, so that stale contents of the
shared array from the first call cannot leak into the second - and checks that a request beyond
the array's capacity is refused with a message naming the limit.  This file is collected last,
and passes both on its own in a fresh process and after the rest of the suite.
"""
import ctypes as C

import pytest
import torch

from longlive_b200 import _lib

pytestmark = pytest.mark.gpu


def _call(fn, x, scale, shift, frame_rows, rule, row_stats=None):
    m, c = x.shape
    mp = (m + 127) // 128 * 128
    codes = torch.full((mp, c // 2), 0xAB, dtype=torch.uint8, device="cuda")
    sf = torch.full((mp * c // 16,), 0x7E, dtype=torch.uint8, device="cuda")
    amax = torch.full((1,), -1.0, dtype=torch.float32, device="cuda")
    y = torch.full((m, c), 7.0, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    args = [x.data_ptr(), m, c, x.stride(0), scale.data_ptr(), shift.data_ptr(), scale.stride(0), frame_rows,
            C.c_float(1e-6), 1, rule, codes.data_ptr(), sf.data_ptr(), amax.data_ptr(), y.data_ptr(), c]
    if row_stats is not None:
        args.append(row_stats.data_ptr())
    args.append(stream)
    rc = fn(*args)
    assert rc == 0, _lib.lib().llnv_last_error()
    torch.cuda.synchronize()
    return codes, sf, amax, y


def test_static_scratch_matches_regular_entry_point_twice():
    lib = _lib.lib()
    g = torch.Generator().manual_seed(77)
    for m, c, frames, rule in ((792, 3072, 3, 3), (130, 512, 2, 0)):       # second call is smaller: stale rows stay behind
        frame_rows = m // frames
        x = (torch.randn(m, c, generator=g) * 2 + 0.5).bfloat16().cuda()
        mod = (torch.randn(frames, 6, c, generator=g) * 0.2).bfloat16().cuda()
        scale, shift = mod[:, 1], mod[:, 0]
        ws = torch.empty(2 * m, dtype=torch.float32, device="cuda")
        ref = _call(lib.llnv_adaln_quantize_nvfp4, x, scale, shift, frame_rows, rule, row_stats=ws)
        free_before = torch.cuda.mem_get_info()[0]
        got = _call(lib.llnv_adaln_quantize_nvfp4_static, x, scale, shift, frame_rows, rule)
        for a, b in zip(ref, got):
            assert torch.equal(a, b)
        assert float(got[2].item()) > 0
        # the outputs above are this test's own allocations; the entry point itself must not have
        # taken device memory from the driver (allow the allocator's granularity for the outputs)
        assert free_before - torch.cuda.mem_get_info()[0] <= 64 << 20


def test_static_scratch_rejects_oversized_requests():
    lib = _lib.lib()
    limit = lib.llnv_static_max_rows()
    assert limit == 16384
    m, c = limit + 1, 64
    x = torch.zeros(m, c, dtype=torch.bfloat16, device="cuda")
    mod = torch.zeros(1, c, dtype=torch.bfloat16, device="cuda")
    codes = torch.empty((m + 127) // 128 * 128, c // 2, dtype=torch.uint8, device="cuda")
    sf = torch.empty(codes.shape[0] * c // 16, dtype=torch.uint8, device="cuda")
    amax = torch.zeros(1, dtype=torch.float32, device="cuda")
    rc = lib.llnv_adaln_quantize_nvfp4_static(x.data_ptr(), m, c, c, mod.data_ptr(), mod.data_ptr(), c, m, C.c_float(1e-6), 1, 3,
                                              codes.data_ptr(), sf.data_ptr(), amax.data_ptr(), None, 0, None)
    assert rc == -1
    msg = lib.llnv_last_error().decode()
    assert "16384" in msg and "exceeds" in msg
