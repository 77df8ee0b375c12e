"""nvfp4_quantize_static: the quantiser for hosts that cannot allocate.

Some callers reach this library from a place where they may not call an allocator (a plug-in inside another
framework's callback, a replayed step with a frozen memory plan, a process whose device memory was handed out up
front).  The variant under test keeps the amax scratch inside the library image.  It must give exactly the bytes of
nvfp4_quantize, also on a second call that finds the scratch as the first call left it."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call_static(native, x, signs, sr, rht, seed, packed, scales, pts):
    mp, kp = native.round128(x.shape[0]), native.round128(x.shape[1])
    with torch.cuda.device(x.device):
        native.check(native.lib().nvfp4_quantize_static(
            x.data_ptr(), native.dtype_code(x), x.shape[0], x.shape[1], x.stride(0), x.stride(1), mp, kp, sr, int(rht), seed,
            signs.data_ptr(), None, packed.data_ptr(), scales.data_ptr(), pts.data_ptr(), native.stream_of(x)))


def test_static_scratch_variant_matches_the_allocating_entry_point(native):
    g = torch.Generator().manual_seed(42)
    signs = (torch.randint(0, 2, (16,), generator=g).float() * 2 - 1).cuda()
    cases = [((193, 129), torch.bfloat16, 0, False, False), ((1024, 2048), torch.bfloat16, native.Q_SR_HASH, True, False),
             ((300, 520), torch.float32, native.Q_SR_PHILOX, True, False),
             ((520, 300), torch.bfloat16, native.Q_SR_HASH, True, True), ((129, 193), torch.float32, 0, False, True)]
    # outputs are allocated by the test up front: the entry point itself never allocates
    # the last flag asks for a transposed view (row stride 1) of a contiguous tensor of the swapped shape
    for shape, dtype, sr, rht, transposed in cases:
        mp, kp = native.round128(shape[0]), native.round128(shape[1])
        packed = torch.empty((mp, kp // 2), dtype=torch.uint8, device="cuda")
        scales = torch.empty((mp // 128 * 32, kp // 64 * 16), dtype=torch.uint8, device="cuda")
        pts = torch.empty((), dtype=torch.float32, device="cuda")
        for call in range(2):   # two calls in a row: the second one inherits the first one's scratch contents
            x = (torch.randn(shape[::-1] if transposed else shape, generator=g) * (1.0 + 3.0 * call)).to(dtype).cuda()
            if transposed:
                x = x.t()
                assert x.stride(0) == 1 and tuple(x.shape) == shape
            want = native.quantize(x, signs, mp, kp, sr, rht, 77 + call)
            packed.fill_(0xCD); scales.fill_(0xCD); pts.fill_(-1.0)
            _call_static(native, x, signs, sr, rht, 77 + call, packed, scales, pts)
            torch.cuda.synchronize()
            assert pts.item() == want[2].item()
            assert torch.equal(packed, want[0]) and torch.equal(scales, want[1])


def test_static_variant_rejects_sizes_beyond_its_limit(native):
    handle = native.lib()
    limit = handle.nvfp4_quantize_static_max_elements()
    assert limit == 1 << 31
    x = torch.zeros((16, 16), dtype=torch.bfloat16, device="cuda")
    signs = torch.ones(16, device="cuda")
    buf = torch.empty(16, dtype=torch.uint8, device="cuda")
    rc = handle.nvfp4_quantize_static(x.data_ptr(), native.BF16, 1 << 20, 1 << 12, 1 << 12, 1, 1 << 20, 1 << 12, 0, 0, 0,
                                      signs.data_ptr(), None, buf.data_ptr(), buf.data_ptr(), buf.data_ptr(), None)
    assert rc == 1 and b"exceed the limit" in handle.nvfp4_last_error()
