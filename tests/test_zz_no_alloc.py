"""The allocation-free one-pole entry point (dgc_onepole_fwd_static) against the context-based one.

Some hosts call the filter from a real-time audio thread, where cudaMalloc (and therefore creating or
growing a context) is off limits.  That entry point keeps its scratch in a fixed device array inside the
library; here it is driven through the C ABI twice in a row -- the second call reuses the array while it
still holds the first call's carries -- and compared with dgc_onepole_fwd, plus the size limit.
This file sorts last on purpose: a run that stops at the first failure has then run every other test.
"""
import ctypes as C

import numpy as np
import pytest

import dgen_b200

pytestmark = pytest.mark.gpu
f32 = np.float32


def test_static_scratch_onepole_matches_context_version_twice():
    import torch
    lib = dgen_b200.load()
    ctx = dgen_b200.Context(0)
    stream = torch.cuda.current_stream().cuda_stream
    err = C.create_string_buffer(256)
    rng = np.random.default_rng(42)
    for B, T, a in ((4, 100000, 0.9), (2, 5000, -0.6)):   # second call: fewer chunks, stale tail in the array
        x = torch.from_numpy(rng.standard_normal((B, T)).astype(f32)).cuda()
        want = ctx.onepole_fwd(x, a)
        got = torch.full((B, T), float("nan"), device="cuda")
        rc = lib.dgc_onepole_fwd_static(stream, x.data_ptr(), B, T, a, got.data_ptr(), err, 256)
        assert rc == 0, err.value.decode()
        torch.cuda.synchronize()
        w, g = want.cpu().numpy(), got.cpu().numpy()
        assert np.isfinite(g).all()
        assert np.abs(g - w).max() <= 1e-5 * max(1.0, np.abs(w).max())   # the tolerance of the one-pole parity tests
    ctx.close()


def test_static_scratch_onepole_rejects_oversize_and_null():
    import torch
    lib = dgen_b200.load()
    err = C.create_string_buffer(256)
    x = torch.zeros(8, device="cuda")
    # 40000 voices x 1 chunk > 32768 chunk slots (and > 65535 is also refused): nothing is launched
    rc = lib.dgc_onepole_fwd_static(None, x.data_ptr(), 40000, 8, 0.5, x.data_ptr(), err, 256)
    assert rc == -1 and b"exceeds" in err.value
    rc = lib.dgc_onepole_fwd_static(None, None, 1, 8, 0.5, x.data_ptr(), err, 256)
    assert rc == -1 and b"null" in err.value
    rc = lib.dgc_onepole_fwd_static(None, x.data_ptr(), 1, 0, 0.5, x.data_ptr(), None, 0)
    assert rc == -1


def test_static_scratch_onepole_at_exactly_the_slot_limit_and_in_place():
    """B * ceil(T / 2048) == 32768 chunk slots exactly: the last slot of both halves of the array is used.
    One slot more is refused.  The call runs in place (x_dev == y_dev), which the entry point allows."""
    import torch
    lib = dgen_b200.load()
    ctx = dgen_b200.Context(0)
    err = C.create_string_buffer(256)
    stream = torch.cuda.current_stream().cuda_stream
    B, T = 512, 64 * 2048 - 5                      # 64 chunks per voice (the last one ragged) x 512 voices
    assert B * ((T + 2047) // 2048) == 32768
    x = torch.randn(B, T, device="cuda")
    want = ctx.onepole_fwd(x, 0.95)
    buf = x.clone()
    rc = lib.dgc_onepole_fwd_static(stream, buf.data_ptr(), B, T, C.c_float(0.95), buf.data_ptr(), err, 256)
    assert rc == 0, err.value.decode()
    torch.cuda.synchronize()
    scale = max(1.0, float(want.abs().max()))
    assert float((buf - want).abs().max()) <= 1e-5 * scale
    rc = lib.dgc_onepole_fwd_static(stream, x.data_ptr(), B, T + 2048, C.c_float(0.95), buf.data_ptr(), err, 256)
    assert rc == -1 and b"exceeds" in err.value    # 65 chunks per voice: 33280 slots
    ctx.close()
