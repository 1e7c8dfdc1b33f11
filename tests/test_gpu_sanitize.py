"""GPU parity of the output sanitiser (non-finite -> 0 at the `output` store) against the oracle: bit-exact."""
import numpy as np
import pytest
import torch

import dgen_b200
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
f32 = np.float32


@pytest.fixture(scope="module")
def ctx():
    c = dgen_b200.Context(0)
    yield c
    c.close()


def poisoned(n, seed):
    """Random bit patterns (every exponent, NaN payloads, +-Inf, denormals, -0.0 included) mixed with audio."""
    rng = np.random.default_rng(seed)
    x = rng.standard_normal(n).astype(f32)
    bits = rng.integers(0, 2 ** 32, size=n, dtype=np.uint64).astype(np.uint32)
    pick = rng.random(n) < 0.3
    x.view(np.uint32)[pick] = bits[pick]
    special = np.array([np.inf, -np.inf, np.nan, -0.0, 1e-45, -1e-40, 3.4028235e38], dtype=f32)
    k = min(n, special.size)
    x[:k] = special[:k]
    return x


@pytest.mark.parametrize("n", [0, 1, 3, 4, 5, 255, 1024, 4099, 1 << 20, (1 << 22) + 7])
@pytest.mark.parametrize("offset", [0, 1, 3])
def test_sanitize_bit_exact(ctx, n, offset):
    import torch
    x = poisoned(n + offset, 17 * n + offset)
    want = orc.sanitize(x[offset:].copy())
    buf = torch.from_numpy(x).cuda()
    out = torch.full((n + offset,), 7.0, device="cuda")
    ctx.sanitize(buf[offset:], out[offset:])
    ctx.sync()
    got = out.cpu().numpy()
    assert np.array_equal(got[offset:].view(np.uint32), want.view(np.uint32))
    assert np.all(got[:offset] == 7.0)  # nothing written before the slice
    # in place, and with input / output misaligned relative to each other (scalar path)
    ctx.sanitize(buf[offset:])
    ctx.sync()
    assert np.array_equal(buf.cpu().numpy()[offset:].view(np.uint32), want.view(np.uint32))
    if n > 8:
        src = torch.from_numpy(x).cuda()
        dst = torch.zeros(n + offset + 2, device="cuda")
        ctx.sanitize(src[offset:], dst[offset + 1:offset + 1 + n])
        ctx.sync()
        assert np.array_equal(dst.cpu().numpy()[offset + 1:offset + 1 + n].view(np.uint32), want.view(np.uint32))


def test_sanitize_is_idempotent_and_clears_render_poison(ctx):
    """Size-independent property at the full render size: sanitising twice equals sanitising once, and the
    result holds no non-finite value."""
    import torch
    x = poisoned(16 * 64000, 5)
    d = torch.from_numpy(x).cuda()
    once = ctx.sanitize(d.clone())
    twice = ctx.sanitize(once.clone())
    ctx.sync()
    assert torch.equal(once.view(torch.int32), twice.view(torch.int32))
    assert bool(torch.isfinite(once).all())
    keep = torch.isfinite(d)
    assert torch.equal(once[keep].view(torch.int32), d[keep].view(torch.int32))


@pytest.mark.parametrize("T,shape", [(1, (1,)), (1000, (1,)), (64000, (3, 5)), (513, (700,)), (70000, (2,))])
def test_reduce_frames_sums_per_frame_tensors_in_a_fixed_order(T, shape):
    """dgc_reduce_frames: the frame-by-frame accumulation of per-frame parameter gradients
    (Sources/DGen/Emit+State.swift:50-115) against a float64 sum; repeated calls give identical bits."""
    ctx = dgen_b200.Context(0)
    rng = np.random.default_rng(T)
    x = (rng.standard_normal((T,) + shape) * 10).astype(np.float32)
    X = torch.from_numpy(x).cuda()
    a = ctx.reduce_frames(X, scale=0.5)
    b = ctx.reduce_frames(X, scale=0.5)
    want = 0.5 * x.astype(np.float64).sum(axis=0)
    assert tuple(a.shape) == shape and torch.equal(a, b)
    assert np.abs(a.cpu().numpy() - want).max() <= 1e-6 * max(1.0, np.abs(want).max())
    acc = torch.ones(shape, device="cuda")
    ctx.reduce_frames(X, out=acc, accumulate=True)
    assert np.abs(acc.cpu().numpy() - (1.0 + 2.0 * want)).max() <= 1e-5 * max(1.0, np.abs(want).max())
    ctx.close()


def test_step_recording_of_plain_library_calls_and_its_error_reports():
    """dgc_graph_*: any sequence of entry points recorded on a non-default stream replays with refilled inputs; the
    misuse cases come back as errors, not as a broken context."""
    ctx = dgen_b200.Context(0)
    x = torch.randn(4000, 6, device="cuda")
    x[5, 2] = float("nan")
    clean, total = torch.empty_like(x), torch.empty(6, device="cuda")
    with pytest.raises(dgen_b200.DgenCudaError):           # the context is bound to the default stream here
        with ctx.record():
            pass
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with ctx.on_stream(s), torch.cuda.stream(s):
        ctx.sanitize(x, clean)                             # first use outside the recording (scratch allocation)
        ctx.reduce_frames(clean, out=total)
        with ctx.record() as rec:
            ctx.sanitize(x, clean)
            ctx.reduce_frames(clean, out=total)
            with pytest.raises(dgen_b200.DgenCudaError):   # no nested recording
                ctx.check(ctx.lib.dgc_graph_begin(ctx.h))
        g = rec.graph
        assert g.nodes >= 3
        for k in range(3):
            x.normal_()
            x[k, 0] = float("inf")
            g.launch()
            s.synchronize()
            ref = torch.where(torch.isfinite(x), x, torch.zeros_like(x))
            assert torch.equal(clean, ref)
            assert torch.allclose(total, ref.double().sum(0).float(), rtol=1e-5, atol=1e-4)
        with pytest.raises(dgen_b200.DgenCudaError):       # end without begin
            out = dgen_b200._vp()
            ctx.check(ctx.lib.dgc_graph_end(ctx.h, dgen_b200.C.byref(out)))
        g.close()
    assert ctx.sanitize(x.clone()) is not None             # the context still works
    ctx.close()
