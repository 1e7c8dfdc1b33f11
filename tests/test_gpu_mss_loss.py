"""GPU parity of the multi-scale spectral loss against the CPU oracle (through the C ABI)."""
import numpy as np
import pytest

import dgen_b200
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
f32 = np.float32


@pytest.fixture(scope="module")
def ctx():
    c = dgen_b200.Context(0)
    yield c
    c.close()


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("N", [16, 32, 64, 128, 256, 512, 1024, 2048])
def test_single_scale_partials_match_oracle(ctx, N):
    rng = np.random.default_rng(N)
    B, T, hop = 3, 5000 if N <= 256 else 9000, N // 4
    x = rng.standard_normal((B, T)).astype(f32)
    y = (0.5 * rng.standard_normal((B, T))).astype(f32)
    _, part = ctx.mss_loss_fwd(dev(x), dev(y), sizes=(N,), want_partial=True)
    part = part.cpu().numpy()
    H = (T + hop - 1) // hop
    lin_o = orc.spectral_loss(x, y, N, hop, want_partial=True)[1]
    log_o = orc.spectral_loss(x, y, N, hop, use_log=True, want_partial=True)[1]
    lin_g, log_g = part[:H * B].reshape(H, B), part[H * B:].reshape(H, B)
    # relative loss error tolerance of the path: 1e-4
    assert np.abs(lin_g - lin_o).max() < 1e-4 * np.abs(lin_o).max()
    assert np.abs(log_g - log_o)[1:].max() < 1e-4 * np.abs(log_o).max()


def test_multi_scale_total_matches_oracle_fp32_and_fp64(ctx):
    rng = np.random.default_rng(7)
    B, T = 4, 16000
    x = rng.standard_normal((B, T)).astype(f32)
    y = rng.standard_normal((B, T)).astype(f32)
    got = float(ctx.mss_loss_fwd(dev(x), dev(y)).cpu()[0])
    want = orc.mss_loss(x, y)
    want64 = orc.mss_loss(x, y, double=True)
    assert abs(got - want) < 1e-4 * abs(want)
    assert abs(got - want64) < 1e-4 * abs(want64)


def test_identical_signals_give_zero_and_short_render_skips_long_windows(ctx):
    rng = np.random.default_rng(1)
    x = rng.standard_normal((2, 1000)).astype(f32)
    # prediction and target share one complex FFT, so identical inputs cancel to rounding, not to 0.0
    # (the reference's own test accepts 0.01: Tests/DGenLazyTests/BatchedSpectralLossTests.swift:174-191)
    assert abs(float(ctx.mss_loss_fwd(dev(x), dev(x)).cpu()[0])) < 1e-5
    y = rng.standard_normal((2, 1000)).astype(f32)
    got = float(ctx.mss_loss_fwd(dev(x), dev(y)).cpu()[0])   # 2048 and 1024 are longer than T: skipped
    want = orc.mss_loss(x, y)
    assert abs(got - want) < 1e-4 * abs(want)


def test_loss_is_bit_deterministic(ctx):
    rng = np.random.default_rng(2)
    x, y = dev(rng.standard_normal((3, 8000)).astype(f32)), dev(rng.standard_normal((3, 8000)).astype(f32))
    a = ctx.mss_loss_fwd(x, y).cpu().numpy()
    b = ctx.mss_loss_fwd(x, y).cpu().numpy()
    assert a.tobytes() == b.tobytes()
