"""Signal.noise() on the device (dgc_noise_fill).
NOISE_STREAM: the reference's xorshift32 stream, bit for bit against the oracle's serial generator, at lengths that
cross run and block boundaries, for seeds including 0 (reseeded to 1) -- the jump-ahead matrices are exact or the
streams differ in every bit.  NOISE_GAUSSIAN: a restatement in numpy from the same serial generator (hash of
(seed, voice) -> state, values 2n and 2n+1 through Box-Muller), to single-precision rounding of log/cos, plus the
moments of a long fill."""
import numpy as np
import pytest
import torch

import dgen_b200
from oracle import oracle as orc

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ctx():
    c = dgen_b200.Context(0)
    yield c
    c.close()


@pytest.mark.parametrize("seed,T,B", [(1, 1, 1), (0, 63, 2), (12345, 64, 1), (0xDEADBEEF, 65, 3), (7, 4097, 2),
                                      (2463534242, 64000, 2), (99, 262144 + 17, 1)])
def test_stream_noise_is_the_reference_stream_bit_for_bit(ctx, seed, T, B):
    want, _ = orc.noise_xorshift(seed if seed else 1, T)
    got = ctx.noise_fill(seed, B, T)
    ctx.sync()
    got = got.cpu().numpy()
    for b in range(B):
        assert np.array_equal(got[b].view(np.uint32), want.view(np.uint32)), (seed, T, b)
    assert got.min() > 0.0 and got.max() <= 1.0


def _voice_state(seed, b):
    m = 0xFFFFFFFF
    z = (seed + 0x9E3779B9 * (b + 1)) & m
    z = ((z ^ (z >> 16)) * 0x85EBCA6B) & m
    z = ((z ^ (z >> 13)) * 0xC2B2AE35) & m
    z ^= z >> 16
    return z or 1


def test_gaussian_noise_follows_its_definition_and_has_unit_moments(ctx):
    seed, B, T, sigma = 2024, 3, 5000, 0.3
    got = ctx.noise_fill(seed, B, T, mode=dgen_b200.NOISE_GAUSSIAN, sigma=sigma)
    ctx.sync()
    got = got.cpu().numpy().astype(np.float64)
    for b in range(B):
        u, _ = orc.noise_xorshift(_voice_state(seed, b), 2 * T)
        u = u.astype(np.float64)
        want = sigma * np.sqrt(-2.0 * np.log(u[0::2])) * np.cos(2.0 * np.pi * u[1::2])
        # fast log and cosine on the device: absolute error of a few 1e-6 at sigma = 0.3
        assert np.abs(got[b] - want).max() < 2e-5, b
    big = ctx.noise_fill(5, 16, 64000, mode=dgen_b200.NOISE_GAUSSIAN, sigma=1.0)
    ctx.sync()
    assert abs(float(big.mean())) < 5e-3
    assert abs(float(big.std()) - 1.0) < 5e-3
    rows = big.cpu().numpy()
    c = np.corrcoef(rows)                               # voices are independent streams
    assert np.abs(c - np.eye(16)).max() < 0.03
    assert abs(float((rows[:, 1:] * rows[:, :-1]).mean())) < 5e-3      # white: no lag-1 correlation


def test_noise_fill_rejects_bad_arguments(ctx):
    out = torch.empty(4, device="cuda")
    assert ctx.lib.dgc_noise_fill(ctx.h, 1, 2, 1, 4, 1.0, out.data_ptr()) == -1
    assert ctx.lib.dgc_noise_fill(ctx.h, 1, 0, 0, 4, 1.0, out.data_ptr()) == -1
    assert ctx.lib.dgc_noise_fill(ctx.h, 1, 0, 1, 4, 1.0, None) == -1


def test_host_step_with_device_noise_and_resident_target_matches_the_uploading_step(ctx):
    """dgc_hn_forward_loss_host with noise_seed set and target_dev given uploads neither the noise nor the target and
    returns the loss of the same step fed the same arrays from the host."""
    rng = np.random.default_rng(3)
    B, T, F, K, NT = 4, 8192, 128, 8, 65
    step = dgen_b200.HnStep()
    step.harm = dgen_b200.HarmonicParams(B, T, K, F, 16000.0, 1.0, dgen_b200.PHASE_SCAN, 0)
    step.fir = dgen_b200.FirParams(B, T, F, NT, 1.0, 1)
    step.mss = dgen_b200.mss_params(B, T, (1024, 256, 64))
    step.nbands = 0
    f0 = rng.uniform(100, 400, (F, B)).astype(np.float32)
    uv = np.ones((F, B), np.float32)
    amps = rng.uniform(0, 1, (F, B, K)).astype(np.float32)
    gain = rng.uniform(0.1, 0.5, (F, B)).astype(np.float32)
    ngain = rng.uniform(0.1, 0.5, (F, B)).astype(np.float32)
    taps = (rng.standard_normal((F, B, NT)) / NT).astype(np.float32)
    target = rng.standard_normal((B, T)).astype(np.float32)
    seed, sigma = 77, 0.25
    noise = ctx.noise_fill(seed, B, T, mode=dgen_b200.NOISE_GAUSSIAN, sigma=sigma)
    ctx.sync()
    noise_h = noise.cpu().numpy()
    want = ctx.hn_forward_loss_host(step, f0, uv, amps, gain, ngain, taps, None, noise_h, target)
    tgt_dev = torch.from_numpy(target).cuda()
    step.noise_seed, step.noise_mode, step.noise_sigma = seed, dgen_b200.NOISE_GAUSSIAN, sigma
    step.target_dev = tgt_dev.data_ptr()
    got = ctx.hn_forward_loss_host(step, f0, uv, amps, gain, ngain, taps, None, None, None)
    assert got == want
