"""GPU parity of buffer -> FFT -> magnitude and of the partitioned convolution against the oracle."""
import os

import numpy as np
import pytest

import dgen_b200
from dgen_b200 import workloads as wl
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
f32 = np.float32
GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_artefacts.npz"))


@pytest.fixture(scope="module")
def ctx():
    c = dgen_b200.Context(0)
    yield c
    c.close()


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("N,hop,T,V", [(16, 8, 100, 1), (64, 16, 1000, 3), (1024, 256, 5000, 2), (2048, 1024, 9000, 1),
                                       (256, 256, 1000, 1), (128, 32, 129, 2)])
def test_stft_mag_matches_oracle(ctx, N, hop, T, V):
    rng = np.random.default_rng(N + T)
    x = rng.standard_normal((V, T)).astype(f32)
    win = orc.hann_periodic(N)
    for w in (None, win):
        want = np.stack([orc.buffer_fft_mag(x[v], N, hop, w) for v in range(V)])
        got = ctx.stft_mag(dev(x), N, hop, None if w is None else dev(w)).cpu().numpy()
        assert got.shape == want.shape
        assert np.abs(got - want).max() < 2e-5 * np.abs(want).max()


def test_partconv_reproduces_the_reference_generated_artefact(ctx):
    """The reference's own emitted code for partitioned convolution (spectral-effect fixture, N=16 hop=8
    gain=0.5, 32-tap IR) run on the reference harness input: tests/golden/ref_artefacts.npz."""
    ir = np.zeros(32, f32)
    ir[0], ir[8], ir[16], ir[24] = 1.0, 0.35, 0.15, 0.05
    got = ctx.partconv(dev(GOLD["input"].reshape(1, -1)), dev(ir), 16, 8, gain=0.5).cpu().numpy()[0]
    assert np.abs(got - GOLD["spectral_effect"]).max() < 2e-5  # the reference's fixture tolerance


@pytest.mark.parametrize("N,hop,T,V,irlen", [(64, 32, 3000, 2, 200), (2048, 1024, 20000, 2, 9000),
                                             (256, 64, 2000, 1, 256), (128, 64, 1000, 3, 1)])
def test_partconv_matches_oracle(ctx, N, hop, T, V, irlen):
    rng = np.random.default_rng(N + T)
    x = rng.standard_normal((V, T)).astype(f32)
    ir = (rng.standard_normal(irlen) * np.exp(-np.arange(irlen) / max(1.0, irlen / 4))).astype(f32)
    want = np.stack([orc.partitioned_convolve(x[v], ir, N, hop) for v in range(V)])
    got = ctx.partconv(dev(x), dev(ir), N, hop).cpu().numpy()
    assert np.abs(got - want).max() < 1e-4 * max(1.0, np.abs(want).max())


def test_partconv_configuration_slice(ctx):
    """Hop-gated partitioned FFT convolution configuration (N=2048, hop=1024, 2 s IR at 48 kHz, RT60 1.2 s),
    two voices of 1.5 s so that the oracle finishes in seconds."""
    d = wl.partconv_inputs(20260003, V=2, T=72000)
    want = np.stack([orc.partitioned_convolve(d["x"][v], d["ir"], d["N"], d["hop"]) for v in range(2)])
    got = ctx.partconv(dev(d["x"]), dev(d["ir"]), d["N"], d["hop"]).cpu().numpy()
    assert np.abs(got - want).max() < 1e-4 * max(1.0, np.abs(want).max())


def test_stft_rejects_bad_sizes(ctx):
    import torch
    x = torch.zeros(1, 100, device="cuda")
    with pytest.raises(dgen_b200.DgenCudaError):
        ctx.stft_mag(x, 100, 10)
    with pytest.raises(dgen_b200.DgenCudaError):
        ctx.stft_mag(x, 4096, 10)
