"""GPU gradients of the synthesis (harmonic bank, noise FIR, partitioned convolution, heads) against the fp64
autograd evaluation of the same graph (oracle/torch_oracle.py); tolerance 1e-3 relative."""
import numpy as np
import pytest
import torch

import dgen_b200
from dgen_b200 import workloads as wl
from oracle import torch_oracle as to

pytestmark = pytest.mark.gpu
f32 = np.float32


@pytest.fixture(scope="module")
def ctx():
    c = dgen_b200.Context(0)
    yield c
    c.close()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def rel_err(got, want):
    return np.abs(got - want).max() / max(np.abs(want).max(), 1e-30)


@pytest.mark.parametrize("shape", [dict(B=2, T=4096, K=100, F=64), dict(B=3, T=3000, K=7, F=33),
                                   dict(B=1, T=2000, K=130, F=9), dict(B=2, T=1500, K=20, F=1500)])
def test_harmonic_render_backward(ctx, shape):
    d = wl.harmonic_noise_inputs(21, sr=16000.0, **shape)
    rng = np.random.default_rng(1)
    g = rng.standard_normal((d["B"], d["T"])).astype(f32)
    rows = to.rows_of(d["F"], d["T"])
    amps = to.t64(d["amps"]).requires_grad_(True)
    out = to.harmonic_render(to.t64(d["f0"]), to.t64(d["uv"]), amps, to.t64(d["gain"]), d["T"], d["sr"], rows)
    (out * to.t64(g)).sum().backward()
    got = ctx.harmonic_render_bwd(dev(d["f0"]), dev(d["uv"]), dev(d["amps"]), dev(d["gain"]), dev(g), d["T"], d["sr"])
    assert rel_err(got.cpu().numpy(), amps.grad.numpy()) < 1e-3
    # the same gradient walking the phases of the per-voice scan of the fundamental
    got = ctx.harmonic_render_bwd(dev(d["f0"]), dev(d["uv"]), dev(d["amps"]), dev(d["gain"]), dev(g), d["T"], d["sr"],
                                  phase_mode=dgen_b200.PHASE_FUNDAMENTAL)
    assert rel_err(got.cpu().numpy(), amps.grad.numpy()) < 1e-3
    # and the form a training step uses: the forward is handed the scratch, leaves its per-frame sums there, and the
    # backward that is told so reads them instead of reducing over its lanes -- the same gradient
    import ctypes as C
    B, T, K, F = d["B"], d["T"], d["K"], d["F"]
    hp = dgen_b200.HarmonicParams(B, T, K, F, d["sr"], 1.0, dgen_b200.PHASE_FUNDAMENTAL, 0)
    scratch = torch.empty(int(ctx.lib.dgc_harmonic_bwd_scratch_floats(C.byref(hp))), device="cuda")
    D = {k: dev(d[k]) for k in ("f0", "uv", "amps", "gain")}
    audio = ctx.harmonic_render(D["f0"], D["uv"], D["amps"], D["gain"], T, d["sr"],
                                phase_mode=dgen_b200.PHASE_FUNDAMENTAL, scratch=scratch)
    plain = ctx.harmonic_render(D["f0"], D["uv"], D["amps"], D["gain"], T, d["sr"], phase_mode=dgen_b200.PHASE_FUNDAMENTAL)
    assert torch.equal(audio, plain)                      # keeping the sums does not change the audio
    gp = torch.empty(F, B, K, device="cuda")
    gd = dev(g)
    ctx.check(ctx.lib.dgc_harmonic_render_bwd_prepared(ctx.h, C.byref(hp), D["f0"].data_ptr(), D["uv"].data_ptr(),
                                                       D["amps"].data_ptr(), D["gain"].data_ptr(), gd.data_ptr(),
                                                       scratch.data_ptr(), gp.data_ptr()))
    ctx.sync()
    assert rel_err(gp.cpu().numpy(), amps.grad.numpy()) < 1e-3
    assert rel_err(gp.cpu().numpy(), got.cpu().numpy()) < 2e-5


@pytest.mark.parametrize("B,T,F,NT", [(2, 3000, 50, 257), (1, 1000, 5, 17), (2, 2049, 300, 64)])
def test_fir_noise_backward(ctx, B, T, F, NT):
    rng = np.random.default_rng(T)
    taps = rng.standard_normal((F, B, NT)).astype(f32)
    noise = rng.standard_normal((B, T)).astype(f32)
    ng = rng.uniform(0.2, 1, (F, B)).astype(f32)
    g = rng.standard_normal((B, T)).astype(f32)
    rows = to.rows_of(F, T)
    tt = to.t64(taps).requires_grad_(True)
    (to.fir_noise(to.t64(noise), tt, to.t64(ng), rows) * to.t64(g)).sum().backward()
    got = ctx.fir_noise_bwd(dev(noise), dev(ng), dev(g), F, NT)
    assert rel_err(got.cpu().numpy(), tt.grad.numpy()) < 1e-3


@pytest.mark.parametrize("N,hop,T,V,irlen", [(64, 32, 3000, 2, 200), (2048, 1024, 20000, 2, 9000), (128, 64, 1000, 3, 1),
                                             (256, 64, 2100, 1, 300)])
def test_partconv_backward(ctx, N, hop, T, V, irlen):
    rng = np.random.default_rng(N + T)
    x = rng.standard_normal((V, T)).astype(f32)
    ir = (rng.standard_normal(irlen) * np.exp(-np.arange(irlen) / max(1.0, irlen / 4))).astype(f32)
    g = rng.standard_normal((V, T)).astype(f32)
    xt, it = to.t64(x).requires_grad_(True), to.t64(ir).requires_grad_(True)
    (to.partconv(xt, it, N, hop, gain=0.8) * to.t64(g)).sum().backward()
    gx, gir = ctx.partconv_bwd(dev(x), dev(ir), N, hop, dev(g), gain=0.8)
    assert rel_err(gx.cpu().numpy(), xt.grad.numpy()) < 1e-3
    assert rel_err(gir.cpu().numpy(), it.grad.numpy()) < 1e-3


def test_heads_forward_and_backward(ctx):
    rng = np.random.default_rng(4)
    M, K, NB = 777, 100, 65
    z = (2 * rng.standard_normal((M, K + NB))).astype(f32)
    ga, gb = rng.standard_normal((M, K)).astype(f32), rng.standard_normal((M, NB)).astype(f32)
    zt = to.t64(z).requires_grad_(True)
    a64, b64 = to.heads(zt, K)
    ((a64 * to.t64(ga)).sum() + (b64 * to.t64(gb)).sum()).backward()
    amps, bands = ctx.heads_fwd(dev(z), K)
    assert rel_err(amps.cpu().numpy(), a64.detach().numpy()) < 1e-5
    assert rel_err(bands.cpu().numpy(), b64.detach().numpy()) < 1e-5
    gz = ctx.heads_bwd(dev(z), dev(ga), dev(gb))
    assert rel_err(gz.cpu().numpy(), zt.grad.numpy()) < 1e-3


def test_backward_kernels_are_deterministic(ctx):
    d = wl.harmonic_noise_inputs(5, B=2, T=4096, K=100, F=64)
    g = dev(np.random.default_rng(0).standard_normal((2, 4096)).astype(f32))
    args = (dev(d["f0"]), dev(d["uv"]), dev(d["amps"]), dev(d["gain"]), g, d["T"], d["sr"])
    a = ctx.harmonic_render_bwd(*args).cpu().numpy()
    b = ctx.harmonic_render_bwd(*args).cpu().numpy()
    assert np.array_equal(a, b)


def temporal_grad_scan_reference(g, reset, scale):
    """The reference's reverse loop, literally (Sources/DGen/Emit+TemporalGradient.swift:60-88), in float64."""
    E, T = g.shape
    out = np.zeros((E, T), np.float64)
    for e in range(E):
        carry = 0.0
        for n in range(T - 1, -1, -1):
            active = 0.0 if (reset is not None and reset[n] > 0) else carry
            out[e, n] = active
            carry = float(g[e, n]) + active
    return out * scale


@pytest.mark.parametrize("E,T,density", [(1, 1, 1.0), (3, 7, 0.3), (2, 1025, 0.01), (4, 3000, 0.2), (2, 40000, 0.0005),
                                         (1, 5000, 1.0), (2, 2048, 0.0)])
def test_temporal_grad_scan_with_resets_follows_the_reference_loop(ctx, E, T, density):
    """A reset at frame r cuts the sum for earlier frames after g[r] and zeroes out[r]; runs of resets, resets on the
    first and last frame, a reset on every frame, none at all."""
    rng = np.random.default_rng(T)
    g = rng.standard_normal((E, T)).astype(f32)
    reset = (rng.uniform(size=T) < density).astype(f32)
    if T > 4:
        reset[0] = 1.0
        reset[T - 1] = 1.0 if density > 0 else 0.0
        reset[T // 2] = -1.0            # not a reset: the test is > 0
    want = temporal_grad_scan_reference(g, reset, 1.0 / 44100.0)
    got = ctx.temporal_grad_scan(dev(g), 1.0 / 44100.0, reset=dev(reset)).cpu().numpy()
    assert np.abs(got - want).max() <= 1e-6 * max(np.abs(want).max(), 1e-12)
    assert np.all(got[:, reset > 0] == 0.0)


def test_temporal_grad_scan_is_the_exclusive_reverse_sum(ctx):
    """temporalGradScan without resets (Sources/DGen/Emit+TemporalGradient.swift:60-88): out[n] = sum_{m>n} g[m]."""
    rng = np.random.default_rng(3)
    for E, T in [(1, 1), (3, 7), (2, 1025), (5, 64000)]:
        g = rng.standard_normal((E, T)).astype(f32)
        want = (np.cumsum(g[:, ::-1].astype(np.float64), axis=1)[:, ::-1] - g) / 48000.0
        got = ctx.temporal_grad_scan(dev(g), 1.0 / 48000.0).cpu().numpy()
        assert np.abs(got - want).max() <= 1e-6 * max(np.abs(want).max(), 1e-30), (E, T)


@pytest.mark.parametrize("B,T,K,F", [(2, 4096, 12, 32), (3, 5000, 40, 17), (1, 64000, 100, 1000)])
def test_harmonic_f0_gradient_against_fp64_autograd(ctx, B, T, K, F):
    """d loss / d f0 through the phases (phasor temporal gradient + sin + sum + sampleRow backward) against the
    fp64 autograd evaluation of the same graph: 1e-3 relative to the largest entry."""
    d = wl.harmonic_noise_inputs(50 + K, B=B, T=T, K=K, F=F)
    rng = np.random.default_rng(K)
    g = rng.standard_normal((B, T)).astype(f32)
    f0 = to.t64(d["f0"]).requires_grad_(True)
    audio = to.harmonic_render(f0, to.t64(d["uv"]), to.t64(d["amps"]), to.t64(d["gain"]), T, d["sr"], to.rows_of(F, T))
    (audio * to.t64(g)).sum().backward()
    want = f0.grad.numpy()
    got = ctx.harmonic_f0_bwd(dev(d["f0"]), dev(d["uv"]), dev(d["amps"]), dev(d["gain"]), dev(g), T, d["sr"]).cpu().numpy()
    err = np.abs(got - want).max() / np.abs(want).max()
    print("f0 grad rel err %.2e" % err)
    assert err < 1e-3
