"""GPU parity of the oscillator bank, noise FIR and clocks against the CPU oracle (through the C ABI)."""
import numpy as np
import pytest

import dgen_b200
from dgen_b200 import workloads as wl
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


def test_clock_accum_bit_exact(ctx):
    for incr, mn, mx, T in ((0.1, 0.0, 1.0, 4096), (1.0, 0.0, 79.0, 1000), (0.37, -2.0, 3.0, 5000)):
        got = ctx.clock_accum(incr, mn, mx, T).cpu().numpy()
        assert np.array_equal(got, orc.accum(incr, mn, mx, T))


def test_playhead_bit_exact(ctx):
    for F, T in ((1000, 64000), (250, 16000), (1, 512), (7, 1001)):
        assert np.array_equal(ctx.playhead(F, T).cpu().numpy(), orc.playhead(F, T))


def test_osc_bank_const_deterministic_matches_oracle(ctx):
    # the oscillator-bank -> filter -> FFT configuration: 64 partials, 110*k Hz, 1/k, sr 44100, 65536 frames
    c = wl.osc_filter_fft_inputs()
    want = orc.osc_bank_const(c["freq"], c["amp"], c["T"], c["sr"], stateful=False)
    got = ctx.osc_bank_const(dev(c["freq"]), dev(c["amp"]), c["T"], c["sr"], dgen_b200.PHASE_DETERMINISTIC)
    assert np.abs(got.cpu().numpy() - want).max() < 1e-4  # forward audio tolerance of the path: 1e-4


def test_osc_bank_const_sequential_matches_oracle(ctx):
    c = wl.osc_filter_fft_inputs(T=16384)
    want = orc.osc_bank_const(c["freq"], c["amp"], c["T"], c["sr"], stateful=True)
    got = ctx.osc_bank_const(dev(c["freq"]), dev(c["amp"]), c["T"], c["sr"], dgen_b200.PHASE_SEQUENTIAL)
    assert np.abs(got.cpu().numpy() - want).max() < 2e-5


def test_known_answers_through_the_abi(ctx):
    # Tests/DGenLazyTests/CBackendTests.swift:63-76: 1 Hz at sr 4 -> 0, 1, 0, -1
    for mode in (dgen_b200.PHASE_DETERMINISTIC, dgen_b200.PHASE_SEQUENTIAL):
        got = ctx.osc_bank_const(dev(np.array([1.0], f32)), dev(np.array([1.0], f32)), 4, 4.0, mode).cpu().numpy()
        assert np.allclose(got, [0, 1, 0, -1], atol=1e-4)


def _render_both(ctx, d, mode, noise=True):
    T, sr = d["T"], d["sr"]
    taps = wl.taps_from_bands(d) if noise else None
    want = orc.harmonic_noise_render(d["f0"], d["uv"], d["amps"], d["gain"], d["noise_gain"], taps,
                                     d["noise"] if noise else None, T, sr)
    audio = ctx.harmonic_render(dev(d["f0"]), dev(d["uv"]), dev(d["amps"]), dev(d["gain"]), T, sr, phase_mode=mode)
    if noise:
        taps_dev = ctx.bands_to_taps(dev(d["bands"]), dev(d["W"]))
        assert np.abs(taps_dev.cpu().numpy() - taps).max() < 1e-5
        ctx.fir_noise(dev(d["noise"]), taps_dev, dev(d["noise_gain"]), out=audio, accumulate=True)
    ctx.sync()
    return audio.cpu().numpy(), want


@pytest.mark.parametrize("F,B,NB,NT", [(500, 40, 65, 257), (333, 61, 65, 257), (211, 33, 33, 129), (130, 9, 80, 400),
                                       (700, 3, 65, 130)])
def test_band_to_tap_map_at_scale_against_a_double_precision_product(ctx, F, B, NB, NT, monkeypatch):
    """The plain single-precision tile kernel of the map (forced here; the default where the tensor-core kernel does
    not apply, up to 1024 output tiles): row counts that are no multiple of the 128-row tile, tap counts with a
    one-column remainder tile (257 = 2 x 128 + 1), a two-column one (130) and a wide ragged one (400), band counts
    up to the shared-memory limit of the kernel (80).  Single-precision accumulation in band order: within a few
    ulps of the double-precision product."""
    monkeypatch.setenv("DGC_TAP_MAP", "tile")
    assert F * B * NB * NT >= 1 << 24
    rng = np.random.default_rng(F)
    bands = rng.uniform(0, 1, (F, B, NB)).astype(f32)
    W = rng.standard_normal((NT, NB)).astype(f32)
    want = bands.reshape(F * B, NB).astype(np.float64) @ W.astype(np.float64).T
    got = ctx.bands_to_taps(dev(bands), dev(W)).cpu().numpy().reshape(F * B, NT)
    scale = np.abs(want).max()
    assert np.abs(got - want).max() < 2e-6 * scale
    # the matrix of the synthetic workload as well (windowed frequency sampling)
    d = wl.harmonic_noise_inputs(5, B=B, T=1024, K=4, F=F, nbands=NB, taps=NT)
    got = ctx.bands_to_taps(dev(d["bands"]), dev(d["W"])).cpu().numpy()
    assert np.abs(got - wl.taps_from_bands(d)).max() < 1e-5


@pytest.mark.parametrize("rows,NB,NT", [(1010, 65, 257), (2100, 65, 257), (40001, 33, 128), (20000, 32, 136),
                                        (9000, 72, 137), (30011, 65, 300), (64000, 65, 257), (5000, 40, 1024),
                                        (100, 72, 2400), (129, 64, 2100)])
def test_band_to_tap_map_on_the_persistent_tensor_core_kernel(ctx, rows, NB, NT, monkeypatch):
    """32 to 72 bands and at least 128 taps: the matmul entry point (forced here for every size; the default beyond
    1024 output tiles) runs the map on the persistent short-reduction tensor-core kernel (3xTF32 with rounded
    parts).  One row tile and several per CTA (the accumulators and the copy stages alternate),
    rows that end inside a tile, up to eight leftover columns computed as plain dot products (257, 136), a ragged
    last column block (137, 300), more column blocks than a few (1024), fewer rows than one tile and a second tile
    of a single row (100 and 129 rows), band counts of every alignment.  The result
    stays within a few single-precision ulps of the double-precision product, and the same call twice gives the same
    bits."""
    assert rows * NB * NT >= 1 << 24, "below 2^24 multiply-adds the map does not run as a matmul"
    rng = np.random.default_rng(rows + NB + NT)
    bands = rng.uniform(0, 1, (rows, 1, NB)).astype(f32)
    W = rng.standard_normal((NT, NB)).astype(f32)
    want = bands.reshape(rows, NB).astype(np.float64) @ W.astype(np.float64).T
    monkeypatch.setenv("DGC_TAP_MAP", "tc")
    before = ctx.gemm_path_counts()
    got_dev = ctx.bands_to_taps(dev(bands), dev(W))
    got = got_dev.cpu().numpy().reshape(rows, NT)
    after = ctx.gemm_path_counts()
    assert sum(after) == sum(before) + 1, "the map did not go through the matmul entry point"
    assert np.abs(got - want).max() < 2e-6 * np.abs(want).max()
    again = ctx.bands_to_taps(dev(bands), dev(W)).cpu().numpy().reshape(rows, NT)
    assert np.array_equal(got, again)


@pytest.mark.parametrize("shape", [dict(B=2, T=4096, K=100, F=64), dict(B=3, T=5000, K=7, F=33),
                                   dict(B=1, T=1000, K=1, F=2), dict(B=2, T=2048, K=130, F=40),
                                   dict(B=1, T=640, K=300, F=11)])
def test_harmonic_render_sequential_matches_oracle(ctx, shape):
    d = wl.harmonic_noise_inputs(11, sr=16000.0, **shape)
    got, want = _render_both(ctx, d, dgen_b200.PHASE_SEQUENTIAL, noise=False)
    assert np.abs(got - want).max() < 2e-5


def test_harmonic_noise_render_full_config_both_phase_modes(ctx):
    """The batched harmonic+noise configuration at full size (B=16, T=64000, K=100, 65 bands, 257 taps)."""
    d = wl.harmonic_noise_inputs(20260001)
    got, want = _render_both(ctx, d, dgen_b200.PHASE_SEQUENTIAL)
    err_seq = np.abs(got - want).max()
    got2, _ = _render_both(ctx, d, dgen_b200.PHASE_SCAN)
    err_scan = np.abs(got2 - want).max()
    got3, _ = _render_both(ctx, d, dgen_b200.PHASE_FUNDAMENTAL)
    err_fund = np.abs(got3 - want).max()
    print("max abs err: sequential %.3g, scan %.3g, fundamental %.3g" % (err_seq, err_scan, err_fund))
    assert err_seq < 2e-5
    assert err_scan < 1e-4  # the stated forward tolerance
    assert err_fund < 1e-4  # one scan per voice: also drops the rounding of each partial's own increment


@pytest.mark.parametrize("shape", [dict(B=2, T=4096, K=100, F=64), dict(B=3, T=5000, K=7, F=33),
                                   dict(B=1, T=1000, K=1, F=2), dict(B=2, T=2048, K=130, F=40),
                                   dict(B=1, T=640, K=300, F=11), dict(B=2, T=70001, K=100, F=300)])
def test_harmonic_render_fundamental_mode_matches_oracle(ctx, shape):
    """The per-voice scan of the fundamental: partial k reads its phase as k times one 64-bit running sum."""
    d = wl.harmonic_noise_inputs(13, sr=16000.0, **shape)
    got, want = _render_both(ctx, d, dgen_b200.PHASE_FUNDAMENTAL, noise=False)
    assert np.abs(got - want).max() < 1e-4
    got_scan, _ = _render_both(ctx, d, dgen_b200.PHASE_SCAN, noise=False)
    assert np.abs(got - got_scan).max() < 1e-4


def test_fundamental_mode_out_of_range_f0(ctx):
    """Fundamentals at and above the sample rate, zero and negative ones: the phase stays defined (fraction of
    f0 / sr), partials above Nyquist are masked exactly as in the other modes."""
    d = wl.harmonic_noise_inputs(17, B=4, T=4096, K=20, F=32, sr=16000.0)
    d["f0"][:, 1] = 0.0
    d["f0"][:, 2] *= 40.0          # up to and beyond the sample rate
    d["f0"][::2, 3] = -50.0
    got, want = _render_both(ctx, d, dgen_b200.PHASE_FUNDAMENTAL, noise=False)
    assert np.isfinite(got).all()
    assert np.abs(got[:2] - want[:2]).max() < 1e-4
    got_scan, _ = _render_both(ctx, d, dgen_b200.PHASE_SCAN, noise=False)
    assert np.abs(got - got_scan).max() < 2e-4


def test_fir_noise_ragged_and_short(ctx):
    for B, T, F, NT in ((2, 3000, 50, 257), (1, 100, 5, 17), (2, 2049, 9, 64), (1, 5000, 1, 33)):
        rng = np.random.default_rng(T)
        taps = rng.standard_normal((F, B, NT)).astype(f32)
        noise = rng.standard_normal((B, T)).astype(f32)
        ng = rng.uniform(0, 1, (F, B)).astype(f32)
        K = 1
        z = np.zeros((F, B), f32)
        want = orc.harmonic_noise_render(z + 100, z, np.ones((F, B, K), f32), z, ng, taps, noise, T, 16000.0)
        got = ctx.fir_noise(dev(noise), dev(taps), dev(ng)).cpu().numpy()
        scale = max(1.0, np.abs(want).max())
        assert np.abs(got - want).max() < 2e-5 * scale


def test_render_is_deterministic(ctx):
    d = wl.harmonic_noise_inputs(5, B=2, T=8192, K=100, F=128)
    a = ctx.harmonic_render(dev(d["f0"]), dev(d["uv"]), dev(d["amps"]), dev(d["gain"]), d["T"], d["sr"]).cpu().numpy()
    b = ctx.harmonic_render(dev(d["f0"]), dev(d["uv"]), dev(d["amps"]), dev(d["gain"]), d["T"], d["sr"]).cpu().numpy()
    assert np.array_equal(a, b)


def test_bad_arguments_return_errors(ctx):
    import torch
    with pytest.raises(dgen_b200.DgenCudaError):
        ctx.osc_bank_const(torch.zeros(1, device="cuda"), torch.zeros(1, device="cuda"), 0, 44100.0)
    with pytest.raises(dgen_b200.DgenCudaError):
        ctx.clock_accum(1.0, 1.0, 1.0, 16)


def test_device_resident_composite_equals_the_staged_calls(ctx):
    """dgc_hn_forward_loss (two branches on two streams, joined at the loss) against the same step made of the
    single entry points on one stream: identical loss, identical audio."""
    import ctypes as C
    import torch
    B, T, K, F, NB, NT = 3, 9000, 40, 70, 9, 33
    d = wl.harmonic_noise_inputs(61, B=B, T=T, K=K, F=F, nbands=NB, taps=NT)
    D = {k: dev(v) for k, v in d.items() if isinstance(v, np.ndarray)}
    target = dev(np.random.default_rng(2).standard_normal((B, T)).astype(f32) * f32(0.1))
    audio = ctx.harmonic_render(D["f0"], D["uv"], D["amps"], D["gain"], T, d["sr"])
    ctx.fir_noise(D["noise"], ctx.bands_to_taps(D["bands"], D["W"]), D["noise_gain"], out=audio, accumulate=True)
    want = float(ctx.mss_loss_fwd(audio, target, sizes=(512, 128, 64)).cpu()[0])
    st = dgen_b200.HnStep()
    st.harm = dgen_b200.HarmonicParams(B, T, K, F, d["sr"], 1.0, dgen_b200.PHASE_SCAN, 0)
    st.fir = dgen_b200.FirParams(B, T, F, NT, 0.12, 1)
    st.mss = dgen_b200.mss_params(B, T, (512, 128, 64))
    st.nbands = NB
    for want_audio in (False, True):
        out = torch.empty(B, T, device="cuda") if want_audio else None
        for _ in range(3):          # repeated calls reuse the side stream and events
            loss, _ = ctx.hn_forward_loss(st, D["f0"], D["uv"], D["amps"], D["gain"], D["noise_gain"], D["bands"], D["W"],
                                          D["noise"], target, audio=out)
        ctx.sync()
        assert float(loss.cpu()[0]) == want
        if want_audio:
            assert torch.equal(out, audio)


def test_two_host_buffer_steps_in_flight_equal_the_blocking_call(ctx):
    """dgc_hn_forward_loss_host_submit / _wait: different batches alternate over the two slots; every loss (and the
    audio read back) equals the blocking host-buffer call on the same batch; a slot cannot be resubmitted before its
    wait, and the blocking call refuses to run while steps are in flight."""
    import torch
    B, T, K, F, NB, NT = 3, 9000, 40, 70, 9, 33
    st = dgen_b200.HnStep()
    st.harm = dgen_b200.HarmonicParams(B, T, K, F, 16000.0, 1.0, dgen_b200.PHASE_SCAN, 0)
    st.fir = dgen_b200.FirParams(B, T, F, NT, 0.12, 1)
    st.mss = dgen_b200.mss_params(B, T, (512, 128, 64))
    st.nbands = NB
    pin = lambda a: torch.from_numpy(np.ascontiguousarray(a)).pin_memory()
    order = ("f0", "uv", "amps", "gain", "noise_gain", "bands", "W", "noise")
    batches, want, want_audio = [], [], []
    for i in range(5):
        d = wl.harmonic_noise_inputs(70 + i, B=B, T=T, K=K, F=F, nbands=NB, taps=NT)
        P = [pin(d[k]) for k in order] + [pin(np.random.default_rng(i).standard_normal((B, T)).astype(f32) * f32(0.1))]
        batches.append(P)
        a = pin(np.zeros((B, T), f32))
        want.append(ctx.hn_forward_loss_host(st, *P, audio_out=a))
        want_audio.append(a.numpy().copy())
    got = [None] * 5
    audio = [pin(np.zeros((B, T), f32)) for _ in range(2)]
    ctx.hn_forward_loss_host_submit(st, *batches[0], 0, audio_out=audio[0])
    with pytest.raises(dgen_b200.DgenCudaError):
        ctx.hn_forward_loss_host_submit(st, *batches[1], 0)            # slot 0 is still in flight
    with pytest.raises(dgen_b200.DgenCudaError):
        ctx.hn_forward_loss_host(st, *batches[1])                      # blocking call while a step is in flight
    for i in range(1, 5):
        ctx.hn_forward_loss_host_submit(st, *batches[i], i % 2, audio_out=audio[i % 2])
        got[i - 1] = ctx.hn_forward_loss_host_wait((i - 1) % 2)
        assert np.array_equal(audio[(i - 1) % 2].numpy(), want_audio[i - 1])
    got[4] = ctx.hn_forward_loss_host_wait(0)
    assert got == want
    with pytest.raises(dgen_b200.DgenCudaError):
        ctx.hn_forward_loss_host_wait(1)                               # nothing submitted on slot 1 any more
    assert ctx.hn_forward_loss_host(st, *batches[2]) == want[2]        # the blocking call works again
