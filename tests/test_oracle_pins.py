"""Pins the CPU oracle (oracle/dgen_oracle.c) to the reference.

Sources of truth used here:
  * known-answer values of the reference's C-backend tests
    (Tests/DGenLazyTests/CBackendTests.swift:46-76),
  * outputs of the reference's own generated C artefacts (toolchain/generated/hermetic/*.c) run
    with the reference harness's inputs, committed as tests/golden/ref_artefacts.npz by
    tests/golden/make_golden.py, and re-run live when oracle/_ref exists,
  * mathematical identities for the FFT host service (vs numpy) and overlap-add gain
    (Tests/DGenTests/AcceleratedFFTTests.swift:11-140: peak = N/hop within 0.1).
"""
import os

import numpy as np
import pytest

from oracle import oracle as orc

GOLD = np.load(os.path.join(os.path.dirname(__file__), "golden", "ref_artefacts.npz"))
f32 = np.float32


def test_phasor_known_answers():
    # CBackendTests.testSignalPhasor: 100 Hz at sr 1000 -> 0, .1, .5, .9 at frames 0,1,5,9 (1e-4)
    ph = orc.phasor_stateful(np.full((12, 1), 100.0, f32), 1000.0)[:, 0]
    for i, v in ((0, 0.0), (1, 0.1), (5, 0.5), (9, 0.9)):
        assert abs(ph[i] - v) < 1e-4
    # scalar accum form of the same thing
    ac = orc.accum(f32(100.0) / f32(1000.0), 0.0, 1.0, 12)
    assert np.array_equal(ac, ph)


def test_sine_known_answers():
    # CBackendTests.testSignalSineWave: 1 Hz at sr 4 -> 0, 1, 0, -1 (1e-4)
    a = orc.osc_bank_const([1.0], [1.0], 4, 4.0, stateful=True)
    assert np.allclose(a, [0, 1, 0, -1], atol=1e-4)
    a = orc.osc_bank_const([1.0], [1.0], 4, 4.0, stateful=False)
    assert np.allclose(a, [0, 1, 0, -1], atol=1e-4)


def _scalar_synth_restated(n, sr):
    ph = orc.phasor_stateful(np.full((n + 1, 1), 220.0, f32), sr)[:, 0]
    p = ph[:n].astype(np.float64)
    fund = np.sin(p * 6.283185)
    harm = np.cos(p * 12.56637)
    return ph, (0.2 * np.tanh(1.75 * (fund + 0.125 * harm))).astype(f32)


def test_stateful_phasor_matches_reference_artefact_bit_exactly():
    """scalar-synth: the phasor state the reference's emitted code leaves after 8192 frames equals the
    oracle's phase, bit for bit; audio agrees to the polynomial-sin error class (2e-6)."""
    n = GOLD["scalar_synth"].size
    ph, audio = _scalar_synth_restated(n, 48000.0)
    assert ph[n] == GOLD["scalar_synth_final_phase"][0]
    assert np.abs(audio - GOLD["scalar_synth"]).max() < 2e-6


def test_history_feedback_matches_reference_artefact():
    """feedback-delay-effect: out = mix(x, d, wet), d[n] = w[n-37], w[n] = x[n] + fb*d[n-1]
    (one-sample history delay)."""
    x = GOLD["input"]
    n = x.size
    fb, wet, D = f32(0.35), f32(0.4), 37
    w = np.zeros(n, f32)
    d = np.zeros(n, f32)
    for i in range(n):
        prev = d[i - 1] if i > 0 else f32(0)
        w[i] = x[i] + fb * prev
        d[i] = w[i - D] if i >= D else f32(0)
    out = x * (f32(1) - wet) + d * wet
    assert np.abs(out - GOLD["feedback_delay"]).max() < 1e-6


def test_row_lerp_matches_reference_artefact():
    """wavetable-instrument: `peek` reads a [16 x 2] table at a fractional sample index with the arithmetic
    sampleRow shares -- wrap into [0, rows), floor row, next row wrapping to 0 at the end, (1 - frac) * lo + frac * hi
    (toolchain/generated/hermetic/wavetable-instrument.c: t28..t69; Sources/DGen/Emit+RowSelection.swift:166-199).
    The oracle's orc_sample_row on the artefact's own table and phase reproduces the artefact's audio."""
    gold, mem = GOLD["wavetable_instrument"], GOLD["wavetable_memory"]
    n = gold.size
    freq, wave, gain = f32(mem[32]), f32(mem[33]), f32(mem[34])
    ph = orc.phasor_stateful(np.full((n, 1), freq, f32), 48000.0)[:, 0]
    idx = ((ph - np.floor(ph)) * f32(16.0)).astype(f32)
    table = np.stack([mem[0:16], mem[16:32]], axis=1).astype(f32)            # [sample][wave] = memory[16 * wave + sample]
    rows = orc.sample_row(table, idx)                                        # [n][2]: both waves at the sample index
    w = f32(min(max(wave, f32(0)), f32(1)))
    wl = f32(np.floor(w))
    wf = f32(w - wl)
    hi = int(min(wl + 1, 1))
    out = gain * ((rows[:, int(wl)] * (f32(1) - wf)).astype(f32) + (rows[:, hi] * wf).astype(f32)).astype(f32)
    assert np.abs(out.astype(f32) - gold).max() < 1e-7
    # the wrap of the upper row: the last sample interpolates towards sample 0
    k = int(np.argmax(idx >= 15.0))
    assert idx[k] >= 15.0 and abs(rows[k, 0] - ((f32(1) - (idx[k] - 15)) * table[15, 0] + (idx[k] - 15) * table[0, 0])) < 1e-6


def test_partitioned_convolve_matches_reference_artefact():
    """spectral-effect: bufferView ring + hop counter + Hann + FFT + partitioned MAC + IFFT +
    overlapAdd, N=16 hop=8 gain=0.5, 32-tap IR (toolchain/fixtures/spectral-effect.lisp)."""
    ir = np.zeros(32, f32)
    ir[0], ir[8], ir[16], ir[24] = 1.0, 0.35, 0.15, 0.05
    out = orc.partitioned_convolve(GOLD["input"], ir, 16, 8, gain=0.5)
    assert np.abs(out - GOLD["spectral_effect"]).max() < 2e-6


@pytest.mark.skipif(not orc.ref_available(), reason="oracle/_ref not built")
def test_golden_file_is_what_the_artefacts_produce_now():
    import importlib.util
    spec = importlib.util.spec_from_file_location(
        "make_golden", os.path.join(os.path.dirname(__file__), "golden", "make_golden.py"))
    mg = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mg)
    m = mg.memory_for("spectral-effect")
    out = orc.ref_run("spectral-effect", m, mg.harness_input(8192), 128, 64, 48000.0)
    assert np.array_equal(out, GOLD["spectral_effect"])
    m = mg.memory_for("scalar-synth")
    out = orc.ref_run("scalar-synth", m, None, 128, 64, 48000.0)
    assert np.array_equal(out, GOLD["scalar_synth"])


@pytest.mark.parametrize("N", [2, 16, 64, 1024, 2048])
def test_fft_service_is_the_unnormalised_dft(N):
    rng = np.random.default_rng(N)
    re, im = rng.standard_normal(N).astype(f32), rng.standard_normal(N).astype(f32)
    R, I = orc.fft(re, im)
    ref = np.fft.fft(re.astype(np.float64) + 1j * im)
    scale = np.abs(ref).max()
    assert np.abs(R - ref.real).max() < 2e-6 * scale and np.abs(I - ref.imag).max() < 2e-6 * scale
    r2, i2 = orc.fft(R, I, inverse=True)  # both directions unnormalised: round trip = N * x
    assert np.abs(r2 / N - re).max() < 1e-5 and np.abs(i2 / N - im).max() < 1e-5


def test_fft_ifft_overlap_add_gain_is_n_over_hop():
    # AcceleratedFFTTests: buffer -> FFT -> IFFT(1/N) -> overlapAdd of a constant 1.0 reaches N/hop
    N, hop, T = 64, 16, 512
    H = T // hop
    frames = np.zeros((H, N), f32)
    for h in range(H):
        f = h * hop
        w = np.array([1.0 if f - N + 1 + i >= 0 else 0.0 for i in range(N)], f32)
        R, I = orc.fft(w, np.zeros(N, f32))
        r, _ = orc.fft(R, I, inverse=True)
        frames[h] = r / N
    out = orc.overlap_add(frames, T, hop)
    assert abs(out[N * 2:].max() - N / hop) < 0.1


def test_hann_tables():
    # SpectralLossGradientTests.swift:129-157 uses 0.5*(1-cos(2 pi n/(N-1))) for the loss window
    w = orc.hann_symmetric(8)
    assert np.allclose(w, 0.5 * (1 - np.cos(2 * np.pi * np.arange(8) / 7)), atol=1e-7)
    assert w[0] == 0 and abs(w[-1]) < 1e-7
    # toolchain_harness.c kSpectralHann: hann(16) periodic as the reference evaluates it in Float
    gold = np.array([0.0, 0.038060218, 0.14644659, 0.3086583, 0.49999997, 0.69134164, 0.8535534, 0.96193975,
                     1.0, 0.9619398, 0.85355353, 0.69134176, 0.5, 0.30865842, 0.14644668, 0.038060308], f32)
    assert np.abs(orc.hann_periodic(16) - gold).max() < 1.5e-7


def test_spectral_loss_semantics():
    # BatchedSpectralLossTests: identical signals -> 0; batched == mean of per-voice scalar losses;
    rng = np.random.default_rng(3)
    B, T, N, hop = 3, 256, 64, 16
    x = rng.standard_normal((B, T)).astype(f32)
    y = rng.standard_normal((B, T)).astype(f32)
    assert orc.spectral_loss(x, x, N, hop) == 0.0
    tot, part = orc.spectral_loss(x, y, N, hop, want_partial=True)
    singles = [orc.spectral_loss(x[b:b + 1], y[b:b + 1], N, hop) for b in range(B)]
    assert abs(tot - np.mean(singles)) < 1e-4 * abs(tot)
    # independent check of one hop frame against numpy's rfft
    h = 9
    f = h * hop
    win = orc.hann_symmetric(N).astype(np.float64)
    seg = lambda s: np.abs(np.fft.rfft(s[f - N + 1:f + 1].astype(np.float64) * win))
    for b in range(B):
        assert abs(part[h, b] - np.abs(seg(x[b]) - seg(y[b])).sum()) < 1e-3
    # first hop frame: only x[0] * hann[N-1] = 0 contributes
    assert abs(part[0]).max() < 1e-5
    lg = orc.spectral_loss(x, y, N, hop, use_log=True)
    lg64 = orc.spectral_loss(x, y, N, hop, use_log=True, double=True)
    assert abs(lg - lg64) < 1e-4 * abs(lg64)


def test_biquad_lowpass_coefficients():
    # RBJ low-pass with the op's fixed 2*pi/44100 constant (Sources/DGen/HigherOps.swift:447)
    fc, q = 1000.0, 0.707
    w = fc * 2 * np.pi / 44100
    al = np.sin(w) / (2 * q)
    a0 = 1 + al
    want = [(1 - np.cos(w)) / 2 / a0, (1 - np.cos(w)) / a0, (1 - np.cos(w)) / 2 / a0, -2 * np.cos(w) / a0, (1 - al) / a0]
    assert np.allclose(orc.biquad_coef(fc, q, double=True), want, rtol=1e-9)
    assert np.allclose(orc.biquad_coef(fc, q), want, rtol=2e-5)
    # DC gain of a low-pass is 1
    y = orc.biquad(np.ones(4000, f32), fc, q)
    assert abs(y[-1] - 1) < 1e-3


def test_sample_row_wraps_ceil_to_row_zero():
    tab = np.array([[0.0, 10.0], [1.0, 20.0], [2.0, 30.0]], f32)
    out = orc.sample_row(tab, np.array([0.0, 0.5, 2.0, 2.5], f32))
    assert np.allclose(out, [[0, 10], [0.5, 15], [2, 30], [1.0, 20.0]])


def test_playhead_is_sequential_fp32():
    F, T = 1000, 64000
    p = orc.playhead(F, T)
    step = f32(F - 1) / f32(T - 1)
    s = f32(0)
    for n in range(2000):
        assert p[n] == s
        s = f32(s + step)
    assert p.max() <= f32(F - 1) - f32(1e-4) + 1e-6
    # the sequential fp32 clock drifts from n*step by a sizeable fraction of a control frame
    assert np.abs(p[:60000] - np.arange(60000) * float(step)).max() > 0.05


def test_noise_prng_range_and_determinism():
    a, s = orc.noise_xorshift(0, 1000)
    b, _ = orc.noise_xorshift(0, 1000)
    assert np.array_equal(a, b) and a.min() > 0 and a.max() < 1.0 + 1e-7 and s != 0


def test_adam_first_step_is_lr_sign():
    th = np.array([1.0, -2.0, 3.0], f32)
    g = np.array([0.5, -0.25, 2.0], f32)
    m = np.zeros(3, f32)
    v = np.zeros(3, f32)
    orc.adam(th, g, m, v, 1)
    assert np.allclose(th, [1 - 1e-3, -2 + 1e-3, 3 - 1e-3], atol=1e-6)
