"""Ring / hold ops through the C ABI against the frame-by-frame restatement (oracle/stateful_ops.py).

Tolerances: the delay gathers interpolate with one fused multiply-add where the restatement rounds the two
products separately -> 1e-6 relative to the signal scale; fixed spectrum delay and latch move values without
arithmetic -> bit exact; compressor 1e-4 relative (log10 / pow of two math libraries; the reference's own
cross-backend tolerance for it is 1e-3, Tests/DGenLazyTests/AudioEffectsTests.swift:168-210)."""
import numpy as np
import pytest
import torch

import dgen_b200
from oracle import stateful_ops as so

pytestmark = pytest.mark.gpu
f32 = np.float32


@pytest.fixture(scope="module")
def ctx():
    c = dgen_b200.Context(0)
    yield c
    c.close()


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def close(got, want, rel):
    got = got.cpu().numpy()
    return np.abs(got - want).max() <= rel * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("mode", ["scalar", "per_frame", "per_frame_lane", "per_lane"])
def test_delay_line_modes(ctx, mode):
    rng = np.random.default_rng(11)
    T, lanes, R = 700, 5, 64
    x = rng.standard_normal((T, lanes)).astype(f32)
    if mode == "scalar":
        d_or, d_dev = 10.5, 10.5
    elif mode == "per_frame":
        d = rng.uniform(-3.0, 80.0, T).astype(f32)
        d_or, d_dev = d, dev(d)
    elif mode == "per_frame_lane":
        d = rng.uniform(-3.0, 80.0, (T, lanes)).astype(f32)
        d[::7] = np.floor(d[::7])                    # whole delays too, among them the clamped maximum
        d_or, d_dev = d, dev(d)
    else:
        d = np.asarray([0.0, 5.0, 9.25, 63.0, 200.0], f32)
        d_or, d_dev = np.tile(d, (T, 1)), dev(d)
    want, _, _ = so.delay_line(x, d_or, R)
    got = ctx.delay_line(dev(x), d_dev, R, per_lane=(mode == "per_lane"))
    assert close(got, want, 1e-6)


def test_delay_line_reference_ramps(ctx):
    # Tests/DGenLazyTests/TensorDelayTests.swift:83-131
    T = 64
    x = (np.arange(T, dtype=f32)[:, None] * np.asarray([2.0, 5.0], f32)[None, :]).astype(f32)
    y = ctx.delay_line(dev(x), dev(np.asarray([5.0, 9.0], f32)), 512, per_lane=True).cpu().numpy()
    n = np.arange(T)
    assert np.abs(y[:, 0] - np.where(n >= 5, 2.0 * (n - 5), 0)).max() <= 1e-3
    assert np.abs(y[:, 1] - np.where(n >= 9, 5.0 * (n - 9), 0)).max() <= 1e-3
    y = ctx.delay_line(dev(x), 1000.0, 32).cpu().numpy()          # clamped to max_delay - 1
    assert np.abs(y[:, 0] - np.where(n >= 31, 2.0 * (n - 31), 0)).max() <= 1e-3


@pytest.mark.parametrize("splits", [(113, 187), (20, 10, 270), (64, 64, 172)])
def test_delay_line_state_across_calls(ctx, splits):
    """Blocks shorter and longer than the ring: outputs, ring and head continue exactly as one long call."""
    rng = np.random.default_rng(5)
    T, lanes, R = sum(splits), 3, 37
    x = rng.standard_normal((T, lanes)).astype(f32)
    d = rng.uniform(-2.0, 45.0, (T, lanes)).astype(f32)
    want, ring_w, head_w = so.delay_line(x, d, R)
    ring = torch.zeros(lanes, R, device="cuda")
    head = torch.zeros(1, device="cuda")
    outs, o = [], 0
    for n in splits:
        outs.append(ctx.delay_line(dev(x[o:o + n]), dev(d[o:o + n]), R, ring=ring, head=head))
        o += n
    assert close(torch.cat(outs), want, 1e-6)
    assert np.array_equal(ring.cpu().numpy(), ring_w) and float(head.cpu()[0]) == head_w


def test_delay_line_large_against_gather(ctx):
    """A size the frame loop cannot reach in seconds: against a vectorised gather of the same definition."""
    rng = np.random.default_rng(6)
    T, lanes, R = 200000, 64, 4096
    x = rng.standard_normal((T, lanes)).astype(f32)
    d = rng.uniform(0.0, R + 10.0, T).astype(f32)
    got = ctx.delay_line(dev(x), dev(d), R).cpu().numpy()
    dc = np.clip(d, 0, R - 1).astype(f32)
    k = np.floor(dc).astype(np.int64)
    frac = (dc - k).astype(f32)[:, None]
    n = np.arange(T)
    xp = np.concatenate([np.zeros((R + 1, lanes), f32), x])
    k1 = np.where(k + 1 >= R, 0, k + 1)
    s0, s1 = xp[n - k + R + 1], xp[n - k1 + R + 1]
    want = s0 * (1 - frac) + s1 * frac
    assert np.abs(got - want).max() <= 1e-6 * np.abs(want).max()


def test_spectrum_delay_fixed_and_modulated(ctx):
    rng = np.random.default_rng(8)
    H, N, hops = 90, 48, 5
    spec = rng.standard_normal((H, N)).astype(f32)
    want, ring_w, row_w = so.spectrum_delay(spec, hops)
    ring, row = torch.zeros(hops + 1, N, device="cuda"), torch.zeros(1, device="cuda")
    a = ctx.spectrum_delay(dev(spec[:33]), hops, ring=ring, row=row)
    b = ctx.spectrum_delay(dev(spec[33:36]), hops, ring=ring, row=row)       # shorter than the ring
    c = ctx.spectrum_delay(dev(spec[36:]), hops, ring=ring, row=row)
    assert np.array_equal(torch.cat([a, b, c]).cpu().numpy(), want)
    assert np.array_equal(ring.cpu().numpy(), ring_w) and float(row.cpu()[0]) == row_w
    d = rng.uniform(-1.0, hops + 1.5, H).astype(f32)
    d[::5] = np.floor(d[::5])
    want, ring_w, row_w = so.spectrum_delay_mod(spec, d, hops)
    ring.zero_()
    row.zero_()
    a = ctx.spectrum_delay(dev(spec[:41]), hops, delay=dev(d[:41]), ring=ring, row=row)
    b = ctx.spectrum_delay(dev(spec[41:]), hops, delay=dev(d[41:]), ring=ring, row=row)
    assert close(torch.cat([a, b]), want, 1e-6)
    assert np.array_equal(ring.cpu().numpy(), ring_w) and float(row.cpu()[0]) == row_w
    # Tests/DGenTests/SpectrumDelayTests.swift:9-150: a constant delay of one hop equals the fixed one-hop delay
    one = ctx.spectrum_delay(dev(spec), 3, delay=dev(np.full(H, 1.0, f32))).cpu().numpy()
    assert np.array_equal(one[1:], spec[:-1]) and np.all(one[0] == 0)


@pytest.mark.parametrize("T,lanes,shared", [(1, 1, True), (1000, 7, True), (1000, 7, False), (70000, 3, False),
                                            (129, 300, False), (50000, 1, True)])
def test_latch_bit_exact(ctx, T, lanes, shared):
    rng = np.random.default_rng(T + lanes)
    v = rng.standard_normal((T, lanes)).astype(f32)
    # sparse triggers, with long gaps that span many chunks and some lanes that never trigger
    c = np.where(rng.random(T if shared else (T, lanes)) < 0.004, 1.0, rng.choice([0.0, -1.0], T if shared else (T, lanes))).astype(f32)
    if not shared and lanes > 1:
        c[:, 1] = 0
    st = rng.standard_normal(lanes).astype(f32)
    want, st_w = so.latch(v, c, st)
    state = dev(st)
    got = ctx.latch(dev(v), dev(c), state=state)
    assert np.array_equal(got.cpu().numpy(), want) and np.array_equal(state.cpu().numpy(), st_w)
    # a second block continues from the held value
    v2 = rng.standard_normal((64, lanes)).astype(f32)
    c2 = np.zeros(64 if shared else (64, lanes), f32)
    want2, _ = so.latch(v2, c2, st_w)
    assert np.array_equal(ctx.latch(dev(v2), dev(c2), state=state).cpu().numpy(), want2)


@pytest.mark.parametrize("ratio,thr,knee,att,rel", [(4.0, -20.0, 6.0, 0.005, 0.05), (20.0, -10.0, 0.1, 0.001, 0.01),
                                                    (4.0, -20.0, 20.0, 0.01, 0.1)])
def test_compressor(ctx, ratio, thr, knee, att, rel):
    # parameter sets of Tests/DGenLazyTests/AudioEffectsTests.swift:168-210
    rng = np.random.default_rng(21)
    sr, B, T = 44100.0, 6, 3000
    t = np.arange(T, dtype=f32) / f32(sr)
    x = np.stack([(a * np.sin(2 * np.pi * f * t) * (1.0 + 0.5 * np.sin(2 * np.pi * 3.0 * t))).astype(f32)
                  for a, f in zip([0.9, 0.5, 0.1, 0.01, 1.5, 0.3], [440.0, 220.0, 1000.0, 50.0, 3000.0, 777.0])])
    x[5] = (0.3 * rng.standard_normal(T)).astype(f32)
    want, s_w = so.compressor(x, ratio, thr, knee, att, rel, sr)
    state = torch.zeros(B, device="cuda")
    a = ctx.compressor(dev(x[:, :1111]), ratio, thr, knee, att, rel, sr, state=state)
    b = ctx.compressor(dev(x[:, 1111:]), ratio, thr, knee, att, rel, sr, state=state)
    got = torch.cat([a, b], dim=1)
    assert close(got, want, 1e-4)
    assert np.allclose(state.cpu().numpy(), s_w, rtol=1e-4, atol=1e-5)
    side = np.roll(x, 1, axis=0)
    want, _ = so.compressor(x, ratio, thr, knee, att, rel, sr, sidechain=side)
    assert close(ctx.compressor(dev(x), ratio, thr, knee, att, rel, sr, sidechain=dev(side)), want, 1e-4)


def test_argument_errors(ctx):
    x = torch.zeros(8, 2, device="cuda")
    with pytest.raises(dgen_b200.DgenCudaError):
        ctx.delay_line(x, 1.0, 1)                                  # max_delay must be > 1
    with pytest.raises(dgen_b200.DgenCudaError):
        ctx.spectrum_delay(x, 0)                                   # hops must be >= 1
    with pytest.raises(dgen_b200.DgenCudaError):
        ctx.check(ctx.lib.dgc_delay_line(ctx.h, x.data_ptr(), x.data_ptr(), 0, 8, 2, 16, x.data_ptr(), None,
                                         torch.empty_like(x).data_ptr()))     # ring without head


# ---- standalone spectral blocks and the phase vocoder ----------------------------------------------------------
from oracle import oracle as orc


def oracle_stft(x, N, hop, window):
    T = x.size
    H = (T + hop - 1) // hop
    re, im = np.zeros((H, N), f32), np.zeros((H, N), f32)
    xp = np.concatenate([np.zeros(N - 1, f32), x])
    for h in range(H):
        w = xp[h * hop:h * hop + N]          # bufferView: element i of hop frame f = x[f - N + 1 + i]
        if window is not None:
            w = (w * window).astype(f32)
        re[h], im[h] = orc.fft(w, np.zeros(N, f32))
    return re, im


def oracle_istft_ola(re, im, T, hop, window, gain=1.0):
    H, N = re.shape
    frames = np.zeros((H, N), f32)
    for h in range(H):
        r, _ = orc.fft(re[h], im[h], inverse=True)
        r = (r * f32(1.0 / N)).astype(f32)          # the reference scales the inverse transform by 1/N
        if window is not None:
            r = (r * window).astype(f32)
        frames[h] = (r * f32(gain)).astype(f32)
    return orc.overlap_add(frames, T, hop)


def test_oracle_fft_inverse_is_unnormalised():
    re, im = orc.fft(np.asarray([1, 0, 0, 0, 0, 0, 0, 0] * 2, f32), np.zeros(16, f32))
    r, _ = orc.fft(re, im, inverse=True)
    assert abs(r[0] - 16.0) < 1e-4      # so oracle_istft_ola applies the 1/N itself


@pytest.mark.parametrize("N,hop,T,V", [(16, 8, 200, 1), (256, 64, 5000, 3), (1024, 256, 16000, 2), (2048, 1024, 9000, 1)])
def test_stft_fwd_and_istft_ola(ctx, N, hop, T, V):
    rng = np.random.default_rng(N + T)
    x = rng.standard_normal((V, T)).astype(f32)
    win = orc.hann_periodic(N)
    re, im = ctx.stft(dev(x), N, hop, window=dev(win))
    for v in range(V):
        wr, wi = oracle_stft(x[v], N, hop, win)
        scale = max(np.abs(wr).max(), np.abs(wi).max())
        assert np.abs(re[v].cpu().numpy() - wr).max() <= 2e-6 * scale * np.log2(N)
        assert np.abs(im[v].cpu().numpy() - wi).max() <= 2e-6 * scale * np.log2(N)
    # inverse of ARBITRARY (non-Hermitian) spectra: the real part of the inverse transform is kept
    sr = rng.standard_normal(tuple(re.shape)).astype(f32)
    si = rng.standard_normal(tuple(re.shape)).astype(f32)
    y = ctx.istft_ola(dev(sr), dev(si), T, hop, window=dev(win), gain=0.5)
    for v in range(V):
        want = oracle_istft_ola(sr[v], si[v], T, hop, win, 0.5)
        assert np.abs(y[v].cpu().numpy() - want).max() <= 2e-6 * max(1.0, np.abs(want).max()) * np.log2(N)
    # Tests/DGenLazyTests/AcceleratedFFTTests.swift:11-140: FFT -> IFFT -> overlap-add of unwindowed frames scales the
    # signal by N / hop once every frame is covered by N / hop windows
    re, im = ctx.stft(dev(x), N, hop)
    back = ctx.istft_ola(re, im, T, hop).cpu().numpy()
    # window h = x[h*hop-N+1 .. h*hop], laid back at h*hop .. h*hop+N-1: a delay of N - 1 frames
    d = N - 1
    lo, hi = d + N, T - N
    if hi > lo:
        assert np.abs(back[:, lo:hi] - (N / hop) * x[:, lo - d:hi - d]).max() <= 1e-4 * (N / hop) * np.abs(x).max()


def test_phase_vocoder_against_restatement(ctx):
    rng = np.random.default_rng(77)
    V, H, N, hop = 3, 40, 64, 16
    re = rng.standard_normal((V, H, N)).astype(f32)
    im = rng.standard_normal((V, H, N)).astype(f32)
    ratio = np.stack([np.full(H, 1.0, f32), np.full(H, 1.5, f32), (0.5 + rng.random(H)).astype(f32)])
    ratio[2, 5] = -3.0                                # raised to 1e-4: nothing in range but bin 0
    state = torch.zeros(V, 2 * N + 1, device="cuda")
    a_re, a_im = ctx.phase_vocoder(dev(re[:, :17]), dev(im[:, :17]), dev(ratio[:, :17]), hop, state=state)
    b_re, b_im = ctx.phase_vocoder(dev(re[:, 17:]), dev(im[:, 17:]), dev(ratio[:, 17:]), hop, state=state)
    got_re, got_im = torch.cat([a_re, b_re], 1).cpu().numpy(), torch.cat([a_im, b_im], 1).cpu().numpy()
    for v in range(V):
        w_re, w_im, st = so.phase_vocoder(re[v], im[v], ratio[v], hop)
        err = np.maximum(np.abs(got_re[v] - w_re), np.abs(got_im[v] - w_im))
        # the synthesis phase accumulates over the hops; a phase difference within rounding of +-pi flips a wrap in
        # one implementation and not in the other, a 2 pi (ratio - 1) jump for that bin: bound the bulk tightly
        assert np.quantile(err, 0.995) <= 2e-4 * np.abs(w_re).max(), v
        assert float(state[v, 2 * N].cpu()) == 1.0
    # ratio 1 returns the input (the synthesis phase tracks the analysis phase)
    assert np.abs(got_re[0] - re[0]).max() <= 1e-4 * np.abs(re[0]).max()
    assert np.abs(got_im[0] - im[0]).max() <= 1e-4 * np.abs(im[0]).max()
    # one ratio for all voices and hops
    o_re, _ = ctx.phase_vocoder(dev(re), dev(im), 1.5, hop)
    w_re, _, _ = so.phase_vocoder(re[1], im[1], np.full(H, 1.5, f32), hop)
    assert np.quantile(np.abs(o_re[1].cpu().numpy() - w_re), 0.995) <= 2e-4 * np.abs(w_re).max()


def test_pitch_shift_chain_moves_a_sinusoid(ctx):
    """Tests/DGenTests/PhaseVocoderTests.swift:99-150: buffer -> FFT -> phase vocoder -> IFFT -> overlap-add; an octave
    up roughly doubles the zero-crossing rate of a sinusoid, ratio 1 keeps it."""
    sr, T, N, hop = 44100.0, 32768, 1024, 256
    t = np.arange(T, dtype=f32) / f32(sr)
    x = np.sin(2 * np.pi * 440.0 * t).astype(f32)[None, :]
    win = dev(orc.hann_periodic(N))
    re, im = ctx.stft(dev(x), N, hop, window=win)

    def crossings(ratio):
        o_re, o_im = ctx.phase_vocoder(re, im, ratio, hop)
        y = ctx.istft_ola(o_re, o_im, T, hop, window=win).cpu().numpy()[0, 4096:-4096]
        assert np.isfinite(y).all() and np.abs(y).max() > 0.01
        return int(np.sum(np.signbit(y[1:]) != np.signbit(y[:-1])))

    same, up = crossings(1.0), crossings(2.0)
    base = int(np.sum(np.signbit(x[0, 4097:-4096]) != np.signbit(x[0, 4096:-4097])))
    assert abs(same - base) <= 0.02 * base
    assert 1.8 * base <= up <= 2.2 * base
