"""The restatement of the ring / hold ops (oracle/stateful_ops.py) against the known answers the reference's own
tests hold for them: delayed ramps (Tests/DGenLazyTests/TensorDelayTests.swift:55-131), the hop staircase of the
spectrum delay (Tests/DGenTests/SpectrumDelayTests.swift:9-150), and the latch's hold semantics
(Sources/DGen/Definitions.swift:104-113)."""
import numpy as np

from oracle import stateful_ops as so

f32 = np.float32


def ramp(T, factors):
    return (np.arange(T, dtype=f32)[:, None] * np.asarray(factors, f32)[None, :]).astype(f32)


def delayed_ramp(T, factor, delay):
    n = np.arange(T)
    return np.where(n >= delay, factor * (n - delay), 0.0).astype(f32)


def test_tensor_delay_scalar_time_delays_lanes_independently():
    y, _, _ = so.delay_line(ramp(64, [2.0, 5.0]), 10.0, 88000 // 64)
    assert np.abs(y[:, 0] - delayed_ramp(64, 2.0, 10)).max() <= 1e-3
    assert np.abs(y[:, 1] - delayed_ramp(64, 5.0, 10)).max() <= 1e-3


def test_tensor_delay_per_lane_times():
    y, _, _ = so.delay_line(ramp(64, [2.0, 5.0]), np.tile(np.asarray([5.0, 9.0], f32), (64, 1)), 512)
    assert np.abs(y[:, 0] - delayed_ramp(64, 2.0, 5)).max() <= 1e-3
    assert np.abs(y[:, 1] - delayed_ramp(64, 5.0, 9)).max() <= 1e-3


def test_tensor_delay_fractional_time_interpolates():
    y, _, _ = so.delay_line(ramp(64, [1.0, 1.0]), 10.5, 512)
    n = np.arange(12, 64)
    assert np.abs(y[12:, 0] - (n - 10.5)).max() <= 1e-3


def test_tensor_delay_clamps_oversized_time():
    y, _, _ = so.delay_line(ramp(64, [1.0, 1.0]), 1000.0, 32)
    assert np.abs(y[:, 0] - delayed_ramp(64, 1.0, 31)).max() <= 1e-3


def test_delay_state_carries_across_calls():
    rng = np.random.default_rng(3)
    x = rng.standard_normal((300, 3)).astype(f32)
    d = rng.uniform(-2.0, 45.0, (300, 3)).astype(f32)
    whole, ring_w, head_w = so.delay_line(x, d, 37)
    a, ring, head = so.delay_line(x[:113], d[:113], 37)
    b, ring, head = so.delay_line(x[113:], d[113:], 37, ring, head)
    assert np.array_equal(np.concatenate([a, b]), whole)
    assert np.array_equal(ring, ring_w) and head == head_w


def test_spectrum_delay_reads_hops_ago():
    hop, hops_back, N, H = 4, 2, 16, 8
    spec = np.repeat((np.arange(H, dtype=f32) * hop)[:, None], N, axis=1)
    out, _, _ = so.spectrum_delay(spec, hops_back)
    for h in range(hops_back, H):
        assert abs(out[h].mean() - (h - hops_back) * hop) <= 1e-3
    assert np.all(out[:hops_back] == 0)


def test_spectrum_delay_mod_constant_delay_of_one_matches_fixed_delay():
    hop, N, H = 4, 16, 8
    spec = np.repeat((np.arange(H, dtype=f32) * hop)[:, None], N, axis=1)
    out, _, _ = so.spectrum_delay_mod(spec, np.full(H, 1.0, f32), 3)
    fixed, _, _ = so.spectrum_delay(spec, 1)
    assert np.array_equal(out, fixed)
    for h in range(1, H):
        assert abs(out[h].mean() - (h - 1) * hop) <= 1e-3


def test_latch_holds_last_triggered_value():
    v = np.arange(1, 11, dtype=f32)[:, None]
    c = np.asarray([0, 0, 1, 0, 0, -1, 1, 0, 0, 0], f32)
    y, st = so.latch(v, c, state=np.asarray([7.5], f32))
    assert y[:, 0].tolist() == [7.5, 7.5, 3, 3, 3, 3, 7, 7, 7, 7] and st[0] == 7


def test_compressor_leaves_quiet_signals_alone_and_reduces_loud_ones():
    sr = 44100.0
    t = np.arange(4096, dtype=f32) / f32(sr)
    quiet = (0.01 * np.sin(2 * np.pi * 440.0 * t)).astype(f32)[None, :]     # -40 dB: below the knee
    loud = (0.9 * np.sin(2 * np.pi * 440.0 * t)).astype(f32)[None, :]
    yq, _ = so.compressor(quiet, 4.0, -20.0, 6.0, 0.005, 0.05, sr)
    mask = np.abs(quiet) >= 1e-5     # below the detector floor the op emits the floor itself
    assert np.allclose(yq[mask], quiet[mask], rtol=2e-5, atol=1e-7)
    yl, s = so.compressor(loud, 4.0, -20.0, 6.0, 0.005, 0.05, sr)
    assert np.abs(yl[:, 2048:]).max() < 0.5 * np.abs(loud).max() and s[0] > 0
    assert np.all(np.sign(yl) == np.sign(loud))
