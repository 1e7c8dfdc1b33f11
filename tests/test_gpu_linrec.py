"""GPU parity of the linear-recurrence scans (one-pole, biquad bank forward and BPTT) against the oracle."""
import numpy as np
import pytest
import torch

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


@pytest.mark.parametrize("B,T,a", [(1, 65536, 0.9), (3, 5000, 0.5), (2, 1, 0.9), (2, 2049, -0.7), (1, 300000, 0.99)])
def test_onepole_matches_oracle(ctx, B, T, a):
    rng = np.random.default_rng(T)
    x = rng.standard_normal((B, T)).astype(f32)
    want = np.stack([orc.onepole(x[b], a) for b in range(B)])
    got = ctx.onepole_fwd(dev(x), a).cpu().numpy()
    assert np.abs(got - want).max() < 1e-5 * max(1.0, np.abs(want).max())


def test_osc_filter_fft_configuration(ctx):
    """Oscillator bank (64 partials, 110k Hz, 1/k) -> one-pole y = x + 0.9 y1 -> buffer(1024, hop 256) -> FFT
    -> magnitude, 65536 frames at 44.1 kHz: audio and per-hop magnitude frames against the oracle."""
    c = wl.osc_filter_fft_inputs()
    audio_o = orc.onepole(orc.osc_bank_const(c["freq"], c["amp"], c["T"], c["sr"]), c["pole"])
    mags_o = orc.buffer_fft_mag(audio_o, c["N"], c["hop"])
    osc = ctx.osc_bank_const(dev(c["freq"]), dev(c["amp"]), c["T"], c["sr"], dgen_b200.PHASE_DETERMINISTIC)
    audio = ctx.onepole_fwd(osc.view(1, -1), c["pole"])
    mags = ctx.stft_mag(audio, c["N"], c["hop"])
    ctx.sync()
    assert np.abs(audio.cpu().numpy()[0] - audio_o).max() < 1e-4
    assert mags.shape == (1, 256, 513)
    assert np.abs(mags.cpu().numpy()[0] - mags_o).max() < 1e-4 * np.abs(mags_o).max()


@pytest.mark.parametrize("B,T,L,mode", [(2, 3000, 5, 0.0), (1, 512, 130, 0.0), (2, 1025, 3, 1.0), (1, 700, 4, 2.0),
                                        (1, 2048, 6, 5.0), (3, 1, 2, 0.0)])
def test_biquad_forward_matches_oracle(ctx, B, T, L, mode):
    d = wl.biquad_bank_inputs(17, B=B, L=L, T=T)
    want = orc.biquad_bank(d["x"], d["cutoff"], d["q"], mode=mode)              # [B][L][T]
    got = ctx.biquad_fwd(dev(d["x"]), dev(d["cutoff"]), dev(d["q"]), mode=mode)  # [B][T][L]
    got = got.cpu().numpy().transpose(0, 2, 1)
    # scalar-vs-lane tolerance of the reference's own tests is 1e-4..1e-6 (TensorBiquadTests.swift:72-221)
    assert np.abs(got - want).max() < 1e-4 * max(1.0, np.abs(want).max())


@pytest.mark.parametrize("mode,gain", [(0.0, 0.7), (1.0, 1.0), (2.0, 1.3), (3.0, 1.0), (4.0, 1.0), (5.0, 0.5),
                                       (6.0, 2.0), (6.0, 0.4), (7.0, 2.0), (7.0, 0.25), (5.5, 1.5), (6.5, 1.5)])
def test_biquad_all_eight_modes_forward_and_gradients(ctx, mode, gain):
    """Graph.biquad documents eight filter types (Sources/DGen/HigherOps.swift:388-398): the shelves (6 high, 7 low)
    take their boost / cut from `gain` through A = sqrt(|gain|) and carry their own normalisation; a fractional
    mode follows the graph's selector and `>= 6` / `>= 7` switches literally.  Forward against the oracle's
    restatement of the coefficient graph, BPTT gradients against its fp64 evaluation."""
    B, T, L = 2, 3000, 12
    d = wl.biquad_bank_inputs(41, B=B, L=L, T=T)
    x, q = d["x"], d["q"]
    cut = np.exp(np.random.default_rng(7).uniform(np.log(400.0), np.log(8000.0), L)).astype(f32)
    want = orc.biquad_bank(x, cut, q, gain=gain, mode=mode)                                  # [B][L][T]
    y = ctx.biquad_fwd(dev(x), dev(cut), dev(q), gain=gain, mode=mode)
    got = y.cpu().numpy().transpose(0, 2, 1)
    assert np.abs(got - want).max() < 1e-4 * max(1.0, np.abs(want).max())
    target = orc.biquad_bank(x, cut * f32(1.05), q * f32(0.9), gain=gain, mode=mode)
    scale = 1.0 / (B * T)
    loss64, gc64, gq64 = orc.biquad_bank_mse_grad(x, cut, q, target, scale=scale, gain=gain, mode=mode)
    gc, gq, loss = ctx.biquad_mse_bwd(dev(x), dev(cut), dev(q), y, dev(target.transpose(0, 2, 1)), loss_scale=scale,
                                      gain=gain, mode=mode)
    assert abs(float(loss.cpu()[0]) - loss64) < 1e-3 * abs(loss64)
    assert np.abs(gc.cpu().numpy() - gc64).max() < 2e-3 * np.abs(gc64).max()
    assert np.abs(gq.cpu().numpy() - gq64).max() < 2e-3 * np.abs(gq64).max()


def test_biquad_mode_out_of_range_is_refused(ctx):
    d = wl.biquad_bank_inputs(3, B=1, L=2, T=64)
    with pytest.raises(dgen_b200.DgenCudaError):
        ctx.biquad_fwd(dev(d["x"]), dev(d["cutoff"]), dev(d["q"]), mode=8.0)


@pytest.mark.parametrize("B,L,cuts", [(2, 8, (700, 1300, 512)), (1, 130, (1024, 1024)), (2, 16, (1, 2, 3, 2048, 5)),
                                      (64, 1024, (1024, 512))])
def test_biquad_state_cells_continue_across_calls(ctx, B, L, cuts):
    """Consecutive calls over consecutive blocks with the history cells carried (preserveState,
    Sources/DGenLazy/Realize.swift:551-553) equal one call over the whole signal -- also across the tensor-core
    first pass (the last case), ragged blocks and blocks of one or two frames."""
    import torch
    T = int(sum(cuts))
    d = wl.biquad_bank_inputs(23, B=B, L=L, T=T)
    x, cut, q = dev(d["x"]), dev(d["cutoff"]), dev(d["q"])
    whole = ctx.biquad_fwd(x, cut, q)
    state = torch.zeros(B, 4, L, device="cuda")
    n0, parts = 0, []
    for n in cuts:
        parts.append(ctx.biquad_fwd(x[:, n0:n0 + n].contiguous(), cut, q, state=state))
        n0 += n
    got = torch.cat(parts, dim=1)
    scale = max(1.0, float(whole.abs().max()))
    # the two runs cut the signal into chunks at different places, so they round differently: 5e-5 covers the
    # recurrence's own rounding noise for the bank's sharpest lanes (50 Hz, Q 8) in single precision
    assert float((got - whole).abs().max()) <= 5e-5 * scale
    ctx.sync()
    st = state.cpu().numpy()
    w = whole.cpu().numpy()
    assert np.abs(st[:, 0] - w[:, T - 1]).max() <= 5e-5 * scale and np.abs(st[:, 1] - w[:, T - 2]).max() <= 5e-5 * scale
    assert np.array_equal(st[:, 2], np.repeat(d["x"][:, T - 1:T], L, axis=1))
    assert np.array_equal(st[:, 3], np.repeat(d["x"][:, T - 2:T - 1], L, axis=1))


def test_biquad_control_rate_coefficients_by_blocks(ctx):
    """Coefficients that change at control rate: one call per control block with that block's cutoff and Q, the
    history cells carried across -- against the reference recurrence with the coefficient graph evaluated per
    frame (Sources/DGen/HigherOps.swift:401-570) on piecewise-constant cutoff / Q."""
    import torch
    B, L, blocks, n = 1, 6, 5, 600
    T = blocks * n
    rng = np.random.default_rng(9)
    x = rng.standard_normal((B, T)).astype(f32)
    cuts = np.exp(rng.uniform(np.log(300.0), np.log(6000.0), (blocks, L))).astype(f32)
    qs = np.exp(rng.uniform(np.log(0.5), np.log(6.0), (blocks, L))).astype(f32)
    want = np.zeros((T, L), f32)
    for l in range(L):
        x1 = x2 = y1 = y2 = f32(0)
        for t in range(T):
            b0, b1, b2, a1, a2 = [f32(v) for v in orc.biquad_coef(cuts[t // n, l], qs[t // n, l], 1.0, 0.0)]
            x0 = x[0, t]
            v = f32(f32(f32(x2 * b2) + f32(x1 * b1)) + f32(x0 * b0)) - f32(f32(y2 * a2) + f32(y1 * a1))
            want[t, l] = v
            x2, x1, y2, y1 = x1, x0, y1, f32(v)
    state = torch.zeros(B, 4, L, device="cuda")
    parts = [ctx.biquad_fwd(dev(x[:, k * n:(k + 1) * n]), dev(cuts[k]), dev(qs[k]), state=state) for k in range(blocks)]
    got = torch.cat(parts, dim=1).cpu().numpy()[0]
    assert np.abs(got - want).max() <= 1e-4 * max(1.0, np.abs(want).max())


def test_onepole_state_cell_continues_across_calls(ctx):
    import torch
    B, cuts = 3, (5000, 1, 2047, 2049, 300)
    T = int(sum(cuts))
    x = torch.randn(B, T, device="cuda")
    whole = ctx.onepole_fwd(x, 0.97)
    state = torch.zeros(B, device="cuda")
    n0, parts = 0, []
    for n in cuts:
        parts.append(ctx.onepole_fwd(x[:, n0:n0 + n].contiguous(), 0.97, state=state))
        n0 += n
    got = torch.cat(parts, dim=1)
    assert float((got - whole).abs().max()) <= 1e-5 * max(1.0, float(whole.abs().max()))
    assert torch.equal(state, got[:, -1])


def test_biquad_lanes_are_independent(ctx):
    """Lane independence is exact (Tests/DGenLazyTests/TensorBiquadGradientTests.swift)."""
    d = wl.biquad_bank_inputs(3, B=2, L=8, T=2000)
    full = ctx.biquad_fwd(dev(d["x"]), dev(d["cutoff"]), dev(d["q"])).cpu().numpy()
    for l in (0, 5):
        one = ctx.biquad_fwd(dev(d["x"]), dev(d["cutoff"][l:l + 1]), dev(d["q"][l:l + 1])).cpu().numpy()
        assert np.array_equal(one[:, :, 0], full[:, :, l])


@pytest.mark.parametrize("B,T,L", [(2, 4000, 6), (1, 513, 3), (3, 1500, 40)])
def test_biquad_bptt_gradients_match_fp64_and_finite_differences(ctx, B, T, L):
    """Cutoffs from 400 Hz up: below that the reference's single-precision coefficient formula
    (1 - cos(w), Sources/DGen/HigherOps.swift:447-452) loses up to 3 digits by cancellation, so no
    single-precision evaluation of the graph can sit within 1e-3 of a double-precision one."""
    d = wl.biquad_bank_inputs(29, B=B, L=L, T=T)
    x, q = d["x"], d["q"]
    cut = np.exp(np.random.default_rng(L).uniform(np.log(400.0), np.log(8000.0), L)).astype(f32)
    target = orc.biquad_bank(x, cut * f32(1.05), q)                             # [B][L][T]
    scale = 1.0 / (B * T)
    loss64, gc64, gq64 = orc.biquad_bank_mse_grad(x, cut, q, target, scale=scale)
    y = ctx.biquad_fwd(dev(x), dev(cut), dev(q))
    gc, gq, loss = ctx.biquad_mse_bwd(dev(x), dev(cut), dev(q), y, dev(target.transpose(0, 2, 1)), loss_scale=scale)
    gc, gq, loss = gc.cpu().numpy(), gq.cpu().numpy(), float(loss.cpu()[0])
    own = ((y.cpu().numpy().astype(np.float64) - target.transpose(0, 2, 1)) ** 2).sum() * scale
    assert abs(loss - own) < 1e-5 * own                     # the reduction itself
    assert abs(loss - loss64) < 1e-3 * abs(loss64)
    # gradient tolerance of the path: 1e-3 relative to the fp64 evaluation
    assert np.abs(gc - gc64).max() < 1e-3 * np.abs(gc64).max()
    assert np.abs(gq - gq64).max() < 1e-3 * np.abs(gq64).max()
    # finite-difference check of the fp64 loss on one lane
    l = int(np.argmax(np.abs(gc64)))
    h = float(cut[l]) * 1e-5
    cp, cm = cut.astype(np.float64).copy(), cut.astype(np.float64).copy()
    cp[l] += h
    cm[l] -= h
    lp = ((orc.biquad_bank(x, cp, q, double=True) - target) ** 2).sum() * scale
    lm = ((orc.biquad_bank(x, cm, q, double=True) - target) ** 2).sum() * scale
    fd = (lp - lm) / (2 * h)
    assert abs(fd - gc[l]) < 2e-3 * abs(fd)


def test_biquad_bptt_full_cutoff_range_is_finite_and_close(ctx):
    """The biquad-bank configuration's own parameter range (50..8000 Hz, Q 0.5..8): gradients agree with
    the fp64 evaluation to the accuracy the single-precision coefficient formula allows."""
    d = wl.biquad_bank_inputs(20260002, B=2, L=64, T=8192)
    x, cut, q = d["x"], d["cutoff"], d["q"]
    target = orc.biquad_bank(x, cut * f32(1.05), q)
    scale = 1.0 / (2 * 8192)
    loss64, gc64, gq64 = orc.biquad_bank_mse_grad(x, cut, q, target, scale=scale)
    y = ctx.biquad_fwd(dev(x), dev(cut), dev(q))
    gc, gq, loss = ctx.biquad_mse_bwd(dev(x), dev(cut), dev(q), y, dev(target.transpose(0, 2, 1)), loss_scale=scale)
    gc, gq = gc.cpu().numpy(), gq.cpu().numpy()
    assert np.isfinite(gc).all() and np.isfinite(gq).all()
    assert abs(float(loss.cpu()[0]) - loss64) < 2e-2 * loss64
    ok = cut >= 400.0
    assert np.abs(gc - gc64)[ok].max() < 2e-3 * np.abs(gc64)[ok].max()
    assert np.abs(gq - gq64)[ok].max() < 2e-3 * np.abs(gq64)[ok].max()
    assert np.abs(gc - gc64).max() < 0.1 * np.abs(gc64).max()


@pytest.mark.parametrize("B,T,L", [(2, 4000, 6), (1, 513, 3), (2, 1500, 200)])
def test_biquad_backward_for_an_arbitrary_upstream_gradient(ctx, B, T, L):
    """dgc_biquad_bwd takes dL/dy of any loss.  With gy = 2 scale (y - target) it must reproduce the MSE entry point's
    coefficient gradients; dL/dx is the sum over lanes of the TRANSPOSED filters applied to gy, which for a filter
    started from rest is the same filter run on the time-reversed gradient (fp64 restatement), tolerance 1e-3."""
    d = wl.biquad_bank_inputs(31, B=B, L=L, T=T)
    x, q = d["x"], d["q"]
    cut = np.exp(np.random.default_rng(L + 1).uniform(np.log(400.0), np.log(8000.0), L)).astype(f32)
    target = orc.biquad_bank(x, cut * f32(1.05), q).transpose(0, 2, 1)          # [B][T][L]
    scale = 1.0 / (B * T)
    X, C_, Q_ = dev(x), dev(cut), dev(q)
    y = ctx.biquad_fwd(X, C_, Q_)
    gc0, gq0, _ = ctx.biquad_mse_bwd(X, C_, Q_, y, dev(target), loss_scale=scale)
    gy = (2.0 * scale) * (y - dev(target))
    gc, gq, gx = ctx.biquad_bwd(X, C_, Q_, y, gy)
    # (the two round g differently -- the MSE entry point forms 2 scale (y - t) inside the sweep -- and the sums over
    # frames cancel: compare against the largest gradient)
    assert float((gc - gc0).abs().max()) <= 1e-4 * float(gc0.abs().max())
    assert float((gq - gq0).abs().max()) <= 1e-4 * float(gq0.abs().max())
    gcn, gqn, none = ctx.biquad_bwd(X, C_, Q_, y, gy, want_grad_x=False)
    assert none is None and torch.equal(gcn, gc) and torch.equal(gqn, gq)
    g64 = gy.cpu().numpy().astype(np.float64)
    want = np.zeros((B, T))
    for b in range(B):
        for l in range(L):
            want[b] += orc.biquad(g64[b, ::-1, l].copy(), float(cut[l]), float(q[l]), double=True)[::-1]
    got = gx.cpu().numpy()
    assert np.abs(got - want).max() < 1e-3 * np.abs(want).max()
    # a second, unrelated upstream gradient: linear in gy
    rng = np.random.default_rng(5)
    g2 = dev(rng.standard_normal((B, T, L)).astype(f32))
    a_c, a_q, a_x = ctx.biquad_bwd(X, C_, Q_, y, g2)
    s_c, s_q, s_x = ctx.biquad_bwd(X, C_, Q_, y, gy + g2)
    assert torch.allclose(s_x, gx + a_x, rtol=0, atol=2e-5 * float(s_x.abs().max()))
    assert torch.allclose(s_c, gc + a_c, rtol=1e-3, atol=1e-6 * float(s_c.abs().max()))


@pytest.mark.parametrize("B,T,a", [(1, 1, 0.9), (3, 5000, 0.9), (2, 70001, 0.999), (4, 2048 * 3, -0.5)])
def test_onepole_backward(ctx, B, T, a):
    """lam[n] = gy[n] + a lam[n+1]: the forward scan on the time-reversed gradient (oracle), and
    dL/da = sum lam[n] y[n-1] against its fp64 value and a finite difference of the fp64 filter."""
    rng = np.random.default_rng(T)
    x = rng.standard_normal((B, T)).astype(f32)
    gy = rng.standard_normal((B, T)).astype(f32)
    y = ctx.onepole_fwd(dev(x), a)
    gx, ga = ctx.onepole_bwd(dev(gy), a, y=y)
    gx_only, none = ctx.onepole_bwd(dev(gy), a)
    assert none is None and torch.equal(gx_only, gx)
    got = gx.cpu().numpy()
    for b in range(B):
        want = orc.onepole(gy[b, ::-1].copy(), a)[::-1]
        assert np.abs(got[b] - want).max() <= 1e-5 * max(1.0, np.abs(want).max())
    y64 = np.stack([orc.onepole(x[b].astype(np.float64), a, double=True) for b in range(B)])
    lam64 = np.stack([orc.onepole(gy[b, ::-1].astype(np.float64).copy(), a, double=True)[::-1] for b in range(B)])
    ga64 = (lam64[:, 1:] * y64[:, :-1]).sum(axis=1)
    assert np.abs(ga.cpu().numpy() - ga64).max() <= 1e-3 * max(1e-6, np.abs(ga64).max())
    if T > 1:
        h = 1e-6
        f = lambda aa: sum((orc.onepole(x[b].astype(np.float64), aa, double=True) * gy[b]).sum() for b in range(B))
        fd = (f(a + h) - f(a - h)) / (2 * h)
        assert abs(fd - ga64.sum()) <= 1e-4 * max(1.0, abs(fd))
