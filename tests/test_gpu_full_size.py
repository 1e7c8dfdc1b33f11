"""The other configurations of the path at their FULL sizes, through properties that do not need the oracle to
run at that size: exact lane / voice independence against a small run of the same kernel (which the oracle
tests cover), linearity, time-shift invariance by a whole number of hops, and a slice against the oracle.

  biquad bank:       256 lanes x 32 voices x 262144 frames (8.6 GB of lane signals), forward and BPTT
  partitioned conv:  16 voices x 480000 frames, 96000-tap impulse response (94 partitions of 1024, N = 2048)
  oscillator bank -> one-pole -> FFT: 64 partials, 65536 frames (against the oracle directly, see test_gpu_linrec)
  forward + loss:    256 voices x 64000 frames x 100 partials on one GPU, the throughput target's own configuration
"""
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
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_biquad_bank_full_size_forward_and_bptt(ctx):
    d = wl.biquad_bank_inputs(20260002)              # B=32, L=256, T=262144
    B, L, T = d["B"], d["L"], d["T"]
    x, cut, q = dev(d["x"]), dev(d["cutoff"]), dev(d["q"])
    y = ctx.biquad_fwd(x, cut, q)                    # [B][T][L], 8.6 GB
    ctx.sync()
    assert y.shape == (B, T, L) and bool(torch.isfinite(y).all())
    # lane and voice independence is exact: 32 lanes of four voices, run alone over the full length (large enough
    # to take the same route as the full bank: chunk end states by the tensor-core product)
    lanes32, voices4 = list(range(3, 256, 8)), [0, 9, 22, 31]
    sub32 = ctx.biquad_fwd(x[voices4].contiguous(), cut[lanes32].contiguous(), q[lanes32].contiguous())
    ctx.sync()
    for i, b in enumerate(voices4):
        assert torch.equal(sub32[i], y[b][:, lanes32]), b
    del sub32
    # three lanes of two voices: a bank this small gets its chunk end states from the serial recurrence instead;
    # the two routes agree to rounding
    lanes, voices = [0, 131, 255], [0, 31]
    sub = ctx.biquad_fwd(x[voices].contiguous(), cut[lanes].contiguous(), q[lanes].contiguous())
    ctx.sync()
    for i, b in enumerate(voices):
        ref = y[b][:, lanes]
        assert float((sub[i] - ref).abs().max()) < 2e-5 * max(1.0, float(ref.abs().max())), b
    # the head of one voice against the oracle (the chunked scan must agree with the serial recurrence)
    want = orc.biquad_bank(d["x"][0:1, :6000], d["cutoff"][lanes], d["q"][lanes])[0].T   # [frames][lanes]
    got = sub[0, :6000].cpu().numpy()
    assert np.abs(got - want).max() < 1e-4 * max(1.0, np.abs(want).max())
    got_full = y[0, :6000][:, lanes].cpu().numpy()
    assert np.abs(got_full - want).max() < 1e-4 * max(1.0, np.abs(want).max())
    # the WHOLE length against the serial recurrence of the oracle, last chunk included, for lanes that span the
    # parameter range -- the lowest cutoff, the highest Q (poles closest to the unit circle: the double-precision
    # carry over 512 chunks is what keeps these right), the highest cutoff, the lowest Q, and two in between
    cn, qn = d["cutoff"], d["q"]
    span = sorted({int(np.argmin(cn)), int(np.argmax(qn)), int(np.argmax(cn)), int(np.argmin(qn)),
                   int(np.argmin(cn / qn)), 77, 200})
    want_full = orc.biquad_bank(d["x"][0:1], cn[span], qn[span])[0].T                      # [T][lanes]
    got_full = y[0][:, span].cpu().numpy()
    # The yardstick.  For poles this close to the unit circle (60 Hz, Q 7.7: radius 0.9994) the single-precision
    # recurrence carries its own rounding noise: run serially in fp32 it sits 1.7e-4 away from the exact response
    # of the very same fp32 coefficients (the recurrence in double).  Two fp32 evaluations that round in different
    # places cannot be asked to agree better than that, so each lane is held to: within 1e-4 of the serial fp32
    # recurrence, OR no farther from the exact response than the serial fp32 recurrence is itself (+ 20 %).
    exact = np.stack([orc.biquad_exact_response(d["x"][0], cn[l], qn[l]) for l in span], axis=1)   # [T][lanes] f64
    scale = np.maximum(1.0, np.abs(want_full).max(axis=0))
    err = np.abs(got_full - want_full).max(axis=0) / scale
    noise = np.abs(want_full - exact).max(axis=0) / scale
    err_exact = np.abs(got_full - exact).max(axis=0) / scale
    print("full-length biquad, lanes %s (cutoff %s, Q %s):\n  vs serial fp32 %s\n  serial fp32 vs exact %s\n  ours vs exact %s"
          % (span, np.round(cn[span], 1), np.round(qn[span], 2), err, noise, err_exact))
    assert ((err < 1e-4) | (err_exact < 1.2 * noise)).all(), (err, noise, err_exact)
    assert (err < 1e-4 + 2.0 * noise).all()
    tail = slice(T - 600, T)                                                                # the last chunk
    assert (np.abs(got_full[tail] - exact[tail]).max(axis=0) / scale < 1e-4 + 1.2 * noise).all()
    # BPTT over the whole length for those lanes (one voice) against the fp64 evaluation of the recurrence
    tspan = orc.biquad_bank(d["x"][0:1], cn[span] * f32(1.05), qn[span])                    # [1][lanes][T]
    l64, gc64, gq64 = orc.biquad_bank_mse_grad(d["x"][0:1], cn[span], qn[span], tspan, scale=1.0 / T)
    ys = ctx.biquad_fwd(x[0:1].contiguous(), dev(cn[span]), dev(qn[span]))
    g1, g2, l1 = ctx.biquad_mse_bwd(x[0:1].contiguous(), dev(cn[span]), dev(qn[span]), ys,
                                    dev(tspan.transpose(0, 2, 1)), loss_scale=1.0 / T)
    ctx.sync()
    g1, g2 = g1.cpu().numpy(), g2.cpu().numpy()
    # 1e-3 where the single-precision coefficient formula allows it (cutoff >= 400 Hz, see test_gpu_linrec.py)
    hi = cn[span] >= 400.0
    rel_c, rel_q = np.abs(g1 - gc64) / np.abs(gc64).max(), np.abs(g2 - gq64) / np.abs(gq64).max()
    print("full-length BPTT vs fp64: rel err cutoff %s, q %s" % (rel_c, rel_q))
    assert abs(float(l1.cpu()[0]) - l64) < 1e-3 * abs(l64)
    assert (rel_c[hi] < 1e-3).all() and (rel_q[hi] < 1e-3).all()
    assert (rel_c < 5e-2).all() and (rel_q < 5e-2).all()
    del ys
    # BPTT at full size: gradients of the lanes above equal those of the small bank run alone (per-lane sums over
    # voices and frames do not mix lanes), up to the split of the voice sum
    target = ctx.biquad_fwd(x, cut * 1.05, q)
    gc, gq, loss = ctx.biquad_mse_bwd(x, cut, q, y, target, loss_scale=1.0 / (B * T))
    tsub = ctx.biquad_fwd(x, (cut * 1.05)[lanes].contiguous(), q[lanes].contiguous())
    ysub = ctx.biquad_fwd(x, cut[lanes].contiguous(), q[lanes].contiguous())
    gcs, gqs, _ = ctx.biquad_mse_bwd(x, cut[lanes].contiguous(), q[lanes].contiguous(), ysub, tsub,
                                     loss_scale=1.0 / (B * T))
    ctx.sync()
    assert bool(torch.isfinite(gc).all()) and bool(torch.isfinite(gq).all()) and float(loss.cpu()[0]) > 0
    assert torch.allclose(gc[lanes], gcs, rtol=1e-4, atol=0) and torch.allclose(gq[lanes], gqs, rtol=1e-4, atol=0)
    del y, target


def test_partitioned_convolution_full_size_properties(ctx):
    d = wl.partconv_inputs(20260003)                 # V=16, T=480000, IR 96000, N=2048, hop=1024
    V, T, N, hop = d["V"], d["T"], d["N"], d["hop"]
    x, ir = dev(d["x"]), dev(d["ir"])
    y = ctx.partconv(x, ir, N, hop)
    ctx.sync()
    assert y.shape == (V, T) and bool(torch.isfinite(y).all())
    # voices are independent (exactly): two voices run alone
    ysub = ctx.partconv(x[[3, 15]].contiguous(), ir, N, hop)
    assert torch.equal(ysub[0], y[3]) and torch.equal(ysub[1], y[15])
    # linear in the input and in the impulse response
    x2 = torch.roll(x, 7, dims=0)
    ylin = ctx.partconv(x + 2.0 * x2, ir, N, hop)
    y2 = ctx.partconv(x2, ir, N, hop)
    scale = float(y.abs().max())
    assert float((ylin - (y + 2.0 * y2)).abs().max()) < 2e-5 * scale
    assert float((ctx.partconv(x, 0.5 * ir, N, hop) - 0.5 * y).abs().max()) < 1e-6 * scale
    # a delay of the input by a whole number of hops delays the output by the same amount
    shift = 3 * hop
    xs = torch.zeros_like(x)
    xs[:, shift:] = x[:, :-shift]
    ys = ctx.partconv(xs, ir, N, hop)
    ctx.sync()
    assert float((ys[:, shift:] - y[:, :-shift]).abs().max()) < 2e-5 * scale
    assert float(ys[:, :shift - N].abs().max()) == 0.0     # nothing before the delayed input reaches a window
    # head of one voice against the oracle (94 partitions in play after 96000 frames: take 1.2 s)
    want = orc.partitioned_convolve(d["x"][3, :57600], d["ir"], N, hop)
    got = ctx.partconv(x[3:4, :57600].contiguous(), ir, N, hop).cpu().numpy()[0]
    assert np.abs(got - want).max() < 1e-4 * max(1.0, np.abs(want).max())


def test_onepole_long_signals(ctx):
    """64 voices x 1 Mi frames (256 MB, twice L2; 512 chunks per voice carried in sequence) against the serial
    recurrence of the oracle on a few voices, and a ragged length that leaves a partial last chunk."""
    rng = np.random.default_rng(12)
    for B, T, a in [(64, 1 << 20, 0.9), (48, (1 << 20) - 777, 0.999)]:
        x = rng.standard_normal((B, T)).astype(f32)
        y = ctx.onepole_fwd(dev(x), a).cpu().numpy()
        for b in (0, B // 2, B - 1):
            want = orc.onepole(x[b], a)
            assert np.abs(y[b] - want).max() <= 1e-4 * max(1.0, np.abs(want).max()), (B, T, b)


def test_forward_loss_256_voices_against_16_voice_runs_and_the_oracle(ctx):
    """The throughput target's configuration, 256 voices x 64000 frames through ONE composite call, checked by
    properties and slices.  At this size the step takes other code paths than at 16 voices (the band -> tap map on
    the tensor-core matmul instead of the tile kernel, the FIR after the render on one stream adding into its output
    instead of beside it with a summing pass, the 80-register FIR build), so:
      * voice independence: the audio of voices 32..47 and 240..255 inside the 256-voice step equals a 16-voice
        step over those voices alone to single-precision accumulation differences (the 3xTF32 map);
      * the loss is a mean over voices: the 256-voice loss equals the mean of the sixteen 16-voice losses;
      * two voices of the 256-voice audio against the CPU oracle (the same bound as the 2-voice test);
      * the same call twice gives bit-identical audio and loss."""
    B, T, K, F, NB, NT, sr = 256, 64000, 100, 1000, 65, 257, 16000.0
    d = wl.harmonic_noise_inputs(4242, B=B, T=T, K=K, F=F, sr=sr, nbands=NB, taps=NT)
    rng = np.random.default_rng(9)
    target = (rng.standard_normal((B, T)) * 0.1).astype(f32)

    def step_for(b):
        st = dgen_b200.HnStep()
        st.harm = dgen_b200.HarmonicParams(b, T, K, F, sr, 1.0, dgen_b200.PHASE_FUNDAMENTAL, 0)
        st.fir = dgen_b200.FirParams(b, T, F, NT, 0.12, 1)
        st.mss = dgen_b200.mss_params(b, T)
        st.nbands = NB
        return st

    def run(sl):
        n = sl.stop - sl.start
        args = [dev(d[k][:, sl]) for k in ("f0", "uv", "amps", "gain", "noise_gain", "bands")]
        out = torch.empty(n, T, device="cuda")
        loss, _ = ctx.hn_forward_loss(step_for(n), *args, dev(d["W"]), dev(d["noise"][sl]), dev(target[sl]), audio=out)
        ctx.sync()
        return out, float(loss.cpu()[0])

    full, loss_full = run(slice(0, B))
    again, loss_again = run(slice(0, B))
    assert torch.equal(full, again) and loss_full == loss_again
    losses = []
    for c in range(B // 16):
        sl = slice(16 * c, 16 * c + 16)
        part, l = run(sl)
        losses.append(l)
        if c in (2, 15):
            err = float((part - full[sl]).abs().max())
            assert err < 5e-6, (c, err)
    assert abs(np.mean(losses) - loss_full) < 1e-6 * abs(loss_full)
    taps = wl.taps_from_bands({k: (v[:, 100:102] if k == "bands" else v) for k, v in d.items()})
    want = orc.harmonic_noise_render(d["f0"][:, 100:102], d["uv"][:, 100:102], d["amps"][:, 100:102],
                                     d["gain"][:, 100:102], d["noise_gain"][:, 100:102], taps, d["noise"][100:102], T, sr)
    got = full[100:102].cpu().numpy()
    assert np.abs(got - want).max() < 1e-4
