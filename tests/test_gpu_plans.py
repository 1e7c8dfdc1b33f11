"""Block plans through the C ABI (dgc_plan_run): the configurations of the path written as the ordered block lists a
host's matcher would hand over -- recognised primitives and generated blocks over ONE arena, every buffer an offset
-- and checked against the CPU oracle and against the same primitives called one by one.  The training step
(the fifth configuration) is a plan too: dgc_hn_train_plan, exercised by tests/test_gpu_train_step.py."""
import ctypes as C

import numpy as np
import pytest
import torch

import dgen_b200
from dgen_b200 import (PLAN_ADD, PLAN_BANDS_TO_TAPS, PLAN_BIQUAD_FWD, PLAN_BIQUAD_MSE_BWD, PLAN_BLOCK, PLAN_FIR_NOISE,
                       PLAN_FORK, PLAN_HARMONIC_RENDER, PLAN_JOIN, PLAN_MSS_LOSS_FWD, PLAN_ONEPOLE, PLAN_OSC_BANK_CONST,
                       PLAN_PARTCONV, PLAN_SANITIZE, PLAN_STFT_MAG, Plan, PlanStep, plan_step)
from dgen_b200 import workloads as wl
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
f32 = np.float32


@pytest.fixture(scope="module")
def ctx():
    c = dgen_b200.Context(0)
    yield c
    c.close()


class Arena:
    """A dgc_arena with a bump allocator for the test's buffers (256-byte aligned, like a cell allocator would)."""

    def __init__(self, ctx, nfloats):
        self.ctx, self.used, self.n = ctx, 0, nfloats
        self.h = C.c_void_p()
        ctx.check(ctx.lib.dgc_arena_create(ctx.h, nfloats, C.byref(self.h)))

    def take(self, n):
        off = self.used
        self.used += (int(n) + 63) & ~63
        assert self.used <= self.n
        return off

    def put(self, array):
        a = np.ascontiguousarray(array, f32).reshape(-1)
        off = self.take(a.size)
        self.ctx.check(self.ctx.lib.dgc_arena_upload(self.h, off, a.ctypes.data_as(C.c_void_p), a.size))
        return off

    def get(self, off, shape, dtype=f32):
        n = int(np.prod(shape)) * (2 if dtype == np.float64 else 1)
        out = np.empty(n, f32)
        self.ctx.check(self.ctx.lib.dgc_arena_download(self.h, off, out.ctypes.data_as(C.c_void_p), n))
        return out.view(dtype).reshape(shape)

    def run(self, steps, modules=None, kernels=None, first=0, count=-1):
        arr = (PlanStep * len(steps))(*steps)
        mods = (C.c_void_p * len(modules))(*[m.h for m in modules]) if modules else None
        names = (C.c_char_p * len(kernels))(*[k.encode() for k in kernels]) if kernels else None
        plan = Plan(arr, len(steps), mods, names, len(kernels) if kernels else 0)
        self.keep = (arr, mods, names, plan)
        self.ctx.check(self.ctx.lib.dgc_plan_run(self.ctx.h, self.h, C.byref(plan), first, count))
        return plan

    def close(self):
        self.ctx.lib.dgc_arena_destroy(self.h)


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def test_oscillator_filter_fft_configuration_as_a_plan(ctx):
    """64 partials -> one-pole -> buffer(1024, hop 256) -> FFT magnitudes: three blocks, one arena."""
    c = wl.osc_filter_fft_inputs(T=16384)
    K, T, N, hop = c["K"], c["T"], c["N"], c["hop"]
    H = (T + hop - 1) // hop
    ar = Arena(ctx, 1 << 20)
    freq, amp = ar.put(c["freq"]), ar.put(c["amp"])
    osc, y, mags = ar.take(T), ar.take(T), ar.take(H * (N // 2 + 1))
    ar.run([plan_step(PLAN_OSC_BANK_CONST, a=(freq, amp, osc), i=(K, T, dgen_b200.PHASE_DETERMINISTIC), f=(c["sr"],)),
            plan_step(PLAN_ONEPOLE, a=(osc, y, None), i=(1, T), f=(c["pole"],)),
            plan_step(PLAN_STFT_MAG, a=(y, None, mags), i=(1, T, N, hop))])
    ctx.sync()
    want_osc = orc.osc_bank_const(c["freq"], c["amp"], T, c["sr"], stateful=False)
    want_y = orc.onepole(want_osc, c["pole"])
    want_m = orc.buffer_fft_mag(want_y, N, hop)
    assert np.abs(ar.get(y, (T,)) - want_y).max() < 1e-4
    got_m = ar.get(mags, (H, N // 2 + 1))
    assert np.abs(got_m - want_m).max() < 1e-4 * np.abs(want_m).max()
    ar.close()


def test_harmonic_noise_loss_configuration_as_a_plan(ctx):
    """Noise branch on the side stream beside the harmonic branch, joined, summed, scored: the loss equals the
    library's composite entry point bit for bit and the oracle within the path's tolerance."""
    B, T, K, F, NB, NT = 3, 9000, 40, 70, 9, 33
    sizes = (512, 128, 64)
    d = wl.harmonic_noise_inputs(61, B=B, T=T, K=K, F=F, nbands=NB, taps=NT)
    target = (np.random.default_rng(2).standard_normal((B, T)) * 0.1).astype(f32)
    ar = Arena(ctx, 1 << 22)
    o = {k: ar.put(d[k]) for k in ("f0", "uv", "amps", "gain", "noise_gain", "bands", "W", "noise")}
    tg = ar.put(target)
    taps, harm, noise_out, loss = ar.take(F * B * NT), ar.take(B * T), ar.take(B * T), ar.take(2)
    mss_i = (B, T, len(sizes), 4) + sizes
    steps = [plan_step(PLAN_FORK),
             plan_step(PLAN_BANDS_TO_TAPS, a=(o["bands"], o["W"], taps), i=(F * B, NB, NT), stream=1),
             plan_step(PLAN_FIR_NOISE, a=(o["noise"], taps, o["noise_gain"], noise_out), i=(B, T, F, NT, 0), f=(0.12,),
                       stream=1),
             plan_step(PLAN_HARMONIC_RENDER, a=(o["f0"], o["uv"], o["amps"], o["gain"], None, harm),
                       i=(B, T, K, F, dgen_b200.PHASE_SCAN, 0), f=(d["sr"], 1.0)),
             plan_step(PLAN_JOIN),
             plan_step(PLAN_ADD, a=(harm, noise_out, harm, B * T)),
             plan_step(PLAN_MSS_LOSS_FWD, a=(harm, tg, None, loss), i=mss_i, f=(1.0, 1.0))]
    for _ in range(2):
        ar.run(steps)
    ctx.sync()
    got_loss = float(ar.get(loss, (1,), np.float64)[0])
    st = dgen_b200.HnStep()
    st.harm = dgen_b200.HarmonicParams(B, T, K, F, d["sr"], 1.0, dgen_b200.PHASE_SCAN, 0)
    st.fir = dgen_b200.FirParams(B, T, F, NT, 0.12, 1)
    st.mss = dgen_b200.mss_params(B, T, sizes)
    st.nbands = NB
    D = {k: dev(d[k]) for k in ("f0", "uv", "amps", "gain", "noise_gain", "bands", "W", "noise")}
    comp, _ = ctx.hn_forward_loss(st, D["f0"], D["uv"], D["amps"], D["gain"], D["noise_gain"], D["bands"], D["W"], D["noise"],
                                  dev(target))
    ctx.sync()
    assert got_loss == float(comp.cpu()[0])
    audio = ar.get(harm, (B, T))
    want = orc.harmonic_noise_render(d["f0"], d["uv"], d["amps"], d["gain"], d["noise_gain"], wl.taps_from_bands(d),
                                     d["noise"], T, d["sr"])
    assert np.abs(audio - want).max() < 1e-4
    want_loss = orc.mss_loss(audio, target, sizes=sizes)
    assert abs(got_loss - want_loss) < 1e-4 * abs(want_loss)
    ar.close()


def test_biquad_bank_and_partitioned_convolution_as_plans(ctx):
    B, L, T = 2, 16, 3000
    d = wl.biquad_bank_inputs(17, B=B, L=L, T=T)
    ar = Arena(ctx, 1 << 22)
    x, cut, q = ar.put(d["x"]), ar.put(d["cutoff"]), ar.put(d["q"])
    target_np = orc.biquad_bank(d["x"], d["cutoff"] * f32(1.05), d["q"]).transpose(0, 2, 1)
    tg = ar.put(target_np)
    y, gc, gq, loss = ar.take(B * T * L), ar.take(L), ar.take(L), ar.take(2)
    scale = 1.0 / (B * T)
    ar.run([plan_step(PLAN_BIQUAD_FWD, a=(x, cut, q, None, None, y), i=(B, T, L), f=(1.0, 0.0)),
            plan_step(PLAN_BIQUAD_MSE_BWD, a=(x, cut, q, y, tg, None, gc, gq, loss), i=(B, T, L), f=(1.0, 0.0, scale))])
    ctx.sync()
    want = orc.biquad_bank(d["x"], d["cutoff"], d["q"]).transpose(0, 2, 1)
    assert np.abs(ar.get(y, (B, T, L)) - want).max() < 1e-4 * max(1.0, np.abs(want).max())
    yd = ctx.biquad_fwd(dev(d["x"]), dev(d["cutoff"]), dev(d["q"]))
    g1, g2, l1 = ctx.biquad_mse_bwd(dev(d["x"]), dev(d["cutoff"]), dev(d["q"]), yd, dev(target_np), loss_scale=scale)
    assert np.array_equal(ar.get(gc, (L,)), g1.cpu().numpy()) and np.array_equal(ar.get(gq, (L,)), g2.cpu().numpy())
    assert float(ar.get(loss, (1,), np.float64)[0]) == float(l1.cpu()[0])
    # partitioned convolution, wet added to a buffer that holds the dry signal
    V, Tc, irl, N, hop = 2, 6000, 700, 256, 128
    rng = np.random.default_rng(4)
    xs, ir = rng.standard_normal((V, Tc)).astype(f32), (rng.standard_normal(irl) * np.exp(-np.arange(irl) / 150.0)).astype(f32)
    px, pir, out = ar.put(xs), ar.put(ir), ar.put(xs)
    ar.run([plan_step(PLAN_PARTCONV, a=(px, pir, None, out), i=(V, Tc, irl, N, hop, 1), f=(1.0,))])
    ctx.sync()
    want = xs + np.stack([orc.partitioned_convolve(xs[v], ir, N, hop) for v in range(V)])
    assert np.abs(ar.get(out, (V, Tc)) - want).max() < 1e-4 * max(1.0, np.abs(want).max())
    ar.close()


def test_generated_blocks_between_primitives(ctx):
    """A leftover elementwise block (gain and soft clip, emitted from an op list and compiled in process) between two
    primitives, and a sequential block with a state cell after them: oscillator -> y = tanh(2 x) -> one-pole ->
    feedback block z[n] = y[n] + 0.5 z[n-1] written as history read / write ops."""
    c = wl.osc_filter_fft_inputs(T=4096, K=8)
    K, T = c["K"], c["T"]
    ar = Arena(ctx, 1 << 18)
    freq, amp = ar.put(c["freq"]), ar.put(c["amp"] * f32(0.3))
    osc, shaped, y, cell, z = ar.take(T), ar.take(T), ar.take(T), ar.put(np.zeros(1, f32)), ar.take(T)
    elementwise = [("LOAD", osc), ("CONST", 0, 0, 0, 2.0), ("MUL", 0, 1), ("TANH", 2), ("STORE", shaped, 3)]
    sequential = [("HISTORY_READ", cell), ("CONST", 0, 0, 0, 0.5), ("MUL", 0, 1), ("LOAD", y), ("ADD", 3, 2),
                  ("HISTORY_WRITE", cell, 4), ("STORE_FRAME_LANE", z, 5)]
    m1 = ctx.compile_block(elementwise, name="blk_shape")
    m2 = ctx.compile_block(sequential, name="blk_feedback", sequential=True)
    steps = [plan_step(PLAN_OSC_BANK_CONST, a=(freq, amp, osc), i=(K, T, dgen_b200.PHASE_DETERMINISTIC), f=(c["sr"],)),
             plan_step(PLAN_BLOCK, i=(0, 0, T, 0)),
             plan_step(PLAN_ONEPOLE, a=(shaped, y, None), i=(1, T), f=(0.5,)),
             plan_step(PLAN_BLOCK, i=(1, 1, T, 1)),
             plan_step(PLAN_SANITIZE, a=(z, z, T))]
    ar.run(steps, modules=[m1, m2], kernels=["blk_shape", "blk_feedback"])
    ctx.sync()
    want_osc = orc.osc_bank_const(c["freq"], c["amp"] * f32(0.3), T, c["sr"], stateful=False)
    want_shaped = np.tanh(f32(2.0) * want_osc).astype(f32)
    want_y = orc.onepole(want_shaped, 0.5)
    want_z = orc.onepole(want_y, 0.5)
    assert np.abs(ar.get(shaped, (T,)) - want_shaped).max() < 1e-4
    assert np.abs(ar.get(z, (T,)) - want_z).max() < 1e-4
    assert abs(float(ar.get(cell, (1,))[0]) - float(want_z[-1])) < 1e-4      # the state cell holds the last output
    m1.close()
    m2.close()
    ar.close()


def test_plan_errors_name_the_step_and_launch_nothing_after_it(ctx):
    ar = Arena(ctx, 4096)
    x, y = ar.take(1024), ar.take(1024)
    good = plan_step(PLAN_ONEPOLE, a=(x, y, None), i=(1, 1024), f=(0.5,))
    beyond = plan_step(PLAN_ONEPOLE, a=(x, 4000, None), i=(1, 1024), f=(0.5,))
    before = ctx.launch_count()
    with pytest.raises(dgen_b200.DgenCudaError, match="step 1.*beyond the arena"):
        ar.run([good, beyond, good])
    assert ctx.launch_count() - before == 3                       # only step 0 (three kernels) was enqueued
    with pytest.raises(dgen_b200.DgenCudaError, match="step 0.*before a FORK"):
        ar.run([plan_step(PLAN_ONEPOLE, a=(x, y, None), i=(1, 1024), f=(0.5,), stream=1)])
    with pytest.raises(dgen_b200.DgenCudaError, match="step 0.*unknown op"):
        ar.run([plan_step(99)])
    with pytest.raises(dgen_b200.DgenCudaError, match="step 0.*no generated kernel"):
        ar.run([plan_step(PLAN_BLOCK, i=(0, 0, 16, 0))])
    with pytest.raises(dgen_b200.DgenCudaError, match="step 0.*required buffer"):
        ar.run([plan_step(PLAN_ONEPOLE, a=(x, None, None), i=(1, 1024), f=(0.5,))])
    ar.run([good])                                                # the context and the arena still work
    ctx.sync()
    ar.close()


def test_a_plan_is_recorded_once_and_replayed(ctx):
    T = 8192
    ar = Arena(ctx, 1 << 16)
    x, y, z = ar.put(np.random.default_rng(0).standard_normal(T).astype(f32)), ar.take(T), ar.take(T)
    steps = [plan_step(PLAN_ONEPOLE, a=(x, y, None), i=(1, T), f=(0.9,)),
             plan_step(PLAN_ONEPOLE, a=(y, z, None), i=(1, T), f=(-0.5,))]
    ar.run(steps)
    ctx.sync()
    want = ar.get(z, (T,)).copy()
    stream = torch.cuda.Stream()
    with ctx.on_stream(stream), torch.cuda.stream(stream):
        with ctx.record() as rec:
            ar.run(steps)
        ctx.check(ctx.lib.dgc_arena_zero(ar.h))                   # wipes x, y, z ...
        new_x = np.random.default_rng(1).standard_normal(T).astype(f32)
        ctx.check(ctx.lib.dgc_arena_upload(ar.h, x, new_x.ctypes.data_as(C.c_void_p), T))
        rec.graph.launch()
        stream.synchronize()
        got = ar.get(z, (T,))
        rec.graph.close()
    assert np.abs(got - orc.onepole(orc.onepole(new_x, 0.9), -0.5)).max() < 1e-4
    assert not np.array_equal(got, want)
    ar.close()
