"""Generated elementwise blocks through the C ABI: CUDA C as a renderer would emit it for a block that no
primitive covers is compiled in process (dgc_module_compile), launched over device memory (dgc_launch) and
checked against numpy; the image path (dgc_module_load) takes the committed PTX of the same kind of block."""
import ctypes as C
import os

import numpy as np
import pytest
import torch

import dgen_b200

pytestmark = pytest.mark.gpu
f32 = np.float32
HERE = os.path.dirname(os.path.abspath(__file__))

# what the C renderer writes as a frame loop over arena cells (Sources/DGen/Renderer/CRenderer.swift:479-1307),
# with the loop replaced by the thread index: out = tanh(a * gain + b), then the output sanitiser
BLOCK_SRC = r"""
extern "C" __global__ void dgen_block_7(float *memory, int a_off, int b_off, int out_off, float gain, int frameCount) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= frameCount) return;
  float t1 = memory[a_off + i], t2 = memory[b_off + i];
  float t3 = tanhf(t1 * gain + t2);
  unsigned bits = __float_as_uint(t3);
  memory[out_off + i] = ((bits & 0x7f800000u) == 0x7f800000u) ? 0.0f : t3;
}
extern "C" __global__ void dgen_block_8(const float *x, float *y, int n) {
  int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) y[i] = x[i] * x[i];
}
"""


@pytest.fixture(scope="module")
def ctx():
    c = dgen_b200.Context(0)
    yield c
    c.close()


def test_compiled_block_runs_over_an_arena(ctx):
    n = 100003
    rng = np.random.default_rng(1)
    a, b = rng.standard_normal(n).astype(f32), rng.standard_normal(n).astype(f32)
    a[5] = np.inf
    b[5] = -np.inf          # inf - inf -> NaN -> sanitised to 0
    mem = torch.zeros(3 * n, device="cuda")
    mem[:n] = torch.from_numpy(a).cuda()
    mem[n:2 * n] = torch.from_numpy(b).cuda()
    m = ctx.compile_module(BLOCK_SRC)
    m.launch("dgen_block_7", (n + 255) // 256, 256, [mem, C.c_int(0), C.c_int(n), C.c_int(2 * n), C.c_float(0.5), C.c_int(n)])
    ctx.sync()
    got = mem[2 * n:].cpu().numpy()
    with np.errstate(invalid="ignore"):
        want = np.tanh((a * f32(0.5) + b).astype(np.float64))
    want[~np.isfinite(want)] = 0.0
    assert np.abs(got - want).max() < 2e-6
    assert got[5] == 0.0
    # a second kernel of the same module, torch tensors as plain pointers
    x = torch.arange(1000, device="cuda", dtype=torch.float32)
    y = torch.empty_like(x)
    m.launch("dgen_block_8", 4, 256, [x, y, C.c_int(1000)])
    ctx.sync()
    assert torch.equal(y, x * x)
    m.close()


def test_errors_are_reported_not_thrown_across_the_abi(ctx):
    with pytest.raises(dgen_b200.DgenCudaError, match="does not compile"):
        ctx.compile_module("extern \"C\" __global__ void k(float *x) { x[0] = undefined_symbol; }")
    m = ctx.compile_module(BLOCK_SRC)
    with pytest.raises(dgen_b200.DgenCudaError, match="no kernel"):
        m.launch("not_there", 1, 32, [C.c_int(0)])
    m.close()
    with pytest.raises(dgen_b200.DgenCudaError, match="dgc_module_load"):
        ctx.load_module(b"this is not device code\0")
    # the context is still usable after the refused calls
    t = torch.ones(8, device="cuda")
    ctx.sanitize(t)
    ctx.sync()


def test_ptx_image_path(ctx):
    """dgc_module_load on PTX text (tests/golden/scale_block_sm100a.ptx, made from scale_block.cu by
    tests/golden/make_ptx.sh)."""
    ptx = open(os.path.join(HERE, "golden", "scale_block_sm100a.ptx")).read()
    m = ctx.load_module(ptx)
    x = torch.linspace(-1, 1, 4097, device="cuda")
    y = torch.empty_like(x)
    m.launch("dgen_scale_block", (4097 + 127) // 128, 128, [x, y, C.c_float(3.0), C.c_int(4097)])
    ctx.sync()
    assert torch.equal(y, x * 3.0)
    m.close()


# ---- op lists -> emitted CUDA C -> NVRTC -> launch, against a numpy interpreter of the same ops ----------------
def interpret(ops, mem, count):
    """float32 evaluation of an op list with the emitter's semantics (one rounding per operation)."""
    f = np.float32
    mem = mem.copy()
    i = np.arange(count)
    v = []
    with np.errstate(all="ignore"):
        for o in ops:
            o = tuple(o) + (0,) * (5 - len(o))
            op, a, b, c, imm = o
            A = v[a] if op not in ("CONST", "LOAD", "LOAD_SCALAR", "FRAME_INDEX", "STORE", "OUTPUT") else None
            B = v[b] if op in ("ADD", "SUB", "MUL", "DIV", "MOD", "POW", "MIN", "MAX", "ATAN2", "AND", "OR", "XOR", "GT",
                               "GTE", "LTE", "LT", "EQ", "GSWITCH", "STORE", "OUTPUT") else None
            one = lambda m: np.where(m, f(1), f(0)).astype(f)
            r = {
                "CONST": lambda: np.full(count, f(imm), f), "LOAD": lambda: mem[a + i], "LOAD_SCALAR": lambda: np.full(count, mem[a], f),
                "FRAME_INDEX": lambda: i.astype(f), "ADD": lambda: A + B, "SUB": lambda: A - B, "MUL": lambda: A * B,
                "DIV": lambda: A / B, "MOD": lambda: np.fmod(A, B), "POW": lambda: np.power(A, B), "MIN": lambda: np.fmin(A, B),
                "MAX": lambda: np.fmax(A, B), "ATAN2": lambda: np.arctan2(A, B), "AND": lambda: one((A != 0) & (B != 0)),
                "OR": lambda: one((A != 0) | (B != 0)), "XOR": lambda: one((A != 0) ^ (B != 0)), "GT": lambda: one(A > B),
                "GTE": lambda: one(A >= B), "LTE": lambda: one(A <= B), "LT": lambda: one(A < B), "EQ": lambda: one(A == B),
                "ABS": lambda: np.abs(A), "SIGN": lambda: np.sign(A), "FLOOR": lambda: np.floor(A), "CEIL": lambda: np.ceil(A),
                "ROUND": lambda: np.where(A >= 0, np.floor(A + f(0.5)), np.ceil(A - f(0.5))), "SIN": lambda: np.sin(A),
                "COS": lambda: np.cos(A), "TAN": lambda: np.tan(A), "ATAN": lambda: np.arctan(A), "TANH": lambda: np.tanh(A),
                "EXP": lambda: np.exp(A), "LOG": lambda: np.log(A), "LOG10": lambda: np.log10(A), "SQRT": lambda: np.sqrt(A),
                "GSWITCH": lambda: np.where(v[a] > 0, v[b], v[c]), "STORE": lambda: B, "OUTPUT": lambda: np.where(np.isfinite(B), B, f(0)),
            }[op]().astype(f)
            if op in ("STORE", "OUTPUT"):
                mem[a + i] = r
            v.append(r)
    return mem


def test_emitted_block_matches_a_float32_interpreter(ctx):
    n = 5000
    rng = np.random.default_rng(11)
    mem = np.zeros(4 * n + 8, f32)
    mem[:n] = rng.standard_normal(n)
    mem[n:2 * n] = rng.uniform(0.1, 4.0, n)
    mem[4 * n] = 0.75
    ops = [("LOAD", 0), ("LOAD", n), ("LOAD_SCALAR", 4 * n), ("CONST", 0, 0, 0, 0.5), ("CONST", 0, 0, 0, 2.0),
           ("MUL", 0, 2), ("ADD", 5, 1), ("TANH", 6), ("SIN", 0), ("COS", 1), ("MUL", 8, 9), ("SUB", 10, 7),
           ("ABS", 11), ("SQRT", 12), ("LOG", 1), ("EXP", 8), ("DIV", 15, 1), ("POW", 1, 4), ("POW", 1, 3),
           ("MIN", 16, 17), ("MAX", 19, 18), ("FLOOR", 0), ("CEIL", 0), ("GT", 0, 3), ("LTE", 0, 3), ("AND", 23, 24),
           ("OR", 23, 24), ("XOR", 23, 24), ("GSWITCH", 0, 13, 14), ("ATAN2", 0, 1), ("SIGN", 0), ("ATAN", 0),
           ("MOD", 1, 3), ("ADD", 28, 29), ("ADD", 33, 32), ("ADD", 34, 20), ("STORE", 2 * n, 35),
           ("DIV", 0, 21), ("OUTPUT", 3 * n, 37), ("FRAME_INDEX",), ("EQ", 39, 21), ("LOG10", 1), ("ROUND", 0), ("TAN", 31)]
    want = interpret(ops, mem, n)
    d = torch.from_numpy(mem).cuda()
    m = ctx.compile_block(ops, "blk")
    m.launch("blk", (n + 255) // 256, 256, [d, C.c_int(n)])
    ctx.sync()
    got = d.cpu().numpy()
    # +, -, *, / round identically; the library transcendentals differ from numpy's by a few ulp, and the
    # compiler may contract a * b + c (as the reference's own build does)
    err = np.abs(got - want) / np.maximum(1.0, np.abs(want))
    assert np.isfinite(got[3 * n:4 * n]).all()          # x / floor(x) hits 0 / 0 and x / 0: sanitised at the output
    assert err.max() < 5e-6, (err.max(), np.argmax(err))
    m.close()


# ---- blocks with state cells: one thread per lane, the frame loop inside ------------------------------------------
def test_sequential_block_history_feedback_against_the_one_pole_restatement(ctx):
    """y = x + 0.9 * y1 (Sources/DGenLazy/Signal.swift:265-278 one-pole through historyRead / historyWrite), a lane
    per voice; the state cell continues across two launches."""
    from oracle import oracle as orc
    frames, lanes = 3000, 37
    rng = np.random.default_rng(3)
    x = rng.standard_normal((frames, lanes)).astype(f32)
    X, S, Y = 0, frames * lanes, frames * lanes + lanes
    ops = [("LOAD_FRAME_LANE", X), ("HISTORY_READ", S), ("CONST", 0, 0, 0, 0.9), ("MUL", 1, 2), ("ADD", 0, 3),
           ("HISTORY_WRITE", S, 4), ("STORE_FRAME_LANE", Y, 5)]
    m = ctx.compile_block(ops, "onepole_block", sequential=True)
    mem = torch.zeros(2 * frames * lanes + lanes, device="cuda")
    mem[:frames * lanes] = torch.from_numpy(x.reshape(-1)).cuda()
    half = frames // 2
    # first half, then the second half continuing from the stored state (the frame-lane cells are offset by hand)
    m.launch("onepole_block", (lanes + 63) // 64, 64, [mem, C.c_int(half), C.c_int(lanes)])
    ops2 = [("LOAD_FRAME_LANE", X + half * lanes)] + ops[1:6] + [("STORE_FRAME_LANE", Y + half * lanes, 5)]
    m2 = ctx.compile_block(ops2, "onepole_block_b", sequential=True)
    m2.launch("onepole_block_b", (lanes + 63) // 64, 64, [mem, C.c_int(frames - half), C.c_int(lanes)])
    ctx.sync()
    got = mem[Y:Y + frames * lanes].cpu().numpy().reshape(frames, lanes)
    for l in (0, 17, 36):
        want = orc.onepole(x[:, l], 0.9)
        assert np.abs(got[:, l] - want).max() <= 2e-6 * np.abs(want).max()
    assert np.array_equal(mem[S:S + lanes].cpu().numpy(), got[-1])      # the cell holds the last output
    m.close()
    m2.close()


def test_sequential_block_nonlinear_feedback_phasor_and_latch(ctx):
    """A graph no primitive covers: per-lane phasor -> sine, fed through a saturating feedback loop, sampled and held
    on a shared trigger.  Against a frame-by-frame float32 evaluation of the same ops."""
    frames, lanes, sr = 2000, 50, 44100.0
    rng = np.random.default_rng(4)
    freq = rng.uniform(50.0, 5000.0, lanes).astype(f32)
    drive = rng.uniform(0.5, 3.0, lanes).astype(f32)
    trig = (rng.random(frames) < 0.01).astype(f32)
    reset = np.zeros(frames, f32)
    reset[700] = 1.0
    TRIG, RESET, FREQ, DRIVE = 0, frames, 2 * frames, 2 * frames + lanes
    PH, FB, HOLD = DRIVE + lanes, DRIVE + 2 * lanes, DRIVE + 3 * lanes
    OUT_A = HOLD + lanes
    OUT_B = OUT_A + frames * lanes
    total = OUT_B + frames * lanes
    ops = [("LOAD", TRIG), ("LOAD", RESET), ("LOAD_LANE", FREQ), ("LOAD_LANE", DRIVE),
           ("PHASOR", PH, 2, 1, sr),                      # t4
           ("CONST", 0, 0, 0, 6.28318530717958647692), ("MUL", 4, 5), ("SIN", 6),          # t7 = sin(2 pi phase)
           ("HISTORY_READ", FB), ("CONST", 0, 0, 0, 0.5), ("MUL", 8, 9), ("ADD", 7, 10), ("MUL", 11, 3), ("TANH", 12),
           ("HISTORY_WRITE", FB, 13),                     # t14 = tanh(drive * (s + 0.5 * y1))
           ("LATCH", HOLD, 14, 0),                        # t15
           ("STORE_FRAME_LANE", OUT_A, 14), ("STORE_FRAME_LANE", OUT_B, 15)]
    mem = np.zeros(total, f32)
    mem[TRIG:TRIG + frames], mem[RESET:RESET + frames] = trig, reset
    mem[FREQ:FREQ + lanes], mem[DRIVE:DRIVE + lanes] = freq, drive
    mem[HOLD:HOLD + lanes] = -2.0                         # initial latch content: visible until the first trigger
    d = torch.from_numpy(mem).cuda()
    m = ctx.compile_block(ops, "fb_block", sequential=True)
    m.launch("fb_block", (lanes + 63) // 64, 64, [d, C.c_int(frames), C.c_int(lanes)])
    ctx.sync()
    got = d.cpu().numpy()
    # frame-by-frame evaluation, all lanes at once, single precision
    ph, fb, hold = np.zeros(lanes, f32), np.zeros(lanes, f32), np.full(lanes, -2.0, f32)
    want_a, want_b = np.zeros((frames, lanes), f32), np.zeros((frames, lanes), f32)
    for i in range(frames):
        out_ph = ph
        nxt = (ph + (freq / f32(sr)).astype(f32)).astype(f32)
        nxt = (nxt - np.floor(nxt)).astype(f32)
        nxt = np.where(nxt >= 1, nxt - 1, nxt).astype(f32)
        ph = np.zeros(lanes, f32) if reset[i] > 0 else nxt
        s = np.sin((out_ph * f32(6.28318530717958647692)).astype(f32)).astype(f32)
        y = np.tanh(((s + (fb * f32(0.5)).astype(f32)).astype(f32) * drive).astype(f32)).astype(f32)
        fb = y
        if trig[i] > 0:
            hold = y
        want_a[i], want_b[i] = y, hold
    ga = got[OUT_A:OUT_A + frames * lanes].reshape(frames, lanes)
    gb = got[OUT_B:OUT_B + frames * lanes].reshape(frames, lanes)
    # the phase accumulates in single precision in both; sinf / tanhf of the two math libraries differ by ulps and
    # the loop feeds them back: 1e-4 absolute on outputs in [-1, 1]
    assert np.abs(ga - want_a).max() <= 1e-4
    assert np.abs(gb - want_b).max() <= 1e-4
    assert np.all(gb[0] == -2.0) or trig[0] > 0
    assert np.abs(got[PH:PH + lanes] - ph).max() <= 1e-4 and np.abs(got[FB:FB + lanes] - fb).max() <= 1e-4
    m.close()


def test_sequential_block_biquad_from_ops_against_the_biquad_restatement(ctx):
    """Direct-form-I biquad written as history ops (Sources/DGen/HigherOps.swift:401-570, coefficients given), a lane
    per filter, against the oracle's bank."""
    from oracle import oracle as orc
    frames, lanes = 4000, 24
    rng = np.random.default_rng(6)
    x = rng.standard_normal(frames).astype(f32)
    cutoff = np.exp(rng.uniform(np.log(400.0), np.log(8000.0), lanes)).astype(f32)
    q = np.exp(rng.uniform(np.log(0.5), np.log(8.0), lanes)).astype(f32)
    coef = np.stack([orc.biquad_coef(float(c_), float(q_)) for c_, q_ in zip(cutoff, q)]).astype(f32)   # b0 b1 b2 a1 a2
    X = 0
    CO = frames                                           # 5 planes of per-lane coefficients
    ST = CO + 5 * lanes                                   # x1 x2 y1 y2
    Y = ST + 4 * lanes
    c = lambda j: ("LOAD_LANE", CO + j * lanes)
    ops = [("LOAD", X), c(0), c(1), c(2), c(3), c(4),
           ("HISTORY_READ", ST), ("HISTORY_READ", ST + lanes), ("HISTORY_READ", ST + 2 * lanes),
           ("HISTORY_READ", ST + 3 * lanes),               # t6 x1, t7 x2, t8 y1, t9 y2
           ("MUL", 7, 3), ("MUL", 6, 2), ("ADD", 10, 11), ("MUL", 0, 1), ("ADD", 12, 13),   # t14 = x2 b2 + x1 b1 + x0 b0
           ("MUL", 9, 5), ("MUL", 8, 4), ("ADD", 15, 16), ("SUB", 14, 17),                  # t18 = ... - (y2 a2 + y1 a1)
           ("HISTORY_WRITE", ST + lanes, 6), ("HISTORY_WRITE", ST, 0),
           ("HISTORY_WRITE", ST + 3 * lanes, 8), ("HISTORY_WRITE", ST + 2 * lanes, 18),
           ("STORE_FRAME_LANE", Y, 18)]
    mem = np.zeros(Y + frames * lanes, f32)
    mem[:frames] = x
    for j in range(5):
        mem[CO + j * lanes:CO + (j + 1) * lanes] = coef[:, j]
    d = torch.from_numpy(mem).cuda()
    m = ctx.compile_block(ops, "biquad_block", sequential=True)
    m.launch("biquad_block", 1, 32, [d, C.c_int(frames), C.c_int(lanes)])
    ctx.sync()
    got = d.cpu().numpy()[Y:].reshape(frames, lanes)
    want = orc.biquad_bank(x[None, :], cutoff, q)[0].T    # [frames][lanes]
    assert np.abs(got - want).max() <= 1e-4 * max(1.0, np.abs(want).max())
    m.close()


def test_sequential_block_accum_and_noise_state_ops(ctx):
    """accum (Sources/DGen/Definitions.swift:215-246) against the restatement, and the xorshift noise generator
    (Sources/DGen/Renderer/CRenderer.swift:660-695) bit for bit, a different seed per lane; state cells carry over
    a second launch."""
    from oracle import oracle as orc
    frames, lanes = 1500, 9
    seeds = np.asarray([0, 1, 2, 12345, 0xdeadbeef, 7, 99, 0x7f800001, 0xffc00000], np.uint32)  # incl. NaN / Inf bit patterns
    INCR, ACC, RNG, OUT_A, OUT_N = 0, lanes, 2 * lanes, 3 * lanes, 3 * lanes + 2 * frames * lanes
    incr = np.linspace(0.01, 0.9, lanes).astype(f32)
    ops = [("LOAD_LANE", INCR), ("CONST", 0, 0, 0, 0.0), ("ACCUM", ACC, 0, 1, 3.0), ("NOISE", RNG),
           ("STORE_FRAME_LANE", OUT_A, 2), ("STORE_FRAME_LANE", OUT_N, 3)]
    mem = np.zeros(OUT_N + 2 * frames * lanes, f32)
    mem[INCR:INCR + lanes] = incr
    mem[RNG:RNG + lanes] = seeds.view(f32)
    d = torch.from_numpy(mem).cuda()
    m = ctx.compile_block(ops, "state_ops", sequential=True)
    m.launch("state_ops", 1, 32, [d, C.c_int(frames), C.c_int(lanes)])
    ops2 = ops[:4] + [("STORE_FRAME_LANE", OUT_A + frames * lanes, 2), ("STORE_FRAME_LANE", OUT_N + frames * lanes, 3)]
    m2 = ctx.compile_block(ops2, "state_ops_b", sequential=True)
    m2.launch("state_ops_b", 1, 32, [d, C.c_int(frames), C.c_int(lanes)])
    ctx.sync()
    got = d.cpu().numpy()
    acc = got[OUT_A:OUT_A + 2 * frames * lanes].reshape(2 * frames, lanes)
    noi = got[OUT_N:OUT_N + 2 * frames * lanes].reshape(2 * frames, lanes)
    for l in range(lanes):
        want = orc.accum(float(incr[l]), 0.0, 3.0, 2 * frames)
        assert np.abs(acc[:, l] - want).max() <= 2e-5, l          # the wrap may be contracted to a fused multiply-add
        wn, st = orc.noise_xorshift(int(seeds[l]), 2 * frames)
        assert np.array_equal(noi[:, l], wn), l
        assert got[RNG + l:RNG + l + 1].view(np.uint32)[0] == st
    m.close()
    m2.close()


# ---- the reference's own fixture graphs as op lists, against the outputs of the reference's emitted C ----------
def test_reference_fixture_graphs_as_op_lists_match_the_reference_artefacts(ctx):
    """toolchain/fixtures/scalar-synth.lisp and feedback-delay-effect.lisp are "leftover" graphs (a stateful phasor
    with waveshaping; a delay with one-sample history feedback) that no primitive covers: written as op lists,
    emitted and compiled here, they reproduce the outputs of the reference's own generated C for the same graphs and
    harness inputs (tests/golden/ref_artefacts.npz, made by tests/golden/make_golden.py from
    toolchain/generated/hermetic/*.c).  This pins the emitter to the reference's emitted code, not to an
    interpreter of its own."""
    gold = np.load(os.path.join(HERE, "golden", "ref_artefacts.npz"))
    n, sr = gold["scalar_synth"].size, 48000.0
    # --- scalar-synth: memory[0..2] = freq, drive, gain; cell 3 = phasor state; out at OUT
    OUT = 64
    ops = [("LOAD_SCALAR", 0), ("CONST", 0, 0, 0, 0.0), ("PHASOR", 3, 0, 1, sr),          # 0 1 2: phase
           ("CONST", 0, 0, 0, 6.283185), ("MUL", 2, 3), ("SIN", 4),                        # 3 4 5: fundamental
           ("CONST", 0, 0, 0, 12.56637), ("MUL", 2, 6), ("COS", 7),                        # 6 7 8: harmonic
           ("CONST", 0, 0, 0, 0.125), ("MUL", 8, 9), ("ADD", 5, 10),                       # 9 10 11
           ("LOAD_SCALAR", 1), ("MUL", 12, 11), ("TANH", 13),                              # 12 13 14: shaped
           ("LOAD_SCALAR", 2), ("MUL", 15, 14), ("STORE_FRAME_LANE", OUT, 16)]             # 15 16 17
    mem = torch.zeros(OUT + n, device="cuda")
    mem[:3] = torch.tensor([220.0, 1.75, 0.2])
    m = ctx.compile_block(ops, name="scalar_synth", sequential=True)
    # the harness calls the artefact block by block with the state kept in memory: two calls here, the second
    # continuing from the phasor cell the first one left
    half = n // 2
    m.launch("scalar_synth", 1, 32, [mem, C.c_int(half), C.c_int(1)])
    ctx.sync()
    state_mid = float(mem[3].cpu())
    ops2 = [tuple(o) if o[0] != "STORE_FRAME_LANE" else ("STORE_FRAME_LANE", OUT + half, 16) for o in ops]
    m2 = ctx.compile_block(ops2, name="scalar_synth_b", sequential=True)
    m2.launch("scalar_synth_b", 1, 32, [mem, C.c_int(n - half), C.c_int(1)])
    ctx.sync()
    mem2 = mem
    got = mem[OUT:OUT + n].cpu().numpy()
    assert 0.0 <= state_mid < 1.0
    assert np.abs(got - gold["scalar_synth"]).max() < 2e-6      # the artefact uses a 4-lane polynomial sine
    assert float(mem2[3].cpu()) == float(gold["scalar_synth_final_phase"][0])   # the phasor state, bit for bit
    m.close()
    m2.close()
    # --- feedback-delay-effect: delayed = delay(dry + fb * history, 37); history <- delayed; out = mix(dry, delayed, wet)
    x = gold["input"]
    D, X, W, HIST, OUTF = 37, 128, 128 + n + 64, 8, 128 + 2 * n + 128
    ops = [("LOAD", X), ("HISTORY_READ", HIST), ("LOAD_SCALAR", 1), ("MUL", 2, 1), ("ADD", 0, 3),   # 0..4: w = dry + fb * h
           ("STORE_FRAME_LANE", W, 4),                                                              # 5: the delay's storage
           ("LOAD", W - D), ("HISTORY_WRITE", HIST, 6),                                             # 6 7: delayed = w[n - 37]
           ("LOAD_SCALAR", 2), ("CONST", 0, 0, 0, 1.0), ("SUB", 9, 8), ("MUL", 0, 10), ("MUL", 7, 8),  # 8..12
           ("ADD", 11, 12), ("OUTPUT", OUTF, 13)]
    mem = torch.zeros(OUTF + n, device="cuda")
    mem[:3] = torch.tensor([37.0, 0.35, 0.4])
    mem[X:X + n] = torch.from_numpy(x).cuda()
    m = ctx.compile_block(ops, name="feedback_delay", sequential=True)
    m.launch("feedback_delay", 1, 32, [mem, C.c_int(n), C.c_int(1)])
    ctx.sync()
    got = mem[OUTF:OUTF + n].cpu().numpy()
    assert np.abs(got - gold["feedback_delay"]).max() < 1e-6
    m.close()
