"""ctypes access to the CPU oracle (oracle/dgen_oracle.c) -- TEST INFRASTRUCTURE.

Only tests, the smoke check and the benchmark's CPU-baseline leg may import this module.  It is
the checker for the CUDA kernels, never a fallback for them.

``lib(fast=False)`` returns the strict-IEEE build; ``fast=True`` the build made with the
reference's optimisation policy, used only when timing the CPU baseline.
"""
import ctypes as C
import os
import subprocess

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_libs = {}

f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")
i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")


def build(out_dir=None, march=""):
    """Compile the oracle with the committed Makefile (gcc only)."""
    args = ["make", "-s", "-C", HERE]
    if out_dir:
        os.makedirs(out_dir, exist_ok=True)
        args.append("OUT=" + out_dir)
    if march:
        args.append("MARCH=" + march)
    subprocess.run(args, check=True)


def _declare(L):
    for sfx, ct, p in (("_f32", C.c_float, f32p), ("_f64", C.c_double, f64p)):
        def fn(name, res, args):
            f = getattr(L, name + sfx)
            f.restype = res
            f.argtypes = args
        vp = C.c_void_p
        fn("orc_accum", None, [ct, ct, ct, C.c_int, ct, p, vp])
        fn("orc_phasor_stateful", None, [p, C.c_int, C.c_int, ct, p])
        fn("orc_phasor_deterministic", None, [p, C.c_int, C.c_int, ct, p])
        fn("orc_sample_row", None, [p, C.c_int, C.c_int, p, C.c_int, p])
        fn("orc_playhead", None, [C.c_int, C.c_int, p])
        fn("orc_osc_bank_const", None, [p, p, C.c_int, C.c_int, ct, C.c_int, p])
        fn("orc_onepole", None, [p, C.c_int, ct, ct, p])
        fn("orc_biquad", None, [p, C.c_int, ct, ct, ct, ct, p])
        fn("orc_biquad_coef", None, [ct, ct, ct, ct, p])
        fn("orc_biquad_with_coef", None, [p, C.c_int, p, p])
        fn("orc_biquad_bank", None, [p, C.c_int, C.c_int, C.c_int, p, p, ct, ct, p])
        fn("orc_biquad_bank_mse_grad", C.c_double, [p, C.c_int, C.c_int, C.c_int, p, p, ct, ct, p, ct, p, p])
        fn("orc_fft", None, [p, p, C.c_int, C.c_int])
        fn("orc_hann_periodic", None, [C.c_int, p])
        fn("orc_hann_symmetric", None, [C.c_int, p])
        fn("orc_buffer_fft_mag", None, [p, C.c_int, C.c_int, C.c_int, vp, p])
        fn("orc_overlap_add", None, [p, C.c_int, C.c_int, C.c_int, p])
        fn("orc_partitioned_convolve", None, [p, C.c_int, p, C.c_int, C.c_int, C.c_int, ct, p])
        fn("orc_spectral_loss", C.c_double, [p, p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp])
        fn("orc_mss_loss", C.c_double, [p, p, C.c_int, C.c_int, i32p, C.c_int, C.c_int, ct, ct])
        fn("orc_mss_loss_grad", None, [p, p, C.c_int, C.c_int, i32p, C.c_int, C.c_int, ct, ct, ct, p])
        fn("orc_harmonic_noise_render", None,
           [C.c_int] * 5 + [ct] + [p, p, p, p, p, vp, vp, ct, ct, p, vp])
        fn("orc_adam", None, [p, p, p, p, C.c_size_t, C.c_int, ct, ct, ct, ct])
    L.orc_noise_xorshift.restype = None
    L.orc_noise_xorshift.argtypes = [C.POINTER(C.c_uint32), C.c_int, f32p]
    L.orc_sanitize.restype = None
    L.orc_sanitize.argtypes = [f32p, C.c_size_t]


def lib(fast=False, path=None):
    key = path or ("fast" if fast else "strict")
    if key not in _libs:
        so = path or os.path.join(HERE, "libdgen_oracle_fast.so" if fast else "libdgen_oracle.so")
        if not os.path.exists(so):
            build()
        L = C.CDLL(so)
        _declare(L)
        _libs[key] = L
    return _libs[key]


def _dt(double):
    return (np.float64, "_f64") if double else (np.float32, "_f32")


def _ptr(a):
    return None if a is None else a.ctypes.data_as(C.c_void_p)


# ------------------------------------------------------------------------------------------------
# numpy-level helpers (each allocates its output)
# ------------------------------------------------------------------------------------------------
def accum(incr, mn, mx, T, state0=0.0, double=False, L=None):
    dt, s = _dt(double)
    out = np.empty(T, dt)
    getattr(L or lib(), "orc_accum" + s)(incr, mn, mx, T, state0, out, None)
    return out


def playhead(F, T, double=False, L=None):
    dt, s = _dt(double)
    out = np.empty(T, dt)
    getattr(L or lib(), "orc_playhead" + s)(F, T, out)
    return out


def phasor_stateful(freq, sr, double=False, L=None):
    dt, s = _dt(double)
    freq = np.ascontiguousarray(freq, dt)
    T, lanes = freq.shape
    out = np.empty((T, lanes), dt)
    getattr(L or lib(), "orc_phasor_stateful" + s)(freq, T, lanes, sr, out)
    return out


def phasor_deterministic(freq, T, sr, double=False, L=None):
    dt, s = _dt(double)
    freq = np.ascontiguousarray(freq, dt)
    out = np.empty((T, freq.size), dt)
    getattr(L or lib(), "orc_phasor_deterministic" + s)(freq, T, freq.size, sr, out)
    return out


def sample_row(table, idx, double=False, L=None):
    dt, s = _dt(double)
    table = np.ascontiguousarray(table, dt)
    idx = np.ascontiguousarray(idx, dt)
    rows = table.shape[0]
    cols = table.size // rows
    out = np.empty((idx.size, cols), dt)
    getattr(L or lib(), "orc_sample_row" + s)(table.reshape(rows, cols), rows, cols, idx, idx.size, out)
    return out


def osc_bank_const(freq, amp, T, sr, stateful=False, double=False, L=None):
    dt, s = _dt(double)
    freq = np.ascontiguousarray(freq, dt)
    amp = np.ascontiguousarray(amp, dt)
    out = np.empty(T, dt)
    getattr(L or lib(), "orc_osc_bank_const" + s)(freq, amp, freq.size, T, sr, int(stateful), out)
    return out


def onepole(x, a, y0=0.0, double=False, L=None):
    dt, s = _dt(double)
    x = np.ascontiguousarray(x, dt)
    y = np.empty_like(x)
    getattr(L or lib(), "orc_onepole" + s)(x, x.size, a, y0, y)
    return y


def biquad(x, cutoff, q, gain=1.0, mode=0.0, double=False, L=None):
    dt, s = _dt(double)
    x = np.ascontiguousarray(x, dt)
    y = np.empty_like(x)
    getattr(L or lib(), "orc_biquad" + s)(x, x.size, cutoff, q, gain, mode, y)
    return y


def biquad_coef(cutoff, q, gain=1.0, mode=0.0, double=False, L=None):
    dt, s = _dt(double)
    c = np.empty(5, dt)
    getattr(L or lib(), "orc_biquad_coef" + s)(cutoff, q, gain, mode, c)
    return c  # b0 b1 b2 a1 a2


def biquad_exact_response(x, cutoff, q, gain=1.0, mode=0.0, L=None):
    """The recurrence in double with the SINGLE-precision coefficients of the fp32 graph: what the fp32 filter would
    give without the rounding of its own recurrence.  x [T] -> y [T] float64."""
    coef = biquad_coef(cutoff, q, gain, mode, double=False, L=L).astype(np.float64)
    x = np.ascontiguousarray(x, np.float64)
    y = np.empty_like(x)
    (L or lib()).orc_biquad_with_coef_f64(x, x.size, coef, y)
    return y


def biquad_bank(x, cutoff, q, gain=1.0, mode=0.0, double=False, L=None):
    dt, s = _dt(double)
    x = np.ascontiguousarray(x, dt)
    B, T = x.shape
    cutoff = np.ascontiguousarray(cutoff, dt)
    q = np.ascontiguousarray(q, dt)
    y = np.empty((B, cutoff.size, T), dt)
    getattr(L or lib(), "orc_biquad_bank" + s)(x, B, T, cutoff.size, cutoff, q, gain, mode, y)
    return y


def biquad_bank_mse_grad(x, cutoff, q, target, scale=1.0, gain=1.0, mode=0.0, double=True, L=None):
    """target [B][L][T]. Returns (loss, grad_cutoff[L], grad_q[L])."""
    dt, s = _dt(double)
    x = np.ascontiguousarray(x, dt)
    B, T = x.shape
    cutoff = np.ascontiguousarray(cutoff, dt)
    q = np.ascontiguousarray(q, dt)
    target = np.ascontiguousarray(target, dt)
    gc, gq = np.empty(cutoff.size, dt), np.empty(cutoff.size, dt)
    loss = getattr(L or lib(), "orc_biquad_bank_mse_grad" + s)(x, B, T, cutoff.size, cutoff, q, gain, mode, target,
                                                               scale, gc, gq)
    return loss, gc, gq


def fft(re, im, inverse=False, double=False, L=None):
    dt, s = _dt(double)
    re = np.array(re, dt)
    im = np.array(im, dt)
    getattr(L or lib(), "orc_fft" + s)(re, im, re.size, int(inverse))
    return re, im


def hann_periodic(N, double=False, L=None):
    dt, s = _dt(double)
    w = np.empty(N, dt)
    getattr(L or lib(), "orc_hann_periodic" + s)(N, w)
    return w


def hann_symmetric(N, double=False, L=None):
    dt, s = _dt(double)
    w = np.empty(N, dt)
    getattr(L or lib(), "orc_hann_symmetric" + s)(N, w)
    return w


def buffer_fft_mag(x, N, hop, window=None, double=False, L=None):
    dt, s = _dt(double)
    x = np.ascontiguousarray(x, dt)
    H = (x.size + hop - 1) // hop
    if window is not None:
        window = np.ascontiguousarray(window, dt)
    out = np.empty((H, N // 2 + 1), dt)
    getattr(L or lib(), "orc_buffer_fft_mag" + s)(x, x.size, N, hop, _ptr(window), out)
    return out


def overlap_add(frames, T, hop, double=False, L=None):
    dt, s = _dt(double)
    frames = np.ascontiguousarray(frames, dt)
    out = np.empty(T, dt)
    getattr(L or lib(), "orc_overlap_add" + s)(frames, T, frames.shape[1], hop, out)
    return out


def partitioned_convolve(x, ir, N, hop, gain=1.0, double=False, L=None):
    dt, s = _dt(double)
    x = np.ascontiguousarray(x, dt)
    ir = np.ascontiguousarray(ir, dt)
    out = np.empty_like(x)
    getattr(L or lib(), "orc_partitioned_convolve" + s)(x, x.size, ir, ir.size, N, hop, gain, out)
    return out


def spectral_loss(x1, x2, N, hop, use_log=False, l2=False, double=False, want_partial=False, L=None):
    dt, s = _dt(double)
    x1 = np.ascontiguousarray(x1, dt)
    x2 = np.ascontiguousarray(x2, dt)
    B, T = x1.shape
    H = (T + hop - 1) // hop
    partial = np.empty((H, B), dt) if want_partial else None
    tot = getattr(L or lib(), "orc_spectral_loss" + s)(x1, x2, B, T, N, hop, int(use_log), int(l2), _ptr(partial))
    return (tot, partial) if want_partial else tot


def mss_loss(x1, x2, sizes=(2048, 1024, 512, 256, 128, 64), hop_div=4, w_lin=1.0, w_log=1.0, double=False, L=None):
    dt, s = _dt(double)
    x1 = np.ascontiguousarray(x1, dt)
    x2 = np.ascontiguousarray(x2, dt)
    B, T = x1.shape
    sz = np.asarray(sizes, np.int32)
    return getattr(L or lib(), "orc_mss_loss" + s)(x1, x2, B, T, sz, sz.size, hop_div, w_lin, w_log)


def mss_loss_grad(x1, x2, sizes=(2048, 1024, 512, 256, 128, 64), hop_div=4, w_lin=1.0, w_log=1.0, upstream=1.0,
                  double=True, L=None):
    dt, s = _dt(double)
    x1 = np.ascontiguousarray(x1, dt)
    x2 = np.ascontiguousarray(x2, dt)
    B, T = x1.shape
    sz = np.asarray(sizes, np.int32)
    g = np.empty((B, T), dt)
    getattr(L or lib(), "orc_mss_loss_grad" + s)(x1, x2, B, T, sz, sz.size, hop_div, w_lin, w_log, upstream, g)
    return g


def harmonic_noise_render(f0, uv, amps, gain, noise_gain, taps, noise, T, sr, hscale=1.0, nscale=1.0,
                          double=False, want_phase=False, L=None):
    """f0/uv/gain/noise_gain [F][B]; amps [F][B][K]; taps [F][B][FIR] or None; noise [B][T] or None."""
    dt, s = _dt(double)
    f0 = np.ascontiguousarray(f0, dt)
    F, B = f0.shape
    amps = np.ascontiguousarray(amps, dt)
    K = amps.shape[2]
    uv = np.ascontiguousarray(uv, dt)
    gain = np.ascontiguousarray(gain, dt)
    noise_gain = np.ascontiguousarray(noise_gain, dt)
    FIR = 0
    if taps is not None:
        taps = np.ascontiguousarray(taps, dt)
        noise = np.ascontiguousarray(noise, dt)
        FIR = taps.shape[2]
    audio = np.empty((B, T), dt)
    phase = np.empty((B, K, T), dt) if want_phase else None
    getattr(L or lib(), "orc_harmonic_noise_render" + s)(
        B, T, K, F, FIR, sr, f0, uv, amps, gain, noise_gain, _ptr(taps), _ptr(noise), hscale, nscale, audio,
        _ptr(phase))
    return (audio, phase) if want_phase else audio


def adam(theta, g, m, v, t, lr=1e-3, b1=0.9, b2=0.999, eps=1e-8, double=False, L=None):
    dt, s = _dt(double)
    getattr(L or lib(), "orc_adam" + s)(theta, g, m, v, theta.size, t, lr, b1, b2, eps)


def noise_xorshift(state, T, L=None):
    st = C.c_uint32(state)
    out = np.empty(T, np.float32)
    (L or lib()).orc_noise_xorshift(C.byref(st), T, out)
    return out, st.value


# ------------------------------------------------------------------------------------------------
# The reference's own generated artefacts (oracle/_ref, built by oracle/build_ref.sh)
# ------------------------------------------------------------------------------------------------
REF_DIR = os.path.join(HERE, "_ref")


def sanitize(x, L=None):
    """Non-finite -> 0 in a copy of x (toolchain/include/dgen_runtime.h:72-74)."""
    L = L or lib()
    y = np.ascontiguousarray(x, dtype=np.float32).copy()
    L.orc_sanitize(y, y.size)
    return y


def ref_available():
    return os.path.exists(os.path.join(REF_DIR, "libref_harness.so"))


def ref_run(name, memory, inp, blocks, block_frames, sample_rate=48000.0):
    """Run oracle/_ref/<name>.so like toolchain/harness/toolchain_harness.c does.  memory is updated in place."""
    H = C.CDLL(os.path.join(REF_DIR, "libref_harness.so"))
    H.ref_run.restype = C.c_int
    H.ref_run.argtypes = [C.c_char_p, f32p, C.c_void_p, f32p, C.c_int, C.c_int, C.c_float]
    out = np.zeros(blocks * block_frames, np.float32)
    if inp is not None:
        inp = np.ascontiguousarray(inp, np.float32)
    rc = H.ref_run(os.path.join(REF_DIR, name + ".so").encode(), memory, _ptr(inp), out, blocks, block_frames,
                   sample_rate)
    if rc != 0:
        raise RuntimeError("ref_run(%s) failed: %d" % (name, rc))
    return out
