"""CPU restatement of the reference's remaining stateful ops -- TEST INFRASTRUCTURE.

Only tests may import this module; it is the checker for the CUDA kernels, never a fallback for them.

Every function walks the frames (or hops) one by one and keeps the SAME state cells the reference keeps
(ring buffers, write heads, held values), so ring aliasing and clamping behave as in the emitted code.
Arithmetic is single precision, one rounding per operation (the reference compiles with contraction
allowed, so a fused multiply-add may differ from this by one rounding of the product: tests allow 1e-6
relative).

  delay_line          Sources/DGen/HigherOps+DelayLine.swift:33-65, emission Sources/DGen/Emit.swift:331-403
  spectrum_delay      Sources/DGen/HigherOps+SpectrumDelay.swift:20-85, emission Sources/DGen/Emit.swift:405-440
  spectrum_delay_mod  Sources/DGen/HigherOps+SpectrumDelay.swift:87-135, emission Sources/DGen/Emit.swift:442-512
  latch               Sources/DGen/Definitions.swift:104-113 (scalar), Sources/DGen/Emit+State.swift:225-262 (tensor)
  compressor          Sources/DGen/HigherOps.swift:566-651
"""
import numpy as np

f32 = np.float32


def delay_line(x, delay, max_delay, ring=None, wpos=0.0):
    """x [T][lanes]; delay scalar, [T] (one time per frame, all lanes) or [T][lanes]; -> (y [T][lanes], ring, wpos).

    Per frame: every lane writes its sample at the shared head, then reads at head - delay with linear
    interpolation between the two bracketing ring slots, then the head advances (write before read: a delay of
    0 returns the current sample).  delay is clamped to [0, max_delay - 1]; the second slot of a delay of
    max_delay - 1 wraps onto the slot just written (its weight is 0 there)."""
    x = np.ascontiguousarray(x, f32)
    T, lanes = x.shape
    d = np.broadcast_to(np.asarray(delay, f32).reshape((-1, 1)) if np.ndim(delay) == 1 else np.asarray(delay, f32),
                        (T, lanes))
    ring = np.zeros((lanes, max_delay), f32) if ring is None else np.array(ring, f32).reshape(lanes, max_delay)
    wposf = f32(wpos)
    y = np.zeros((T, lanes), f32)
    e = np.arange(lanes)
    max_read = f32(max_delay - 1)
    for n in range(T):
        w = int(wposf)
        ring[:, w] = x[n]
        dr = d[n]
        dc = np.where(dr > max_read, max_read, np.where(dr < f32(0), f32(0), dr)).astype(f32)
        kf = np.floor(dc).astype(f32)
        frac = (dc - kf).astype(f32)
        k = kf.astype(np.int64)
        pos0 = (w - k + max_delay) % max_delay
        pos1 = (w - k - 1 + 2 * max_delay) % max_delay
        s0, s1 = ring[e, pos0], ring[e, pos1]
        y[n] = (s0 * (f32(1) - frac)).astype(f32) + (s1 * frac).astype(f32)
        wposf = f32(0) if wposf + f32(1) >= f32(max_delay) else f32(wposf + f32(1))
    return y, ring, float(wposf)


def spectrum_delay(spec, hops, ring=None, row=0.0):
    """spec [H][N] (one spectrum per hop boundary) -> (out [H][N], ring [hops+1][N], row): the spectrum of
    `hops` hop boundaries ago (zeros until the ring has filled)."""
    spec = np.ascontiguousarray(spec, f32)
    H, N = spec.shape
    rows = hops + 1
    ring = np.zeros((rows, N), f32) if ring is None else np.array(ring, f32).reshape(rows, N)
    rowf = f32(row)
    out = np.zeros((H, N), f32)
    for h in range(H):
        ring[int(rowf)] = spec[h]
        rowf = f32(0) if rowf + f32(1) >= f32(rows) else f32(rowf + f32(1))
        out[h] = ring[int(rowf)]
    return out, ring, float(rowf)


def spectrum_delay_mod(spec, delay, max_hops, ring=None, row=0.0):
    """Fractional, modulated variant: delay [H] in hops, clamped to [0, max_hops]; linear interpolation between
    the spectra floor(delay) and floor(delay) + 1 hops ago."""
    spec = np.ascontiguousarray(spec, f32)
    H, N = spec.shape
    rows = max_hops + 1
    ring = np.zeros((rows, N), f32) if ring is None else np.array(ring, f32).reshape(rows, N)
    rowf = f32(row)
    d = np.broadcast_to(np.asarray(delay, f32), (H,))
    out = np.zeros((H, N), f32)
    for h in range(H):
        ring[int(rowf)] = spec[h]
        rowf = f32(0) if rowf + f32(1) >= f32(rows) else f32(rowf + f32(1))
        dv = d[h]
        dc = f32(max_hops) if dv > f32(max_hops) else (f32(0) if dv < f32(0) else dv)
        kf = f32(np.floor(dc))
        frac = f32(dc - kf)
        k = int(kf)
        base = int(rowf) - 1 + 2 * rows
        near, far = (base - k) % rows, (base - k - 1) % rows
        out[h] = (ring[near] * f32(f32(1) - frac)).astype(f32) + (ring[far] * frac).astype(f32)
    return out, ring, float(rowf)


def latch(value, cond, state=None):
    """value [T][lanes]; cond [T] or [T][lanes]; -> (y [T][lanes], state [lanes]).  y[n] = value[n] where
    cond[n] > 0, else the value held from the last such frame (the initial cell value before any)."""
    value = np.ascontiguousarray(value, f32)
    T, lanes = value.shape
    c = np.asarray(cond, f32)
    c = np.broadcast_to(c.reshape(-1, 1) if c.ndim == 1 else c, (T, lanes))
    held = np.zeros(lanes, f32) if state is None else np.array(state, f32).reshape(lanes)
    y = np.zeros((T, lanes), f32)
    for n in range(T):
        held = np.where(c[n] > f32(0), value[n], held)
        y[n] = held
    return y, held


def compressor(x, ratio, threshold, knee, attack, release, sample_rate, sidechain=None, state=None):
    """x [B][T] -> (y [B][T], state [B]).  The gain computer is per sample; the smoothed gain reduction is the one
    recurrence: s[n] = c * s[n-1] + g[n] * (1 - c) with c the attack coefficient where g[n] > s[n-1], else the
    release coefficient."""
    x = np.ascontiguousarray(x, f32)
    B, T = x.shape
    det = x if sidechain is None else np.ascontiguousarray(sidechain, f32)

    def amp2db(a):
        return (f32(20.0) * np.log10(np.maximum(np.abs(a), f32(1e-5)).astype(f32)).astype(f32)).astype(f32)

    ratio, threshold, knee = f32(ratio), f32(threshold), f32(knee)
    det_db, in_db = amp2db(det), amp2db(x)
    log001 = f32(np.log(f32(0.01)))
    att = f32(np.exp(f32(log001 / f32(f32(attack) * f32(sample_rate)))))
    rel = f32(np.exp(f32(log001 / f32(f32(release) * f32(sample_rate)))))
    knee_half = f32(knee / f32(2))
    knee_start, knee_end = f32(threshold - knee_half), f32(threshold + knee_half)
    with np.errstate(divide="ignore", invalid="ignore"):
        pos = ((det_db - knee_start) / knee).astype(f32)
        interp_ratio = (f32(1) + pos * f32(ratio - f32(1))).astype(f32)
        over = (det_db - (knee_start + pos * f32(threshold - knee_start))).astype(f32)
        hard_ratio = f32(f32(1) - f32(1) / ratio)
        soft_ratio = (f32(1) - f32(1) / interp_ratio).astype(f32)
        hard = ((det_db - threshold) * hard_ratio).astype(f32)
        soft = (over * soft_ratio).astype(f32)
    gr = np.where(det_db <= knee_start, f32(0), np.where(det_db >= knee_end, hard, soft)).astype(f32)
    s = np.zeros(B, f32) if state is None else np.array(state, f32).reshape(B)
    sm = np.zeros((B, T), f32)
    for n in range(T):
        g = gr[:, n]
        a_s = (att * s).astype(f32) + (g * f32(f32(1) - att)).astype(f32)
        r_s = (rel * s).astype(f32) + (g * f32(f32(1) - rel)).astype(f32)
        s = np.where(g > s, a_s, r_s).astype(f32)
        sm[:, n] = s
    att_db = (in_db - sm).astype(f32)
    amp = np.power(f32(10.0), (att_db / f32(20.0)).astype(f32)).astype(f32)
    return (np.sign(x).astype(f32) * amp).astype(f32), s


def _principal_arg(v):
    """Emit+PhaseVocoder.swift:46-53: v - 2 pi round(v / 2 pi), then folded into [-pi, pi]; round is roundf (half away
    from zero)."""
    tau, half = f32(2.0 * np.float32(np.pi)), f32(np.pi)
    q = (v / tau).astype(f32)
    r = (np.sign(q) * np.floor(np.abs(q) + f32(0.5))).astype(f32)
    w = (v - (tau * r).astype(f32)).astype(f32)
    wh = np.where(w > half, (w - tau).astype(f32), w)
    return np.where(w < -half, (wh + tau).astype(f32), wh).astype(f32)


def phase_vocoder(re, im, ratio, hop, state=None):
    """re, im [H][N] (all N bins of each hop's spectrum); ratio [H] -> (out_re, out_im [H][N], state).
    state = (previous analysis phase [N], synthesis phase [N], init flag).  Follows
    Sources/DGen/Emit+PhaseVocoder.swift:32-114 hop by hop."""
    re, im = np.ascontiguousarray(re, f32), np.ascontiguousarray(im, f32)
    H, N = re.shape
    ratio = np.broadcast_to(np.asarray(ratio, f32), (H,))
    if state is None:
        prev, synth, init = np.zeros(N, f32), np.zeros(N, f32), 0.0
    else:
        prev, synth, init = np.array(state[0], f32), np.array(state[1], f32), float(state[2])
    omega_scale = f32(2.0 * np.float32(np.pi) * np.float32(hop) / np.float32(N))
    bins = np.arange(N, dtype=f32)
    out_re, out_im = np.zeros((H, N), f32), np.zeros((H, N), f32)

    def mix(a, b, t):
        return ((a * (f32(1) - t).astype(f32)).astype(f32) + (b * t).astype(f32)).astype(f32)

    for h in range(H):
        mag = np.sqrt((re[h] * re[h]).astype(f32) + (im[h] * im[h]).astype(f32)).astype(f32)
        phase = np.arctan2(im[h], re[h]).astype(f32)
        target = (bins * omega_scale).astype(f32)
        delta = _principal_arg(((phase - prev).astype(f32) - target).astype(f32))
        omega = (target + delta).astype(f32)
        prev = phase
        r = max(f32(ratio[h]), f32(1e-4))
        src = (bins / r).astype(f32)
        in_range = src <= f32(N - 1)
        srcc = np.where(in_range, src, f32(N - 1)).astype(f32)
        fl = np.floor(srcc).astype(f32)
        i0 = fl.astype(np.int64)
        i1 = np.where(i0 < N - 1, i0 + 1, i0)
        frac = (srcc - fl).astype(f32)
        imag_ = mix(mag[i0], mag[i1], frac)
        iom = (mix(omega[i0], omega[i1], frac) * r).astype(f32)
        iph = _principal_arg(mix(prev[i0], prev[i1], frac))
        adv = _principal_arg((synth + iom).astype(f32))
        synth = iph if init == 0.0 else adv
        om = np.where(in_range, imag_, f32(0)).astype(f32)
        out_re[h] = (om * np.cos(synth).astype(f32)).astype(f32)
        out_im[h] = (om * np.sin(synth).astype(f32)).astype(f32)
        init = 1.0
    return out_re, out_im, (prev, synth, init)
