"""Seeded synthetic inputs for the benchmark configurations (numpy, host side).

No dataset is involved: every configuration is defined by shapes and value distributions only.
RNG: numpy Generator(PCG64(seed)); a "target" is the same generator with seed + 1.
"""
import numpy as np

f32 = np.float32


def _smooth(rng, shape, lo=0.0, hi=1.0, span=40):
    """Random control curves along axis 0: piecewise-linear between uniform knots `span` frames apart."""
    F = shape[0]
    nk = F // span + 2
    knots = rng.uniform(lo, hi, (nk,) + tuple(shape[1:]))
    x = np.arange(F) / span
    i = np.floor(x).astype(int)
    fr = (x - i).reshape((F,) + (1,) * (len(shape) - 1))
    return (knots[i] * (1 - fr) + knots[i + 1] * fr).astype(f32)


def band_to_tap_matrix(nbands=65, taps=257):
    """Linear map from band magnitudes to zero-phase FIR taps by frequency sampling: band magnitudes
    are interpolated linearly to (taps-1)/2+1 bins, inverse real FFT of length taps-1, rotated so the
    response is centred, Hann-windowed (symmetric).  Returns W [taps][nbands] float32."""
    n = taps - 1
    nbins = n // 2 + 1
    pos = np.linspace(0, nbands - 1, nbins)
    lo = np.minimum(np.floor(pos).astype(int), nbands - 2)
    fr = pos - lo
    interp = np.zeros((nbins, nbands))
    interp[np.arange(nbins), lo] += 1 - fr
    interp[np.arange(nbins), lo + 1] += fr
    h = np.fft.irfft(interp, n=n, axis=0)            # [n][nbands], zero phase (circular)
    idx = (np.arange(taps) - n // 2) % n
    win = 0.5 * (1 - np.cos(2 * np.pi * np.arange(taps) / (taps - 1)))
    return (h[idx] * win[:, None]).astype(f32)


def harmonic_noise_inputs(seed, B=16, T=64000, K=100, F=1000, sr=16000.0, nbands=65, taps=257):
    """The batched harmonic+noise synthesis configuration.
    f0: log-uniform start in 55..880 Hz, Gaussian random walk of 0.5 semitone per control frame.
    amps: softmax of N(0,1) logits per voice (slowly modulated), gain: loudness envelope in [0,1].
    noise: white N(0, 0.1) per voice; bands: 65 magnitudes in [0,1] per control frame."""
    rng = np.random.Generator(np.random.PCG64(seed))
    start = np.exp(rng.uniform(np.log(55.0), np.log(880.0), B))
    walk = np.cumsum(rng.normal(0.0, 0.5, (F, B)), axis=0)
    walk[0] = 0
    f0 = (start[None, :] * 2.0 ** (walk / 12.0)).astype(f32)
    logits = rng.normal(0.0, 1.0, (1, B, K)) + 0.3 * _smooth(rng, (F, B, K), -1, 1)
    e = np.exp(logits - logits.max(axis=2, keepdims=True))
    amps = (e / e.sum(axis=2, keepdims=True)).astype(f32)
    d = dict(B=B, T=T, K=K, F=F, sr=sr, nbands=nbands, taps=taps)
    d["f0"] = np.ascontiguousarray(f0)
    d["uv"] = np.ones((F, B), f32)
    d["amps"] = np.ascontiguousarray(amps)
    d["gain"] = _smooth(rng, (F, B), 0.0, 1.0)
    d["noise_gain"] = _smooth(rng, (F, B), 0.0, 1.0)
    d["bands"] = _smooth(rng, (F, B, nbands), 0.0, 1.0)
    d["noise"] = rng.normal(0.0, 0.1, (B, T)).astype(f32)
    d["W"] = band_to_tap_matrix(nbands, taps)
    return d


def taps_from_bands(d):
    """Host evaluation of the band -> tap map in float32 accumulation order-independent form."""
    F, B, nb = d["bands"].shape
    return (d["bands"].reshape(F * B, nb).astype(np.float64) @ d["W"].astype(np.float64).T).astype(f32).reshape(
        F, B, d["taps"])


def osc_filter_fft_inputs(K=64, sr=44100.0, T=65536):
    """Oscillator bank -> one-pole -> FFT configuration: partial k at 110*k Hz, amplitude 1/k."""
    k = np.arange(1, K + 1, dtype=f32)
    return dict(freq=(f32(110.0) * k).astype(f32), amp=(f32(1.0) / k).astype(f32), sr=sr, T=T, K=K,
                pole=0.9, N=1024, hop=256)


def biquad_bank_inputs(seed, B=32, L=256, T=262144):
    """Tensor biquad bank: white noise input, cutoff log-uniform 50..8000 Hz, Q log-uniform 0.5..8."""
    rng = np.random.Generator(np.random.PCG64(seed))
    return dict(x=rng.normal(0, 1, (B, T)).astype(f32),
                cutoff=np.exp(rng.uniform(np.log(50.0), np.log(8000.0), L)).astype(f32),
                q=np.exp(rng.uniform(np.log(0.5), np.log(8.0), L)).astype(f32), B=B, L=L, T=T)


def pink_noise(rng, shape):
    """1/f-shaped noise along the last axis (FFT shaping of white noise), unit variance."""
    n = shape[-1]
    X = np.fft.rfft(rng.normal(0, 1, shape), axis=-1)
    f = np.arange(X.shape[-1], dtype=np.float64)
    f[0] = 1.0
    x = np.fft.irfft(X / np.sqrt(f), n=n, axis=-1)
    return (x / x.std(axis=-1, keepdims=True)).astype(f32)


def partconv_inputs(seed, V=16, T=480000, sr=48000.0, ir_seconds=2.0, rt60=1.2):
    """Partitioned convolution: pink-noise input, exponentially decaying white-noise IR."""
    rng = np.random.Generator(np.random.PCG64(seed))
    n_ir = int(ir_seconds * sr)
    t = np.arange(n_ir) / sr
    ir = (rng.normal(0, 1, n_ir) * np.exp(-6.91 * t / rt60)).astype(f32)
    return dict(x=pink_noise(rng, (V, T)), ir=ir, V=V, T=T, N=2048, hop=1024)
