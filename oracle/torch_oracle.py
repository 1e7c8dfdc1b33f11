"""Double-precision host evaluation of the harmonic+noise training graph with automatic
differentiation (PyTorch, CPU) -- TEST INFRASTRUCTURE: the gradient reference for the CUDA backward
kernels ("fp64 host evaluation of the same graph").  Never imported by the product.

Every function restates the forward semantics of the reference graph (file:line in the docstrings);
gradients come from autograd, so they are independent of the hand-derived adjoints in the kernels.
The control clock is taken from the fp32 oracle (oracle.playhead): it is data-independent and its
single-precision rounding is part of the reference semantics.
"""
import numpy as np
import torch

from . import oracle as orc

DT = torch.float64


def t64(a):
    return torch.as_tensor(np.asarray(a), dtype=DT)


def rows_of(F, T):
    """sampleRow positions (Sources/DGen/Emit+RowSelection.swift:166-184) of the control playhead."""
    p = orc.playhead(F, T).astype(np.float64)
    w = np.fmod(p, F)
    w[w < 0] += F
    lo = np.floor(w).astype(np.int64)
    hi = lo + 1
    hi[hi >= F] = 0
    fr = w - lo
    return torch.from_numpy(lo), torch.from_numpy(hi), t64(fr)


def lerp_rows(table, rows):
    lo, hi, fr = rows
    shape = (-1,) + (1,) * (table.dim() - 1)
    return (1 - fr).reshape(shape) * table[lo] + fr.reshape(shape) * table[hi]


def harmonic_render(f0, uv, amps, gain, T, sr, rows, scale=1.0, reference_increments=True):
    """Examples/HarmonicE2E/Synth.swift:47-95. f0/uv/gain [F,B], amps [F,B,K] -> audio [B,T].
    The gradient w.r.t. f0 flows through the phases as the reference's temporal gradient defines it
    (Sources/DGen/Gradients.swift:216-261: exclusive reverse sum of the phase gradients / sr; floor and the
    Nyquist comparison have no gradient).  reference_increments=False evaluates the increments in double
    as well (a smooth function of f0, used for the finite-difference check)."""
    F, B, K = amps.shape
    # The phasor's input is single-precision data in the reference graph (f0 is not a parameter): the
    # per-frame increment is RN(RN(k * f0t) / sr) with f0t the strict single-precision lerp, exactly the
    # values the reference's recurrence adds up (Sources/DGen/Emit+State.swift:322-369).  Only the running sum
    # is carried in double here, so the systematic drift of the rounded increments is part of this
    # evaluation and the (random-walk) rounding of the running phase is not.
    lo, hi, fr = rows
    f32 = np.float32
    fr32 = fr.numpy().astype(f32)[:, None]
    f0n = f0.detach().numpy().astype(f32)
    f0t32 = ((f32(1.0) - fr32) * f0n[lo.numpy()]).astype(f32) + (fr32 * f0n[hi.numpy()]).astype(f32)
    k32 = np.arange(1, K + 1, dtype=f32)
    freq32 = (f0t32[:, :, None] * k32).astype(f32)          # [T,B,K]
    k = torch.arange(1, K + 1, dtype=DT)
    inc_exact = lerp_rows(f0, rows)[:, :, None] * k / sr    # differentiable, double
    if reference_increments:                                # reference values, exact derivative
        inc = t64((freq32 / f32(sr)).astype(f32)) + (inc_exact - inc_exact.detach())
    else:
        inc = inc_exact
    freq = t64(freq32)
    phase = torch.cumsum(inc, 0) - inc                      # phase before the update (first frame 0)
    phase = phase - torch.floor(phase)
    a = lerp_rows(amps, rows) * (freq < sr * 0.5).to(DT)    # Nyquist mask (Synth.swift:161-170)
    a = a / (a.sum(-1, keepdim=True) + 1e-8)
    harm = (torch.sin(2 * np.pi * phase) * a).sum(-1)
    return (harm * lerp_rows(gain, rows) * lerp_rows(uv, rows) * scale).T.contiguous()


def fir_noise(noise, taps, noise_gain, rows, scale=0.12):
    """Synth.swift:97-101: buffer(size: NT) window x per-frame interpolated taps. noise [B,T], taps [F,B,NT]."""
    B, T = noise.shape
    NT = taps.shape[2]
    xp = torch.nn.functional.pad(noise, (NT - 1, 0))
    win = xp.unfold(1, NT, 1)                               # [B,T,NT], element i = x[n-NT+1+i]
    tt = lerp_rows(taps, rows).permute(1, 0, 2)             # [B,T,NT]
    y = (win * tt).sum(-1)
    return y * lerp_rows(noise_gain, rows).T * scale


def hann_periodic(N):
    return t64(orc.hann_periodic(N))


def partconv(x, ir, N, hop, gain=1.0):
    """partitionedConvolve (Sources/DGenLazy/SpectralTensorOps.swift:204-254). x [V,T], ir [L] -> [V,T]."""
    V, T = x.shape
    H = (T + hop - 1) // hop
    K = (ir.numel() + hop - 1) // hop
    w = hann_periodic(N)
    xp = torch.nn.functional.pad(x, (N - 1, H * hop))       # frame h = x[h*hop-(N-1) .. h*hop]
    frames = xp.unfold(1, N, hop)[:, :H] * w                # [V,H,N]
    X = torch.fft.fft(frames.to(torch.complex128), dim=-1)
    irp = torch.nn.functional.pad(ir, (0, K * hop - ir.numel())).reshape(K, hop)
    Hk = torch.fft.fft(torch.nn.functional.pad(irp, (0, N - hop)).to(torch.complex128), dim=-1)  # [K,N]
    Y = torch.zeros_like(X)
    for k in range(min(K, H)):
        Y[:, k:] = Y[:, k:] + X[:, :H - k] * Hk[k]
    y = torch.fft.ifft(Y, dim=-1).real * w * gain           # ifft includes the 1/N
    out = torch.zeros(V, H * hop + N, dtype=DT)
    for h in range(H):                                      # overlapAdd (Sources/DGen/Emit+FFT.swift:6-62)
        out[:, h * hop:h * hop + N] = out[:, h * hop:h * hop + N] + y[:, h]
    return out[:, :T]


def mss_loss(pred, target, sizes=(2048, 1024, 512, 256, 128, 64), hop_div=4, w_lin=1.0, w_log=1.0):
    """Sum over usable window sizes of L1 linear + L1 log-magnitude loss, batch mean, / frames
    (Sources/DGen/Emit+SpectralLoss.swift:719-938, Examples/HarmonicE2E/Trainer.swift:538-588)."""
    B, T = pred.shape
    usable = [n for n in sizes if 1 < n <= T]
    total = torch.zeros((), dtype=DT)
    for N in usable:
        hop = max(1, N // hop_div)
        H = (T + hop - 1) // hop
        w = t64(orc.hann_symmetric(N))

        def mags(x):
            xp = torch.nn.functional.pad(x, (N - 1, H * hop))
            fr = xp.unfold(1, N, hop)[:, :H]
            idx = torch.arange(H)[:, None] * hop - (N - 1) + torch.arange(N)[None, :]
            fr = fr * (idx < T).to(DT) * w
            return torch.fft.rfft(fr, dim=-1).abs()
        m1, m2 = mags(pred), mags(target)
        lin = (m1 - m2).abs().sum()
        lg = (torch.log(m1 + 1e-8) - torch.log(m2 + 1e-8)).abs().sum()
        total = total + (w_lin * lin + w_log * lg) / (B * len(usable) * T)
    return total


def heads(z, K):
    """Examples/HarmonicE2E/Model.swift:102-106 (softplus-normalised amplitudes) + sigmoid band magnitudes."""
    p = torch.nn.functional.softplus(z[:, :K])
    return p / (p.sum(-1, keepdim=True) + 1e-6), torch.sigmoid(z[:, K:])


def mlp(x, weights, biases):
    """tanh trunk + linear head (Model.swift:96-101)."""
    h = x
    for W, b in zip(weights[:-1], biases[:-1]):
        h = torch.tanh(h @ W + b)
    return h @ weights[-1] + biases[-1]
