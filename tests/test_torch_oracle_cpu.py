"""The autograd gradient reference (oracle/torch_oracle.py, fp64) computes the same forward values as the
scalar C oracle in double precision, so its gradients are gradients of the same graph."""
import numpy as np
import torch

from dgen_b200 import workloads as wl
from oracle import oracle as orc
from oracle import torch_oracle as to


def test_forward_values_agree_with_the_c_oracle():
    d = wl.harmonic_noise_inputs(3, B=2, T=2048, K=12, F=33, nbands=9, taps=17)
    rows = to.rows_of(d["F"], d["T"])
    taps = wl.taps_from_bands(d)
    h = to.harmonic_render(to.t64(d["f0"]), to.t64(d["uv"]), to.t64(d["amps"]), to.t64(d["gain"]), d["T"], d["sr"], rows)
    n = to.fir_noise(to.t64(d["noise"]), to.t64(taps), to.t64(d["noise_gain"]), rows)
    want = orc.harmonic_noise_render(d["f0"], d["uv"], d["amps"], d["gain"], d["noise_gain"], taps, d["noise"],
                                     d["T"], d["sr"], double=True)
    # the C oracle's double build also runs the control clock in double; the autograd reference keeps the
    # single-precision clock of the reference semantics, hence 1e-5 rather than 1e-12
    assert np.abs((h + n).numpy() - want).max() < 1e-5

    rng = np.random.default_rng(0)
    x, y = rng.standard_normal((2, 3000)), rng.standard_normal((2, 3000))
    got = float(to.mss_loss(to.t64(x), to.t64(y), sizes=(512, 64, 4096)))
    # the C oracle keeps the reference's Float twiddle table even in its double build: 1e-7 relative
    assert abs(got - orc.mss_loss(x, y, sizes=(512, 64, 4096), double=True)) < 1e-6 * got

    ir = rng.standard_normal(150) * np.exp(-np.arange(150) / 40)
    pc = to.partconv(to.t64(x), to.t64(ir), 64, 32, gain=0.7).numpy()
    want = np.stack([orc.partitioned_convolve(x[v], ir, 64, 32, gain=0.7, double=True) for v in range(2)])
    # window tables: single-precision (Swift Float.pi) in the autograd reference, double in the C build
    assert np.abs(pc - want).max() < 1e-5 * np.abs(want).max()


def test_autograd_loss_gradient_agrees_with_the_c_gradient_oracle():
    rng = np.random.default_rng(1)
    x, y = rng.standard_normal((2, 1500)), rng.standard_normal((2, 1500))
    xt = to.t64(x).requires_grad_(True)
    to.mss_loss(xt, to.t64(y), sizes=(256, 64)).backward()
    want = orc.mss_loss_grad(x, y, sizes=(256, 64))
    assert np.abs(xt.grad.numpy() - want).max() < 1e-5 * np.abs(want).max()


def test_f0_gradient_of_the_autograd_graph_agrees_with_finite_differences():
    """The temporal gradient through the phases (d loss / d f0) of the fp64 graph against central differences
    of the same graph with double-precision increments (a smooth function of f0)."""
    import torch
    F, B, K, T, sr = 6, 2, 5, 512, 16000.0
    rng = np.random.default_rng(9)
    f0 = to.t64(rng.uniform(100.0, 400.0, (F, B)).astype(np.float32)).requires_grad_(True)
    uv, gain = to.t64(rng.uniform(0.5, 1.0, (F, B))), to.t64(rng.uniform(0.5, 1.0, (F, B)))
    amps = to.t64(rng.uniform(0.1, 1.0, (F, B, K)))
    g = to.t64(rng.standard_normal((B, T)))
    rows = to.rows_of(F, T)

    def loss(f):
        return (to.harmonic_render(f, uv, amps, gain, T, sr, rows, reference_increments=False) * g).sum()
    loss(f0).backward()
    got = f0.grad.numpy()
    fd = np.zeros_like(got)
    with torch.no_grad():
        for r in range(F):
            for b in range(B):
                e = torch.zeros_like(f0)
                e[r, b] = 1e-4
                fd[r, b] = float(loss(f0 + e) - loss(f0 - e)) / 2e-4
    assert np.abs(got - fd).max() < 1e-5 * np.abs(fd).max()
