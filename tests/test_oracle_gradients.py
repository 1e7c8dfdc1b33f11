"""The fp64 gradient references of the oracle agree with central finite differences of the fp64 forward."""
import numpy as np

from oracle import oracle as orc


def test_mss_loss_gradient_vs_finite_differences():
    rng = np.random.default_rng(0)
    B, T, sizes = 2, 1500, (512, 64)
    x, y = rng.standard_normal((B, T)), rng.standard_normal((B, T))
    g = orc.mss_loss_grad(x, y, sizes)
    for b, t in ((0, 3), (1, 700), (1, 64), (0, 1024)):
        h = 1e-6
        xp, xm = x.copy(), x.copy()
        xp[b, t] += h
        xm[b, t] -= h
        fd = (orc.mss_loss(xp, y, sizes, double=True) - orc.mss_loss(xm, y, sizes, double=True)) / (2 * h)
        assert abs(g[b, t] - fd) < 1e-5 * max(abs(fd), 1e-6)


def test_biquad_bank_gradient_vs_finite_differences():
    rng = np.random.default_rng(0)
    B, T = 2, 2000
    x = rng.standard_normal((B, T))
    cut, q = np.array([300.0, 2000.0, 7000.0]), np.array([0.7, 3.0, 6.0])
    tgt = orc.biquad_bank(x, cut * 1.05, q, double=True)
    loss, gc, gq = orc.biquad_bank_mse_grad(x, cut, q, tgt)
    f = lambda c, qq: ((orc.biquad_bank(x, c, qq, double=True) - tgt) ** 2).sum()
    assert abs(loss - f(cut, q)) < 1e-9 * loss
    for l in range(3):
        h = cut[l] * 1e-6
        cp, cm = cut.copy(), cut.copy()
        cp[l] += h
        cm[l] -= h
        assert abs((f(cp, q) - f(cm, q)) / (2 * h) - gc[l]) < 1e-5 * abs(gc[l])
        h = q[l] * 1e-6
        qp, qm = q.copy(), q.copy()
        qp[l] += h
        qm[l] -= h
        assert abs((f(cut, qp) - f(cut, qm)) / (2 * h) - gq[l]) < 1e-5 * abs(gq[l])


def test_single_precision_evaluation_of_the_l1_loss_gradient_shows_the_sign_flip_outliers():
    """Why the GPU loss-gradient test bounds a quantile and not the maximum.  The L1 terms carry
    sign(|X1| - |X2|) (and the sign of the log difference): in a bin where the two magnitudes agree to
    single-precision rounding, ANY fp32 evaluation may pick the other sign than the fp64 one, and one flipped bin
    moves every frame of its window by 2 x its weight.  The oracle itself, run in fp32 on the host (no GPU
    involved), shows exactly that against its own fp64 run: all but a fraction of a percent of the frames agree
    to 1e-3 norm-wise, while the worst frames are off by more -- the same picture the CUDA kernels give
    (tests/test_gpu_mss_loss.py::test_backward_matches_fp64_oracle uses the bounds asserted here)."""
    rng = np.random.default_rng(16000)
    B, T, sizes = 3, 16000, (2048, 1024, 512, 256, 128, 64)
    x = rng.standard_normal((B, T)).astype(np.float32)
    y = (0.7 * rng.standard_normal((B, T))).astype(np.float32)
    g64 = orc.mss_loss_grad(x, y, sizes, upstream=2.0, double=True)
    g32 = orc.mss_loss_grad(x, y, sizes, upstream=2.0, double=False)
    err = np.abs(g32.astype(np.float64) - g64)
    keep = err <= np.quantile(err, 0.995)
    bulk = np.linalg.norm(err[keep]) / np.linalg.norm(g64)
    worst = err.max() / np.abs(g64).max()
    typical = np.median(err) / np.abs(g64).max()
    print("fp32 host evaluation vs fp64: bulk (99.5 %%) l2 %.2e, median %.2e, worst frame %.2e" % (bulk, typical, worst))
    assert bulk < 1e-3                      # the bound of the GPU test holds for a plain fp32 evaluation ...
    assert worst < 5e-3
    assert worst > 20 * typical             # ... and its worst frames are outliers, far above the rounding floor
