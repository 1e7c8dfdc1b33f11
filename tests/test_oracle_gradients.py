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
