"""GPU parity of the controller layers (matmul + bias + tanh, backward) and the device Adam step."""
import numpy as np
import pytest

import dgen_b200
from oracle import oracle as orc

pytestmark = pytest.mark.gpu
f32 = np.float32


@pytest.fixture(scope="module")
def ctx():
    c = dgen_b200.Context(0)
    yield c
    c.close()


def dev(a):
    import torch
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


@pytest.mark.parametrize("M,K,N,act", [(1000, 2, 512, 1), (777, 512, 512, 1), (300, 512, 165, 0), (1, 1, 1, 0),
                                       (129, 130, 131, 1), (4096, 512, 512, 1), (2052, 256, 165, 0)])
def test_linear_forward_and_backward_match_fp64(ctx, M, K, N, act):
    rng = np.random.default_rng(M + K + N)
    a = rng.standard_normal((M, K)).astype(f32)
    w = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(f32)
    b = rng.standard_normal(N).astype(f32)
    dc = rng.standard_normal((M, N)).astype(f32)
    z = a.astype(np.float64) @ w.astype(np.float64) + b
    c64 = np.tanh(z) if act else z
    c = ctx.linear_fwd(dev(a), dev(w), dev(b), act)
    # 3xTF32 on the tensor cores: products carry fp32-grade precision, the accumulator in tensor memory
    # truncates, which leaves ~1e-5 relative over a 512-long reduction (forward tolerance of the path: 1e-4)
    assert np.abs(c.cpu().numpy() - c64).max() < 5e-5 * max(1.0, np.abs(z).max())
    da, dw, db = ctx.linear_bwd(dev(a), dev(w), c, dev(dc), act)
    dz = dc * (1 - c64 ** 2) if act else dc.astype(np.float64)
    for got, want in ((da, dz @ w.astype(np.float64).T), (dw, a.astype(np.float64).T @ dz), (db, dz.sum(0))):
        want = np.asarray(want)
        assert np.abs(got.cpu().numpy() - want).max() < 1e-3 * max(1e-6, np.abs(want).max())  # gradient tolerance
    # the transposed copy of the output, and the weight gradient computed from a transposed input
    c2, ct = ctx.linear_fwd(dev(a), dev(w), dev(b), act, want_transposed=True)
    assert torch_equal(c2, c) and torch_equal(ct, c2.t().contiguous())
    _, dw2, _ = ctx.linear_bwd(dev(a), dev(w), c, dev(dc), act, a_t=dev(np.ascontiguousarray(a.T)))
    want = a.astype(np.float64).T @ dz
    assert np.abs(dw2.cpu().numpy() - want).max() < 1e-3 * max(1e-6, np.abs(want).max())


def torch_equal(x, y):
    import torch
    return torch.equal(x, y)


def test_linear_without_bias(ctx):
    rng = np.random.default_rng(0)
    a, w = rng.standard_normal((50, 7)).astype(f32), rng.standard_normal((7, 9)).astype(f32)
    c = ctx.linear_fwd(dev(a), dev(w)).cpu().numpy()
    assert np.abs(c - a @ w).max() < 1e-5


def test_adam_matches_the_reference_operation_order_bit_for_bit(ctx):
    rng = np.random.default_rng(1)
    n = 10007
    th = rng.standard_normal(n).astype(f32)
    m, v = np.zeros(n, f32), np.zeros(n, f32)
    d_th, d_m, d_v = dev(th), dev(m), dev(v)
    for t in (1, 2, 3):
        g = rng.standard_normal(n).astype(f32)
        orc.adam(th, g, m, v, t)
        ctx.adam_step(d_th, dev(g), d_m, d_v, t)
    assert np.array_equal(d_m.cpu().numpy(), m) and np.array_equal(d_v.cpu().numpy(), v)
    assert np.abs(d_th.cpu().numpy() - th).max() <= 1.2e-7 * np.abs(th).max()


def test_linear_backward_is_deterministic(ctx):
    rng = np.random.default_rng(2)
    a, w = dev(rng.standard_normal((999, 64)).astype(f32)), dev(rng.standard_normal((64, 33)).astype(f32))
    dc = dev(rng.standard_normal((999, 33)).astype(f32))
    c = ctx.linear_fwd(a, w)
    r1 = [t.cpu().numpy() for t in ctx.linear_bwd(a, w, c, dc)]
    r2 = [t.cpu().numpy() for t in ctx.linear_bwd(a, w, c, dc)]
    assert all(np.array_equal(x, y) for x, y in zip(r1, r2))
