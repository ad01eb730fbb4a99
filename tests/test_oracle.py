"""Pins the CPU oracle: the known answers the reference's example programs
imply, and independent float64 formulas (numpy / torch autograd)."""
import numpy as np
import pytest
import torch

from util import rel_err


def test_experimental_example_known_answers(orc):
    # src/examples/experimental.zig:19-69: x = sequence(1,1) [3,2], y = sequence(1,1) [2,2],
    # z = inner_product(x, y, "ij,jk->ik"); z.reverse(.keep) with seed grad 1.
    x = orc.sequence(np.empty((3, 2), np.float32), 1.0, 1.0)
    y = orc.sequence(np.empty((2, 2), np.float32), 1.0, 1.0)
    assert x.tolist() == [[1, 2], [3, 4], [5, 6]] and y.tolist() == [[1, 2], [3, 4]]
    z = orc.inner_product(x, y)
    assert z.tolist() == [[7, 10], [15, 22], [23, 34]]
    gz = orc.fill(np.empty_like(z), 1.0)                      # graph.zig:116 seed
    gx = orc.inner_product(gz, y, tb=True, c=np.zeros_like(x), beta=1.0)   # inner_product.zig:283-291
    gy = orc.inner_product(x, gz, ta=True, c=np.zeros_like(y), beta=1.0)   # inner_product.zig:293-300
    assert gx.tolist() == [[3, 7], [3, 7], [3, 7]]
    assert gy.tolist() == [[9, 9], [12, 12]]
    # the forward-mode lines of the same example: reduce + broadcast
    a = orc.reduce_ij_i(y)                                   # "ij->i"
    b = orc.broadcast_j_ij(a, np.empty((3, 2), np.float32))  # "j->ij"
    assert b.tolist() == [[3, 7], [3, 7], [3, 7]]
    c = orc.reduce_ij_j(x)                                   # "ij->j"
    d = orc.broadcast_i_ij(c, np.empty((2, 2), np.float32))  # "i->ij"
    assert d.tolist() == [[9, 9], [12, 12]]


def test_subgraphs_example_values(orc):
    # src/examples/subgraphs.zig:34-46: x = w1 = w2 = 1 (M = 32); z4 = relu(relu(x+w1)+w2) = 3
    one = orc.fill(np.empty(32, np.float32), 1.0)
    z2 = orc.relu(orc.addition(one, one))
    z4 = orc.relu(orc.addition(z2, one))
    assert np.all(z4 == 3.0)
    g4 = orc.fill(np.empty(32, np.float32), 1.0)
    g3 = orc.relu_reverse(orc.addition(z2, one), np.zeros(32, np.float32), g4)
    gw2 = orc.addition(g3, np.zeros(32, np.float32))          # addition.zig:67-81
    assert np.all(gw2 == 1.0)


@pytest.mark.parametrize("dt", [np.float32, np.float64])
def test_elementwise_against_numpy(orc, dt):
    r = np.random.default_rng(0)
    a = r.standard_normal(1000).astype(dt); b = r.standard_normal(1000).astype(dt)
    assert np.array_equal(orc.addition(a, b), a + b)
    assert np.array_equal(orc.subtraction(a, b), a - b)
    assert np.array_equal(orc.hadamard(a, b), a * b)
    assert np.array_equal(orc.negate(a), -a)
    assert np.array_equal(orc.relu(a), np.where(a >= 0, a, 0))
    assert np.array_equal(orc.stepwise(a), (a >= 0).astype(dt))
    assert np.array_equal(orc.copy(a), a)
    assert np.array_equal(orc.translate(a, 0.5), a + dt(0.5))
    assert np.array_equal(orc.dilate(a, 0.5), a * dt(0.5))
    lam, al = 1.0507009873554805, 1.6732632423543772
    a64 = a.astype(np.float64)
    assert rel_err(orc.selu(a), np.where(a64 > 0, lam * a64, lam * al * np.expm1(a64))) < 1e-6
    g = orc.selu_reverse(a, np.zeros_like(a), b)
    assert rel_err(g, b.astype(np.float64) * np.where(a64 > 0, lam, lam * al * np.exp(a64))) < 1e-6


def test_rank2_against_numpy(orc):
    r = np.random.default_rng(1)
    s = r.standard_normal((37, 53))
    assert np.array_equal(orc.permutate_ij_ji(s), s.T)
    d0 = r.standard_normal((53, 37))
    assert np.allclose(orc.permutate_ij_ji(s, d0.copy(), 1.0), s.T + d0)
    assert np.allclose(orc.reduce_ij_i(s), s.sum(1)) and np.allclose(orc.reduce_ij_j(s), s.sum(0))
    v = r.standard_normal(53)
    assert np.allclose(orc.reduce_ij_j(s, v.copy(), 1.0), s.sum(0) + v)
    assert np.array_equal(orc.broadcast_j_ij(v, np.empty((37, 53))), np.broadcast_to(v, (37, 53)))
    u = r.standard_normal(37)
    assert np.allclose(orc.broadcast_i_ij(u, s.copy(), 1.0), u[:, None] + s)
    # NaN in a fresh destination must not leak when alpha == 0
    bad = np.full((53, 37), np.nan)
    assert np.array_equal(orc.permutate_ij_ji(s, bad, 0.0), s.T)


def inverse_axes(perm):
    """numpy `axes` of the permutation whose source dimension i lands at output position perm[i]."""
    axes = [0] * len(perm)
    for i, q in enumerate(perm):
        axes[q] = i
    return axes


def test_general_permutation_against_numpy_and_the_rank2_instance(orc):
    import itertools
    r = np.random.default_rng(11)
    s = r.standard_normal((37, 53))
    assert np.array_equal(orc.permutate(s, [1, 0]), orc.permutate_ij_ji(s))          # pinned rank-2 instance
    for shape in [(3, 4, 5), (2, 1, 7, 3), (2, 3, 2, 3, 2, 3)]:
        x = r.standard_normal(shape).astype(np.float32)
        perms = list(itertools.permutations(range(len(shape))))
        for perm in perms[:: max(1, len(perms) // 24)]:
            ref = np.transpose(x, inverse_axes(perm))
            assert np.array_equal(orc.permutate(x, perm), ref), (shape, perm)
    x = r.standard_normal((3, 4, 5)); d0 = r.standard_normal((5, 3, 4))
    assert np.allclose(orc.permutate(x, [1, 2, 0], d0.copy(), 0.5), np.transpose(x, (2, 0, 1)) + 0.5 * d0)
    bad = np.full((5, 3, 4), np.nan)
    assert np.array_equal(orc.permutate(x, [1, 2, 0], bad, 0.0), np.transpose(x, (2, 0, 1)))


def test_contractions_against_numpy(orc):
    r = np.random.default_rng(2)
    a = r.standard_normal((5, 7)); b = r.standard_normal((7, 3)); c0 = r.standard_normal((5, 3)); bias = r.standard_normal(3)
    assert np.allclose(orc.inner_product(a, b), a @ b)
    assert np.allclose(orc.inner_product(a, b, 0.5, c0.copy(), 2.0), 0.5 * a @ b + 2 * c0)
    assert np.allclose(orc.inner_product(a, np.ascontiguousarray(b.T), tb=True), a @ b)
    assert np.allclose(orc.inner_product(np.ascontiguousarray(a.T), b, ta=True), a @ b)
    assert np.allclose(orc.inner_product(a, b, bias=bias), a @ b + bias)


def test_row_ops_against_torch_autograd(orc):
    torch.manual_seed(0)
    x = torch.randn(9, 33, dtype=torch.float64, requires_grad=True)
    gy = torch.randn(9, 33, dtype=torch.float64)
    y = torch.softmax(x, dim=1)
    y.backward(gy)
    yo = orc.softmax_ij_j(x.detach().numpy())
    assert rel_err(yo, y.detach().numpy()) < 1e-14
    assert rel_err(orc.softmax_ij_j_reverse(yo, gy.numpy()), x.grad.numpy()) < 1e-13
    g0 = np.random.default_rng(3).standard_normal((9, 33))
    assert rel_err(orc.softmax_ij_j_reverse(yo, gy.numpy(), g0.copy(), 1.0), x.grad.numpy() + g0) < 1e-13

    x = torch.randn(9, 33, dtype=torch.float64, requires_grad=True)
    gain = (1 + 0.02 * torch.randn(33, dtype=torch.float64)).requires_grad_()
    eps = 1e-6
    rstd = torch.rsqrt((x * x).mean(1, keepdim=True) + eps)
    y = x * rstd * gain
    y.backward(gy)
    yo, ro = orc.rmsnorm_ij_j(x.detach().numpy(), gain.detach().numpy(), eps)
    assert rel_err(yo, y.detach().numpy()) < 1e-14 and rel_err(ro, rstd.detach().numpy()[:, 0]) < 1e-14
    gx, gg = orc.rmsnorm_ij_j_reverse(x.detach().numpy(), gain.detach().numpy(), gy.numpy(), eps)
    assert rel_err(gx, x.grad.numpy()) < 1e-13 and rel_err(gg, gain.grad.numpy()) < 1e-13


def test_optimizers_against_formulas(orc):
    r = np.random.default_rng(4)
    w = r.standard_normal(100); g = r.standard_normal(100)
    assert np.allclose(orc.sgd(w.copy(), g, 1e-2), w - 1e-2 * g)
    assert np.allclose(orc.sgd(w.copy(), g, 1e-2, -0.5, 0.5), w - 1e-2 * np.clip(g, -0.5, 0.5))
    tw = torch.tensor(w, requires_grad=True)
    opt = torch.optim.Adam([tw], lr=3e-4, betas=(0.9, 0.95), eps=1e-8)
    m = np.zeros(100); v = np.zeros(100); wo = w.copy()
    for step in (1, 2, 3):
        gs = r.standard_normal(100)
        tw.grad = torch.tensor(gs)
        opt.step()
        orc.adam(wo, gs, m, v, 3e-4, 0.9, 0.95, 1e-8, 1.0, step)
    assert rel_err(wo, tw.detach().numpy()) < 1e-12


def _ssd_torch(x, dt, A, Bm, Cm):
    nb, L, H, P = x.shape
    G, N = Bm.shape[2], Bm.shape[3]
    ys = []
    S = torch.zeros(nb, H, N, P, dtype=x.dtype)
    for t in range(L):
        al = torch.exp(dt[:, t] * A)                                     # [nb,H]
        Bt = Bm[:, t].repeat_interleave(H // G, dim=1)                   # [nb,H,N]
        Ct = Cm[:, t].repeat_interleave(H // G, dim=1)
        S = al[..., None, None] * S + dt[:, t][..., None, None] * Bt[..., None] * x[:, t][:, :, None, :]
        ys.append(torch.einsum("bhn,bhnp->bhp", Ct, S))
    return torch.stack(ys, dim=1)


@pytest.mark.parametrize("G", [1, 2])
def test_ssd_oracle_against_torch_autograd(orc, G):
    torch.manual_seed(5)
    nb, L, H, P, N = 2, 12, 4, 3, 5
    x = torch.randn(nb, L, H, P, dtype=torch.float64, requires_grad=True)
    dt = torch.nn.functional.softplus(torch.randn(nb, L, H, dtype=torch.float64) - 1).requires_grad_()
    A = (-torch.exp(torch.rand(H, dtype=torch.float64) * 2)).requires_grad_()
    Bm = torch.randn(nb, L, G, N, dtype=torch.float64, requires_grad=True)
    Cm = torch.randn(nb, L, G, N, dtype=torch.float64, requires_grad=True)
    gy = torch.randn(nb, L, H, P, dtype=torch.float64)
    y = _ssd_torch(x, dt, A, Bm, Cm)
    y.backward(gy)
    n = lambda t: np.ascontiguousarray(t.detach().numpy())
    yo = orc.ssd_forward(n(x), n(dt), n(A), n(Bm), n(Cm))
    assert rel_err(yo, n(y)) < 1e-13
    gx, gdt, gA, gB, gC = orc.ssd_reverse(n(x), n(dt), n(A), n(Bm), n(Cm), n(gy))
    for got, ref, name in [(gx, x.grad, "gx"), (gdt, dt.grad, "gdt"), (gA, A.grad, "gA"), (gB, Bm.grad, "gB"), (gC, Cm.grad, "gC")]:
        assert rel_err(got, n(ref)) < 1e-12, name


def test_batched_contractions_against_numpy(orc):
    r = np.random.default_rng(12)
    a = r.standard_normal((4, 5, 7)); b = r.standard_normal((4, 7, 3)); c0 = r.standard_normal((4, 5, 3))
    assert np.allclose(orc.inner_product_batched(a, b), a @ b)
    assert np.allclose(orc.inner_product_batched(a, b, 0.5, c0.copy(), 2.0), 0.5 * a @ b + 2 * c0)
    assert np.allclose(orc.inner_product_batched(a, np.ascontiguousarray(b.transpose(0, 2, 1)), tb=True), a @ b)
    assert np.allclose(orc.inner_product_batched(np.ascontiguousarray(a.transpose(0, 2, 1)), b, ta=True), a @ b)


def test_c_and_numpy_momentum_agree(orc):
    import ctypes as C
    r = np.random.default_rng(13)
    w = r.standard_normal(100); g = r.standard_normal(100); m = r.standard_normal(100)
    w_ref, m_ref = orc.momentum(w, g, m, 0.1, 0.9, -0.5, 0.5)
    fn = orc.lib().orc_momentum_f64
    fn.restype = None
    wc, mc = w.copy(), m.copy()
    fn(C.c_void_p(wc.ctypes.data), C.c_void_p(g.ctypes.data), C.c_void_p(mc.ctypes.data), C.c_double(0.1), C.c_double(0.9),
       C.c_double(-0.5), C.c_double(0.5), C.c_size_t(100))
    assert np.allclose(wc, w_ref, rtol=0, atol=1e-15) and np.allclose(mc, m_ref, rtol=0, atol=1e-15)
