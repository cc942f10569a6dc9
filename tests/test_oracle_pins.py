"""Pins the CPU oracle: the reference's in-tree known answers, and equivalence to PyTorch CPU on
the reference's own test shapes (PyTorch is the value oracle of every reference test, compared at
mean relative error 1e-4, and 1e-5 for FFT forwards: endia/utils/array_conversions.mojo:63-135)."""
import numpy as np
import pytest
import torch

from conftest import rng, rel_l2


def mean_rel(a, b, eps):
    a = np.asarray(a); b = np.asarray(b)
    return float(np.mean(np.abs(a - b) / np.maximum(np.abs(b), eps)))


def test_readme_known_answers(oracle):
    eo = oracle
    # README.md:62-76: y = sum(x**2) at x = [1,2,3] -> 14, dy/dx = [2,4,6], d sum(dy/dx)/dx = [2,2,2]
    x = eo.Array("[1.0, 2.0, 3.0]", requires_grad=True)
    y = eo.sum(x * x)
    assert y.shape() == [1] and y.v[0] == 14.0
    dy = eo.grad([y], [x], create_graph=True)[0]
    assert dy.v.tolist() == [2.0, 4.0, 6.0]
    d2 = eo.grad([eo.sum(dy)], [x])[0]
    assert d2.v.tolist() == [2.0, 2.0, 2.0]


def test_readme_hessian_known_answer(oracle):
    eo = oracle
    # README.md:106-108: the Hessian of sum(x**2) is 2*I
    x = eo.Array("[1.0, 2.0, 3.0]", requires_grad=True)
    y = eo.sum(x * x)
    y.backward(create_graph=True)
    g = x.grad()
    eo.remove_grad_rec(y)
    g.backward()          # non-scalar output: identity seed -> full Jacobian of g wrt x
    assert np.array_equal(x.grad().v, 2 * np.eye(3, dtype=np.float32))


def test_custom_mul_known_answer(oracle):
    eo = oracle
    # examples/custom_ops_examples/custom_mul.mojo:64-71
    a = eo.Array("[1, 2, 3]", requires_grad=True)
    b = eo.Array("[4, 5, 6]", requires_grad=True)
    c = eo.sum(eo.mul(a, b))
    assert c.v.tolist() == [32.0]
    c.backward()
    assert a.grad().v.tolist() == [4.0, 5.0, 6.0] and b.grad().v.tolist() == [1.0, 2.0, 3.0]


@pytest.mark.parametrize("mode", ["faithful", "fast"])
def test_matmul_fwd_and_grad_vs_torch(oracle, mode):
    eo = oracle
    # tests/test_endia/test_functional/test_binary_ops/test_matmul_op.mojo:18-59
    r = rng(1)
    a = r.standard_normal((2, 30, 40)).astype(np.float32)
    b = r.standard_normal((40, 50)).astype(np.float32)
    eo.config["mode"] = mode
    try:
        A, B = eo.Array(a, requires_grad=True), eo.Array(b, requires_grad=True)
        out = eo.matmul(A, B)
        eo.sum(out).backward()
    finally:
        eo.config["mode"] = "faithful"
    ta, tb = torch.tensor(a, requires_grad=True), torch.tensor(b, requires_grad=True)
    tout = ta @ tb
    tout.sum().backward()
    assert mean_rel(out.v, tout.detach().numpy(), 1e-6) < 1e-4
    assert mean_rel(A.grad().v, ta.grad.numpy(), 1e-6) < 1e-4
    assert B.grad().shape() == [1, 40, 50]          # expanded batch dim is reduced with the dim kept
    assert mean_rel(B.grad().v[0], tb.grad.numpy(), 1e-6) < 1e-4


def test_fast_mode_engines_agree_with_faithful(oracle):
    """Fast mode (what checks the full-size configurations) computes the same product as the
    reference's loop: its C loop with float64 sums and, above config["blas_min_flops"], numpy's float64
    BLAS product both agree with the faithful float32 loop to float32 rounding of the terms."""
    eo = oracle
    r = rng(7)
    a = r.standard_normal((96, 200)).astype(np.float32)
    b = r.standard_normal((200, 64)).astype(np.float32)
    faithful = eo.matmul(eo.Array(a), eo.Array(b)).v
    old = eo.config["blas_min_flops"]
    try:
        eo.config["mode"] = "fast"
        c_loop = eo.matmul(eo.Array(a), eo.Array(b)).v
        eo.config["blas_min_flops"] = 0.0
        blas = eo.matmul(eo.Array(a), eo.Array(b)).v
        blas_t = eo.matmul(eo.Array(a), eo.Array(np.ascontiguousarray(b.T)).T()).v
    finally:
        eo.config["mode"] = "faithful"
        eo.config["blas_min_flops"] = old
    exact = a.astype(np.float64) @ b.astype(np.float64)
    scale = np.abs(a).astype(np.float64) @ np.abs(b).astype(np.float64)
    assert np.array_equal(c_loop, exact.astype(np.float32)) or (np.abs(c_loop - exact) / scale).max() < 1e-7
    assert (np.abs(blas - exact) / scale).max() < 1e-7 and np.array_equal(blas, blas_t)
    assert (np.abs(faithful - exact) / scale).max() < 2e-6


def test_square_weight_quirk_switch(oracle):
    eo = oracle
    r = rng(2)
    g = r.standard_normal((5, 4)).astype(np.float32)
    w = r.standard_normal((4, 4)).astype(np.float32)
    G, W = eo.Array(g), eo.Array(w)
    assert np.allclose(eo.matmul(G, W.T()).v, g @ w.T, atol=1e-5)      # default: the correct product
    eo.config["square_T_quirk"] = True
    try:
        assert np.allclose(eo.matmul(G, W.T()).v, g @ w, atol=1e-5)    # literal reference behaviour
        w2 = r.standard_normal((3, 4)).astype(np.float32)
        g2 = r.standard_normal((5, 4)).astype(np.float32)
        assert np.allclose(eo.matmul(eo.Array(g2), eo.Array(w2).T()).v, g2 @ w2.T, atol=1e-5)
        assert np.allclose(eo.matmul(G, W).v, g @ w, atol=1e-5)        # plain contiguous rhs unaffected
    finally:
        eo.config["square_T_quirk"] = False


UNARY = [("relu", torch.relu), ("tanh", torch.tanh), ("sigmoid", torch.sigmoid),
         ("square", torch.square), ("neg", torch.neg), ("exp", torch.exp),
         ("sin", torch.sin), ("cos", torch.cos), ("sinh", torch.sinh), ("cosh", torch.cosh),
         ("atan", torch.atan), ("reciprocal", torch.reciprocal)]


@pytest.mark.parametrize("name,tfn", UNARY)
def test_unary_fwd_and_grad_vs_torch(oracle, name, tfn):
    eo = oracle
    r = rng(3)
    x = r.standard_normal((2, 30, 40)).astype(np.float32)   # shape of tests/test_endia/test_functional/test_unary_ops/*
    X = eo.Array(x, requires_grad=True)
    out = getattr(eo, name)(X)
    eo.sum(out).backward()
    tx = torch.tensor(x, requires_grad=True)
    tout = tfn(tx)
    tout.sum().backward()
    assert mean_rel(out.v, tout.detach().numpy(), 1e-6) < 1e-4
    assert mean_rel(X.grad().v, tx.grad.numpy(), 1e-6) < 1e-4


@pytest.mark.parametrize("name,tfn", [("tan", torch.tan), ("asin", torch.asin), ("acos", torch.acos)])
def test_bounded_domain_unary_vs_torch(oracle, name, tfn):
    """tan / asin / acos on (-0.9, 0.9) (tests/test_endia/test_functional/test_unary_ops/)."""
    eo = oracle
    x = rng(4).uniform(-0.9, 0.9, (2, 30, 40)).astype(np.float32)
    X = eo.Array(x, requires_grad=True)
    out = getattr(eo, name)(X)
    eo.sum(out).backward()
    tx = torch.tensor(x, requires_grad=True)
    tfn(tx).sum().backward()
    assert mean_rel(out.v, tfn(tx).detach().numpy(), 1e-6) < 1e-4
    assert mean_rel(X.grad().v, tx.grad.numpy(), 1e-6) < 1e-4


def test_variance_std_prod_vs_torch(oracle):
    """reduce_ops/variance_op.mojo:65-79, std_op.mojo, reduce_mul_op.mojo / prod_op.mojo, forward and grad."""
    eo = oracle
    x = rng(5).uniform(0.5, 1.5, (6, 7, 8)).astype(np.float32)
    for unbiased in (True, False):
        X = eo.Array(x, requires_grad=True)
        v = eo.variance(X, [1], unbiased=unbiased)
        sd = eo.std(X, [0, 2], unbiased=unbiased, keepdims=True)
        eo.sum(v).backward()
        tx = torch.tensor(x, requires_grad=True)
        tv = tx.var(1, unbiased=unbiased)
        tv.sum().backward()
        assert v.shape() == [6, 8] and sd.shape() == [1, 7, 1]
        assert mean_rel(v.v, tv.detach().numpy(), 1e-6) < 1e-4
        assert mean_rel(X.grad().v, tx.grad.numpy(), 1e-6) < 1e-4
        assert mean_rel(sd.v, tx.std((0, 2), unbiased=unbiased, keepdim=True).detach().numpy(), 1e-6) < 1e-4
    X = eo.Array(x, requires_grad=True)
    p = eo.reduce_mul(X, [1])
    eo.sum(p).backward()
    tx = torch.tensor(x, requires_grad=True)
    tp = tx.prod(1, keepdim=True)
    tp.sum().backward()
    assert p.shape() == [6, 1, 8] and eo.prod(X).shape() == [1]
    assert mean_rel(p.v, tp.detach().numpy(), 1e-6) < 1e-4
    assert mean_rel(X.grad().v, tx.grad.numpy(), 1e-6) < 1e-4


def test_sqrt_abs_log_on_positive_inputs(oracle):
    eo = oracle
    x = (np.abs(rng(4).standard_normal((40, 50))) + 0.1).astype(np.float32)
    for name, tfn in (("sqrt", torch.sqrt), ("abs", torch.abs), ("log", torch.log)):
        X = eo.Array(x, requires_grad=True)
        out = getattr(eo, name)(X)
        eo.sum(out).backward()
        tx = torch.tensor(x, requires_grad=True)
        tfn(tx).sum().backward()
        assert mean_rel(out.v, tfn(torch.tensor(x)).numpy(), 1e-6) < 1e-4
        assert mean_rel(X.grad().v, tx.grad.numpy(), 1e-6) < 1e-4


BINARY = [("add", torch.add), ("sub", torch.sub), ("mul", torch.mul), ("div", torch.div)]


@pytest.mark.parametrize("name,tfn", BINARY)
def test_binary_broadcast_fwd_and_grad_vs_torch(oracle, name, tfn):
    eo = oracle
    r = rng(5)
    a = r.standard_normal((2, 30, 40)).astype(np.float32)
    b = (r.standard_normal((30, 40)) + 3.0).astype(np.float32)
    A, B = eo.Array(a, requires_grad=True), eo.Array(b, requires_grad=True)
    out = getattr(eo, name)(A, B)
    eo.sum(out).backward()
    ta, tb = torch.tensor(a, requires_grad=True), torch.tensor(b, requires_grad=True)
    tout = tfn(ta, tb)
    tout.sum().backward()
    assert mean_rel(out.v, tout.detach().numpy(), 1e-6) < 1e-4
    assert mean_rel(A.grad().v, ta.grad.numpy(), 1e-6) < 1e-4
    assert B.grad().shape() == [1, 30, 40]
    assert mean_rel(B.grad().v[0], tb.grad.numpy(), 1e-6) < 1e-4


def test_pow_vs_torch(oracle):
    eo = oracle
    r = rng(6)
    a = (np.abs(r.standard_normal((30, 40))) + 0.5).astype(np.float32)
    A = eo.Array(a, requires_grad=True)
    out = A ** 3.0
    eo.sum(out).backward()
    ta = torch.tensor(a, requires_grad=True)
    (ta ** 3.0).sum().backward()
    assert mean_rel(out.v, (a.astype(np.float64) ** 3), 1e-6) < 1e-4
    assert mean_rel(A.grad().v, ta.grad.numpy(), 1e-6) < 1e-4
    # a negative base follows the polar form: |x|^p * cos(pi p)
    assert np.allclose((eo.Array(np.array([-2.0], np.float32)) ** 2.0).v, [4.0], rtol=1e-5)


def test_reduce_and_view_ops_vs_torch(oracle):
    eo = oracle
    r = rng(7)
    x = r.standard_normal((2, 30, 40)).astype(np.float32)
    X = eo.Array(x, requires_grad=True)
    red = eo.reduce_add(X, [1])
    assert red.shape() == [2, 1, 40]                 # reduced dims stay (reduce_add_op.mojo:57-62)
    assert mean_rel(red.v, x.sum(1, keepdims=True), 1e-6) < 1e-4
    m = eo.mean(X, [0, 2])
    assert m.shape() == [30]
    assert mean_rel(m.v, x.mean((0, 2)), 1e-6) < 1e-4
    s = eo.sum(X)
    assert s.shape() == [1]
    p = eo.permute(X, [2, 0, 1])
    assert p.shape() == [40, 2, 30] and p.stride() == [1, 1200, 40]
    e = eo.expand(eo.Array(np.ones(40, np.float32)), [30, 40])
    assert e.shape() == [30, 40] and e.stride() == [0, 1]
    loss = eo.sum(eo.permute(X, [2, 0, 1]) * 2.0)
    loss.backward()
    assert np.allclose(X.grad().v, 2.0)


@pytest.mark.parametrize("shape,dims", [((4096,), [-1]), ((2, 3, 8, 1024), [-2, -1]),
                                        ((2, 2, 4, 16, 64), None)])
def test_fft_forward_vs_numpy(oracle, shape, dims):
    eo = oracle
    # tests/test_endia/test_fft/test_fft.mojo:22, test_fft2.mojo:22-29, test_fftn.mojo:22-30 (rtol 1e-5)
    r = rng(8)
    z = (r.standard_normal(shape) + 1j * r.standard_normal(shape)).astype(np.complex64)
    Z = eo.Array(z)
    y = eo.fftn(Z, dims)
    ref = np.fft.fftn(z.astype(np.complex128), axes=dims)
    assert mean_rel(y.v, ref, 1e-9) < 1e-5
    back = eo.ifftn(y, dims)
    assert rel_l2(back.v, z) < 1e-6


@pytest.mark.parametrize("norm", ["backward", "forward", "ortho"])
@pytest.mark.parametrize("shape,dims", [((8, 64), [-1]), ((4, 16, 32), [0, 2]), ((2, 8, 16), None)])
def test_fft_norm_modes_vs_numpy(oracle, shape, dims, norm):
    """Every `norm` follows numpy.fft, for partial dims too ("backward" is also the reference's
    scaling; the other two deliberately are not, see _norm_divisor), forward values and VJPs."""
    eo = oracle
    r = rng(18)
    z = (r.standard_normal(shape) + 1j * r.standard_normal(shape)).astype(np.complex64)
    w = r.uniform(-1, 1, shape).astype(np.float32)
    for fn, ref in ((eo.fftn, np.fft.fftn), (eo.ifftn, np.fft.ifftn)):
        Z = eo.Array(z, requires_grad=True)
        y = fn(Z, dims, norm)
        assert rel_l2(y.v, ref(z.astype(np.complex128), axes=dims, norm=norm)) < 1e-6
        eo.sum(eo.real(y) * eo.Array(w)).backward()
        want = np.conj(ref(w.astype(np.complex128), axes=dims, norm=norm))   # conj(F(conj(w + 0i)))
        assert rel_l2(Z.grad().v, want) < 1e-6
    with pytest.raises(ValueError):
        eo.fftn(eo.Array(z), dims, "bogus")


def test_fft_vjp_vs_torch(oracle):
    eo = oracle
    r = rng(9)
    z = (r.standard_normal((3, 256)) + 1j * r.standard_normal((3, 256))).astype(np.complex64)
    w = r.uniform(-1, 1, (3, 256)).astype(np.float32)
    Z = eo.Array(z, requires_grad=True)
    loss = eo.sum(eo.real(eo.fft(Z)) * eo.Array(w))
    loss.backward()
    tz = torch.tensor(z, requires_grad=True)
    (torch.fft.fft(tz).real * torch.tensor(w)).sum().backward()
    assert rel_l2(Z.grad().v, tz.grad.numpy()) < 1e-6
    Z2 = eo.Array(z, requires_grad=True)
    eo.sum(eo.square(eo.to_abs(eo.ifft(Z2)))).backward()
    tz2 = torch.tensor(z, requires_grad=True)
    (torch.fft.ifft(tz2).abs() ** 2).sum().backward()
    assert rel_l2(Z2.grad().v, tz2.grad.numpy()) < 1e-5


def test_mlp_adam_step_vs_torch(oracle):
    eo = oracle
    r = rng(0)
    dims = [1, 32, 32, 32, 1]
    Ws, bs = [], []
    for i in range(4):
        lim = np.sqrt(6 / dims[i])
        Ws.append(r.uniform(-lim, lim, (dims[i], dims[i + 1])).astype(np.float32))
        bs.append(r.uniform(-lim, lim, (dims[i + 1],)).astype(np.float32))
    x = r.uniform(0, 1, (128, 1)).astype(np.float32)
    y = np.sin(np.float32(15) * x).astype(np.float32)
    W = [eo.Array(w.copy(), requires_grad=True) for w in Ws]
    B = [eo.Array(b.copy(), requires_grad=True) for b in bs]
    loss = eo.mse(eo.mlp_forward(eo.Array(x), W, B, "relu"), eo.Array(y))
    loss.backward()
    opt = eo.Adam([p for wb in zip(W, B) for p in wb])
    opt.step()
    tW = [torch.tensor(w, requires_grad=True) for w in Ws]
    tB = [torch.tensor(b, requires_grad=True) for b in bs]
    h = torch.tensor(x)
    for i in range(4):
        h = h @ tW[i] + tB[i]
        if i < 3:
            h = torch.relu(h)
    tl = ((h - torch.tensor(y)) ** 2).mean()
    tl.backward()
    torch.optim.Adam([p for wb in zip(tW, tB) for p in wb], lr=1e-3).step()
    assert abs(loss.v[0] - tl.item()) < 1e-6 * max(1.0, abs(tl.item()))
    for i in range(4):
        assert B[i].grad().shape() == [1, dims[i + 1]]      # bias gradient keeps the reduced dim
        assert np.abs(W[i].grad().v - tW[i].grad.numpy()).max() < 1e-5
        assert np.abs(W[i].v - tW[i].detach().numpy()).max() < 1e-6
        assert np.abs(B[i].v - tB[i].detach().numpy()).max() < 1e-6
    assert opt.m[1].shape() == [1, 32] and float(opt.t) == 2.0


def test_second_order_gradient_penalty_vs_torch(oracle):
    eo = oracle
    r = rng(11)
    d = [16, 32, 32, 1]
    Ws = [(r.uniform(-1, 1, (d[i], d[i + 1])) * np.sqrt(6 / d[i])).astype(np.float32) for i in range(3)]
    xs = r.standard_normal((64, 16)).astype(np.float32)
    W = [eo.Array(w.copy(), requires_grad=True) for w in Ws]
    B = [eo.Array(np.zeros(d[i + 1], np.float32), requires_grad=True) for i in range(3)]
    X = eo.Array(xs, requires_grad=True)
    f = eo.mlp_forward(X, W, B, "tanh")
    gx = eo.grad([eo.sum(f)], [X], create_graph=True)[0]
    loss = eo.mean(f, [0, 1]) + 0.1 * (eo.sum(gx * gx) / 64.0)
    grads = eo.grad([loss], W + B)
    tW = [torch.tensor(w, requires_grad=True) for w in Ws]
    tB = [torch.zeros(d[i + 1], requires_grad=True) for i in range(3)]
    tx = torch.tensor(xs, requires_grad=True)
    h = tx
    for i in range(3):
        h = h @ tW[i] + tB[i]
        if i < 2:
            h = torch.tanh(h)
    tgx, = torch.autograd.grad(h.sum(), tx, create_graph=True)
    tloss = h.mean() + 0.1 * (tgx * tgx).sum() / 64
    tg = torch.autograd.grad(tloss, tW + tB)
    assert abs(loss.v[0] - tloss.item()) < 1e-5
    for a, b in zip(grads, tg):
        bn = b.numpy()
        assert np.abs(a.v.reshape(bn.shape) - bn).max() <= 1e-4 * max(np.abs(bn).max(), 1e-6)


def test_oracle_reproduces_golden_fixtures(oracle):
    """The committed fixtures (tests/golden/make_golden.py) pin the oracle against regressions."""
    import os
    from test_gpu_mlp import make_mlp_inputs, train_step, fwd_unfused
    eo = oracle
    here = os.path.join(os.path.dirname(__file__), "golden")
    gold = np.load(os.path.join(here, "c1_mlp_step.npz"))
    Ws, bs, x, y = make_mlp_inputs([1, 32, 32, 32, 1], 128, 0, x_dist="uniform")
    res = train_step(eo, fwd_unfused("relu"), Ws, bs, x, y, steps=1)
    assert np.array_equal(res["loss"], gold["loss"])
    for i in range(8):
        assert np.array_equal(res["grads"][i], gold["grad_%d" % i])
        assert np.array_equal(res["params"][i], gold["param_%d" % i])
    f = np.load(os.path.join(here, "fft_256.npz"))
    Z = eo.Array(f["x"], requires_grad=True)
    Y = eo.fft(Z)
    loss = eo.sum(eo.square(eo.to_abs(Y))) * (1.0 / 256)
    loss.backward()
    assert np.array_equal(Y.to_numpy(), f["y"]) and np.array_equal(Z.grad().to_numpy(), f["grad"])
    assert rel_l2(f["grad"], 2 * f["x"]) < 1e-6
