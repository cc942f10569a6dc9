"""GPU parity of the training-step path (MLP forward, backward, Adam; second order with
create_graph) against the CPU oracle: config c1 at full size, c2 and c3 at reduced sizes with the
oracle and at full size through size-independent identities (the full-size steps against the
oracle: test_gpu_full_size.py)."""
import numpy as np
import pytest

from conftest import rng, max_rel

pytestmark = pytest.mark.gpu
TOL = 1e-4  # max relative error on gradients and updated weights (fp32; GEMMs run the default tensor-core
            # scheme, one tf32 MMA + two bf16 correction MMAs per product, 3xTF32 for N < 256, or FFMA)


def make_mlp_inputs(dims, batch, seed, bias_zero=False, x_dist="normal", out_dim=None):
    """Draw order: weights layer by layer (W then b), then x, then targets."""
    r = rng(seed)
    Ws, bs = [], []
    for i in range(len(dims) - 1):
        lim = np.sqrt(6.0 / dims[i])
        Ws.append(r.uniform(-lim, lim, (dims[i], dims[i + 1])).astype(np.float32))
        b = r.uniform(-lim, lim, (dims[i + 1],)).astype(np.float32)
        bs.append(np.zeros_like(b) if bias_zero else b)
    if x_dist == "uniform":
        x = r.uniform(0, 1, (batch, dims[0])).astype(np.float32)
        y = np.sin(np.float32(15) * x).astype(np.float32)
    else:
        x = r.standard_normal((batch, dims[0])).astype(np.float32)
        y = r.standard_normal((batch, dims[-1])).astype(np.float32)
    return Ws, bs, x, y


def train_step(L, fwd, Ws, bs, x, y, steps=1):
    W = [L.Array(w.copy(), requires_grad=True) for w in Ws]
    B = [L.Array(b.copy(), requires_grad=True) for b in bs]
    params = [p for wb in zip(W, B) for p in wb]
    opt = (L.optim.Adam if hasattr(L, "optim") else L.Adam)(params, lr=1e-3, beta1=0.9, beta2=0.999, eps=1e-8)
    X, Y = L.Array(x), L.Array(y)
    out = {}
    for _ in range(steps):
        loss = L.mse(fwd(L, X, W, B), Y)
        loss.backward()
        out = {"loss": loss.to_numpy(), "loss_shape": loss.shape(),
               "grads": [p.grad().to_numpy() for p in params],
               "grad_shapes": [p.grad().shape() for p in params]}
        opt.step()
        loss.zero_grad()
    out["params"] = [p.to_numpy() for p in params]
    out["m"] = [m.to_numpy() for m in opt.m]
    out["v"] = [v.to_numpy() for v in opt.v]
    out["m_shapes"] = [m.shape() for m in opt.m]
    out["t"] = float(opt.t)
    return out


def fwd_unfused(act):
    def f(L, X, W, B):
        pred = X
        for i in range(len(W)):
            pred = pred @ W[i] + B[i]
            if i < len(W) - 1:
                pred = getattr(L, act)(pred)
        return pred
    return f


def fwd_fused(act):
    def f(L, X, W, B):
        if hasattr(L, "nn"):
            args = [X, None]
            for w, b in zip(W, B):
                args += [w, b]
            return L.nn.mlp(args, activation=act)
        return L.mlp_forward(X, W, B, act)
    return f


def compare_steps(g, o, tol=TOL):
    assert g["loss_shape"] == o["loss_shape"] == [1]
    assert abs(g["loss"][0] - o["loss"][0]) <= tol * abs(o["loss"][0])
    assert g["grad_shapes"] == o["grad_shapes"]
    assert g["m_shapes"] == o["m_shapes"] and g["t"] == o["t"]
    for key in ("grads", "m", "v"):
        for a, b in zip(g[key], o[key]):
            assert max_rel(a, b) < tol, (key, max_rel(a, b))
    # Updated weights: Adam's first steps move a weight by lr*g/(|g|+eps), which is discontinuous
    # at g = 0, so weights whose gradient is within rounding of eps (|g| < 1e-6) can only agree to
    # within the step length; all others must meet the tolerance.
    for a, b, gr in zip(g["params"], o["params"], o["grads"]):
        tiny = np.abs(gr.reshape(b.shape)) < 1e-6
        assert max_rel(np.where(tiny, b, a), b) < tol, ("params", max_rel(np.where(tiny, b, a), b))
        assert np.abs(a - b)[tiny].max(initial=0.0) <= 2.5e-3 * g["t"]


@pytest.mark.parametrize("fused", [False, True])
def test_c1_small_mlp_train_step(nd, oracle, fused):
    """c1: 1->32->32->32->1, ReLU, bias on every layer, batch 128, x ~ U[0,1), y = sin(15x)."""
    Ws, bs, x, y = make_mlp_inputs([1, 32, 32, 32, 1], 128, 0, x_dist="uniform")
    fwd = fwd_fused("relu") if fused else fwd_unfused("relu")
    g = train_step(nd, fwd, Ws, bs, x, y, steps=3)
    o = train_step(oracle, fwd_unfused("relu"), Ws, bs, x, y, steps=3)
    compare_steps(g, o)
    assert g["grad_shapes"][1] == [1, 32] and g["m_shapes"][1] == [1, 32]   # bias gradient keeps its dim


def test_c1_matches_golden_fixture(nd):
    import os
    path = os.path.join(os.path.dirname(__file__), "golden", "c1_mlp_step.npz")
    gold = np.load(path)
    Ws, bs, x, y = make_mlp_inputs([1, 32, 32, 32, 1], 128, 0, x_dist="uniform")
    g = train_step(nd, fwd_fused("relu"), Ws, bs, x, y, steps=1)
    assert abs(g["loss"][0] - gold["loss"][0]) <= TOL * abs(gold["loss"][0])
    for i in range(8):
        assert max_rel(g["grads"][i], gold["grad_%d" % i]) < TOL
        assert max_rel(g["params"][i], gold["param_%d" % i]) < TOL


@pytest.mark.parametrize("act", ["tanh", "sigmoid", "relu"])
@pytest.mark.parametrize("fused", [False, True])
def test_c2_reduced_mlp_train_step(nd, oracle, act, fused):
    """c2 at reduced size (256->512->512->512->256, batch 384, zero bias, N(0,1) data)."""
    Ws, bs, x, y = make_mlp_inputs([256, 512, 512, 512, 256], 384, 0, bias_zero=True)
    oracle.config["mode"] = "fast"
    try:
        o = train_step(oracle, fwd_unfused(act), Ws, bs, x, y)
    finally:
        oracle.config["mode"] = "faithful"
    g = train_step(nd, fwd_fused(act) if fused else fwd_unfused(act), Ws, bs, x, y)
    compare_steps(g, o)


@pytest.mark.parametrize("act", ["tanh", "relu"])
def test_c2_reduced_with_mask_fused_into_dx_product(nd, oracle, act, monkeypatch):
    """The same step with the dX product of each layer applying the lower layer's activation
    derivative and summing its bias gradient in its epilogue (state.fuse_mask_into_dx)."""
    from endia_b200.autograd import state
    monkeypatch.setattr(state, "fuse_mask_into_dx", True)
    # the inputs of test_c2_reduced_mlp_train_step (relu's kink makes other draws flip single units)
    Ws, bs, x, y = make_mlp_inputs([256, 512, 512, 512, 256], 384, 0, bias_zero=True)
    oracle.config["mode"] = "fast"
    try:
        o = train_step(oracle, fwd_unfused(act), Ws, bs, x, y)
    finally:
        oracle.config["mode"] = "faithful"
    launches0 = nd._lib.lib.endia_b200_launch_count()
    g = train_step(nd, fwd_fused(act), Ws, bs, x, y)
    fused_launches = nd._lib.lib.endia_b200_launch_count() - launches0
    compare_steps(g, o)
    monkeypatch.setattr(state, "fuse_mask_into_dx", False)
    launches0 = nd._lib.lib.endia_b200_launch_count()
    train_step(nd, fwd_fused(act), Ws, bs, x, y)
    assert fused_launches < nd._lib.lib.endia_b200_launch_count() - launches0


def second_order(L, Ws, bs, x, fused):
    W = [L.Array(w.copy(), requires_grad=True) for w in Ws]
    B = [L.Array(b.copy(), requires_grad=True) for b in bs]
    X = L.Array(x, requires_grad=True)
    f = (fwd_fused("tanh") if fused else fwd_unfused("tanh"))(L, X, W, B)
    gx = L.grad(outs=[L.sum(f)], inputs=[X], create_graph=True)[0]
    pen = L.sum(gx * gx) / float(x.shape[0])
    loss = L.mean(f, [0, 1]) + 0.1 * pen
    grads = L.grad(outs=[loss], inputs=W + B)
    return {"loss": loss.to_numpy(), "gx": gx.to_numpy(), "grads": [g.to_numpy() for g in grads],
            "shapes": [g.shape() for g in grads]}


@pytest.mark.parametrize("fused", [False, True])
def test_c3_reduced_gradient_penalty(nd, oracle, fused):
    """c3 at reduced size (64->128->128->1, batch 256): loss = mean(f) + 0.1*mean|df/dx|^2 with
    create_graph=True, then backward to the weights (double backward through matmul and tanh)."""
    r = rng(0)
    d = [64, 128, 128, 1]
    Ws = [r.uniform(-np.sqrt(6 / d[i]), np.sqrt(6 / d[i]), (d[i], d[i + 1])).astype(np.float32) for i in range(3)]
    bs = [np.zeros(d[i + 1], np.float32) for i in range(3)]
    x = r.standard_normal((256, 64)).astype(np.float32)
    oracle.config["mode"] = "fast"
    try:
        o = second_order(oracle, Ws, bs, x, False)
    finally:
        oracle.config["mode"] = "faithful"
    g = second_order(nd, Ws, bs, x, fused)
    assert abs(g["loss"][0] - o["loss"][0]) <= TOL * abs(o["loss"][0])
    assert max_rel(g["gx"], o["gx"]) < TOL
    assert g["shapes"] == o["shapes"]
    for a, b in zip(g["grads"], o["grads"]):
        assert max_rel(a, b) < TOL, max_rel(a, b)


def test_fused_tanh_layer_third_order_matches_op_composition(nd):
    """The fused layer's create_graph VJP uses one op for (1 - y^2) * g whose own VJP is again
    differentiable: gradient of a penalty on the second derivative (three nested grad calls),
    fused layers against the same network written op by op."""
    r = rng(5)
    d = [16, 32, 1]
    Ws = [r.uniform(-1, 1, (d[i], d[i + 1])).astype(np.float32) for i in range(2)]
    bs = [r.uniform(-1, 1, d[i + 1]).astype(np.float32) for i in range(2)]
    x = r.standard_normal((24, 16)).astype(np.float32)

    def third(fwd):
        W = [nd.Array(w.copy(), requires_grad=True) for w in Ws]
        B = [nd.Array(b.copy(), requires_grad=True) for b in bs]
        X = nd.Array(x, requires_grad=True)
        f = fwd(nd, X, W, B)
        g1 = nd.grad(outs=[nd.sum(f)], inputs=[X], create_graph=True)[0]
        g2 = nd.grad(outs=[nd.sum(g1 * g1)], inputs=[X], create_graph=True)[0]
        g3 = nd.grad(outs=[nd.sum(g2 * g2)], inputs=W + B[:1])
        return [g1.to_numpy(), g2.to_numpy()] + [g.to_numpy() for g in g3]
    fused, plain = third(fwd_fused("tanh")), third(fwd_unfused("tanh"))
    for a, b in zip(fused, plain):
        assert np.abs(b).max() > 0
        assert max_rel(a, b) < 2e-5, max_rel(a, b)


def test_grad_of_inputs_skips_products_that_cannot_reach_them(nd):
    """grad(outs, inputs) walks only the paths to `inputs`: asking for the input gradient of a
    network runs no weight-gradient product (fewer launches, the weights get no gradient), and the
    input gradient equals the one a full backward() leaves on the input."""
    r = rng(11)
    d = [32, 256, 256, 8]
    Ws = [r.uniform(-0.3, 0.3, (d[i], d[i + 1])).astype(np.float32) for i in range(3)]
    bs = [r.uniform(-0.3, 0.3, d[i + 1]).astype(np.float32) for i in range(3)]
    x = r.standard_normal((128, 32)).astype(np.float32)

    def run(only_input):
        W = [nd.Array(w.copy(), requires_grad=True) for w in Ws]
        B = [nd.Array(b.copy(), requires_grad=True) for b in bs]
        X = nd.Array(x, requires_grad=True)
        out = nd.sum(fwd_fused("tanh")(nd, X, W, B))
        n0 = nd._lib.lib.endia_b200_launch_count()
        if only_input:
            gx = nd.grad(outs=[out], inputs=[X])[0]
        else:
            out.backward()
            gx = X.grad()
        return gx.to_numpy(), nd._lib.lib.endia_b200_launch_count() - n0, [w.has_grad() for w in W]
    g_only, launches_only, has_only = run(True)
    g_all, launches_all, has_all = run(False)
    assert np.array_equal(g_only, g_all)
    assert launches_only < launches_all
    assert has_only == [False] * 3 and has_all == [True] * 3


def test_functional_transforms_known_answers(nd):
    """README.md:62-76, 98-108 and examples/custom_ops_examples/custom_mul.mojo:64-71."""
    def foo(x):
        return nd.sum(x * x)
    x = nd.Array("[1.0, 2.0, 3.0]")
    assert nd.grad(foo)(x).to_numpy().tolist() == [2.0, 4.0, 6.0]
    assert np.array_equal(nd.hessian(foo)(x).to_numpy(), 2 * np.eye(3, dtype=np.float32))
    vg = nd.value_and_grad(lambda args: nd.sum(args[0] * args[1]))([nd.Array("[1, 2, 3]"), nd.Array("[4, 5, 6]")])
    assert vg[0][0].to_numpy().tolist() == [32.0]
    assert vg[1][0].to_numpy().tolist() == [4.0, 5.0, 6.0] and vg[1][1].to_numpy().tolist() == [1.0, 2.0, 3.0]
    a = nd.Array("[1.0, 2.0, 3.0]", requires_grad=True)
    y = nd.sum(a * a)
    dy = nd.grad(outs=[y], inputs=[a], create_graph=True)[0]
    d2 = nd.grad(outs=[nd.sum(dy)], inputs=[a])[0]
    assert dy.to_numpy().tolist() == [2.0, 4.0, 6.0] and d2.to_numpy().tolist() == [2.0, 2.0, 2.0]


def test_grad_accumulates_across_backward_calls(nd):
    a = nd.Array("[1.0, 2.0]", requires_grad=True)
    nd.sum(a * a).backward()
    nd.sum(a * a).backward()
    assert a.grad().to_numpy().tolist() == [4.0, 8.0]     # autograd/functional.mojo:55-57


def test_c2_full_size_gemm_identities(nd):
    """Full c2 layer shapes (batch 8192, 4096x4096): the forward product and both VJP products are
    checked with a Freivalds projection in float64 (u^T (A B) v == (A^T u)^T (B v)), which is
    independent of the problem size, plus linearity of the backward pass in the seed."""
    r = rng(1)
    M, K, N = 8192, 4096, 4096
    x = r.standard_normal((M, K)).astype(np.float32)
    w = r.uniform(-1, 1, (K, N)).astype(np.float32) * np.float32(np.sqrt(6 / K))
    g = r.standard_normal((M, N)).astype(np.float32)
    X, W, G = nd.Array(x), nd.Array(w), nd.Array(g)
    u, v = r.standard_normal(M), r.standard_normal(N)
    uk = r.standard_normal(K)
    y = nd.matmul(X, W).to_numpy().astype(np.float64)
    ref = (x.T.astype(np.float64) @ u) @ (w.astype(np.float64) @ v)
    assert abs(u @ y @ v - ref) <= 1e-4 * max(abs(ref), np.linalg.norm(u) * np.linalg.norm(y @ v) * 1e-3)
    dx = nd.matmul(G, W.T()).to_numpy().astype(np.float64)          # dX = dY W^T
    ref = (g.T.astype(np.float64) @ u) @ (w.T.astype(np.float64) @ uk)
    assert abs(u @ dx @ uk - ref) <= 1e-4 * max(abs(ref), np.linalg.norm(u) * np.linalg.norm(dx @ uk) * 1e-3)
    dw = nd.matmul(X.T(), G).to_numpy().astype(np.float64)          # dW = X^T dY
    ref = (x.astype(np.float64) @ uk) @ (g.astype(np.float64) @ v)
    assert abs(uk @ dw @ v - ref) <= 1e-4 * max(abs(ref), np.linalg.norm(uk) * np.linalg.norm(dw @ v) * 1e-3)
    # sampled entries against exact float64 dot products
    for (i, j) in [(0, 0), (M - 1, N - 1), (4097, 123), (17, 4000)]:
        assert abs(y[i, j] - x[i].astype(np.float64) @ w[:, j]) <= 1e-4 * np.linalg.norm(x[i]) * np.linalg.norm(w[:, j])
    for (i, j) in [(0, 0), (K - 1, N - 1), (1234, 77)]:
        assert abs(dw[i, j] - x[:, i].astype(np.float64) @ g[:, j]) <= 1e-4 * np.linalg.norm(x[:, i]) * np.linalg.norm(g[:, j])


@pytest.mark.parametrize("act,dims,batch", [("relu", [1, 32, 32, 32, 1], 128), ("tanh", [7, 64, 33, 5], 96),
                                            ("sigmoid", [3, 16, 2], 17), ("tanh", [128, 128, 128, 128, 128], 32)])
def test_fused_small_mlp_step_matches_oracle(nd, oracle, act, dims, batch):
    """The single-launch whole-step kernel (c1 and other small networks) over three steps. The last
    case is too large for all its weights to stay in shared memory beside the activations: each
    layer's weights then pass through the staging buffer."""
    Ws, bs, x, y = make_mlp_inputs(dims, batch, 0, x_dist="uniform" if dims[0] == 1 else "normal")
    if dims[0] == 1:
        y = np.sin(np.float32(15) * x).astype(np.float32)
    o = train_step(oracle, fwd_unfused(act), Ws, bs, x, y, steps=3)
    W = [nd.Array(w.copy(), requires_grad=True) for w in Ws]
    B = [nd.Array(b.copy(), requires_grad=True) for b in bs]
    params = [p for wb in zip(W, B) for p in wb]
    opt = nd.optim.Adam(params, lr=1e-3)
    X, Y = nd.Array(x), nd.Array(y)
    for _ in range(3):
        loss = nd.nn.fused_train_step(W, B, X, Y, opt, activation=act)
    g = {"loss": loss.to_numpy(), "loss_shape": loss.shape(), "grads": [p.grad().to_numpy() for p in params],
         "grad_shapes": [p.grad().shape() for p in params], "params": [p.to_numpy() for p in params],
         "m": [m.to_numpy() for m in opt.m], "v": [v.to_numpy() for v in opt.v],
         "m_shapes": [m.shape() for m in opt.m], "t": float(opt.t)}
    compare_steps(g, o)


def test_fused_small_mlp_step_rejects_large_networks(nd):
    W = [nd.Array([512, 16])]
    B = [nd.Array([16])]
    with pytest.raises(nd.EndiaError) as ei:
        nd.nn.fused_train_step(W, B, nd.Array([8, 512]), nd.Array([8, 16]))
    assert ei.value.status == -8


@pytest.mark.parametrize("name,kw", [("SGD", {"lr": 0.1}), ("SGD", {"lr": 0.1, "momentum": 0.9, "weight_decay": 0.01}),
                                     ("SGD", {"lr": 0.1, "weight_decay": 0.01}), ("SGD", {"lr": 0.1, "momentum": 0.9}),
                                     ("RMSprop", {"lr": 0.01}), ("Adagrad", {"lr": 0.1})])
def test_other_optimizers_vs_torch(nd, name, kw):
    """SGD / RMSprop / Adagrad over two steps against torch.optim with the same hyper-parameters."""
    import torch
    r = rng(3)
    w = r.standard_normal((6, 5)).astype(np.float32)
    x = r.standard_normal((9, 6)).astype(np.float32)
    W = nd.Array(w.copy(), requires_grad=True)
    tw = torch.tensor(w.copy(), requires_grad=True)
    opt = getattr(nd.optim, name)([W], **kw)
    tkw = dict(kw)
    if name == "RMSprop":
        tkw["alpha"] = 0.99
    topt = getattr(torch.optim, name)([tw], **tkw)
    for _ in range(2):
        loss = nd.sum(nd.square(nd.Array(x) @ W))
        loss.backward()
        opt.step()
        loss.zero_grad()
        topt.zero_grad()
        ((torch.tensor(x) @ tw) ** 2).sum().backward()
        topt.step()
    assert max_rel(W.to_numpy(), tw.detach().numpy()) < 1e-4


@pytest.mark.parametrize("name", ["SGD", "RMSprop", "Adagrad"])
def test_fused_optimizers_multi_tensor_formulas(nd, name):
    """One launch over a weight (odd size, so the scalar tail runs), and a bias whose gradient is
    (1, N): two steps against the reference's fp32 expressions evaluated in numpy, state shapes
    included (sgd.mojo:40-63, rmsprop.mojo:39-53, adagrad.mojo:36-45)."""
    r = rng(11)
    f32 = np.float32
    w, b = r.standard_normal((37, 29)).astype(f32), r.standard_normal(29).astype(f32)
    W, B = nd.Array(w.copy(), requires_grad=True), nd.Array(b.copy(), requires_grad=True)
    kw = {"SGD": dict(lr=0.05, momentum=0.9, weight_decay=0.01), "RMSprop": dict(lr=0.01, alpha=0.9, eps=1e-8),
          "Adagrad": dict(lr=0.1, eps=1e-10)}[name]
    opt = getattr(nd.optim, name)([W, B], **kw)
    sw, sb = np.zeros_like(w), np.zeros((1, 29), f32)
    for step in range(2):
        gw = r.standard_normal((37, 29)).astype(f32)
        gb = r.standard_normal((1, 29)).astype(f32)
        W.grad_(nd.Array(gw))
        B.grad_(nd.Array(gb))
        opt.step()
        for (p, g, s) in ((w, gw, sw), (b.reshape(1, 29), gb, sb)):
            if name == "SGD":
                s[...] = f32(0.9) * s - f32(0.05) * (g + f32(0.01) * p)
                p += s
            elif name == "RMSprop":
                s[...] = f32(0.9) * s + (f32(1) - f32(0.9)) * g * g
                p -= f32(0.01) * g / (np.sqrt(s) + f32(1e-8))
            else:
                s[...] = s + g * g
                p -= f32(0.1) * g / (np.sqrt(s) + f32(1e-10))
    state = opt.velocity if name == "SGD" else opt.cache
    assert state[1].shape() == [1, 29] and B.shape() == [29]
    assert max_rel(W.to_numpy(), w) < 1e-5 and max_rel(B.to_numpy(), b) < 1e-5
    assert max_rel(state[0].to_numpy(), sw) < 1e-5 and max_rel(state[1].to_numpy(), sb) < 1e-5


BENCH_DIMS = [1, 32, 64, 128, 128, 128, 64, 32, 1]


def _bench_inputs():
    """Network and data of the reference's own benchmark programs
    (benchmarks/mlp_benchmarks/mlp_imp.mojo:20-37): batch 128, x ~ U[0, 1), y = sin(50 (x + 1) / 2)."""
    Ws, bs, x, _ = make_mlp_inputs(BENCH_DIMS, 128, 21, x_dist="uniform")
    y = np.sin(np.float32(50) * (x + np.float32(1)) / np.float32(2)).astype(np.float32)
    return Ws, bs, x, y


def test_reference_benchmark_mlp_imperative(nd, oracle):
    """mlp_imp.mojo:35-75: nn.MLP of the benchmark's depth, mse, backward, Adam.step, three steps."""
    Ws, bs, x, y = _bench_inputs()
    g = train_step(nd, fwd_fused("relu"), Ws, bs, x, y, steps=3)
    o = train_step(oracle, fwd_unfused("relu"), Ws, bs, x, y, steps=3)
    compare_steps(g, o)


def test_reference_benchmark_mlp_functional(nd, oracle):
    """mlp_func.mojo:86-131: value_and_grad of a pure forward function over the argument list
    [x, y, W1, b1, ...] and Adam written as array expressions with in-place updates."""
    Ws, bs, x, y = _bench_inputs()
    args = [nd.Array(x), nd.Array(y)]
    for w, b in zip(Ws, bs):
        args += [nd.Array(w.copy()), nd.Array(b.copy())]

    def fwd(a):
        return nd.mse(nd.nn.mlp([a[0], None] + list(a[2:]), activation="relu"), a[1])

    vag = nd.value_and_grad(fwd)
    f32 = np.float32
    lr, b1, b2, eps = 1e-3, 0.9, 0.999, 1e-8
    m = [nd.Array(a.shape()) for a in args]
    v = [nd.Array(a.shape()) for a in args]
    loss = None
    for t in range(1, 3):
        res = vag(args)
        loss, grads = res[0][0], res[1]
        for i in range(2, len(args)):
            m[i] = b1 * m[i] + float(f32(1) - f32(b1)) * grads[i]
            v[i] = b2 * v[i] + float(f32(1) - f32(b2)) * grads[i] * grads[i]
            m_hat = m[i] / float(f32(1) - f32(b1) ** f32(t))
            v_hat = v[i] / float(f32(1) - f32(b2) ** f32(t))
            args[i] -= lr * m_hat / (nd.sqrt(v_hat) + eps)
    o = train_step(oracle, fwd_unfused("relu"), Ws, bs, x, y, steps=2)
    assert abs(loss.to_numpy()[0] - o["loss"][0]) <= TOL * abs(o["loss"][0])
    for i, (a, ref, gr) in enumerate(zip(args[2:], o["params"], o["grads"])):
        tiny = np.abs(gr.reshape(ref.shape)) < 1e-6
        got = a.to_numpy().reshape(ref.shape)
        assert max_rel(np.where(tiny, ref, got), ref) < TOL, i


def test_captured_step_replays_double_backward(nd):
    """utils.CapturedStep: the create_graph=True step replayed as a CUDA graph gives the eager
    result, and follows its input array when that is refilled in place between replays."""
    import torch
    from endia_b200.utils.general import CapturedStep
    from endia_b200.dist import flat_tensor
    d = [64, 512, 512, 1]
    Ws, bs, x, _ = make_mlp_inputs(d, 512, 5, bias_zero=True)
    W = [nd.Array(w, requires_grad=True) for w in Ws]
    B = [nd.Array(b, requires_grad=True) for b in bs]
    X = nd.Array(x, requires_grad=True)

    def step():
        args = [X, None]
        for w, b in zip(W, B):
            args += [w, b]
        f = nd.nn.mlp(args, activation="tanh")
        gx = nd.grad(outs=[nd.sum(f)], inputs=[X], create_graph=True)[0]
        loss = nd.mean(f, [0, 1]) + 0.1 * (nd.sum(gx * gx) / 512.0)
        return loss, nd.grad(outs=[loss], inputs=W + B)

    loss_e, grads_e = step()
    ref = [loss_e.to_numpy()] + [g.to_numpy() for g in grads_e]
    cap = CapturedStep(step)
    assert cap.launches_per_replay > 20
    loss_c, grads_c = cap()
    got = [loss_c.to_numpy()] + [g.to_numpy() for g in grads_c]
    for a, b in zip(got, ref):
        assert np.array_equal(a, b)
    x2 = rng(6).standard_normal(x.shape).astype(np.float32)
    flat_tensor(X).copy_(torch.from_numpy(x2).reshape(-1))
    loss_c, grads_c = cap()
    got2 = [loss_c.to_numpy()] + [g.to_numpy() for g in grads_c]
    X2 = nd.Array(x2, requires_grad=True)
    X_saved, X = X, X2          # eager run on the new input
    loss_e2, grads_e2 = step()
    for a, b in zip(got2, [loss_e2.to_numpy()] + [g.to_numpy() for g in grads_e2]):
        assert np.array_equal(a, b)


def test_fused_mse_forward_and_vjps(nd, oracle):
    """mse as one fused kernel (loss_ops/mse_op.mojo:18-20): seeded directly, scaled by a later
    op (the VJP then multiplies by the incoming gradient), with a target that needs a gradient,
    through a transposed (non-contiguous) prediction (op composition), and under create_graph."""
    r = rng(41)
    p = r.standard_normal((37, 21)).astype(np.float32)
    t = r.standard_normal((37, 21)).astype(np.float32)

    def run(L, scale, tgrad, transposed, second):
        P = L.Array(p.T.copy() if transposed else p, requires_grad=True)
        T = L.Array(t, requires_grad=tgrad)
        loss = L.mse(P.T() if transposed else P, T)
        if scale:
            loss = loss * 3.0
        if second:
            g = L.grad(outs=[loss], inputs=[P], create_graph=True)[0]
            loss2 = L.sum(g * g)
            g2 = L.grad(outs=[loss2], inputs=[P])[0]
            return [loss.to_numpy(), g.to_numpy(), g2.to_numpy()]
        loss.backward()
        out = [loss.to_numpy(), P.grad().to_numpy()]
        if tgrad:
            out.append(T.grad().to_numpy())
        return out

    for case in [(False, False, False, False), (True, False, False, False), (True, True, False, False),
                 (False, False, True, False), (True, False, False, True)]:
        got, ref = run(nd, *case), run(oracle, *case)
        for a, b in zip(got, ref):
            assert a.shape == b.shape and max_rel(a, b) < 1e-5, case
    launches0 = nd._lib.lib.endia_b200_launch_count()
    P, T = nd.Array(p, requires_grad=True), nd.Array(t)
    nd.mse(P, T).backward()
    assert nd._lib.lib.endia_b200_launch_count() - launches0 <= 4   # fill of the seed, two mse kernels


@pytest.mark.parametrize("opt_name", ["Adam", "SGD", "RMSprop"])
def test_checkpoint_resume_is_bit_exact(nd, tmp_path, opt_name):
    """utils.checkpoint: parameters and optimizer state (Adam's m, v, t with the (1, N) moment shapes
    of the biases) saved after step k; a fresh network that loads them reproduces step k+1 bit for
    bit, weights, state and loss."""
    from endia_b200.utils import checkpoint
    Ws, bs, x, y = make_mlp_inputs([16, 256, 256, 8], 128, 9)
    X, Y = nd.Array(x), nd.Array(y)

    def make():
        W = [nd.Array(w.copy(), requires_grad=True) for w in Ws]
        B = [nd.Array(b.copy(), requires_grad=True) for b in bs]
        params = [p for wb in zip(W, B) for p in wb]
        kw = {"Adam": {}, "SGD": {"momentum": 0.9, "lr": 0.05}, "RMSprop": {}}[opt_name]
        return params, getattr(nd.optim, opt_name)(params, **kw)

    def step(params, opt):
        loss = nd.mse(nd.nn.mlp([X, None] + params, activation="tanh"), Y)
        loss.backward()
        opt.step()
        loss.zero_grad()
        return loss.to_numpy()

    params, opt = make()
    for _ in range(3):
        step(params, opt)
    manifest = checkpoint.save(str(tmp_path / "run"), params, opt)
    assert manifest["optimizer"]["type"] == opt_name and len(manifest["tensors"]) >= 2 * len(params)
    want_loss = step(params, opt)
    want = [p.to_numpy() for p in params]
    params2, opt2 = make()
    checkpoint.load(str(tmp_path / "run"), params2, opt2)
    if opt_name == "Adam":
        assert opt2.t == 4.0 and opt2.m[1].shape() == [1, 256]
    got_loss = step(params2, opt2)
    assert np.array_equal(got_loss, want_loss)
    for a, b in zip([p.to_numpy() for p in params2], want):
        assert np.array_equal(a, b)
    state = "m" if opt_name == "Adam" else ("velocity" if opt_name == "SGD" else "cache")
    for a, b in zip(getattr(opt2, state), getattr(opt, state)):
        assert np.array_equal(a.to_numpy(), b.to_numpy())
    with pytest.raises(nd.EndiaError):
        checkpoint.load(str(tmp_path / "run"), params2[:-1] + [nd.Array([3])], opt2)


def test_torch_bridges(nd):
    """utils.array_conversions (to_torch / from_torch / is_close, array_conversions.mojo:21-135)."""
    import torch
    from endia_b200.utils import array_conversions as ac
    r = rng(12)
    x = r.standard_normal((5, 7)).astype(np.float32)
    z = (r.standard_normal((3, 4)) + 1j * r.standard_normal((3, 4))).astype(np.complex64)
    X = nd.Array(x, requires_grad=True)
    t = ac.to_torch(X)
    assert t.is_cuda and t.requires_grad and np.array_equal(t.detach().cpu().numpy(), x)
    assert np.array_equal(ac.to_torch(X.T()).detach().cpu().numpy(), x.T)
    tz = ac.to_torch(nd.Array(z))
    assert tz.dtype == torch.complex64 and np.array_equal(tz.cpu().numpy(), z)
    back = ac.from_torch(torch.from_numpy(z))
    assert back.is_complex() and back.shape() == [3, 4] and np.array_equal(back.to_numpy(), z)
    assert ac.is_close(nd.tanh(X), torch.tanh(torch.from_numpy(x)))
    view = ac.to_torch(X, copy=False)
    view.mul_(2.0)
    assert np.array_equal(X.to_numpy(), 2 * x)
