"""GPU parity of single ops and their VJPs against the CPU oracle, on the reference's test shapes
and on ragged / edge shapes. Every program is written once against the shared Endia API and run
through both implementations on the same seeded inputs."""
import ctypes as C

import numpy as np
import pytest

from conftest import rng, rel_l2, max_rel

pytestmark = pytest.mark.gpu

TOL = 1e-4  # max relative error (floor = 1e-3 of the tensor's max), fp32 ops


def both(nd, eo, prog, *inputs):
    """Run prog(lib, *arrays) with both libraries; return lists of numpy results."""
    out_g = prog(nd, *[nd.Array(x, requires_grad=True) for x in inputs])
    out_o = prog(eo, *[eo.Array(x.copy(), requires_grad=True) for x in inputs])
    return [(g.to_numpy(), o.to_numpy(), g.shape(), o.shape()) for g, o in zip(out_g, out_o)]


def check(results, tol=TOL):
    for g, o, sg, so in results:
        assert sg == so, "shape metadata differs: %s vs %s" % (sg, so)
        if np.iscomplexobj(o):
            assert rel_l2(g, o) < tol
        else:
            assert max_rel(g, o) < tol, max_rel(g, o)


UNARY = ["neg", "relu", "tanh", "sigmoid", "square", "exp", "conj", "sin", "cos", "sinh", "cosh", "atan",
         "reciprocal"]


@pytest.mark.parametrize("name", UNARY)
def test_unary_fwd_grad(nd, oracle, name):
    x = rng(1).standard_normal((2, 30, 40)).astype(np.float32)

    def prog(L, X):
        y = getattr(L, name)(X)
        L.sum(y).backward()
        return [y, X.grad()]
    check(both(nd, oracle, prog, x))


@pytest.mark.parametrize("name", ["tan", "asin", "acos"])
def test_unary_bounded_domain(nd, oracle, name):
    x = rng(21).uniform(-0.9, 0.9, (2, 30, 40)).astype(np.float32)

    def prog(L, X):
        y = getattr(L, name)(X)
        L.sum(y * y).backward()
        return [y, X.grad()]
    check(both(nd, oracle, prog, x))


@pytest.mark.parametrize("name", ["sinh", "cosh", "tan", "asin", "acos", "atan", "sin", "cos", "reciprocal"])
def test_unary_catalogue_complex(nd, oracle, name):
    """The complex forms the reference defines for these ops (tan, acos, atan act on the real part;
    asin_op.mojo:103-104 has its own pair of formulas)."""
    r = rng(22)
    z = (r.uniform(-0.8, 0.8, (5, 17)) + 1j * r.uniform(-0.8, 0.8, (5, 17))).astype(np.complex64)

    def prog(L, Z):
        return [getattr(L, name)(Z)]
    check(both(nd, oracle, prog, z), 1e-5)


@pytest.mark.parametrize("shape,axes", [((6, 7, 8), [1]), ((128, 40), [0]), ((3, 5000), [1]), ((4, 33), [0, 1])])
def test_variance_std_prod(nd, oracle, shape, axes):
    """variance / std (variance_op.mojo:65-79, std_op.mojo) and reduce_mul / prod with their VJPs."""
    x = rng(23).uniform(0.9, 1.1, shape).astype(np.float32)

    def prog(L, X):
        v = L.variance(X, axes)
        sd = L.std(X, axes, unbiased=False, keepdims=True)
        p = L.reduce_mul(X, axes)
        L.sum(v).backward()
        gv = X.grad()
        X.remove_grad()
        L.sum(p).backward()
        return [v, sd, p, gv, X.grad(), L.prod(X) if X.size() < 300 else p]
    check(both(nd, oracle, prog, x))


def test_comparison_ops(nd):
    a = np.array([[1.0, 2.0, 3.0], [3.0, 2.0, 1.0]], np.float32)
    b = np.array([2.0, 2.0, 2.0], np.float32)
    A, B = nd.Array(a), nd.Array(b)
    for name, fn in [("greater", np.greater), ("greater_equal", np.greater_equal), ("less", np.less),
                     ("less_equal", np.less_equal), ("equal", np.equal), ("not_equal", np.not_equal)]:
        got = getattr(nd, name)(A, B)
        assert got.shape() == [2, 3] and not got.requires_grad()
        assert np.array_equal(got.to_numpy(), fn(a, b).astype(np.float32)), name


def test_forward_mode_matches_reverse_mode(nd):
    """nd.jvp walks the graph forward through every op's jvp rule; for random tangents t and
    cotangents g the two modes must agree on <g, J t> (a chain of elementwise ops, broadcasting,
    reductions, views, a matmul and a fused linear layer; then a transform of a complex array)."""
    r = rng(24)
    x = r.uniform(0.3, 0.9, (6, 8)).astype(np.float32)
    w = r.standard_normal((8, 5)).astype(np.float32)
    b = r.standard_normal(5).astype(np.float32)

    def f(X, W, Bv):
        h = nd.nn.linear(nd.tanh(X) * nd.sinh(X) + nd.sqrt(X) / nd.exp(X), W, Bv, "sigmoid")
        h = nd.matmul(h, W.T()) - nd.atan(X) + nd.reduce_add(nd.square(X), [1])
        z = nd.reshape(nd.permute(h, [1, 0]), [2, 4, 6])
        return nd.squeeze(z * z), nd.mean(nd.log(X) + nd.cos(X) * nd.asin(X), [0])

    X, W, Bv = (nd.Array(v, requires_grad=True) for v in (x, w, b))
    outs = f(X, W, Bv)
    tx, tw, tb = (r.standard_normal(v.shape).astype(np.float32) for v in (x, w, b))
    for out in outs:
        g = r.standard_normal(out.shape()).astype(np.float32)
        jt = nd.jvp(out, [X, W, Bv], [nd.Array(tx), nd.Array(tw), nd.Array(tb)]).to_numpy()
        for p in (X, W, Bv):
            p.remove_grad()
        nd.sum(out * nd.Array(g)).backward()
        lhs = float(np.sum(jt.astype(np.float64) * g))
        rhs = sum(float(np.sum(p.grad().to_numpy().reshape(t.shape).astype(np.float64) * t))
                  for p, t in ((X, tx), (W, tw), (Bv, tb)))
        assert abs(lhs - rhs) <= 1e-4 * max(abs(lhs), abs(rhs), 1.0), (lhs, rhs)
    # y = real(fftn(z)) for complex z: <g, Re F t> = Re <F^H g, t>, and FFTN.vjp returns F^H g
    z = (r.standard_normal((4, 16)) + 1j * r.standard_normal((4, 16))).astype(np.complex64)
    t = (r.standard_normal((4, 16)) + 1j * r.standard_normal((4, 16))).astype(np.complex64)
    g = r.standard_normal((4, 16)).astype(np.float32)
    Z = nd.Array(z, requires_grad=True)
    y = nd.real(nd.fftn(Z))
    jt = nd.jvp(y, [Z], [nd.Array(t)]).to_numpy()
    nd.sum(y * nd.Array(g)).backward()
    lhs = float(np.sum(jt.astype(np.float64) * g))
    rhs = float(np.real(np.vdot(Z.grad().to_numpy().astype(np.complex128), t.astype(np.complex128))))
    assert abs(lhs - rhs) <= 1e-4 * max(abs(lhs), abs(rhs), 1.0), (lhs, rhs)


@pytest.mark.parametrize("name", ["sqrt", "abs", "log", "sign"])
def test_unary_positive_inputs(nd, oracle, name):
    x = (np.abs(rng(2).standard_normal((40, 50))) + 0.1).astype(np.float32)

    def prog(L, X):
        y = getattr(L, name)(X)
        L.sum(y * y).backward()
        return [y, X.grad()]
    check(both(nd, oracle, prog, x))


@pytest.mark.parametrize("name", ["neg", "square", "conj", "abs", "sign", "sqrt", "exp", "log", "tanh"])
def test_unary_complex(nd, oracle, name):
    r = rng(3)
    z = (r.standard_normal((6, 33)) + 1j * r.standard_normal((6, 33))).astype(np.complex64)

    def prog(L, Z):
        return [getattr(L, name)(Z)]
    check(both(nd, oracle, prog, z), tol=2e-5)


def test_relu_sigmoid_reject_complex(nd):
    z = nd.Array(np.ones((4,), np.complex64))
    with pytest.raises(nd.EndiaError):
        nd.relu(z)
    with pytest.raises(nd.EndiaError):
        nd.sigmoid(z)


@pytest.mark.parametrize("name", ["add", "sub", "mul", "div"])
@pytest.mark.parametrize("shapes", [((2, 30, 40), (30, 40)), ((128, 32), (32,)), ((7, 1, 5), (3, 1)),
                                    ((1,), (9, 13)), ((64, 64), (64, 64))])
def test_binary_broadcast_fwd_grad(nd, oracle, name, shapes):
    r = rng(4)
    a = r.standard_normal(shapes[0]).astype(np.float32)
    b = (r.standard_normal(shapes[1]) + 3.0).astype(np.float32)

    def prog(L, A, B):
        y = getattr(L, name)(A, B)
        L.sum(y * y).backward()
        return [y, A.grad(), B.grad()]
    check(both(nd, oracle, prog, a, b))


def test_binary_complex_and_pow(nd, oracle):
    r = rng(5)
    a = (r.standard_normal((5, 17)) + 1j * r.standard_normal((5, 17))).astype(np.complex64)
    b = (r.standard_normal((17,)) + 1j * r.standard_normal((17,)) + 2).astype(np.complex64)
    p = (np.abs(r.standard_normal((5, 17))) + 0.5).astype(np.float32)

    def prog(L, A, B):
        return [L.mul(A, B), L.div(A, B), L.add(A, B), L.sub(A, B)]
    check(both(nd, oracle, prog, a, b), tol=2e-5)

    def prog2(L, P):
        y = P ** 3.0
        L.sum(y).backward()
        return [y, P.grad(), (-P) ** 2.0]
    check(both(nd, oracle, prog2, p))


def test_scalar_operator_sugar(nd, oracle):
    x = rng(6).standard_normal((12, 20)).astype(np.float32)

    def prog(L, X):
        y = (1.0 - 2.0 * X) / 4.0 + X * X - 0.5
        L.sum(y).backward()
        return [y, X.grad()]
    check(both(nd, oracle, prog, x))


@pytest.mark.parametrize("shape,axes", [((2, 30, 40), [1]), ((2, 30, 40), [0, 2]), ((128, 32), [0]),
                                        ((8192, 64), [0]), ((3, 5000), [1]), ((70000,), [0]),
                                        ((4, 3, 2, 5), [1, 3]), ((1, 1), [0, 1])])
def test_reduce_add_mean_sum(nd, oracle, shape, axes):
    x = rng(7).standard_normal(shape).astype(np.float32)

    def prog(L, X):
        red = L.reduce_add(X, axes)
        m = L.mean(X, axes)
        s = L.sum(X * X)
        s.backward()
        return [red, m, s, X.grad()]
    # sums of many terms: the CPU order is sequential, the GPU order a tree -> 1e-4 on the result
    check(both(nd, oracle, prog, x), tol=2e-4)


def test_reduce_complex(nd, oracle):
    r = rng(8)
    z = (r.standard_normal((6, 40)) + 1j * r.standard_normal((6, 40))).astype(np.complex64)

    def prog(L, Z):
        return [L.reduce_add(Z, [0]), L.reduce_add(Z, [1]), L.sum(Z)]
    check(both(nd, oracle, prog, z), tol=2e-5)


def test_view_ops_metadata_and_grads(nd, oracle):
    x = rng(9).standard_normal((2, 30, 40)).astype(np.float32)

    def prog(L, X):
        p = L.permute(X, [2, 0, 1])
        e = L.expand(L.reduce_add(X, [0]), [2, 30, 40])
        u = L.unsqueeze(L.squeeze(L.reduce_add(X, [0, 1])), [0, 2])
        rsh = L.reshape(p, [40, 60])
        y = L.sum(rsh * 2.0) + L.sum(e * X) + L.sum(u)
        y.backward()
        return [p, e, u, rsh, y, X.grad()]
    res = both(nd, oracle, prog, x)
    check(res, tol=2e-4)
    # strides and offsets of the views must agree exactly
    X = nd.Array(x)
    O = oracle.Array(x)
    for fn in (lambda L, A: L.permute(A, [2, 0, 1]), lambda L, A: A.T(),
               lambda L, A: L.expand(L.reduce_add(A, [0]), [2, 30, 40]),
               lambda L, A: L.squeeze(L.reduce_add(A, [0, 1])),
               lambda L, A: L.unsqueeze(L.squeeze(L.reduce_add(A, [0, 1])), [0, 2])):
        g, o = fn(nd, X), fn(oracle, O)
        assert g.shape() == o.shape()
        assert [s for s, e in zip(g.stride(), g.shape()) if e > 1] == \
               [s for s, e in zip(o.stride(), o.shape()) if e > 1]
        assert g.storage_offset() == o.storage_offset()


MM_SHAPES = [((4096, 1024), (1024, 1)), ((4096, 1), (1, 1024)), ((1000, 300), (300, 3)), ((64, 4), (4, 200)),
             ((2, 30, 40), (40, 50)), ((128, 1), (1, 32)), ((128, 32), (32, 32)), ((128, 32), (32, 1)),
             ((1, 1), (1, 1)), ((33, 7), (7, 129)), ((257, 130), (130, 65)), ((3, 2, 9, 5), (2, 5, 4)),
             ((512, 300), (300, 260))]


@pytest.mark.parametrize("shapes", MM_SHAPES)
def test_matmul_fwd_and_vjp(nd, oracle, shapes):
    r = rng(10)
    a = r.standard_normal(shapes[0]).astype(np.float32)
    b = r.standard_normal(shapes[1]).astype(np.float32)

    def prog(L, A, B):
        y = L.matmul(A, B)
        L.sum(y * y).backward()
        return [y, A.grad(), B.grad()]
    oracle.config["mode"] = "fast"
    try:
        check(both(nd, oracle, prog, a, b))
    finally:
        oracle.config["mode"] = "faithful"


def test_matmul_square_weight_is_mathematically_correct(nd):
    r = rng(11)
    g = r.standard_normal((5, 4)).astype(np.float32)
    w = r.standard_normal((4, 4)).astype(np.float32)
    out = nd.matmul(nd.Array(g), nd.Array(w).T()).to_numpy()
    assert np.allclose(out, g @ w.T, atol=1e-5)


def test_matmul_complex(nd, oracle):
    r = rng(12)
    a = (r.standard_normal((9, 20)) + 1j * r.standard_normal((9, 20))).astype(np.complex64)
    b = (r.standard_normal((20, 11)) + 1j * r.standard_normal((20, 11))).astype(np.complex64)

    def prog(L, A, B):
        return [L.matmul(A, B), L.matmul(A, B.T().T())]
    check(both(nd, oracle, prog, a, b), tol=2e-5)


def test_matmul_rejects_bad_shapes(nd):
    with pytest.raises(nd.EndiaError):
        nd.matmul(nd.Array(np.ones((3, 4), np.float32)), nd.Array(np.ones((5, 6), np.float32)))


def _dev(nd, a):
    arr = nd.Array(np.ascontiguousarray(a))
    return arr


@pytest.mark.parametrize("algo", [1])
@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (200, 136, 72), (1, 5, 3), (130, 257, 33)])
def test_gemm_c_abi_all_layouts_with_epilogue(nd, ta, tb, M, N, K, algo):
    """endia_b200_gemm called directly: transposed operands, bias + activation, derivative mask,
    accumulation (beta) and the fused column sum."""
    from endia_b200 import _lib
    from endia_b200._array import stream, alloc
    r = rng(13)
    a = r.standard_normal((K, M) if ta else (M, K)).astype(np.float32)
    b = r.standard_normal((N, K) if tb else (K, N)).astype(np.float32)
    bias = r.standard_normal(N).astype(np.float32)
    saved = r.standard_normal((M, N)).astype(np.float32)
    c0 = r.standard_normal((M, N)).astype(np.float32)
    A, B, BIAS, SAVED, Cd = _dev(nd, a), _dev(nd, b), _dev(nd, bias), _dev(nd, saved), _dev(nd, c0)
    colsum = nd.Array([N])
    scratch = alloc(_lib.lib.endia_b200_gemm_colsum_scratch_bytes(M, N) // 4 + 1)
    epi = _lib.Epilogue()
    epi.alpha, epi.beta = 0.5, 2.0
    epi.bias = BIAS.data_ptr()
    epi.act, epi.dact = _lib.ACT_TANH, _lib.ACT_SIGMOID
    epi.dact_src, epi.ld_dact = SAVED.data_ptr(), N
    epi.colsum, epi.colsum_scratch = colsum.data_ptr(), scratch.data_ptr()
    _lib.call("endia_b200_gemm", ta, tb, M, N, K, A.data_ptr(), a.shape[1], B.data_ptr(), b.shape[1],
              Cd.data_ptr(), N, 1, 0, 0, 0, C.byref(epi), algo, stream())
    am = (a.T if ta else a).astype(np.float64)
    bm = (b.T if tb else b).astype(np.float64)
    v = np.tanh(0.5 * (am @ bm) + bias) * (saved.astype(np.float64) * (1 - saved)) + 2.0 * c0
    assert max_rel(Cd.to_numpy(), v) < TOL
    assert max_rel(colsum.to_numpy(), v.sum(0)) < 2e-4


def test_c_abi_error_codes(nd):
    from endia_b200 import _lib
    from endia_b200._array import stream
    x = nd.Array(np.ones((4, 6), np.complex64))
    y = nd.Array([4, 6], is_complex=True)
    dims = (C.c_int32 * 1)(1)
    st = _lib.lib.endia_b200_fft_c2c(x.desc(), y.desc(), dims, 1, 0, 1.0, None, stream())
    assert st == _lib.EPOW2 and b"power of two" in _lib.lib.endia_b200_last_error()
    st = _lib.lib.endia_b200_gemm(0, 0, 4, 4, 4, x.data_ptr(), 2, x.data_ptr(), 4, y.data_ptr(), 4, 1, 0,
                                  0, 0, None, 0, stream())
    assert st == _lib.EINVAL
    st = _lib.lib.endia_b200_ew_unary(99, x.desc(), y.desc(), stream())
    assert st == _lib.EINVAL
    st = _lib.lib.endia_b200_adam_step_multi(1, None, None, None, None, None, 1e-3, .9, .999, 1e-8, 1., 1., None)
    assert st == _lib.EINVAL


def test_empty_arrays(nd):
    e = nd.Array([0, 5])
    assert nd.add(e, e).shape() == [0, 5]
    assert nd.relu(e).to_numpy().shape == (0, 5)
    m = nd.matmul(nd.Array([0, 3]), nd.Array([3, 4]))
    assert m.shape() == [0, 4]


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(300, 1, 257), (300, 5, 64), (129, 70, 1), (64, 100, 3), (1, 1024, 4096),
                                   (3, 300, 200), (1024, 1, 4096), (4096, 1, 1024), (4096, 1024, 1),
                                   (8, 1024, 512), (4100, 4, 1028), (512, 8, 96), (2, 260, 4100), (700, 2, 8)])
def test_gemm_degenerate_shapes_with_epilogue(nd, ta, tb, M, N, K):
    """N <= 8, M <= 8 and K <= 8 take the one-pass kernels under GEMM_AUTO (rows, tall and outer
    product forms, with and without 16-byte accesses and K ranges over CTAs); bias, activation,
    mask and accumulation are fused there as well."""
    from endia_b200 import _lib
    from endia_b200._array import stream
    r = rng(21)
    a = r.standard_normal((K, M) if ta else (M, K)).astype(np.float32)
    b = r.standard_normal((N, K) if tb else (K, N)).astype(np.float32)
    bias = r.standard_normal(N).astype(np.float32)
    saved = r.standard_normal((M, N)).astype(np.float32)
    c0 = r.standard_normal((M, N)).astype(np.float32)
    A, B, BIAS, SAVED, Cd = _dev(nd, a), _dev(nd, b), _dev(nd, bias), _dev(nd, saved), _dev(nd, c0)
    epi = _lib.Epilogue()
    epi.alpha, epi.beta = 0.5, 2.0
    epi.bias = BIAS.data_ptr()
    epi.act, epi.dact = _lib.ACT_TANH, _lib.ACT_RELU
    epi.dact_src, epi.ld_dact = SAVED.data_ptr(), N
    _lib.call("endia_b200_gemm", ta, tb, M, N, K, A.data_ptr(), a.shape[1], B.data_ptr(), b.shape[1],
              Cd.data_ptr(), N, 1, 0, 0, 0, C.byref(epi), _lib.GEMM_AUTO, stream())
    am = (a.T if ta else a).astype(np.float64)
    bm = (b.T if tb else b).astype(np.float64)
    v = np.tanh(0.5 * (am @ bm) + bias) * (saved > 0) + 2.0 * c0
    assert max_rel(Cd.to_numpy(), v) < TOL


def test_copy_strided_both_sides(nd):
    """endia_b200_copy_strided: strided source into a strided destination (the placement step of
    the slab transpose), complex and real, with and without 128-bit runs."""
    from endia_b200 import _lib
    from endia_b200._array import stream, ArrayShape, Array
    r = rng(12)

    def view(arr, shape, stride, offset):
        v = Array(ArrayShape(shape, stride, offset))
        v.buf = arr.buf
        v.is_complex_flag = arr.is_complex()
        return v

    z = (r.standard_normal((6, 8, 10)) + 1j * r.standard_normal((6, 8, 10))).astype(np.complex64)
    src = nd.Array(z)
    dst_host = np.zeros((6, 16, 10), np.complex64)
    dst = nd.Array(dst_host)
    # rows 2..5 of axis 1 of src -> columns 8..11 of axis 1 of dst
    _lib.call("endia_b200_copy_strided", view(src, [6, 4, 10], [80, 10, 1], 20).desc(),
              view(dst, [6, 4, 10], [160, 10, 1], 80).desc(), stream())
    dst_host[:, 8:12, :] = z[:, 2:6, :]
    assert np.array_equal(dst.to_numpy(), dst_host)
    x = r.standard_normal((5, 7, 9)).astype(np.float32)          # odd run: scalar path
    a, b = nd.Array(x), nd.Array(np.zeros((7, 5, 9), np.float32))
    _lib.call("endia_b200_copy_strided", a.desc(), view(b, [5, 7, 9], [9, 45, 1], 0).desc(), stream())
    assert np.array_equal(b.to_numpy(), x.transpose(1, 0, 2))
    st = _lib.lib.endia_b200_copy_strided(view(a, [5, 9, 7], [63, 1, 9], 0).desc(), b.desc(), stream())
    assert st in (_lib.EINVAL, _lib.ESHAPE)


def test_act_bwd_colsum_writes_operand_parts(nd):
    """endia_b200_act_bwd_colsum_parts: dS, the bias gradient and the bf16 split of dS from one
    pass; the split must equal what endia_b200_bf16_split makes of dS."""
    import torch
    from endia_b200 import _lib
    from endia_b200._array import stream, alloc
    r = rng(41)
    M, N = 96, 256
    h = np.tanh(r.standard_normal((M, N))).astype(np.float32)
    g = r.standard_normal((M, N)).astype(np.float32)
    H, G, DS, DB = nd.Array(h), nd.Array(g), nd.Array([M, N]), nd.Array([1, N])
    scratch = alloc(_lib.lib.endia_b200_act_bwd_colsum_scratch_bytes(M, N) // 4 + 1)
    parts, ref_parts = alloc(M * N), alloc(M * N)
    _lib.call("endia_b200_act_bwd_colsum_parts", _lib.ACT_TANH, H.data_ptr(), G.data_ptr(), DS.data_ptr(),
              DB.data_ptr(), M, N, scratch.data_ptr(), parts.data_ptr(), stream())
    ds = g * (1.0 - h * h)
    assert max_rel(DS.to_numpy(), ds) < 1e-6 and max_rel(DB.to_numpy(), ds.sum(0, keepdims=True)) < 1e-5
    _lib.call("endia_b200_bf16_split", DS.data_ptr(), ref_parts.data_ptr(), M * N, stream())
    assert torch.equal(parts.view(torch.int32), ref_parts.view(torch.int32))
    st = _lib.lib.endia_b200_act_bwd_colsum_parts(_lib.ACT_TANH, H.data_ptr(), G.data_ptr(), DS.data_ptr(), None,
                                                  3, 5, None, parts.data_ptr(), stream())
    assert st == _lib.EINVAL


def test_malloc_quota_refuses_without_exhausting_the_device(nd):
    """Host-injected out-of-memory: with a quota set, endia_b200_malloc refuses a request that
    would exceed it (ENOMEM, message with the figures), frees give the room back, and an absurd
    request without a quota fails cleanly with the same status."""
    from endia_b200 import _lib
    from endia_b200._array import stream
    lib = _lib.lib
    a, b = C.c_void_p(), C.c_void_p()
    _lib.call("endia_b200_set_malloc_quota", 1 << 20)
    try:
        _lib.call("endia_b200_malloc", C.byref(a), 600 << 10, stream())
        assert lib.endia_b200_malloc(C.byref(b), 600 << 10, stream()) == _lib.ENOMEM
        assert b.value is None and b"quota" in lib.endia_b200_last_error()
        _lib.call("endia_b200_free", a, stream())
        _lib.call("endia_b200_malloc", C.byref(b), 600 << 10, stream())
        _lib.call("endia_b200_free", b, stream())
    finally:
        _lib.call("endia_b200_set_malloc_quota", 0)
    assert lib.endia_b200_malloc(C.byref(a), 1 << 50, stream()) == _lib.ENOMEM
    x = nd.Array(np.ones(8, np.float32))
    assert x.to_numpy().sum() == 8.0          # the context is intact
