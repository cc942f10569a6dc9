"""GPU parity of the FFT family and its VJPs against the CPU oracle (float64 radix-2, as the
reference computes it): tolerance 1e-5 relative L2 for complex64 outputs and gradients."""
import numpy as np
import pytest

from conftest import rng, rel_l2

pytestmark = pytest.mark.gpu
TOL = 1e-5


def crandn(r, shape):
    return (r.standard_normal(shape) + 1j * r.standard_normal(shape)).astype(np.complex64)


@pytest.mark.parametrize("n", [1, 2, 4, 8, 16, 32, 64, 128, 256, 512, 1024, 2048, 4096, 8192, 16384, 65536])
def test_fft_1d_all_lengths(nd, oracle, n):
    z = crandn(rng(n), (3, n))
    y = nd.fft(nd.Array(z)).to_numpy()
    ref = oracle.fft(oracle.Array(z)).to_numpy()
    assert rel_l2(y, ref) < TOL
    back = nd.ifft(nd.Array(y)).to_numpy()
    assert rel_l2(back, z) < TOL


@pytest.mark.parametrize("shape,dims", [((4096,), [-1]), ((2, 3, 8, 1024), [-2, -1]), ((2, 2, 4, 16, 64), None),
                                        ((5, 64, 3), [1]), ((16, 7), [0]), ((8, 4, 32), [0, 2]),
                                        ((64, 64, 64), None), ((2, 128, 16), [-2])])
def test_fftn_reference_test_shapes_and_strided_axes(nd, oracle, shape, dims):
    z = crandn(rng(1), shape)
    y = nd.fftn(nd.Array(z), dims).to_numpy()
    ref = oracle.fftn(oracle.Array(z), dims).to_numpy()
    assert rel_l2(y, ref) < TOL
    yi = nd.ifftn(nd.Array(z), dims).to_numpy()
    refi = oracle.ifftn(oracle.Array(z), dims).to_numpy()
    assert rel_l2(yi, refi) < TOL


def test_fft_real_input_and_non_contiguous_view(nd, oracle):
    r = rng(2)
    x = r.standard_normal((6, 256)).astype(np.float32)
    assert rel_l2(nd.fft(nd.Array(x)).to_numpy(), oracle.fft(oracle.Array(x)).to_numpy()) < TOL
    z = crandn(r, (64, 32))
    yt = nd.fft(nd.Array(z).T()).to_numpy()                  # transposed (strided) view as input
    assert rel_l2(yt, oracle.fft(oracle.Array(z).T()).to_numpy()) < TOL


@pytest.mark.parametrize("norm", ["forward", "ortho"])
@pytest.mark.parametrize("shape,dims", [((8, 1024), [-1]), ((4, 16, 64), [0, 2]), ((2, 8, 32), None),
                                        ((2, 1 << 15), [1])])
def test_fft_norm_modes_vs_numpy(nd, shape, dims, norm):
    """norm = "forward" / "ortho" follow numpy.fft (the reference's scaling of these two modes is
    taken for a defect and not reproduced): fft/ifft/fftn/ifftn values and VJPs, partial dims."""
    r = rng(18)
    z = (r.standard_normal(shape) + 1j * r.standard_normal(shape)).astype(np.complex64)
    w = r.uniform(-1, 1, shape).astype(np.float32)
    for fn, ref in ((nd.fftn, np.fft.fftn), (nd.ifftn, np.fft.ifftn)):
        Z = nd.Array(z, requires_grad=True)
        y = fn(Z, dims, norm)
        assert rel_l2(y.to_numpy(), ref(z.astype(np.complex128), axes=dims, norm=norm)) < 2e-6
        nd.sum(nd.real(y) * nd.Array(w)).backward()
        want = np.conj(ref(w.astype(np.complex128), axes=dims, norm=norm))   # conj(F(conj(w + 0i)))
        assert rel_l2(Z.grad().to_numpy(), want) < 2e-6
    if dims is not None and len(dims) == 1:
        y1 = nd.fft(nd.Array(z), dims[0], norm).to_numpy()
        assert rel_l2(y1, np.fft.fft(z.astype(np.complex128), axis=dims[0], norm=norm)) < 2e-6
        y2 = nd.ifft(nd.Array(z), dims[0], norm).to_numpy()
        assert rel_l2(y2, np.fft.ifft(z.astype(np.complex128), axis=dims[0], norm=norm)) < 2e-6
    Z = nd.Array(z, requires_grad=True)
    nd.sum(nd.square(nd.to_abs(nd.fftn(Z, dims, norm)))).backward()      # the fused |y|^2 chain
    s = {"forward": 1.0 / np.prod([shape[d] for d in (dims if dims is not None else range(len(shape)))]),
         "ortho": 1.0}[norm]
    assert rel_l2(Z.grad().to_numpy(), 2.0 * s * z.astype(np.complex128)) < 2e-6   # Parseval


def test_fft_rejects_non_power_of_two(nd):
    with pytest.raises(nd.EndiaError) as ei:
        nd.fft(nd.Array(np.ones((4, 6), np.complex64)))
    assert ei.value.status == -6


@pytest.mark.parametrize("n,batch", [(1024, 4), (1 << 14, 2)])
def test_c4_reduced_fft_loss_and_vjp(nd, oracle, n, batch):
    """c4 at reduced size: loss = sum(|fft(x)|^2) / n; d loss / dx = 2x; ifft(fft(x)) = x."""
    z = crandn(rng(0), (batch, n))

    def prog(L):
        X = L.Array(z, requires_grad=True)
        y = L.fft(X)
        loss = L.sum(L.square(L.to_abs(y))) * (1.0 / n)
        loss.backward()
        return y.to_numpy(), X.grad().to_numpy(), loss.to_numpy(), L.ifft(L.fft(L.Array(z))).to_numpy()
    yg, gg, lg, zg = prog(nd)
    yo, go, lo, zo = prog(oracle)
    assert rel_l2(yg, yo) < TOL and rel_l2(gg, go) < TOL and rel_l2(zg, zo) < TOL
    assert rel_l2(gg, 2 * z) < TOL and rel_l2(zg, z) < TOL
    assert abs(lg[0] - lo[0]) <= 1e-4 * abs(lo[0])


def test_c5_reduced_fftn_loss_and_vjp(nd, oracle):
    """c5 at reduced size (32^3): loss = sum(real(fftn(x)) * w); d loss / dx = F^H (w + 0i)."""
    r = rng(0)
    z = crandn(r, (32, 32, 32))
    w = r.uniform(-1, 1, (32, 32, 32)).astype(np.float32)

    def prog(L):
        X = L.Array(z, requires_grad=True)
        y = L.fftn(X)
        loss = L.sum(L.real(y) * L.Array(w))
        loss.backward()
        return y.to_numpy(), X.grad().to_numpy(), loss.to_numpy()
    yg, gg, lg = prog(nd)
    yo, go, lo = prog(oracle)
    assert rel_l2(yg, yo) < TOL and rel_l2(gg, go) < TOL
    assert abs(lg[0] - lo[0]) <= 1e-4 * max(abs(lo[0]), np.abs(yo).max())
    assert rel_l2(gg, w.size * np.fft.ifftn(w.astype(np.complex128))) < TOL


def test_fft_vjp_with_create_graph(nd, oracle):
    z = crandn(rng(3), (2, 128))

    def prog(L):
        X = L.Array(z, requires_grad=True)
        y = L.sum(L.square(L.to_abs(L.fft(X))))
        g = L.grad(outs=[y], inputs=[X], create_graph=True)[0]
        return g.to_numpy()
    assert rel_l2(prog(nd), prog(oracle)) < TOL


def test_c4_full_size_identities(nd):
    """c4 at full size (32 x 2^20): Parseval, the inverse round trip and the analytic gradient 2x
    are checked without the CPU oracle; one signal is compared with a float64 FFT."""
    n, batch = 1 << 20, 32
    z = crandn(rng(0), (batch, n))
    X = nd.Array(z, requires_grad=True)
    y = nd.fft(X)
    loss = nd.sum(nd.square(nd.to_abs(y))) * (1.0 / n)
    loss.backward()
    yh = y.to_numpy()
    energy = float(np.sum(np.abs(z.astype(np.complex128)) ** 2))
    assert abs(loss.to_numpy()[0] - energy) <= 1e-4 * energy
    assert rel_l2(X.grad().to_numpy(), 2 * z) < TOL
    assert rel_l2(nd.ifft(y).to_numpy(), z) < TOL
    assert rel_l2(yh[5], np.fft.fft(z[5].astype(np.complex128))) < TOL


def test_c5_full_size_identities(nd):
    """c5 at full size (512^3), forward only: the inverse round trip, one output line against a
    float64 evaluation and the DC term (the VJP at this size: test_gpu_full_size.py)."""
    r = rng(0)
    shape = (512, 512, 512)
    z = crandn(r, shape)
    X = nd.Array(z)
    y = nd.fftn(X)
    back = nd.ifftn(y).to_numpy()
    assert rel_l2(back[::37, ::41, :], z[::37, ::41, :]) < TOL
    del back
    # one output line against a float64 evaluation of the separable transform
    yh = y.to_numpy()
    k0, k1 = 3, 500
    e0 = np.exp(-2j * np.pi * k0 * np.arange(512) / 512)
    e1 = np.exp(-2j * np.pi * k1 * np.arange(512) / 512)
    line = np.fft.fft(np.einsum("a,b,abc->c", e0, e1, z.astype(np.complex128)))
    assert rel_l2(yh[k0, k1], line) < TOL
    # DC term = sum of all inputs
    assert abs(yh[0, 0, 0] - z.astype(np.complex128).sum()) <= 1e-4 * np.sqrt(z.size)


def test_fft_matches_golden_fixture(nd):
    import os
    f = np.load(os.path.join(os.path.dirname(__file__), "golden", "fft_256.npz"))
    X = nd.Array(f["x"], requires_grad=True)
    y = nd.fft(X)
    loss = nd.sum(nd.square(nd.to_abs(y))) * (1.0 / 256)
    loss.backward()
    assert rel_l2(y.to_numpy(), f["y"]) < TOL and rel_l2(X.grad().to_numpy(), f["grad"]) < TOL
    assert abs(loss.to_numpy()[0] - f["loss"][0]) <= 1e-4 * abs(f["loss"][0])


@pytest.mark.parametrize("shape,dims", [((4, 1024), [1]), ((8, 16384), [1]), ((16, 32, 64), [0, 1, 2]),
                                        ((6, 256), [1]), ((3, 40), [0])])
def test_fft_reads_real_source_without_copy(nd, shape, dims):
    """endia_b200_fft_c2c with a real contiguous source (complex with zero imaginary part,
    fft_cooley_tukey.mojo:204-206): forward and conjugate direction, fast, four-step and generic
    kernels; shapes whose length is not a power of two are still refused."""
    import ctypes as C
    from endia_b200 import _lib
    from endia_b200._array import stream, alloc
    r = rng(31)
    x = r.standard_normal(shape).astype(np.float32)
    X, Y = nd.Array(x), nd.Array(list(shape), is_complex=True)
    cd = (C.c_int32 * len(dims))(*dims)
    nb = _lib.lib.endia_b200_fft_scratch_bytes(X.desc(), cd, len(dims))
    scratch = alloc(nb // 4 + 1) if nb else None
    sp = scratch.data_ptr() if scratch is not None else None
    if shape == (3, 40):
        st = _lib.lib.endia_b200_fft_c2c(X.desc(), Y.desc(), cd, len(dims), 0, 1.0, sp, stream())
        assert st != 0
        return
    for inverse in (0, 1):
        _lib.call("endia_b200_fft_c2c", X.desc(), Y.desc(), cd, len(dims), inverse, 1.0, sp, stream())
        ref = np.fft.fftn(x.astype(np.float64), axes=dims)
        if inverse:
            ref = np.conj(ref)        # conj(F(conj(x))) with real x
        assert rel_l2(Y.to_numpy(), ref) < 1e-5


def test_real_vjp_gradient_stays_lazy_into_fft(nd):
    """d/dx sum(real(fftn(x)) * w): the gradient of real() is complex(g, 0), which the FFT VJP reads
    from the real array; asking for it as an array gives the same values."""
    from endia_b200._array import LazyComplex
    r = rng(32)
    z = (r.standard_normal((8, 16, 32)) + 1j * r.standard_normal((8, 16, 32))).astype(np.complex64)
    w = r.uniform(-1, 1, (8, 16, 32)).astype(np.float32)
    X = nd.Array(z, requires_grad=True)
    y = nd.fftn(X)
    re = nd.real(y)
    nd.sum(re * nd.Array(w)).backward()
    g = X.grad().to_numpy()
    ref = w.size * np.fft.ifftn(w.astype(np.complex128))
    assert rel_l2(g, ref) < 1e-5
    lz = LazyComplex(nd.Array(w))
    assert not lz.materialised()
    assert np.array_equal(lz.to_numpy(), w.astype(np.complex64)) and lz.materialised()


@pytest.mark.parametrize("shape,dims,real_src", [
    ((8, 65536), [1], False),          # four-step: the last pass reads rows and writes strided
    ((2, 1 << 20), [1], False),        # two 1024-point passes (the c4 passes)
    ((16, 1024), [1], False),          # contiguous rows in and out
    ((512, 32, 16), [0], False),       # strided axis, 512-point lines
    ((64, 128, 256), [0, 1, 2], False),  # last pass on the generic tile kernel (64-point lines)
    ((512, 512, 4), [0, 1], False),
    ((8, 2048), [1], True),            # real source: loss term in a pass of its own
    ((6, 40), [], False),              # nothing to transform
])
def test_fused_fft_entry_point(nd, shape, dims, real_src):
    """endia_b200_fft_c2c_fused: the result equals the plain transform's (times the device scale),
    and both loss terms equal float64 sums over it, whichever kernel runs the last pass."""
    import ctypes as C
    from endia_b200 import _lib
    from endia_b200._array import stream, alloc
    r = rng(len(shape) + shape[-1])
    x = r.standard_normal(shape).astype(np.float32) if real_src else crandn(r, shape)
    w = r.uniform(-1, 1, shape).astype(np.float32)
    X, W = nd.Array(x), nd.Array(w)
    Y0, Y1 = nd.Array(list(shape), is_complex=True), nd.Array(list(shape), is_complex=True)
    G, L = nd.Array(np.array([0.75], np.float32)), nd.Array([1])
    cd = (C.c_int32 * max(len(dims), 1))(*dims)
    nb = _lib.lib.endia_b200_fft_scratch_bytes(X.desc(), cd, len(dims))
    scratch = alloc(nb // 4 + 1) if nb else None
    sp = scratch.data_ptr() if scratch is not None else None
    keep = alloc(_lib.lib.endia_b200_fft_fusion_scratch_bytes() // 4)
    for inverse in (0, 1):
        _lib.call("endia_b200_fft_c2c", X.desc(), Y0.desc(), cd, len(dims), inverse, 0.5, sp, stream())
        y0 = Y0.to_numpy().astype(np.complex128)
        for mode in (1, 2):
            f = _lib.FftFusion()
            f.scale_dev, f.reduce, f.reduce_scale = G.data_ptr(), mode, 2.0
            f.reduce_w, f.reduce_out, f.reduce_scratch = W.data_ptr(), L.data_ptr(), keep.data_ptr()
            _lib.call("endia_b200_fft_c2c_fused", X.desc(), Y1.desc(), cd, len(dims), inverse, 0.5, sp,
                      C.byref(f), stream())
            y1 = Y1.to_numpy().astype(np.complex128)
            assert rel_l2(y1, 0.75 * y0) < 1e-6
            want = 2.0 * (np.sum(np.abs(y1) ** 2) if mode == 1 else np.sum(y1.real * w))
            scale = 2.0 * (np.sum(np.abs(y1) ** 2) if mode == 1 else np.sqrt(np.sum((y1.real * w) ** 2)) * 10)
            assert abs(L.to_numpy()[0] - want) <= 1e-5 * scale, (inverse, mode)
            _lib.call("endia_b200_fft_loss_term", Y1.desc(), mode, W.data_ptr(), L.data_ptr(), 2.0, keep.data_ptr(),
                      stream())
            assert abs(L.to_numpy()[0] - want) <= 1e-5 * scale
    st = _lib.lib.endia_b200_fft_loss_term(X.desc() if real_src else Y1.desc(), 3, None, L.data_ptr(), 1.0,
                                           keep.data_ptr(), stream())
    assert st == _lib.EINVAL


def _fft_programs():
    def c4(L, z, w):
        X = L.Array(z, requires_grad=True)
        y = L.fft(X)
        loss = L.sum(L.square(L.to_abs(y))) * (1.0 / z.shape[-1])
        loss.backward()
        return y, X, loss

    def c5(L, z, w):
        X = L.Array(z, requires_grad=True)
        y = L.fftn(X)
        loss = L.sum(L.real(y) * L.Array(w))
        loss.backward()
        return y, X, loss

    def c5_mean_inverse(L, z, w):
        X = L.Array(z, requires_grad=True)
        y = L.ifftn(X, [0, -1])
        loss = L.mean(L.Array(w) * L.real(y)) * 3.0
        loss.backward()
        return y, X, loss
    return {"c4": c4, "c5": c5, "c5_mean_inverse": c5_mean_inverse}


@pytest.mark.parametrize("prog", ["c4", "c5", "c5_mean_inverse"])
@pytest.mark.parametrize("shape", [(4, 4096), (16, 64, 256), (2, 1 << 17)])
def test_fft_loss_chains_fused_equal_eager(nd, prog, shape, monkeypatch):
    """The two loss chains with their kernels folded into the transforms (the default) against the
    same program run op by op (state.defer_fft_chains off): result, loss and gradient agree, and the
    fused form launches only the transforms and the two finishing sums."""
    from endia_b200.autograd import state
    r = rng(sum(shape))
    z, w = crandn(r, shape), r.uniform(-1, 1, shape).astype(np.float32)
    f = _fft_programs()[prog]
    count = nd._lib.lib.endia_b200_launch_count
    monkeypatch.setattr(state, "defer_fft_chains", False)
    n0 = count()
    y0, X0, l0 = f(nd, z, w)
    eager_launches = count() - n0
    monkeypatch.setattr(state, "defer_fft_chains", True)
    n0 = count()
    y1, X1, l1 = f(nd, z, w)
    fused_launches = count() - n0
    assert fused_launches <= eager_launches - 3, (fused_launches, eager_launches)
    assert rel_l2(y1.to_numpy(), y0.to_numpy()) < 1e-6
    assert rel_l2(X1.grad().to_numpy(), X0.grad().to_numpy()) < 1e-6
    ref = abs(l0.to_numpy()[0]) if prog == "c4" else np.abs(y0.to_numpy()).max()
    assert abs(l1.to_numpy()[0] - l0.to_numpy()[0]) <= 1e-5 * max(ref, abs(l0.to_numpy()[0]))


def test_deferred_fft_results_behave_like_arrays(nd, oracle):
    """A deferred transform or chain member gives its values whenever they are asked for: before or
    after the fused loss, through two losses on one transform (the lazily scaled gradient is then
    written out and added), under create_graph, and after its input was rewritten in place."""
    r = rng(77)
    z, w = crandn(r, (8, 512)), r.uniform(-1, 1, (8, 512)).astype(np.float32)
    X = nd.Array(z, requires_grad=True)
    y = nd.fft(X)
    a = nd.to_abs(y)
    loss = nd.sum(nd.square(a)) + nd.sum(nd.real(y) * nd.Array(w))
    assert rel_l2(a.to_numpy(), np.abs(np.fft.fft(z.astype(np.complex128)))) < TOL   # asked for after the fused sum
    loss.backward()
    Xo = oracle.Array(z, requires_grad=True)
    yo = oracle.fft(Xo)
    lo = oracle.sum(oracle.square(oracle.to_abs(yo))) + oracle.sum(oracle.real(yo) * oracle.Array(w))
    lo.backward()
    assert rel_l2(X.grad().to_numpy(), Xo.grad().to_numpy()) < TOL
    assert abs(loss.to_numpy()[0] - lo.to_numpy()[0]) <= 1e-5 * abs(lo.to_numpy()[0])
    # create_graph: the fused node's VJP is the composition of differentiable ops
    X2 = nd.Array(z, requires_grad=True)
    l2 = nd.sum(nd.square(nd.to_abs(nd.fft(X2))))
    g = nd.grad(outs=[l2], inputs=[X2], create_graph=True)[0]
    assert rel_l2(g.to_numpy(), 2 * 512 * z) < TOL
    # an in-place update of the input runs the pending transform first
    X3 = nd.Array(z)
    y3 = nd.fft(X3)
    X3 -= nd.Array(np.ones((8, 512), np.complex64))
    assert rel_l2(y3.to_numpy(), np.fft.fft(z.astype(np.complex128))) < TOL
    assert rel_l2(nd.fft(X3).to_numpy(), np.fft.fft(z.astype(np.complex128) - 1)) < TOL
