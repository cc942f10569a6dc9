"""The tcgen05 3xTF32 GEMM through the C ABI: all four operand layouts, ragged sizes and the fused
epilogue, against float64 products. 3xTF32 keeps ~21 mantissa bits per product, so the error bound
is a few 1e-6 of the natural scale of each dot product (|a|.|b|)."""
import ctypes as C

import numpy as np
import pytest

from conftest import rng, max_rel

pytestmark = pytest.mark.gpu


def run_gemm(nd, a, b, ta, tb, algo, epi=None, c0=None):
    from endia_b200 import _lib
    from endia_b200._array import stream
    M = a.shape[1] if ta else a.shape[0]
    K = a.shape[0] if ta else a.shape[1]
    N = b.shape[0] if tb else b.shape[1]
    A, B = nd.Array(a), nd.Array(b)
    Cd = nd.Array(c0) if c0 is not None else nd.Array([M, N])
    _lib.call("endia_b200_gemm", ta, tb, M, N, K, A.data_ptr(), a.shape[1], B.data_ptr(), b.shape[1],
              Cd.data_ptr(), N, 1, 0, 0, 0, C.byref(epi) if epi is not None else None, algo, stream())
    _lib.call("endia_b200_device_status", stream())
    return Cd.to_numpy()


def dot_scale(am, bm):
    """|a_i|.|b_j| for every output element: the scale float32 dot products are accurate to."""
    return np.abs(am).astype(np.float64) @ np.abs(bm).astype(np.float64)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(128, 128, 32), (256, 256, 64), (384, 512, 256), (200, 328, 100),
                                   (1024, 1024, 1024), (136, 260, 36), (256, 1024, 4096), (200, 136, 2048)])
def test_3xtf32_all_layouts(nd, ta, tb, M, N, K):
    from endia_b200 import _lib
    if not _lib.lib.endia_b200_has_tcgen05():
        pytest.fail("library built without the tcgen05 GEMM")
    check_layout_case(nd, ta, tb, M, N, K, _lib.GEMM_3XTF32, 5e-6)


@pytest.mark.parametrize("ta,tb", [(0, 0), (0, 1), (1, 0), (1, 1)])
@pytest.mark.parametrize("M,N,K", [(256, 256, 64), (384, 512, 256), (200, 328, 100), (1024, 1024, 1024),
                                   (136, 260, 36), (256, 1024, 4096), (1000, 520, 2048)])
def test_tf32_bf16x2_all_layouts(nd, ta, tb, M, N, K):
    """One tf32 MMA plus two bf16 correction MMAs per product: the correction operands carry 8
    bits, so the bound is 2^-19 of |a||b| per product in the worst case (measured far below)."""
    from endia_b200 import _lib
    check_layout_case(nd, ta, tb, M, N, K, _lib.GEMM_TF32_BF16X2, 8e-6)


def test_tf32_bf16x2_needs_wide_output(nd):
    from endia_b200 import _lib
    from endia_b200._array import stream
    A, B, Cd = nd.Array([256, 64]), nd.Array([64, 128]), nd.Array([256, 128])
    st = _lib.lib.endia_b200_gemm(0, 0, 256, 128, 64, A.data_ptr(), 64, B.data_ptr(), 128, Cd.data_ptr(), 128,
                                  1, 0, 0, 0, None, _lib.GEMM_TF32_BF16X2, stream())
    assert st == _lib.EINVAL


def check_layout_case(nd, ta, tb, M, N, K, algo, bound):
    from endia_b200 import _lib
    r = rng(M + N + K)
    a = r.standard_normal((K, M) if ta else (M, K)).astype(np.float32)
    b = r.standard_normal((N, K) if tb else (K, N)).astype(np.float32)
    out = run_gemm(nd, a, b, ta, tb, algo)
    am = (a.T if ta else a).astype(np.float64)
    bm = (b.T if tb else b).astype(np.float64)
    ref = am @ bm
    err = np.abs(out - ref) / dot_scale(am, bm)
    print("max error / (|a|.|b|): %.3g" % err.max())
    assert err.max() < bound, err.max()          # plain tf32 would be ~1e-3
    ffma = run_gemm(nd, a, b, ta, tb, _lib.GEMM_FFMA)
    assert max_rel(out, ffma) < 1e-4


@pytest.mark.parametrize("scheme", ["3xtf32", "tf32_bf16x2"])
@pytest.mark.parametrize("ta,tb,alpha", [(1, 0, 1.0), (0, 1, 0.5)])
def test_halved_reduction(nd, ta, tb, alpha, scheme):
    """81 tiles of 256 x 256 fill the last round of CTA pairs badly: the persistent kernel halves K
    and the two halves are added into a zeroed C by the copy engine. The result must not depend on
    which half lands first, so two runs agree bit for bit; C starts out as garbage."""
    from endia_b200 import _lib
    r = rng(77)
    M = N = 2304
    K = 4096
    a = r.standard_normal((K, M) if ta else (M, K)).astype(np.float32)
    b = r.standard_normal((N, K) if tb else (K, N)).astype(np.float32)
    epi = _lib.Epilogue()
    epi.alpha, epi.beta = alpha, 0.0
    junk = np.full((M, N), 1e30, np.float32)
    algo = _lib.GEMM_3XTF32 if scheme == "3xtf32" else _lib.GEMM_TF32_BF16X2
    out = run_gemm(nd, a, b, ta, tb, algo, epi=epi, c0=junk)
    out2 = run_gemm(nd, a, b, ta, tb, algo, epi=epi, c0=junk)
    assert np.array_equal(out, out2)
    am = (a.T if ta else a).astype(np.float64)
    bm = (b.T if tb else b).astype(np.float64)
    rows = slice(0, M, 7)        # every 7th row keeps the float64 product short
    ref = alpha * (am[rows] @ bm)
    err = np.abs(out[rows] - ref) / dot_scale(am[rows], bm)
    assert err.max() < (5e-6 if scheme == "3xtf32" else 8e-6), err.max()


def test_3xtf32_fused_epilogue(nd):
    from endia_b200 import _lib
    r = rng(5)
    M, N, K = 256, 384, 160
    a = r.standard_normal((M, K)).astype(np.float32)
    b = r.standard_normal((K, N)).astype(np.float32) * np.float32(0.1)
    bias = r.standard_normal(N).astype(np.float32)
    saved = r.uniform(0.1, 0.9, (M, N)).astype(np.float32)
    c0 = r.standard_normal((M, N)).astype(np.float32)
    BIAS, SAVED = nd.Array(bias), nd.Array(saved)
    epi = _lib.Epilogue()
    epi.alpha, epi.beta = 0.5, 2.0
    epi.bias = BIAS.data_ptr()
    epi.act, epi.dact = _lib.ACT_TANH, _lib.ACT_SIGMOID
    epi.dact_src, epi.ld_dact = SAVED.data_ptr(), N
    out = run_gemm(nd, a, b, 0, 0, _lib.GEMM_3XTF32, epi=epi, c0=c0)
    v = np.tanh(0.5 * (a.astype(np.float64) @ b) + bias) * (saved.astype(np.float64) * (1 - saved)) + 2.0 * c0
    assert max_rel(out, v) < 1e-4


@pytest.mark.parametrize("algo_name", ["3xtf32", "tf32_bf16x2"])
@pytest.mark.parametrize("M,N,K,tb", [(512, 384, 256, 1), (300, 260, 96, 0), (1024, 1024, 512, 1)])
def test_tensor_core_epilogue_mask_and_bias_gradient(nd, M, N, K, tb, algo_name):
    """dS = (dY . W^T) * act'(h) with the bias gradient colsum(dS) from the same launch: the
    backward mask and the column reduction fused into the store of the dX product
    (tanh_op.mojo:92, expand_op.mojo:121-126)."""
    from endia_b200 import _lib
    from endia_b200._array import alloc
    algo = _lib.GEMM_3XTF32 if algo_name == "3xtf32" else _lib.GEMM_TF32_BF16X2
    r = rng(M + N)
    a = r.standard_normal((M, K)).astype(np.float32)
    b = (r.standard_normal((N, K) if tb else (K, N)) * 0.1).astype(np.float32)
    h = np.tanh(r.standard_normal((M, N))).astype(np.float32)
    H, colsum = nd.Array(h), nd.Array([N])
    scratch = alloc(_lib.lib.endia_b200_gemm_colsum_scratch_bytes(M, N) // 4 + 1)
    epi = _lib.Epilogue()
    epi.alpha, epi.beta = 1.0, 0.0
    epi.dact, epi.dact_src, epi.ld_dact = _lib.ACT_TANH, H.data_ptr(), N
    epi.colsum, epi.colsum_scratch = colsum.data_ptr(), scratch.data_ptr()
    out = run_gemm(nd, a, b, 0, tb, algo, epi=epi)
    bm = (b.T if tb else b).astype(np.float64)
    v = (a.astype(np.float64) @ bm) * (1.0 - h.astype(np.float64) ** 2)
    assert max_rel(out, v) < 1e-4
    assert max_rel(colsum.to_numpy(), v.sum(0)) < 1e-4


@pytest.mark.parametrize("ta,tb,K", [(1, 0, 16384 + 96), (0, 1, 24576)])
def test_auto_long_reduction_runs(nd, ta, tb, K):
    """K > 8192 under GEMM_AUTO: the two-CTA kernel drains its accumulators after runs of 2048 and
    adds the runs (and the K ranges of a product with few tiles) in order, so the product is
    reproducible and as accurate as a short one."""
    from endia_b200 import _lib
    r = rng(K)
    M, N = 384, 512
    a = r.standard_normal((K, M) if ta else (M, K)).astype(np.float32)
    b = r.standard_normal((N, K) if tb else (K, N)).astype(np.float32)
    junk = np.full((M, N), -7e29, np.float32)
    launches0 = _lib.lib.endia_b200_launch_count()
    out = run_gemm(nd, a, b, ta, tb, _lib.GEMM_AUTO, c0=junk)
    # two splits + one GEMM (K ranges as work items) + the kernel that adds the ranges; no FFMA tiles
    assert _lib.lib.endia_b200_launch_count() - launches0 <= 4
    out2 = run_gemm(nd, a, b, ta, tb, _lib.GEMM_AUTO, c0=junk)
    assert np.array_equal(out, out2)
    am = (a.T if ta else a).astype(np.float64)
    bm = (b.T if tb else b).astype(np.float64)
    err = np.abs(out - am @ bm) / dot_scale(am, bm)
    assert err.max() < 8e-6, err.max()
    # the truncation bias of one long accumulation would show as a negative mean relative error
    rel = (out - am @ bm) / np.maximum(np.abs(am @ bm), 1e-3 * dot_scale(am, bm))
    assert abs(np.median(rel)) < 3e-5


def test_3xtf32_long_k_error_growth(nd):
    """dW reduces over the batch: K = 8192 must still meet the gradient tolerance."""
    from endia_b200 import _lib
    r = rng(6)
    M, N, K = 256, 256, 8192
    a = r.standard_normal((K, M)).astype(np.float32)
    b = r.standard_normal((K, N)).astype(np.float32)
    out = run_gemm(nd, a, b, 1, 0, _lib.GEMM_3XTF32)
    ref = a.T.astype(np.float64) @ b.astype(np.float64)
    assert max_rel(out, ref) < 1e-4
    assert (np.abs(out - ref) / dot_scale(a.T, b)).max() < 5e-6
    # Beyond K = 8192 the default algorithm choice goes back to exact fp32 accumulation.
    a2 = r.standard_normal((16384, 128)).astype(np.float32)
    b2 = r.standard_normal((16384, 128)).astype(np.float32)
    out2 = run_gemm(nd, a2, b2, 1, 0, _lib.GEMM_AUTO)
    assert max_rel(out2, a2.T.astype(np.float64) @ b2.astype(np.float64)) < 2e-5


def test_auto_falls_back_to_ffma_for_unaligned_or_small(nd):
    from endia_b200 import _lib
    r = rng(7)
    a = r.standard_normal((130, 33)).astype(np.float32)       # lda = 33: not 16-byte aligned rows
    b = r.standard_normal((33, 257)).astype(np.float32)
    out = run_gemm(nd, a, b, 0, 0, _lib.GEMM_AUTO)
    assert max_rel(out, a.astype(np.float64) @ b) < 1e-4
    from endia_b200._array import stream
    A, B, Cd = nd.Array(a), nd.Array(b), nd.Array([130, 257])
    st = _lib.lib.endia_b200_gemm(0, 0, 130, 257, 33, A.data_ptr(), 33, B.data_ptr(), 257, Cd.data_ptr(),
                                  257, 1, 0, 0, 0, None, _lib.GEMM_3XTF32, stream())
    assert st == _lib.EINVAL


def test_weight_operand_parts_written_by_adam(nd):
    """Adam leaves the bf16 split of each updated weight matrix behind (bf16(w) and
    bf16(w - tf32(w))); the next products with that weight (plain and transposed) read it, and any
    other in-place update drops it."""
    import torch
    r = rng(9)
    w = r.standard_normal((256, 384)).astype(np.float32)
    x = r.standard_normal((512, 256)).astype(np.float32)
    g = r.standard_normal((512, 384)).astype(np.float32)
    W = nd.Array(w, requires_grad=True)
    W.grad_(nd.Array(r.standard_normal((256, 384)).astype(np.float32)))
    nd.optim.Adam([W]).step()
    assert getattr(W, "_pair16", None) is not None
    wn32 = W.to_numpy()
    wn = wn32.astype(np.float64)
    pair = W._pair16.view(torch.bfloat16).float().cpu().numpy().reshape(2, 256, 384)
    hi = (wn32.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)
    assert np.array_equal(pair[0], torch.from_numpy(wn32).to(torch.bfloat16).float().numpy())
    assert np.array_equal(pair[1], torch.from_numpy(wn32 - hi).to(torch.bfloat16).float().numpy())
    y = nd.matmul(nd.Array(x), W).to_numpy()
    dx = nd.matmul(nd.Array(g), W.T()).to_numpy()
    assert max_rel(y, x.astype(np.float64) @ wn) < 2e-5
    assert max_rel(dx, g.astype(np.float64) @ wn.T) < 2e-5
    W -= nd.Array(np.ones((256, 384), np.float32))
    assert W._pair16 is None and W._tf32_lo is None
    assert max_rel(nd.matmul(nd.Array(x), W).to_numpy(), x.astype(np.float64) @ (wn - 1.0)) < 2e-5


@pytest.mark.parametrize("algo_name", ["3xtf32", "tf32_bf16x2"])
@pytest.mark.parametrize("K,tb", [(4096, 0), (6144 + 96, 1), (16384, 0)])
def test_short_accumulation_runs_with_nonlinear_epilogue(nd, K, tb, algo_name):
    """The two-CTA kernel cuts every reduction into runs of 2048: with a bias, an activation, a
    derivative mask and the column sums in the epilogue the earlier runs leave bare sums in C and
    the last run adds them before the epilogue. Forward form (bias + tanh) and backward form
    (mask + bias gradient), C pre-filled with garbage."""
    from endia_b200 import _lib
    from endia_b200._array import alloc
    algo = _lib.GEMM_3XTF32 if algo_name == "3xtf32" else _lib.GEMM_TF32_BF16X2
    r = rng(K + tb)
    M, N = 300, 520
    a = r.standard_normal((M, K)).astype(np.float32)
    b = (r.standard_normal((N, K) if tb else (K, N)) / np.sqrt(K)).astype(np.float32)
    bias = r.standard_normal(N).astype(np.float32)
    h = np.tanh(r.standard_normal((M, N))).astype(np.float32)
    bm = (b.T if tb else b).astype(np.float64)
    prod = a.astype(np.float64) @ bm
    junk = np.full((M, N), 3e30, np.float32)
    BIAS, H, colsum = nd.Array(bias), nd.Array(h), nd.Array([N])
    epi = _lib.Epilogue()
    epi.alpha, epi.beta, epi.bias, epi.act = 1.0, 0.0, BIAS.data_ptr(), _lib.ACT_TANH
    out = run_gemm(nd, a, b, 0, tb, algo, epi=epi, c0=junk)
    # (the bf16 correction products carry 8 bits: up to 2^-19 of |a||b| per product, sqrt(K) larger
    # relative to a sum of random signs)
    bound = 4e-5 if algo_name == "3xtf32" else 6e-5
    assert max_rel(out, np.tanh(prod + bias)) < bound
    scratch = alloc(_lib.lib.endia_b200_gemm_colsum_scratch_bytes(M, N) // 4 + 1)
    epi = _lib.Epilogue()
    epi.alpha, epi.beta = 1.0, 0.0
    epi.dact, epi.dact_src, epi.ld_dact = _lib.ACT_TANH, H.data_ptr(), N
    epi.colsum, epi.colsum_scratch = colsum.data_ptr(), scratch.data_ptr()
    out = run_gemm(nd, a, b, 0, tb, algo, epi=epi, c0=junk)
    v = prod * (1.0 - h.astype(np.float64) ** 2)
    assert max_rel(out, v) < bound
    assert max_rel(colsum.to_numpy(), v.sum(0)) < bound


@pytest.mark.parametrize("algo_name", ["3xtf32", "tf32_bf16x2"])
def test_accumulator_truncation_bias_is_bounded_by_the_run_length(nd, algo_name):
    """Sums of same-sign terms show the round-toward-zero bias of the tensor-core accumulator most
    clearly: one accumulation over K = 8192 on the two-CTA kernel is off by -5.5e-5 of the result
    (measured), linear in K. With runs of 2048 added in fp32 the mean relative error stays at the
    level of one run (-1.3e-5), for a plain product and under an epilogue."""
    from endia_b200 import _lib
    algo = _lib.GEMM_3XTF32 if algo_name == "3xtf32" else _lib.GEMM_TF32_BF16X2
    r = rng(123)
    M, N, K = 2048, 2048, 8192          # 128 CTAs' worth of tiles: the two-CTA kernel on both schemes
    a = r.uniform(0.5, 1.5, (M, K)).astype(np.float32)
    b = r.uniform(0.5, 1.5, (K, N)).astype(np.float32)
    rows = slice(0, M, 16)
    ref = a[rows].astype(np.float64) @ b.astype(np.float64)
    out = run_gemm(nd, a, b, 0, 0, algo)
    bias_plain = np.mean((out[rows] - ref) / ref)
    BIAS = nd.Array(np.zeros(N, np.float32))
    epi = _lib.Epilogue()
    epi.alpha, epi.beta, epi.bias, epi.act = 1.0, 0.0, BIAS.data_ptr(), _lib.ACT_RELU
    out = run_gemm(nd, a, b, 0, 0, algo, epi=epi)
    bias_epi = np.mean((out[rows] - ref) / ref)
    print("mean relative error of a same-sign sum, K = 8192: plain %.2e, with epilogue %.2e" % (bias_plain, bias_epi))
    assert abs(bias_plain) < 2e-5 and abs(bias_epi) < 2e-5


def test_bounded_wait_gives_up_and_the_context_stays_usable(nd):
    """A device-side wait that can never complete (a barrier nothing arrives at, limited to a
    thousand polls) runs out: the kernel returns, endia_b200_device_status reports ETIMEOUT exactly
    once, and a tensor-core product afterwards is still correct."""
    from endia_b200 import _lib
    from endia_b200._array import stream
    assert _lib.lib.endia_b200_device_status(stream()) == 0
    _lib.call("endia_b200_selftest_wait_timeout", 1000, stream())
    assert _lib.lib.endia_b200_device_status(stream()) == _lib.ETIMEOUT
    assert b"wait" in _lib.lib.endia_b200_last_error()
    assert _lib.lib.endia_b200_device_status(stream()) == 0            # reported once, then cleared
    assert _lib.lib.endia_b200_selftest_wait_timeout(0, stream()) == _lib.EINVAL
    r = rng(5)
    a = r.standard_normal((256, 128)).astype(np.float32)
    b = r.standard_normal((128, 256)).astype(np.float32)
    out = run_gemm(nd, a, b, 0, 0, _lib.GEMM_TF32_BF16X2)
    assert max_rel(out, a.astype(np.float64) @ b.astype(np.float64)) < 2e-5


@pytest.mark.parametrize("M,N,K,algo_name", [(512, 512, 4096, "tf32_bf16x2"), (300, 520, 96, "3xtf32"),
                                             (256, 128, 64, "3xtf32"), (64, 40, 16, "ffma")])
def test_epilogue_writes_operand_parts_of_the_output(nd, M, N, K, algo_name):
    """epi.c16: the bf16 split of the stored C (what the products that read C as an operand need)
    comes out of the same call, from the two-CTA kernel's epilogue (first two cases: two
    accumulation runs with the bare-sum round trip, and a single run) or from a split pass where
    another kernel runs; bit for bit what endia_b200_bf16_split gives on the output."""
    import torch
    from endia_b200 import _lib
    from endia_b200._array import stream, alloc
    algo = {"3xtf32": _lib.GEMM_3XTF32, "tf32_bf16x2": _lib.GEMM_TF32_BF16X2, "ffma": _lib.GEMM_FFMA}[algo_name]
    r = rng(M + K)
    a = r.standard_normal((M, K)).astype(np.float32)
    b = (r.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32)
    bias = r.standard_normal(N).astype(np.float32)
    A, B, BIAS, Cd = nd.Array(a), nd.Array(b), nd.Array(bias), nd.Array([M, N])
    parts, want = alloc(M * N), alloc(M * N)
    epi = _lib.Epilogue()
    epi.alpha, epi.beta, epi.bias, epi.act, epi.c16 = 1.0, 0.0, BIAS.data_ptr(), _lib.ACT_TANH, parts.data_ptr()
    _lib.call("endia_b200_gemm", 0, 0, M, N, K, A.data_ptr(), K, B.data_ptr(), N, Cd.data_ptr(), N, 1, 0, 0, 0,
              C.byref(epi), algo, stream())
    _lib.call("endia_b200_bf16_split", Cd.data_ptr(), want.data_ptr(), M * N, stream())
    assert torch.equal(parts.view(torch.int32), want.view(torch.int32))
    ref = np.tanh(a.astype(np.float64) @ b.astype(np.float64) + bias)
    assert max_rel(Cd.to_numpy(), ref) < 6e-5


@pytest.mark.parametrize("algo_name", ["auto", "3xtf32", "tf32_bf16x2"])
@pytest.mark.parametrize("M,N,K,ta,tb", [(1024, 1024, 4096, 1, 0), (256, 1024, 4096, 1, 0), (4096, 256, 2048, 0, 1),
                                         (300, 260, 2048 + 32, 0, 0), (300, 259, 2048, 0, 1),
                                         (520, 300, 8192 + 64, 1, 1)])
def test_few_tiles_long_reduction_takes_k_ranges(nd, M, N, K, ta, tb, algo_name):
    """A product with few 256 x 256 tiles and K >= 2048 runs on the two-CTA kernel with K ranges as
    extra work items; their bare sums are added in order by the finishing kernel, which applies the
    whole epilogue (here alpha, bias, tanh and accumulation into C). Same bits on every run."""
    from endia_b200 import _lib
    algo = {"auto": _lib.GEMM_AUTO, "3xtf32": _lib.GEMM_3XTF32, "tf32_bf16x2": _lib.GEMM_TF32_BF16X2}[algo_name]
    r = rng(M + N + K)
    a = r.standard_normal((K, M) if ta else (M, K)).astype(np.float32)
    b = (r.standard_normal((N, K) if tb else (K, N)) / np.sqrt(K)).astype(np.float32)
    bias = r.standard_normal(N).astype(np.float32)
    c0 = r.standard_normal((M, N)).astype(np.float32)
    am = (a.T if ta else a).astype(np.float64)
    bm = (b.T if tb else b).astype(np.float64)
    out = run_gemm(nd, a, b, ta, tb, algo)
    assert max_rel(out, am @ bm) < 4e-5
    BIAS = nd.Array(bias)
    epi = _lib.Epilogue()
    epi.alpha, epi.beta, epi.bias, epi.act = 0.5, 2.0, BIAS.data_ptr(), _lib.ACT_TANH
    want = np.tanh(0.5 * (am @ bm) + bias) + 2.0 * c0
    out1 = run_gemm(nd, a, b, ta, tb, algo, epi=epi, c0=c0)
    out2 = run_gemm(nd, a, b, ta, tb, algo, epi=epi, c0=c0)
    assert max_rel(out1, want) < 4e-5
    assert np.array_equal(out1, out2)
