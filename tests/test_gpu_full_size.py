"""GPU parity at the FULL sizes of the configurations against the CPU oracle in fast mode (the
reference's op sequence with float64 sums, large products through a float64 BLAS):

  c2  MLP 1024->4096->4096->4096->1024, tanh, zero bias, batch 8192, MSE + one Adam step: loss, all
      eight gradients, updated weights and both Adam moments, on BOTH tensor-core schemes
      (tf32 + two bf16 correction MMAs, and 3xTF32);
  c3  MLP 256->1024->1024->1, tanh, batch 4096, gradient penalty with create_graph=True: loss, the
      input gradient and every parameter gradient;
  c5  512^3 fftn with loss = sum(real(fftn(x)) * w): the forward result and the gradient
      x.grad = N * ifftn(w) on sampled lines evaluated in float64.

Tolerance: 1e-4 max relative error on gradients and updated weights (entries below the tensor's RMS
are judged on the RMS scale, see conftest.max_rel), 1e-5 relative L2 for the FFT. The unfloored
per-element relative error is reported as percentiles next to it."""
import numpy as np
import pytest

from conftest import rng, max_rel, rel_l2
from test_gpu_mlp import make_mlp_inputs, train_step, fwd_fused, fwd_unfused, compare_steps, second_order, TOL

pytestmark = pytest.mark.gpu

C2_DIMS, C2_BATCH = [1024, 4096, 4096, 4096, 1024], 8192
C3_DIMS, C3_BATCH = [256, 1024, 1024, 1], 4096


def unfloored_percentiles(a, b):
    """Percentiles (50, 99, 99.9) and the maximum of |a-b| / |b| over the entries with b != 0."""
    a = np.asarray(a, np.float64).reshape(-1)
    b = np.asarray(b, np.float64).reshape(-1)
    nz = b != 0
    rel = np.abs(a[nz] - b[nz]) / np.abs(b[nz])
    if rel.size == 0:
        return [0.0, 0.0, 0.0, 0.0]
    return [float(v) for v in np.percentile(rel, [50, 99, 99.9])] + [float(rel.max())]


@pytest.fixture(scope="module")
def c2_case(oracle):
    Ws, bs, x, y = make_mlp_inputs(C2_DIMS, C2_BATCH, 0, bias_zero=True)
    oracle.config["mode"] = "fast"
    try:
        o = train_step(oracle, fwd_unfused("tanh"), Ws, bs, x, y)
    finally:
        oracle.config["mode"] = "faithful"
    return Ws, bs, x, y, o


@pytest.mark.parametrize("scheme", ["tf32_bf16x2", "3xtf32"])
def test_c2_full_size_train_step(nd, c2_case, scheme, monkeypatch, record_property):
    """One full-size c2 training step from the seeded weights on the named tensor-core scheme."""
    from endia_b200 import _lib
    from endia_b200.autograd import state
    Ws, bs, x, y, o = c2_case
    monkeypatch.setattr(state, "gemm_algo", _lib.GEMM_TF32_BF16X2 if scheme == "tf32_bf16x2" else _lib.GEMM_3XTF32)
    g = train_step(nd, fwd_fused("tanh"), Ws, bs, x, y)
    compare_steps(g, o)
    assert g["grad_shapes"][1] == [1, 4096] and g["grad_shapes"][0] == [1024, 4096]
    worst = {}
    for key in ("grads", "params"):
        for i, (a, b) in enumerate(zip(g[key], o[key])):
            if i % 2 == 0:      # the weight matrices (biases start at zero, their gradients are covered above)
                worst["%s[%d]" % (key, i)] = unfloored_percentiles(a, b)
    record_property("unfloored_rel_p50_p99_p999_max", worst)
    print("\nc2 full size, %s: unfloored relative error [p50, p99, p99.9, max] per tensor:" % scheme)
    for k, v in worst.items():
        print("  %-10s %s" % (k, " ".join("%.2e" % e for e in v)))
    # the unfloored error: half of the entries of every weight gradient agree to better than 5e-5 of
    # their own magnitude and 99 % to 2e-3 (entries far below the tensor's RMS are cancellation
    # residues: float32 dot products, the FFMA kernel's included, are not accurate relative to those)
    assert all(v[0] < 5e-5 and v[1] < 2e-3 for k, v in worst.items() if k.startswith("grads"))


@pytest.mark.parametrize("fused", [True, False])
def test_c3_full_size_gradient_penalty(nd, oracle, fused):
    """c3 at full size: loss = mean(f) + 0.1 * mean |df/dx|^2 through create_graph=True, then the
    gradients of all six parameters (double backward through the matmul and tanh VJPs)."""
    r = rng(0)
    d = C3_DIMS
    Ws = [r.uniform(-np.sqrt(6 / d[i]), np.sqrt(6 / d[i]), (d[i], d[i + 1])).astype(np.float32) for i in range(3)]
    bs = [np.zeros(d[i + 1], np.float32) for i in range(3)]
    x = r.standard_normal((C3_BATCH, d[0])).astype(np.float32)
    oracle.config["mode"] = "fast"
    try:
        o = second_order(oracle, Ws, bs, x, False)
    finally:
        oracle.config["mode"] = "faithful"
    g = second_order(nd, Ws, bs, x, fused)
    assert abs(g["loss"][0] - o["loss"][0]) <= TOL * abs(o["loss"][0])
    assert max_rel(g["gx"], o["gx"]) < TOL
    assert g["shapes"] == o["shapes"] == [[256, 1024], [1024, 1024], [1024, 1], [1, 1024], [1, 1024], [1, 1]]
    for a, b in zip(g["grads"], o["grads"]):
        assert max_rel(a, b) < TOL, max_rel(a, b)


def _line(arr, k0, k1, n):
    """Line arr[k0, k1, :] of a contiguous [n, n, n] complex device array as numpy."""
    from endia_b200.dist import flat_tensor
    off = 2 * (k0 * n * n + k1 * n)
    return flat_tensor(arr)[off:off + 2 * n].cpu().numpy().view(np.complex64)


def _contract_axis0(e, arr):
    """sum_a e[a] * arr[a, :, :] in float64, a few planes at a time (no full-size float64 copy)."""
    acc = np.zeros(arr.shape[1:], np.complex128)
    for a in range(0, arr.shape[0], 64):
        acc += np.tensordot(e[a:a + 64], arr[a:a + 64].astype(np.complex128), axes=(0, 0))
    return acc


def test_c5_full_size_forward_and_vjp(nd):
    """c5 at full size: y = fftn(x) and x.grad of loss = sum(real(y) * w), which is
    conj(fftn(conj(w + 0i))) = N * ifftn(w) (fftn_op.mojo:43-49). Lines of both are evaluated in
    float64 from the separable definition, and the loss from <x, x.grad>."""
    r = rng(0)
    n = 512
    z = (r.standard_normal((n, n, n), dtype=np.float32)
         + 1j * r.standard_normal((n, n, n), dtype=np.float32)).astype(np.complex64)
    w = r.uniform(-1, 1, (n, n, n)).astype(np.float32)
    X = nd.Array(z, requires_grad=True)
    y = nd.fftn(X)
    loss = nd.sum(nd.real(y) * nd.Array(w))
    loss.backward()
    gx = X.grad()
    assert gx.shape() == [n, n, n] and gx.is_complex()
    ar = np.arange(n)
    for (k0, k1) in [(3, 500), (0, 0), (257, 64)]:
        e0 = np.exp(-2j * np.pi * k0 * ar / n)
        e1 = np.exp(-2j * np.pi * k1 * ar / n)
        # forward line y[k0, k1, :] = fft_c( sum_ab x[a,b,c] e0[a] e1[b] )
        line = np.fft.fft(e1 @ _contract_axis0(e0, z))
        assert rel_l2(_line(y, k0, k1, n), line) < 1e-5
        # gradient line gx[k0, k1, :] = sum_abc w[a,b,c] exp(+2 pi i (k0 a + k1 b + k c) / n)
        gline = n * np.fft.ifft(np.conj(e1) @ _contract_axis0(np.conj(e0), w))
        assert rel_l2(_line(gx, k0, k1, n), gline) < 1e-5
    # loss = sum_k real(y_k) w_k = Re <w, F x> = Re <F^H w, x> = Re sum_x conj(gx) x
    gh = gx.to_numpy()
    ref_loss = 0.0
    for a in range(0, n, 32):
        ref_loss += float(np.real(np.vdot(gh[a:a + 32].astype(np.complex128), z[a:a + 32].astype(np.complex128))))
    # the loss is a sum of n^3 terms of size ~ n^1.5 with random signs: judged on its spread
    spread = float(n) ** 3 * 0.577
    assert abs(loss.to_numpy()[0] - ref_loss) <= 1e-4 * max(abs(ref_loss), spread)
