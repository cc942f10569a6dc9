"""The allocation-free MSE entry point (endia_b200_mse_fwd_bwd_noalloc) against the regular one.

Some hosts cannot allocate device memory around a call (their runtime owns the device heap, or they
sit in a section where cudaMalloc is not allowed), so this variant keeps its partial sums in a fixed
array inside the library. The file name sorts last on purpose: the entry point shares that array
between calls, and running after every other test shows that earlier use of the library does not
disturb it. It must also pass alone in a fresh process (its first call performs the set-up)."""
import numpy as np
import pytest

from conftest import rng

pytestmark = pytest.mark.gpu
TOL = 1e-4  # same relative tolerance as the other fp32 parity tests


def _run_pair(nd, n, seed, with_grad):
    from endia_b200 import _lib
    from endia_b200._array import alloc, stream
    r = rng(seed)
    p = r.standard_normal(n).astype(np.float32)
    t = r.standard_normal(n).astype(np.float32)
    P, T = nd.Array(p), nd.Array(t)
    loss_a, loss_b = nd.Array([1]), nd.Array([1])
    d_a, d_b = nd.Array([n]), nd.Array([n])
    scratch = alloc(_lib.lib.endia_b200_mse_scratch_bytes(n) // 4 + 1)
    _lib.call("endia_b200_mse_fwd_bwd", P.data_ptr(), T.data_ptr(), n, 1.0, loss_a.data_ptr(),
              d_a.data_ptr() if with_grad else None, scratch.data_ptr(), stream())
    _lib.call("endia_b200_mse_fwd_bwd_noalloc", P.data_ptr(), T.data_ptr(), n, 1.0, loss_b.data_ptr(),
              d_b.data_ptr() if with_grad else None, stream())
    la, lb = loss_a.to_numpy()[0], loss_b.to_numpy()[0]
    exact = float(np.mean((p.astype(np.float64) - t) ** 2))
    assert abs(lb - la) <= TOL * abs(la)
    assert abs(lb - exact) <= TOL * exact
    if with_grad:
        ga, gb = d_a.to_numpy(), d_b.to_numpy()
        assert np.abs(gb - ga).max() <= TOL * np.abs(ga).max()
        assert np.abs(gb - 2.0 * (p - t) / n).max() <= TOL * np.abs(ga).max()


def test_noalloc_mse_matches_regular_entry_point_twice_in_a_row(nd):
    # Two calls back to back: a large problem first, then a smaller one that reuses only the front
    # of the shared array (stale partials behind it must not leak into the result).
    _run_pair(nd, 8192 * 1024, 1, with_grad=True)
    _run_pair(nd, 128 * 33 + 5, 2, with_grad=True)
    _run_pair(nd, 7, 3, with_grad=False)


def test_noalloc_mse_rejects_sizes_beyond_its_fixed_scratch(nd):
    from endia_b200 import _lib
    from endia_b200._array import stream
    x = nd.Array([8])
    st = _lib.lib.endia_b200_mse_fwd_bwd_noalloc(x.data_ptr(), x.data_ptr(), 16777216 + 1, 1.0,
                                                 x.data_ptr(), None, stream())
    assert st == _lib.ELIMIT
    assert b"16777216" in _lib.lib.endia_b200_last_error()
