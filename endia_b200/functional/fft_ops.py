"""Complex FFT family and its VJPs (endia/functional/fft_ops/): fft, ifft, fft2, ifft2, fftn,
ifftn. Power-of-two lengths only, like the reference (fft_cooley_tukey.mojo:227-235).

Normalisation follows the usual convention for every `norm`: "backward" scales the inverse by
1/n, "forward" scales the forward transform by 1/n, "ortho" scales both by 1/sqrt(n), with n the
product of the transformed lengths. (The reference's "forward"/"ortho" branches divide by the
whole array size and treat every unknown string as ortho, fft_cooley_tukey.mojo:210-217.)
"""
import ctypes as C
import math

from .. import _lib
from .._array import Array, ArrayShape, alloc, stream
from ..autograd import state as _state
from ._utils import op_array, setup_shape_and_data
from .unary_ops import conj

_NORMS = {"backward": 0, "forward": 1, "ortho": 2}


def encode_fft_params(dims, norm):
    """meta_data = [ndims, dims..., norm code] (fft_ops/utils.mojo:193-208)."""
    if norm not in _NORMS:
        raise _lib.EndiaError(_lib.EINVAL, "fft: unknown norm %r" % (norm,))
    return [len(dims)] + list(dims) + [_NORMS[norm]]


def _norm_dims(x, dims):
    nd = x.ndim()
    if dims is None or len(dims) == 0:
        return list(range(nd))
    out = []
    for d in dims:
        d2 = d + nd if d < 0 else d
        if d2 < 0 or d2 >= nd:
            raise _lib.EndiaError(_lib.EINVAL, "Invalid dimension")
        out.append(d2)
    return out


def _scale(n, norm, inverse):
    if norm == "ortho":
        return 1.0 / math.sqrt(n)
    if (norm == "backward") == bool(inverse):
        return 1.0 / n
    return 1.0


def run_fft(src, dst, dims, direction_inverse, scale):
    """Enqueue one C-ABI transform of `src` (complex, any strides) into `dst` (contiguous)."""
    cd = (C.c_int32 * len(dims))(*dims)
    sd, dd = src.desc(), dst.desc()
    nbytes = _lib.lib.endia_b200_fft_scratch_bytes(sd, cd, len(dims))
    scratch = alloc((nbytes + 3) // 4) if nbytes else None
    timer = _state.fft_timer
    if timer is not None:
        timer.start(16.0 * src.size())   # algorithmic bytes: one read and one write of the array
    _lib.call("endia_b200_fft_c2c", sd, dd, cd, len(dims), 1 if direction_inverse else 0,
              float(scale), scratch.data_ptr() if scratch is not None else None, stream())
    if timer is not None:
        timer.stop()


def _as_complex(x):
    """The transform's source: a complex array, or a contiguous real one, which the kernels read
    as complex with a zero imaginary part (fft_cooley_tukey.mojo:204-206) without a copy."""
    from .._array import LazyComplex
    from ._utils import contiguous
    if isinstance(x, LazyComplex) and not x.materialised():
        return contiguous(x.re_part)
    if x.is_complex():
        return x
    return contiguous(x)


def _transform(x, dims, norm, inverse):
    """Gradient-free transform used by the forward callables and the fused VJPs."""
    dims = _norm_dims(x, dims)
    n = 1
    for d in dims:
        n *= x.shape()[d]
    out = Array(ArrayShape(x.shape()))
    out.is_complex_flag = True
    setup_shape_and_data(out)
    if out.size():
        run_fft(_as_complex(x), out, dims, inverse, _scale(n, norm, inverse))
    return out


def _fft_node(x, dims, norm, inverse):
    dims_l = list(dims) if dims is not None else []

    def call(curr, args):
        setup_shape_and_data(curr)
        d = _norm_dims(args[0], dims_l)
        n = 1
        for a in d:
            n *= args[0].shape()[a]
        if curr.size():
            run_fft(_as_complex(args[0]), curr, d, inverse, _scale(n, norm, inverse))

    def vjp(primals, grad, out):
        # FFTN.vjp = conj(fftn(conj(grad))) (fftn_op.mojo:43-49); IFFTN.vjp = conj(ifftn(conj(grad)))
        # (ifftn_op.mojo:42-48). Without create_graph both conjugations are fused into the
        # transform's load and store (conj o F o conj = opposite-direction transform).
        if _state.create_graph:
            inner = ifftn if inverse else fftn
            return [conj(inner(conj(grad), dims_l, norm))]
        d = _norm_dims(grad, dims_l)
        n = 1
        for a in d:
            n *= grad.shape()[a]
        res = Array(ArrayShape(grad.shape()))
        res.is_complex_flag = True
        setup_shape_and_data(res)
        if res.size():
            run_fft(_as_complex(grad), res, d, not inverse, _scale(n, norm, inverse))
        return [res]
    return op_array(ArrayShape(x.shape()), [x], "ifftn" if inverse else "fftn", call, vjp=vjp,
                    meta_data=encode_fft_params(dims_l, norm), is_complex_p=True)


def fftn(x, dims=None, norm="backward"):
    return _fft_node(x, dims, norm, False)


def ifftn(x, dims=None, norm="backward"):
    return _fft_node(x, dims, norm, True)


def fft(x, dim=-1, norm="backward"):
    return fftn(x, [dim], norm)


def ifft(x, dim=-1, norm="backward"):
    return ifftn(x, [dim], norm)


def fft2(x, dims=(-2, -1), norm="backward"):
    return fftn(x, list(dims), norm)


def ifft2(x, dims=(-2, -1), norm="backward"):
    return ifftn(x, list(dims), norm)
