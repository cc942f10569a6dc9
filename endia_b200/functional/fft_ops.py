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
    """Factor applied to a transform over n points. "backward" is the reference's scaling (nothing
    forward, 1/n inverse). "forward" and "ortho" follow numpy.fft; the reference instead divides the
    input by the size of the whole array, takes any other string for "ortho"
    (fft_cooley_tukey.mojo:208-215) and still applies ifftn's 1/prod(n) (ifftn_op.mojo:67-77), which
    is taken for a defect and not reproduced."""
    if norm == "ortho":
        return 1.0 / math.sqrt(n)
    if (norm == "backward") == bool(inverse):
        return 1.0 / n
    return 1.0


def run_fft(src, dst, dims, direction_inverse, scale, scale_dev=None, reduce=0, reduce_w=None, reduce_out=None):
    """Enqueue one C-ABI transform of `src` (complex, any strides, or contiguous real) into `dst`
    (contiguous). `scale_dev` (a one-element device Array) is multiplied into the scale by the last
    pass; `reduce` / `reduce_w` / `reduce_out` fuse a loss term into that pass (endia_b200_fft_fusion)."""
    cd = (C.c_int32 * len(dims))(*dims)
    sd, dd = src.desc(), dst.desc()
    nbytes = _lib.lib.endia_b200_fft_scratch_bytes(sd, cd, len(dims))
    scratch = alloc((nbytes + 3) // 4) if nbytes else None
    fusion = None
    keep = None
    if scale_dev is not None or reduce:
        fusion = _lib.FftFusion()
        fusion.scale_dev = scale_dev.data_ptr() if scale_dev is not None else None
        fusion.reduce = int(reduce)
        fusion.reduce_scale = 1.0
        if reduce:
            keep = alloc((_lib.lib.endia_b200_fft_fusion_scratch_bytes() + 3) // 4)
            fusion.reduce_scratch = keep.data_ptr()
            fusion.reduce_out = reduce_out.data_ptr()
            fusion.reduce_w = reduce_w.data_ptr() if reduce_w is not None else None
    timer = _state.fft_timer
    if timer is not None:
        timer.start(16.0 * src.size())   # algorithmic bytes: one read and one write of the array
    _lib.call("endia_b200_fft_c2c_fused", sd, dd, cd, len(dims), 1 if direction_inverse else 0,
              float(scale), scratch.data_ptr() if scratch is not None else None,
              C.byref(fusion) if fusion is not None else None, stream())
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


def _vjp_source(grad):
    """(source array, device scale or None, host factor) of the transform a VJP runs on `grad`: a
    gradient that is still a LazyScaled product is read through its source and the scale."""
    from ._deferred import LazyScaled
    from ._utils import contiguous
    if isinstance(grad, LazyScaled) and not grad.materialised():
        src = grad.src if grad.src.is_complex() else contiguous(grad.src)
        return src, contiguous(grad.g), grad.factor
    return _as_complex(grad), None, 1.0


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


def run_root_fused(y, kind, w, loss_out):
    """Enqueue the pending transform `y` (a Deferred of kind "fft") with the loss term `kind`
    (1: sum |y|^2, 2: sum real(y) * w) summed into loss_out in its last pass."""
    src, d, inverse, scale = y._fft_args
    y._thunk = None
    setup_shape_and_data(y)
    run_fft(_as_complex(src), y, d, inverse, scale, reduce=kind, reduce_w=w, reduce_out=loss_out)


def loss_pass(y, kind, w, loss_out):
    """The same loss term in one pass over a transform result that exists already."""
    keep = alloc((_lib.lib.endia_b200_fft_fusion_scratch_bytes() + 3) // 4)
    _lib.call("endia_b200_fft_loss_term", y.desc(), int(kind), w.data_ptr() if w is not None else None,
              loss_out.data_ptr(), 1.0, keep.data_ptr(), stream())


_MAX_LINE = 4096      # longest line one kernel pass transforms; longer ones split into two passes


def _check_lengths(x, d):
    """The checks of endia_b200_fft_c2c that depend on the shape only, made when the op is created
    (the transform itself may run later): power-of-two lengths (fft_cooley_tukey.mojo:227-235) and
    the length limits of the kernels."""
    if len(set(d)) != len(d):
        raise _lib.EndiaError(_lib.EINVAL, "fft: a dim is listed twice")
    shape = x.shape()
    for a in d:
        n = shape[a]
        if n < 1 or n & (n - 1):
            raise _lib.EndiaError(_lib.EPOW2, "fft: length %d of dim %d is not a power of two" % (n, a))
        if n > _MAX_LINE:
            inner = 1
            for e in shape[a + 1:]:
                inner *= e
            if n > _MAX_LINE * _MAX_LINE or inner != 1:
                raise _lib.EndiaError(_lib.ELIMIT, "fft: lengths above %d are supported on the innermost axis only "
                                                   "(up to %d)" % (_MAX_LINE, _MAX_LINE * _MAX_LINE))


def _fft_node(x, dims, norm, inverse):
    from ._deferred import Deferred
    from .._array import watch_input
    dims_l = list(dims) if dims is not None else []
    d = _norm_dims(x, dims_l)
    _check_lengths(x, d)
    n = 1
    for a in d:
        n *= x.shape()[a]
    scale = _scale(n, norm, inverse)

    def call(curr, args):
        setup_shape_and_data(curr)
        if curr.size():
            run_fft(_as_complex(args[0]), curr, d, inverse, scale)

    def vjp(primals, grad, out):
        # FFTN.vjp = conj(fftn(conj(grad))) (fftn_op.mojo:43-49); IFFTN.vjp = conj(ifftn(conj(grad)))
        # (ifftn_op.mojo:42-48). Without create_graph both conjugations are fused into the
        # transform's load and store (conj o F o conj = opposite-direction transform).
        if _state.create_graph:
            inner = ifftn if inverse else fftn
            return [conj(inner(conj(grad), dims_l, norm))]
        res = Array(ArrayShape(grad.shape()))
        res.is_complex_flag = True
        setup_shape_and_data(res)
        if res.size():
            src, scale_dev, factor = _vjp_source(grad)
            run_fft(src, res, d, not inverse, scale * factor, scale_dev=scale_dev)
        return [res]
    res = op_array(ArrayShape(x.shape()), [x], "ifftn" if inverse else "fftn", call, vjp=vjp,
                   jvp=lambda p, t: (ifftn if inverse else fftn)(t[0], dims_l, norm),     # the transform is linear
                   meta_data=encode_fft_params(dims_l, norm), is_complex_p=True, deferred="fft")
    if isinstance(res, Deferred) and res.pending():
        res._fft_args = (x, d, inverse, scale)
        watch_input(x, res)
    return res


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
