"""Sum reductions (endia/functional/reduce_ops/): reduce_add keeps reduced dims as 1; sum and
mean squeeze afterwards, so a full reduction has shape [1]."""
from .. import _lib
from .._array import ArrayShape, alloc, stream
from ._utils import op_array, setup_shape_and_data
from .view_ops import expand, squeeze


def reduce_add(arg0, axis):
    """Sum over `axis`, reduced dims kept with extent 1 (reduce_add_op.mojo:39-62); the vjp
    expands the gradient back to the primal's shape (:234)."""
    nd = arg0.ndim()
    axes = sorted(set(a + nd if a < 0 else a for a in axis))
    shape = [1 if i in axes else s for i, s in enumerate(arg0.shape())]
    mask = 0
    for a in axes:
        mask |= 1 << a
    if len(axes) == nd:
        # the full sum of one of the FFT loss chains is taken inside the transform (_deferred.py)
        from ._deferred import is_pending, fused_loss
        if is_pending(arg0, "abs2") or is_pending(arg0, "rew"):
            fused = fused_loss(arg0, shape)
            if fused is not None:
                return fused

    def call(curr, args):
        setup_shape_and_data(curr)
        if curr.size() == 0:
            return
        d = args[0].desc()
        nbytes = _lib.lib.endia_b200_reduce_scratch_bytes(d, mask)
        scratch = alloc((nbytes + 3) // 4) if nbytes else None
        _lib.call("endia_b200_reduce_add", d, mask, curr.data_ptr(),
                  scratch.data_ptr() if scratch is not None else None, stream())

    def vjp(primals, grad, out):
        return [expand(grad, primals[0].array_shape())]
    return op_array(ArrayShape(shape), [arg0], "reduce_add", call, vjp=vjp,
                    jvp=lambda p, t: reduce_add(t[0], axes))


def sum(arg0):
    """Sum over all axes; shape [1] (sum_op.mojo:35-62, squeeze keeps the last dim)."""
    return squeeze(reduce_add(arg0, list(range(arg0.ndim()))))


def mean(arg0, axes=None, keepdims=False):
    """reduce_add / (size_in / size_out) (mean_op.mojo:35-65)."""
    if axes is None:
        axes = list(range(arg0.ndim()))
    res = reduce_add(arg0, axes)
    divisor = float(arg0.size() / res.size())
    out = res / divisor
    return out if keepdims else squeeze(out)


def reduce_mul(arg0, axis):
    """Product over `axis`, reduced dims kept with extent 1 (reduce_ops/reduce_mul_op.mojo). The VJP is
    the derivative of the product, expand(grad * out) / x; the reference's own VJP returns the
    expanded gradient unchanged (reduce_mul_op.mojo:238-255), which is reduce_add's."""
    if arg0.is_complex():
        raise _lib.EndiaError(_lib.EINVAL, "reduce_mul: real arrays only")
    nd = arg0.ndim()
    axes = sorted(set(a + nd if a < 0 else a for a in axis))
    shape = [1 if i in axes else s for i, s in enumerate(arg0.shape())]
    mask = 0
    for a in axes:
        mask |= 1 << a

    def call(curr, args):
        setup_shape_and_data(curr)
        if curr.size() == 0:
            return
        d = args[0].desc()
        nbytes = _lib.lib.endia_b200_reduce_scratch_bytes(d, mask)
        scratch = alloc((nbytes + 3) // 4) if nbytes else None
        _lib.call("endia_b200_reduce_mul", d, mask, curr.data_ptr(),
                  scratch.data_ptr() if scratch is not None else None, stream())

    def vjp(primals, grad, out):
        from .binary_ops import mul, div
        return [div(expand(mul(grad, out), primals[0].array_shape()), primals[0])]
    return op_array(ArrayShape(shape), [arg0], "reduce_mul", call, vjp=vjp)


def prod(arg0):
    """Product over all axes; shape [1] (reduce_ops/prod_op.mojo)."""
    return squeeze(reduce_mul(arg0, list(range(arg0.ndim()))))


def variance(arg0, axes=None, unbiased=True, keepdims=False):
    """reduce_add((x - mean)^2) / (n - 1), or / n when not unbiased, n = elements per output
    (reduce_ops/variance_op.mojo:65-79); a composition of differentiable ops."""
    if axes is None:
        axes = list(range(arg0.ndim()))
    res = reduce_add(arg0, axes)
    n = float(arg0.size() / res.size())
    divisor = n - 1.0 if unbiased else n
    mean_res = res / n
    diff = arg0 - mean_res
    var = reduce_add(diff * diff, axes) / divisor
    return var if keepdims else squeeze(var)


def std(arg0, axes=None, unbiased=True, keepdims=False):
    """sqrt(variance) (reduce_ops/std_op.mojo)."""
    from .unary_ops import sqrt
    return sqrt(variance(arg0, axes, unbiased, keepdims))
