"""Zero-copy view ops (endia/functional/view_ops/): a view shares the base's device buffer and
only rewrites shape, stride and offset."""
from .. import _lib
from .._array import Array, ArrayShape, compute_stride
from ._utils import op_array, default_vjp, contiguous


def _view_call(curr, args):
    curr.buf = args[0].buf
    curr.base_ = args[0].base()


def _norm_axes(axes, ndim):
    return [a + ndim if a < 0 else a for a in axes]


# ---------------------------------------------------------------------------- expand
def _expand_shape(src, target_shape, ignore_axes):
    """Expand.compute_shape (view_ops/expand_op.mojo:36-84): new leading dims and stretched
    size-1 dims get stride 0. The source offset is kept (the reference resets it to 0)."""
    s_shape, s_stride = src.shape(), src.stride()
    ignore = _norm_axes(ignore_axes, len(s_shape))
    diff = len(target_shape) - len(s_shape)
    if diff < 0:
        raise _lib.EndiaError(_lib.ESHAPE, "Error in broadcast_shape_to: source rank exceeds target rank")
    shape = list(target_shape[:diff])
    stride = [0] * diff
    for i in range(len(s_shape)):
        if i in ignore or s_shape[i] == target_shape[i + diff]:
            shape.append(s_shape[i])
            stride.append(s_stride[i])
        elif s_shape[i] == 1:
            shape.append(target_shape[i + diff])
            stride.append(0)
        else:
            raise _lib.EndiaError(_lib.ESHAPE, "Error in broadcast_shape_to: Incompatible shapes for broadcasting")
    return ArrayShape(shape, stride, src.storage_offset())


def _expand_vjp(primals, grad, out):
    # Reduce over the stretched axes; reduced dims are kept as 1, so a bias gradient has shape
    # (1, N) (expand_op.mojo:121-126, reduce_add_op.mojo:57-62).
    from .reduce_ops import reduce_add
    axes = [i for i, st in enumerate(out.stride()) if st == 0]
    return [reduce_add(grad, axes)]


def expand(arg0, array_shape, ignore_axes=()):
    """Broadcast view of arg0 to `array_shape` (an ArrayShape or a list); returns arg0 itself when
    rank and all non-ignored extents already match (expand_op.mojo:161-172)."""
    target = array_shape.shape if isinstance(array_shape, ArrayShape) else list(array_shape)
    ignore = _norm_axes(list(ignore_axes), arg0.ndim())
    if arg0.ndim() == len(target):
        if all(i in ignore or a == t for i, (a, t) in enumerate(zip(arg0.shape(), target))):
            return arg0
    ig = tuple(ignore_axes)
    return op_array(_expand_shape(arg0, target, ignore_axes), [arg0], "brdcst", _view_call,
                    vjp=_expand_vjp, is_view=True, jvp=lambda p, t: expand(t[0], target, ig))


broadcast_to = expand


def expand_as(arg0, arg1):
    return expand(arg0, arg1.array_shape())


# --------------------------------------------------------------------------- permute
def _perm_axes(axis, ndim):
    """`axis` lists the order of the trailing len(axis) dims (permute_op.mojo:48-60)."""
    if len(axis) > ndim:
        raise _lib.EndiaError(_lib.EINVAL, "Error: Number of axes in the list exceeds the number of dimensions of the ArrayShape")
    perm = list(range(ndim))
    for i, a in enumerate(axis):
        perm[ndim - len(axis) + i] = a + ndim if a < 0 else a
    return perm


def permute(arg0, axis):
    perm = _perm_axes(list(axis), arg0.ndim())
    sh, st = arg0.shape(), arg0.stride()
    shape = ArrayShape([sh[p] for p in perm], [st[p] for p in perm], arg0.storage_offset())
    ax = list(axis)
    return op_array(shape, [arg0], "permute", _view_call,
                    vjp=lambda primals, grad, out: [permute_inv(grad, ax)], is_view=True,
                    jvp=lambda p, t: permute(t[0], ax))


def permute_inv(arg0, axis):
    """Inverse of permute(., axis) (permute_op.mojo:239-357)."""
    perm = _perm_axes(list(axis), arg0.ndim())
    sh, st = arg0.shape(), arg0.stride()
    shape, stride = [0] * len(perm), [0] * len(perm)
    for i, p in enumerate(perm):
        shape[p] = sh[i]
        stride[p] = st[i]
    ax = list(axis)
    return op_array(ArrayShape(shape, stride, arg0.storage_offset()), [arg0], "permute_inv", _view_call,
                    vjp=lambda primals, grad, out: [permute(grad, ax)], is_view=True,
                    jvp=lambda p, t: permute_inv(t[0], ax))


def transpose(arg0, axis1=-1, axis2=-2):
    nd = arg0.ndim()
    a1, a2 = (axis1 + nd) % nd, (axis2 + nd) % nd
    perm = list(range(nd))
    perm[a1], perm[a2] = perm[a2], perm[a1]
    return permute(arg0, perm)


swapaxes = transpose


# ------------------------------------------------------------------ squeeze / unsqueeze
def _squeezable_axes(shape):
    """Every size-1 dim, except that when all dims are 1 the last one stays
    (view_ops/squeeze_op.mojo:34-43)."""
    axes = [i for i, s in enumerate(shape) if s == 1]
    if len(axes) == len(shape) and axes:
        axes.pop()
    return axes


def squeeze(arg0):
    axes = _squeezable_axes(arg0.shape())
    sh, st = arg0.shape(), arg0.stride()
    keep = [i for i in range(len(sh)) if i not in axes]
    shape = ArrayShape([sh[i] for i in keep], [st[i] for i in keep], arg0.storage_offset())
    return op_array(shape, [arg0], "squeeze", _view_call,
                    vjp=lambda primals, grad, out: [unsqueeze(grad, axes)], is_view=True,
                    jvp=lambda p, t: squeeze(t[0]))


def unsqueeze(arg0, axis):
    """Insert size-1 dims at the listed positions (view_ops/unsqueeze_op.mojo:42-74)."""
    axis = list(axis)
    sh, st = arg0.shape(), arg0.stride()
    if not axis:
        shape, stride = list(sh), list(st)
    else:
        shape = [-1] * (axis[-1] + 1)
        stride = [-1] * (axis[-1] + 1)
        for x in axis:
            shape[x] = 1
        idx = 0
        for i in range(len(shape)):
            if shape[i] == -1:
                shape[i], stride[i] = sh[idx], st[idx]
                idx += 1
        shape += sh[idx:]
        stride += st[idx:]
        if stride and stride[-1] == -1:
            stride[-1] = 1
        for i in range(len(stride) - 2, -1, -1):
            if stride[i] == -1:
                stride[i] = stride[i + 1]
    return op_array(ArrayShape(shape, stride, arg0.storage_offset()), [arg0], "unsqueeze", _view_call,
                    vjp=lambda primals, grad, out: [squeeze(grad)], is_view=True,
                    jvp=lambda p, t: unsqueeze(t[0], axis))


# --------------------------------------------------------------------------- reshape
def reshape(arg0, shape):
    """View when the source is contiguous, else a copy first (view_ops/view_op.mojo:62-84);
    one extent may be -1."""
    shape = list(shape)
    if -1 in shape:
        known = 1
        for s in shape:
            if s != -1:
                known *= s
        shape[shape.index(-1)] = arg0.size() // known if known else 0
    n = 1
    for s in shape:
        n *= s
    if n != arg0.size():
        raise _lib.EndiaError(_lib.ESHAPE, "reshape: cannot view %s as %s" % (arg0.shape(), shape))
    src = contiguous_op(arg0)
    prim_shape = arg0.shape()
    return op_array(ArrayShape(shape, compute_stride(shape), src.storage_offset()), [src], "reshape",
                    _view_call, vjp=lambda primals, grad, out: [reshape(grad, prim_shape)], is_view=True,
                    jvp=lambda p, t: reshape(t[0], shape))


view = reshape


def flatten(arg0):
    return reshape(arg0, [arg0.size()])


def contiguous_op(arg0):
    """Differentiable contiguous(): identity for contiguous arrays, else a gathered copy node."""
    if arg0.is_contiguous():
        return arg0

    def fwd(curr, args):
        c = contiguous(args[0])
        curr.buf = c.buf
    return op_array(ArrayShape(arg0.shape()), [arg0], "contiguous", fwd,
                    vjp=lambda primals, grad, out: [grad], jvp=lambda p, t: t[0])


# ------------------------------------------------------------------------ real / imag
def real(arg0):
    """Float view of the real parts: strides and offset doubled, is_complex cleared
    (view_ops/real_op.mojo:43-52, 110); vjp = complex(grad, 0) (:75-77)."""
    if not arg0.is_complex():
        return arg0
    shape = ArrayShape(arg0.shape(), [2 * s for s in arg0.stride()], 2 * arg0.storage_offset())

    def vjp(primals, grad, out):
        from .init_ops import complex as make_complex
        from ..autograd import state as _state
        from .._array import LazyComplex
        from ._utils import contiguous
        if not _state.create_graph and not grad.is_complex():
            return [LazyComplex(contiguous(grad))]   # complex(grad, 0), written only if read as such
        return [make_complex(grad, expand(Array([1]), grad.shape()))]
    from ._deferred import is_pending
    defer = {}
    if is_pending(arg0, "abs"):
        defer = {"deferred": "absr", "root": arg0.root}
    elif is_pending(arg0, "fft"):
        defer = {"deferred": "re", "root": arg0}
    res = op_array(shape, [arg0], "real", _view_call, vjp=vjp, is_view=True, jvp=lambda p, t: real(t[0]), **defer)
    res.is_complex_flag = False
    return res


def imag(arg0):
    """Float view of the imaginary parts; not differentiable in the reference
    (view_ops/imag_op.mojo:61-62 uses the default vjp)."""
    if not arg0.is_complex():
        return Array(arg0.shape())
    shape = ArrayShape(arg0.shape(), [2 * s for s in arg0.stride()], 2 * arg0.storage_offset() + 1)
    res = op_array(shape, [arg0], "imag", _view_call, vjp=default_vjp, is_view=True)
    res.is_complex_flag = False
    return res


def detach(arg0):
    """Same storage, no graph (view_ops/detach_op.mojo)."""
    res = Array(ArrayShape(arg0.shape(), arg0.stride(), arg0.storage_offset()))
    res.buf = arg0.buf
    res.base_ = arg0.base()
    res.is_view = True
    res.is_complex_flag = arg0.is_complex()
    return res
