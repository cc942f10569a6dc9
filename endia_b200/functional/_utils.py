"""Op registration and storage helpers: the operator boundary of Endia
(endia/functional/_utils.mojo:79-326) with device storage. An op is a forward callable that
fills `curr`'s buffer by enqueuing kernels, plus a VJP written in differentiable ops so that
`create_graph=True` yields graphs of gradients.
"""
from .. import _lib
from .._array import Array, ArrayShape, alloc, compute_stride, stream, drop_operand_parts


def clone_shape(array_shape):
    return ArrayShape(array_shape.shape)


def setup_shape_and_data(curr):
    """Allocate `curr`'s storage for its shape (functional/_utils.mojo:319-326). The reference
    zero-fills; here every forward kernel writes its whole output instead."""
    if curr.buf is None:
        curr.buf = alloc(curr.size() * (2 if curr.is_complex() else 1))


def op_array(array_shape, args, name, callable, vjp=None, jvp=None, is_view=False, meta_data=None,
             is_complex_p=False, kwargs=None, deferred=None, root=None, w=None):
    """Create the result node of an op and run its forward (functional/_utils.mojo:208-316).

    requires_grad is the OR over the args and the complex flag is the OR over the args (or
    forced); graph edges and the VJP are stored only when a gradient can flow (:262-272).
    `deferred` names the node's place in one of the FFT loss chains (functional/_deferred.py): the
    forward then runs when the result's storage is first asked for."""
    from ..autograd import state as _state
    if deferred is not None and _state.defer_fft_chains:
        from ._deferred import Deferred
        curr = Deferred(array_shape)
        curr.kind, curr.root, curr.w = deferred, root, w
    else:
        deferred = None
        curr = Array(array_shape)
    curr.name = name
    curr.is_view = is_view
    curr.meta_data = list(meta_data) if meta_data else []
    curr.is_complex_flag = bool(is_complex_p) or any(a.is_complex() for a in args)
    curr.requires_grad_flag = any(a.requires_grad() for a in args)
    if curr.requires_grad_flag:
        curr.args_ = list(args)
        curr.vjp_ = vjp
        curr.jvp_ = jvp
    if deferred is not None:
        curr._thunk = lambda: callable(curr, args)
    else:
        callable(curr, args)
    return curr


def default_vjp(primals, grad, out):
    """Pass-through used by non-differentiable ops (_array.mojo:43-47)."""
    print("Attention: Default vjp is being used!")
    return [grad for _ in primals]


def broadcast_shapes(s0, s1):
    """Right-aligned numpy broadcasting (endia/utils/_array_shape.mojo:366-411)."""
    n = max(len(s0), len(s1))
    out = []
    for i in range(n):
        a = s0[len(s0) - n + i] if len(s0) - n + i >= 0 else None
        b = s1[len(s1) - n + i] if len(s1) - n + i >= 0 else None
        if a is None:
            out.append(b)
        elif b is None:
            out.append(a)
        elif a == b or b == 1:
            out.append(a)
        elif a == 1:
            out.append(b)
        else:
            raise _lib.EndiaError(_lib.ESHAPE, "Error: Incompatible shapes for broadcasting: %s %s" % (s0, s1))
    return out


def launch_unary(opcode, src, dst):
    _lib.call("endia_b200_ew_unary", opcode, src.desc(), dst.desc(), stream())


def launch_binary(opcode, a, b, dst):
    _lib.call("endia_b200_ew_binary", opcode, a.desc(), b.desc(), dst.desc(), stream())


def copy(arg):
    """Fresh contiguous array with arg's logical contents (functional/_utils.mojo:179-199)."""
    out = Array(ArrayShape(arg.shape()))
    out.is_complex_flag = arg.is_complex()
    setup_shape_and_data(out)
    if out.size():
        launch_unary(_lib.UN_COPY, arg, out)
    return out


def contiguous(arg):
    """`arg` itself when already contiguous, else a gathered copy (functional/_utils.mojo:201-205)."""
    return arg if arg.is_contiguous() else copy(arg)


def copy_into(src, dst):
    """Flat copy of src's logical elements into dst's storage (execute_copy_raw as used by the
    in-place operators, _array.mojo:998-1006). dst keeps its own shape; sizes must match."""
    if src.size() != dst.size():
        raise _lib.EndiaError(_lib.ESHAPE, "in-place update: size mismatch %s vs %s" % (src.shape(), dst.shape()))
    if not dst.is_contiguous():
        raise _lib.EndiaError(_lib.EINVAL, "in-place update of a non-contiguous view is not supported")
    s = contiguous(src)
    from .._array import flush_readers
    flush_readers(dst)        # deferred kernels that read the old contents run first
    w = 2 if dst.is_complex() else 1
    if s.is_complex() != dst.is_complex():
        raise _lib.EndiaError(_lib.EINVAL, "in-place update: complex flag mismatch")
    _lib.call("endia_b200_d2d", dst.data_ptr(), s.data_ptr(), dst.size() * w * 4, stream())
    drop_operand_parts(dst)   # cached GEMM operand parts no longer match the storage
