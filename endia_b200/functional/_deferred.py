"""Deferred kernels around the FFT: the loss on a transform's result and the gradient that flows
back into its VJP transform are folded into the transforms themselves.

The reference evaluates every op eagerly (functional/_utils.mojo:315), so `sum(square(to_abs(
fft(x))))` or `sum(real(fftn(x)) * w)` makes four to six passes over arrays of the transform's size
in each direction. Here the ops of exactly these chains return `Deferred` arrays: ordinary graph
nodes (args, VJP, shape) whose forward kernel has not been enqueued yet. A deferred array runs its
own kernel the moment anything asks for its storage, so every other use behaves as before. When a
full `reduce_add` meets one of the two chains, the transform is enqueued with the loss term summed
in the store of its last pass (endia_b200_fft_c2c_fused), and the node it returns hands the VJP of
the transform a `LazyScaled` gradient (2*g*y, resp. complex(g*w, 0)) that the VJP transform reads
through its `scale_dev` argument: no elementwise pass is left in either direction.
With create_graph=True the fused node's VJP is the reference's composition of differentiable ops.
"""
from .. import _lib
from .._array import Array, ArrayShape


class Deferred(Array):
    """An op result whose forward kernel is enqueued on first access of `buf`.

    kind: "fft" (a transform), "abs" (abs of one), "absr" (real(abs) = to_abs), "abs2"
    (square(to_abs)), "re" (real of a transform), "rew" (real(...) * w); `root` is the transform,
    `w` the real weight array of "rew"."""
    kind = None
    root = None
    w = None

    def __init__(self, array_shape):
        super().__init__(array_shape)
        self._buf = None
        self._thunk = None

    @property
    def buf(self):
        if self._buf is None and self._thunk is not None:
            thunk, self._thunk = self._thunk, None
            thunk()
        return self._buf

    @buf.setter
    def buf(self, value):
        self._buf = value

    def pending(self):
        return self._buf is None and self._thunk is not None


def is_pending(arr, kind):
    return isinstance(arr, Deferred) and arr.kind == kind and arr.pending()


class LazyScaled(Array):
    """factor * g[0] * src as a complex array that is only written when something asks for its
    storage: `g` is a one-element device array (the gradient arriving at a fused loss node), `src`
    a complex array, or a real one standing for complex(src, 0). Its usual consumer, the VJP
    transform of FFTN / IFFTN, reads `src` itself and takes factor and g as the transform's scale."""

    def __init__(self, src, g, factor):
        super().__init__(ArrayShape(src.shape()))
        self.is_complex_flag = True
        self.name = "scaled"
        self.src, self.g, self.factor = src, g, float(factor)
        self._buf = None

    @property
    def buf(self):
        if self._buf is None and self.src is not None:
            from .binary_ops import fused_binary
            from .init_ops import complex as make_complex, full
            from .view_ops import expand
            from ._utils import contiguous
            f = fused_binary(_lib.BIN_MUL, contiguous(self.g), full([1], self.factor))     # [1] real
            if self.src.is_complex():
                fc = make_complex(f, Array(f.shape()))                                    # f + 0i
                self._buf = fused_binary(_lib.BIN_MUL, self.src, fc).buf
            else:
                re = fused_binary(_lib.BIN_MUL, contiguous(self.src), f)
                self._buf = make_complex(re, expand(Array([1]), re.shape())).buf
        return self._buf

    @buf.setter
    def buf(self, value):
        self._buf = value

    def materialised(self):
        return self._buf is not None


def fused_loss(node, axes_shape):
    """reduce_add over all axes of a pending "abs2" / "rew" chain: one op node on the transform's
    result y with the loss term taken in the transform's last pass. Returns None when the chain
    cannot be fused (the caller then reduces the materialised array)."""
    from ..autograd import state as _state
    from ._utils import op_array, setup_shape_and_data
    from .fft_ops import run_root_fused, loss_pass
    root = node.root
    kind = 1 if node.kind == "abs2" else 2
    w = node.w
    if root is None or not isinstance(root, Deferred) or root.kind != "fft":
        return None
    if kind == 2 and (w is None or w.is_complex() or not w.is_contiguous() or w.shape() != root.shape()):
        return None

    def call(curr, args):
        curr.is_complex_flag = False       # (op_array takes the flag from y)
        setup_shape_and_data(curr)
        y = args[0]
        if y.pending():
            run_root_fused(y, kind, w, curr)        # the transform itself, loss term in its last pass
        else:
            loss_pass(y, kind, w, curr)             # y exists already: one pass over it

    def vjp(primals, grad, out):
        y = primals[0]
        if _state.create_graph:
            # the reference's chain, in differentiable ops (square_op.mojo:96, real_op.mojo:75-77,
            # abs_op.mojo:93; mul_op.mojo:125-128)
            from .binary_ops import mul
            from .unary_ops import sign, abs as abs_op
            from .view_ops import real, expand
            from .init_ops import complex as make_complex
            if kind == 1:
                a = real(abs_op(y))
                ga = mul(2.0 * a, grad)
                gz = make_complex(ga, expand(Array([1]), ga.shape()))
                return [mul(sign(y), gz)]
            gr = mul(w, grad)
            return [make_complex(gr, expand(Array([1]), gr.shape()))]
        if kind == 1:
            return [LazyScaled(y, grad, 2.0)]        # 2 |y| * sign(y) * g = 2 g y
        return [LazyScaled(w, grad, 1.0)]            # complex(g * w, 0)
    res = op_array(ArrayShape(axes_shape), [root], "fft_loss", call, vjp=vjp)
    res.is_complex_flag = False
    return res
