"""Unary elementwise ops (endia/functional/unary_ops/); VJPs are compositions of ops."""
from .. import _lib
from .._array import Array, ArrayShape
from ..autograd import state as _state
from ._utils import op_array, setup_shape_and_data, launch_unary


def _unary_call(opcode):
    def call(curr, args):
        setup_shape_and_data(curr)
        if curr.size():
            launch_unary(opcode, args[0], curr)
    return call


def unary_op_array(arg0, name, opcode, vjp, jvp=None, **defer):
    return op_array(ArrayShape(arg0.shape()), [arg0], name, _unary_call(opcode), vjp=vjp, jvp=jvp, **defer)


def _m(a, b):
    from .binary_ops import mul
    return mul(a, b)


def _fused(opcode, a, b):
    from .binary_ops import fused_binary
    return fused_binary(opcode, a, b)


def neg(arg0):
    return unary_op_array(arg0, "neg", _lib.UN_NEG, lambda p, g, o: [neg(g)],     # neg_op.mojo:91
                          jvp=lambda p, t: neg(t[0]))


def _relu_vjp(primals, grad, out):
    # greater(x, 0) * grad, strict > (relu_op.mojo:95)
    if not _state.create_graph:
        return [_fused(_lib.BIN_RELU_BWD, primals[0], grad)]
    from .comparison_ops import greater
    from .binary_ops import mul
    return [mul(greater(primals[0], Array([primals[0].shape()[-1]])), grad)]


def relu(arg0):
    if arg0.is_complex():
        raise _lib.EndiaError(_lib.EINVAL, "Warning: Relu does not support complex numbers")  # relu_op.mojo:51-52
    def jvp(p, t):
        from .comparison_ops import greater
        return _m(greater(p[0], Array([p[0].shape()[-1]])), t[0])
    return unary_op_array(arg0, "relu", _lib.UN_RELU, _relu_vjp, jvp=jvp)


def _tanh_vjp(primals, grad, out):
    # (1 - square(tanh(x))) * grad, tanh recomputed from the primal (tanh_op.mojo:92)
    if not _state.create_graph and not primals[0].is_complex():
        return [_fused(_lib.BIN_TANH_BWD, primals[0], grad)]
    from .binary_ops import mul
    return [mul(1.0 - square(tanh(primals[0])), grad)]


def tanh(arg0):
    return unary_op_array(arg0, "tanh", _lib.UN_TANH, _tanh_vjp,
                          jvp=lambda p, t: _m(1.0 - square(tanh(p[0])), t[0]))        # tanh_op.mojo:56-73


def _sigmoid_vjp(primals, grad, out):
    # out * (1 - out) * grad (sigmoid_op.mojo:98)
    if not _state.create_graph:
        return [_fused(_lib.BIN_SIGMOID_BWD, out, grad)]
    from .binary_ops import mul
    return [mul(mul(out, 1.0 - out), grad)]


def sigmoid(arg0):
    if arg0.is_complex():
        raise _lib.EndiaError(_lib.EINVAL, "Warning: Sigmoid does not support complex numbers")  # sigmoid_op.mojo:49-50
    def jvp(p, t):
        sg = sigmoid(p[0])
        return _m(_m(sg, 1.0 - sg), t[0])
    return unary_op_array(arg0, "sigmoid", _lib.UN_SIGMOID, _sigmoid_vjp, jvp=jvp)


def _square_vjp(primals, grad, out):
    # 2 * x * grad (square_op.mojo:96); one fused pass when no graph of the gradient is kept
    if not _state.create_graph:
        return [_fused(_lib.BIN_SQUARE_BWD, primals[0], grad)]
    from .binary_ops import mul
    return [mul(2.0 * primals[0], grad)]


def square(arg0):
    from ._deferred import is_pending
    if is_pending(arg0, "absr"):       # square(to_abs(fft(x))): see _deferred.py
        return unary_op_array(arg0, "square", _lib.UN_SQUARE, _square_vjp, deferred="abs2", root=arg0.root)
    return unary_op_array(arg0, "square", _lib.UN_SQUARE, _square_vjp, jvp=lambda p, t: _m(2.0 * p[0], t[0]))


def sqrt(arg0):
    from .binary_ops import div
    return unary_op_array(arg0, "sqrt", _lib.UN_SQRT, lambda p, g, o: [div(g, 2.0 * sqrt(p[0]))],  # sqrt_op.mojo:91
                          jvp=lambda p, t: div(t[0], 2.0 * sqrt(p[0])))


def conj(arg0):
    return unary_op_array(arg0, "conj", _lib.UN_CONJ, lambda p, g, o: [conj(g)],  # conj_op.mojo
                          jvp=lambda p, t: conj(t[0]))


def sign(arg0):
    from ._utils import default_vjp
    return unary_op_array(arg0, "sign", _lib.UN_SIGN, default_vjp)  # sign_op.mojo: default vjp


def _abs_vjp(primals, grad, out):
    # sign(x) * grad (abs_op.mojo:93); one fused pass when no graph of the gradient is kept
    if not _state.create_graph:
        return [_fused(_lib.BIN_ABS_BWD, primals[0], grad)]
    from .binary_ops import mul
    return [mul(sign(primals[0]), grad)]


def abs(arg0):
    from ._deferred import is_pending
    if is_pending(arg0, "fft"):
        return unary_op_array(arg0, "abs", _lib.UN_ABS, _abs_vjp, deferred="abs", root=arg0)
    return unary_op_array(arg0, "abs", _lib.UN_ABS, _abs_vjp, jvp=lambda p, t: _m(sign(p[0]), t[0]))


def to_abs(arg0):
    """abs as a real array (abs_op.mojo:157)."""
    from .view_ops import real
    return real(abs(arg0))


def exp(arg0):
    from .binary_ops import mul
    return unary_op_array(arg0, "exp", _lib.UN_EXP, lambda p, g, o: [mul(exp(p[0]), g)],
                          jvp=lambda p, t: mul(exp(p[0]), t[0]))


def log(arg0):
    from .binary_ops import div
    return unary_op_array(arg0, "log", _lib.UN_LOG, lambda p, g, o: [div(g, p[0])],  # log_op.mojo:91
                          jvp=lambda p, t: div(t[0], p[0]))


def sin(arg0):
    from .binary_ops import mul
    return unary_op_array(arg0, "sin", _lib.UN_SIN, lambda p, g, o: [mul(cos(p[0]), g)],
                          jvp=lambda p, t: mul(cos(p[0]), t[0]))


def cos(arg0):
    from .binary_ops import mul
    return unary_op_array(arg0, "cos", _lib.UN_COS, lambda p, g, o: [mul(neg(sin(p[0])), g)],
                          jvp=lambda p, t: mul(neg(sin(p[0])), t[0]))


def reciprocal(arg0):
    from .binary_ops import div
    return unary_op_array(arg0, "reciprocal", _lib.UN_RECIPROCAL,
                          lambda p, g, o: [div(neg(g), square(p[0]))],
                          jvp=lambda p, t: div(neg(t[0]), square(p[0])))


def sinh(arg0):
    """vjp cosh(x) * grad (sinh_op.mojo:68, 88)."""
    return unary_op_array(arg0, "sinh", _lib.UN_SINH, lambda p, g, o: [_m(cosh(p[0]), g)],
                          jvp=lambda p, t: _m(cosh(p[0]), t[0]))


def cosh(arg0):
    """vjp sinh(x) * grad (cosh_op.mojo:69, 89)."""
    return unary_op_array(arg0, "cosh", _lib.UN_COSH, lambda p, g, o: [_m(sinh(p[0]), g)],
                          jvp=lambda p, t: _m(sinh(p[0]), t[0]))


def tan(arg0):
    """vjp grad * (1 + out^2) (tan_op.mojo:81). The jvp is (1 + tan(x)^2) * dx; the reference's line
    `1 + square(tan(x)) * dx` (tan_op.mojo:65) binds the product first."""
    return unary_op_array(arg0, "tan", _lib.UN_TAN, lambda p, g, o: [_m(g, 1.0 + square(o))],
                          jvp=lambda p, t: _m(1.0 + square(tan(p[0])), t[0]))


def asin(arg0):
    """vjp grad / sqrt(1 - x^2) (asin_op.mojo:83); the jvp is the same factor (the reference writes
    1 / cos(x), asin_op.mojo:67, which is the derivative of another function)."""
    from .binary_ops import div
    return unary_op_array(arg0, "asin", _lib.UN_ASIN, lambda p, g, o: [div(g, sqrt(1.0 - square(p[0])))],
                          jvp=lambda p, t: div(t[0], sqrt(1.0 - square(p[0]))))


def acos(arg0):
    """vjp -grad / sqrt(1 - x^2) (acos_op.mojo:71, 91)."""
    from .binary_ops import div
    return unary_op_array(arg0, "acos", _lib.UN_ACOS, lambda p, g, o: [div(neg(g), sqrt(1.0 - square(p[0])))],
                          jvp=lambda p, t: div(neg(t[0]), sqrt(1.0 - square(p[0]))))


def atan(arg0):
    """vjp grad / (1 + x^2) (atan_op.mojo:69, 85)."""
    from .binary_ops import div
    return unary_op_array(arg0, "atan", _lib.UN_ATAN, lambda p, g, o: [div(g, 1.0 + square(p[0]))],
                          jvp=lambda p, t: div(t[0], 1.0 + square(p[0])))
