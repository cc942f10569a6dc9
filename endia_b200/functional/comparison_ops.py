"""Comparison ops (endia/functional/comparison_ops/): 1.0 / 0.0 arrays, not differentiable."""
from .. import _lib
from .._array import ArrayShape
from ._utils import op_array, setup_shape_and_data, broadcast_shapes, launch_binary
from .view_ops import expand


def _compare(arg0, arg1, name, opcode):
    shape = broadcast_shapes(arg0.shape(), arg1.shape())
    a0, a1 = expand(arg0, shape), expand(arg1, shape)

    def call(curr, args):
        setup_shape_and_data(curr)
        if curr.size():
            launch_binary(opcode, args[0], args[1], curr)
    res = op_array(ArrayShape(shape), [a0, a1], name, call)
    res.requires_grad_flag = False
    res.clear_args()
    return res


def greater(arg0, arg1):
    """arg0 > arg1 elementwise (comparison_ops/greater_op.mojo:46-60); the result carries no graph."""
    return _compare(arg0, arg1, "greater", _lib.BIN_GREATER)


def greater_equal(arg0, arg1):
    """comparison_ops/greater_equal_op.mojo"""
    return _compare(arg0, arg1, "greater_equal", _lib.BIN_GREATER_EQUAL)


def less(arg0, arg1):
    """comparison_ops/less_op.mojo"""
    return _compare(arg0, arg1, "less", _lib.BIN_LESS)


def less_equal(arg0, arg1):
    """comparison_ops/less_equal_op.mojo"""
    return _compare(arg0, arg1, "less_equal", _lib.BIN_LESS_EQUAL)


def equal(arg0, arg1):
    """comparison_ops/equal_op.mojo"""
    return _compare(arg0, arg1, "equal", _lib.BIN_EQUAL)


def not_equal(arg0, arg1):
    """comparison_ops/not_equal_op.mojo"""
    return _compare(arg0, arg1, "not_equal", _lib.BIN_NOT_EQUAL)
