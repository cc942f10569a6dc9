"""Comparison ops (endia/functional/comparison_ops/): 1.0 / 0.0 arrays, not differentiable."""
from .. import _lib
from .._array import ArrayShape
from ._utils import op_array, setup_shape_and_data, broadcast_shapes, launch_binary
from .view_ops import expand


def greater(arg0, arg1):
    """arg0 > arg1 elementwise (comparison_ops/greater_op.mojo:46-60); the result carries no graph."""
    shape = broadcast_shapes(arg0.shape(), arg1.shape())
    a0, a1 = expand(arg0, shape), expand(arg1, shape)

    def call(curr, args):
        setup_shape_and_data(curr)
        if curr.size():
            launch_binary(_lib.BIN_GREATER, args[0], args[1], curr)
    res = op_array(ArrayShape(shape), [a0, a1], "greater", call)
    res.requires_grad_flag = False
    res.clear_args()
    return res
