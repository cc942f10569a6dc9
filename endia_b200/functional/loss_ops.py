"""Losses (endia/functional/loss_ops/)."""
from .. import _lib
from .._array import Array, ArrayShape, alloc, stream
from ..autograd import state as _state
from ._utils import op_array, setup_shape_and_data
from .binary_ops import sub, mul, add, fused_binary
from .reduce_ops import sum


def _mse_composed(pred, target):
    diff = sub(pred, target)
    return sum(mul(diff, diff)) / float(pred.size())


def mse(pred, target):
    """sum((pred - target) * (pred - target)) / pred.size(), shape [1] (loss_ops/mse_op.mojo:18-20).

    Two real contiguous arrays of one shape run as ONE fused kernel (endia_b200_mse_fwd_bwd) that
    also writes d loss / d pred = 2 (pred - target) / n, which the VJP hands on as it is: the
    reference's chain of sub, mul, reduce, div and their five VJP passes become two launches. With
    create_graph=True the VJP is the differentiable composition of the same formula. Any other
    operands use the op composition."""
    if (pred.is_complex() or target.is_complex() or pred.shape() != target.shape() or pred.size() == 0
            or not pred.is_contiguous() or not target.is_contiguous()):
        return _mse_composed(pred, target)
    n = pred.size()

    def call(curr, args):
        setup_shape_and_data(curr)
        p, t = args
        dpred = None
        if curr.requires_grad_flag:
            dpred = Array(ArrayShape(p.shape()))
            dpred.name = "mse_vjp"
            setup_shape_and_data(dpred)
        scratch = alloc((_lib.lib.endia_b200_mse_scratch_bytes(n) + 3) // 4)
        _lib.call("endia_b200_mse_fwd_bwd", p.data_ptr(), t.data_ptr(), n, 1.0, curr.data_ptr(),
                  dpred.data_ptr() if dpred is not None else None, scratch.data_ptr(), stream())
        curr._dpred = dpred

    def vjp(primals, grad, out):
        p, t = primals
        zero = Array(0)
        if _state.create_graph:
            # d/dp sum(d*d)/n = (d + d) * (grad/n): mul_op.mojo:125-128 applied to both operands of d*d
            d = sub(p, t)
            gp = mul(add(d, d), grad / float(n))
        elif getattr(grad, "_is_ones_seed", False):
            gp = out._dpred            # the seed of backward() is ones(1): nothing to multiply
        else:
            gp = fused_binary(_lib.BIN_MUL, out._dpred, grad)
        gt = zero
        if t.requires_grad():
            from .unary_ops import neg
            gt = neg(gp)
        return [gp if p.requires_grad() else zero, gt]
    return op_array(ArrayShape([1]), [pred, target], "mse", call, vjp=vjp)
