"""Losses (endia/functional/loss_ops/)."""
from .binary_ops import sub, mul
from .reduce_ops import sum


def mse(pred, target):
    """sum((pred - target) * (pred - target)) / pred.size()  (loss_ops/mse_op.mojo:18-20)."""
    diff = sub(pred, target)
    return sum(mul(diff, diff)) / float(pred.size())
