"""Free-function ops of Endia (endia/functional/__init__.mojo)."""
from ._utils import (op_array, setup_shape_and_data, clone_shape, contiguous, copy, default_vjp,
                     broadcast_shapes)
from .binary_ops import add, sub, mul, div, pow_to, pow, matmul
from .comparison_ops import greater, greater_equal, less, less_equal, equal, not_equal
from .unary_ops import (neg, relu, tanh, sigmoid, square, sqrt, conj, sign, abs, to_abs, exp, log,
                        sin, cos, reciprocal, sinh, cosh, tan, asin, acos, atan)
from .reduce_ops import reduce_add, sum, mean, reduce_mul, prod, variance, std
from .view_ops import (expand, broadcast_to, expand_as, permute, permute_inv, transpose, swapaxes,
                       squeeze, unsqueeze, reshape, view, flatten, real, imag, detach, contiguous_op)
from .loss_ops import mse
from .init_ops import (full, zeros, ones, zeros_like, ones_like, eye, arange, linspace, randu, randn,
                       rand_he_normal, rand_he_uniform, rand_xavier_uniform, rand_xavier_normal,
                       rand_lecun_uniform, rand_lecun_normal, complex, manual_seed)
from .fft_ops import fft, ifft, fft2, ifft2, fftn, ifftn
