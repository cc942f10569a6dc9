"""Array constructors (endia/functional/init_ops/init_ops.mojo). Random initialisers draw from a
seedable numpy generator on the host (the reference reseeds from the clock on every call,
init_ops.mojo:230,260, so its streams cannot be reproduced)."""
import math

import numpy as np

from .. import _lib
from .._array import Array, ArrayShape, stream
from ._utils import op_array, setup_shape_and_data, launch_unary, launch_binary

_rng = np.random.Generator(np.random.PCG64(0))


def manual_seed(seed):
    global _rng
    _rng = np.random.Generator(np.random.PCG64(seed))


def full(shape, value, requires_grad=False):
    shape = [shape] if isinstance(shape, int) else list(shape)
    out = Array(ArrayShape(shape))
    setup_shape_and_data(out)
    if out.size():
        _lib.call("endia_b200_fill", out.data_ptr(), out.size(), 0, float(value), 0.0, stream())
    out.requires_grad_flag = requires_grad
    return out


def zeros(shape, requires_grad=False):
    return full(shape, 0.0, requires_grad)


def ones(shape, requires_grad=False):
    return full(shape, 1.0, requires_grad)


def zeros_like(arg0):
    return Array(arg0.shape(), is_complex=arg0.is_complex())


def ones_like(arg0):
    return ones(arg0.shape())


def eye(n, requires_grad=False):
    out = Array(ArrayShape([n, n]))
    setup_shape_and_data(out)
    if n:
        _lib.call("endia_b200_eye", out.data_ptr(), n, stream())
    out.requires_grad_flag = requires_grad
    return out


def arange(start, end, step=1.0, requires_grad=False):
    return Array(np.arange(start, end, step, dtype=np.float32), requires_grad=requires_grad)


def linspace(start, end, steps, requires_grad=False):
    return Array(np.linspace(start, end, steps, dtype=np.float32), requires_grad=requires_grad)


def randu(shape, min=0.0, max=1.0, requires_grad=False):
    return Array(_rng.uniform(min, max, size=tuple(shape)).astype(np.float32), requires_grad=requires_grad)


def randn(shape, mean=0.0, std=1.0, requires_grad=False):
    return Array((_rng.standard_normal(size=tuple(shape)) * std + mean).astype(np.float32),
                 requires_grad=requires_grad)


def rand_he_normal(shape, fan_in, requires_grad=False):
    return randn(shape, 0.0, math.sqrt(2.0 / fan_in), requires_grad)


def rand_he_uniform(shape, fan_in, requires_grad=False):
    limit = math.sqrt(6.0 / fan_in)  # init_ops.mojo:307
    return randu(shape, -limit, limit, requires_grad)


def rand_xavier_uniform(shape, fan_in, fan_out, requires_grad=False):
    limit = math.sqrt(6.0 / (fan_in + fan_out))
    return randu(shape, -limit, limit, requires_grad)


def rand_xavier_normal(shape, fan_in, fan_out, requires_grad=False):
    return randn(shape, 0.0, math.sqrt(2.0 / (fan_in + fan_out)), requires_grad)


def rand_lecun_uniform(shape, fan_in, requires_grad=False):
    limit = math.sqrt(3.0 / fan_in)
    return randu(shape, -limit, limit, requires_grad)


def rand_lecun_normal(shape, fan_in, requires_grad=False):
    return randn(shape, 0.0, math.sqrt(1.0 / fan_in), requires_grad)


def complex(real, imag):
    """Interleave two real arrays of equal shape into a complex array; a fresh leaf without graph
    (init_ops.mojo:419-433)."""
    if real.shape() != imag.shape():
        raise _lib.EndiaError(_lib.ESHAPE, "complex: real and imaginary parts must have the same shape")
    out = Array(ArrayShape(real.shape()))
    out.is_complex_flag = True
    setup_shape_and_data(out)
    if out.size() == 0:
        return out
    from .view_ops import expand
    launch_binary(_lib.BIN_COMPLEX, real, imag, out)
    return out
