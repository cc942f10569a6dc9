"""endia_b200: B200-native device path for Endia's reverse-mode hot path, behind Endia's own API
(`import endia_b200 as nd`): Array/Tensor, the functional ops, backward/grad/jacobian/hessian,
nn.MLP, optim.Adam and the FFT family. Every computation runs in hand-written sm_100a CUDA kernels
through the C ABI of libendia_b200.so; there is no CPU fallback."""
from ._lib import EndiaError
from ._array import Array, Tensor, ndarray, ArrayShape
from .functional import *  # noqa: F401,F403
from .functional import sum, abs, pow, complex  # noqa: F401  (shadow builtins on purpose, as Endia does)
from .autograd.functional import backward, jacrev, grad, jacobian, hessian, value_and_grad, Callable, jvp
from . import nn, optim
from .autograd import state as config
