"""SGD (momentum, weight decay), RMSprop and Adagrad (endia/optim/sgd.mojo:17-63,
rmsprop.mojo:17-53, adagrad.mojo:17-45), each step one fused multi-tensor launch. The state arrays
take the broadcast shape of (state, grad) like the reference's array expressions do: a bias
gradient is (1, N), so the velocity / cache of a bias becomes (1, N)."""
import ctypes as C

from .. import _lib
from .._array import Array, ArrayShape, stream, drop_operand_parts, flush_readers
from ..functional._utils import contiguous, broadcast_shapes


class _FusedOptimizer:
    """Pointer tables and checks shared by the fused optimizers."""

    def __init__(self, params):
        self.params = list(params)
        self.grad_scale = 1.0

    def _tables(self, state):
        n = len(self.params)
        grads = []
        for p in self.params:
            flush_readers(p)
            if not p.is_contiguous():
                raise _lib.EndiaError(_lib.EINVAL, "optimizer: parameters must be contiguous arrays")
            g = contiguous(p.grad())   # zeros when no gradient is stored (_array.mojo:695-698)
            if g.size() != p.size():
                raise _lib.EndiaError(_lib.ESHAPE, "optimizer: gradient %s does not match parameter %s" % (
                    g.shape(), p.shape()))
            grads.append(g)
        P = (C.c_void_p * n)(*[p.data_ptr() for p in self.params])
        G = (C.c_void_p * n)(*[g.data_ptr() for g in grads])
        S = (C.c_void_p * n)(*[s.data_ptr() for s in state]) if state else None
        numel = (C.c_int64 * n)(*[p.size() for p in self.params])
        return n, P, G, S, numel, grads

    def _after(self, state, grads):
        for s, g in zip(state, grads):
            s.array_shape_ = ArrayShape(broadcast_shapes(s.shape(), g.shape()))
        for p in self.params:
            drop_operand_parts(p)   # the storage changed
            p.clear_args()


class SGD(_FusedOptimizer):
    def __init__(self, params, lr=0.01, momentum=0.0, weight_decay=0.0):
        super().__init__(params)
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        self.velocity = [Array(p.shape()) for p in self.params] if momentum > 0 else []

    def step(self):
        n, P, G, S, numel, grads = self._tables(self.velocity)
        _lib.call("endia_b200_sgd_step_multi", n, P, G, S, numel, self.lr, self.momentum, self.weight_decay,
                  self.grad_scale, stream())
        self._after(self.velocity, grads)


class RMSprop(_FusedOptimizer):
    def __init__(self, params, lr=0.01, alpha=0.99, eps=1e-8):
        super().__init__(params)
        self.lr, self.alpha, self.eps = lr, alpha, eps
        self.cache = [Array(p.shape()) for p in self.params]

    def step(self):
        n, P, G, S, numel, grads = self._tables(self.cache)
        _lib.call("endia_b200_rmsprop_step_multi", n, P, G, S, numel, self.lr, self.alpha, self.eps,
                  self.grad_scale, stream())
        self._after(self.cache, grads)


class Adagrad(_FusedOptimizer):
    def __init__(self, params, lr=0.01, eps=1e-10):
        super().__init__(params)
        self.lr, self.eps = lr, eps
        self.cache = [Array(p.shape()) for p in self.params]

    def step(self):
        n, P, G, S, numel, grads = self._tables(self.cache)
        _lib.call("endia_b200_adagrad_step_multi", n, P, G, S, numel, self.lr, self.eps, self.grad_scale,
                  stream())
        self._after(self.cache, grads)
