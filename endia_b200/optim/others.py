"""SGD (momentum, weight decay), RMSprop and Adagrad (endia/optim/sgd.mojo:17-63,
rmsprop.mojo:17-53, adagrad.mojo:17-45), written like the reference as array expressions over the
elementwise device kernels; in-place updates copy into the parameter's storage."""
from .._array import Array
from ..functional.unary_ops import sqrt


class SGD:
    def __init__(self, params, lr=0.01, momentum=0.0, weight_decay=0.0):
        self.params = list(params)
        self.lr, self.momentum, self.weight_decay = lr, momentum, weight_decay
        self.velocity = [Array(p.shape()) for p in self.params] if momentum > 0 else []

    def step(self):
        for i, p in enumerate(self.params):
            g = p.grad()
            if self.weight_decay > 0:
                g = g + self.weight_decay * p
            if self.momentum > 0:
                self.velocity[i] = self.momentum * self.velocity[i] - self.lr * g
                self.velocity[i].clear_args()
                p += self.velocity[i]
            else:
                p -= self.lr * g
            p.clear_args()


class RMSprop:
    def __init__(self, params, lr=0.01, alpha=0.99, eps=1e-8):
        self.params = list(params)
        self.lr, self.alpha, self.eps = lr, alpha, eps
        self.cache = [Array(p.shape()) for p in self.params]

    def step(self):
        for i, p in enumerate(self.params):
            g = p.grad()
            self.cache[i] = self.alpha * self.cache[i] + (1 - self.alpha) * g * g
            self.cache[i].clear_args()
            p -= self.lr * g / (sqrt(self.cache[i]) + self.eps)
            p.clear_args()


class Adagrad:
    def __init__(self, params, lr=0.01, eps=1e-10):
        self.params = list(params)
        self.lr, self.eps = lr, eps
        self.cache = [Array(p.shape()) for p in self.params]

    def step(self):
        for i, p in enumerate(self.params):
            g = p.grad()
            self.cache[i] = self.cache[i] + g * g
            self.cache[i].clear_args()
            p -= self.lr * g / (sqrt(self.cache[i]) + self.eps)
            p.clear_args()
