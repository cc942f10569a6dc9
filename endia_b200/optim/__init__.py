"""Optimizers (endia/optim/)."""
from .adam import Adam
from .others import SGD, RMSprop, Adagrad
