"""Optimizers (endia/optim/)."""
from .adam import Adam
