"""Neural-network layer of Endia (endia/nn/): MLP module and functional mlp."""
from .modules import MLP, mlp, linear, fused_train_step, SmallMLPStep
