"""Process-wide switches read by the VJPs."""
import os

from .. import _lib

# True while a backward pass runs with create_graph=True: VJPs then build differentiable
# compositions instead of fused single-pass kernels.
create_graph = False
# GEMM algorithm handed to endia_b200_gemm (AUTO = tcgen05 3xTF32 when the shape allows).
gemm_algo = _lib.GEMM_AUTO
# Let the dX product of a fused linear layer apply the lower layer's activation-derivative mask and
# sum its bias gradient in its epilogue (ENDIA_B200_FUSE_MASK=1); off: a separate fused kernel.
fuse_mask_into_dx = os.environ.get("ENDIA_B200_FUSE_MASK", "0") == "1"
# Keep the tf32 low part of an op result beside it after its first use as a GEMM operand.
cache_tf32_lo = True
# Optional object with start(flops) / stop() called around every GEMM launch (benchmarks bracket
# the launches with events on the launching stream).
gemm_timer = None
# Same hook around every FFT call: start(algorithmic_bytes) / stop().
fft_timer = None
# Ops of the FFT loss chains (fft -> abs -> real -> square -> sum, fft -> real -> * w -> sum) return
# deferred arrays so that the loss term and its gradient are folded into the transforms
# (functional/_deferred.py); ENDIA_B200_FFT_FUSE=0 runs every op eagerly.
defer_fft_chains = os.environ.get("ENDIA_B200_FFT_FUSE", "1") != "0"
# A list while utils.CapturedStep captures a step (None otherwise): the leaf arrays whose GEMM
# operand parts were computed inside the capture and are shared by the products of that step.
capture_parts = None
# While a reverse walk runs for grad(outs, inputs): the ids of the nodes whose value depends on one of
# `inputs` (None: every gradient is computed). wants_grad() is what the VJPs whose operands' gradients
# are expensive (matrix products) ask instead of requires_grad().
grad_wanted = None


def wants_grad(arr):
    return arr.requires_grad() and (grad_wanted is None or id(arr) in grad_wanted)
