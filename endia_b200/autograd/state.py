"""Process-wide switches read by the VJPs."""
from .. import _lib

# True while a backward pass runs with create_graph=True: VJPs then build differentiable
# compositions instead of fused single-pass kernels.
create_graph = False
# GEMM algorithm handed to endia_b200_gemm (AUTO = tcgen05 3xTF32 when the shape allows).
gemm_algo = _lib.GEMM_AUTO
