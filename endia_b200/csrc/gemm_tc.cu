// Placeholder for the tcgen05 3xTF32 GEMM (filled in by gemm_tc.cu proper).
#include "common.cuh"
#include "gemm.cuh"
namespace eb {
bool tc_gemm_supported(const GemmParams &, int, int, int64_t) { return false; }
int launch_gemm_tc(const GemmParams &, int, int, cudaStream_t) {
  set_error("tcgen05 GEMM not built");
  return ENDIA_B200_EINVAL;
}
}  // namespace eb
extern "C" int endia_b200_has_tcgen05(void) { return 0; }
