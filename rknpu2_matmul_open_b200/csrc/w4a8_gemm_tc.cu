// w4a8_gemm_tc.cu -- tcgen05 W4A8 GEMM (large-batch path).  Placeholder until the
// kernel lands: reports "unsupported" so every geometry runs on the mma.sync kernel.
#include "w4a8_device.h"
namespace rkb200 {
bool gemm_tc_supported(const GemmParams&) { return false; }
cudaError_t launch_gemm_tc(const GemmParams&, cudaStream_t, bool) { return cudaErrorNotSupported; }
} // namespace rkb200
