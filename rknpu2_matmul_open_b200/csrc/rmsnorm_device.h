// rmsnorm_device.h -- device side of the residual add + RMSNorm operator (rk_npu_add_rmsnorm_f16.h).
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace rkb200 {

struct AddRmsNormParams {
    const uint4* x;          // 16-byte chunks of 8 fp16 values, in either layout
    const uint4* residual;
    uint4* residual_out;
    uint4* norm_out;
    const uint4* gamma;      // [D / 8] chunks, by d
    int M, D;
    float eps;
    int row_major;           // 0: block-8 (D/8, M, 8); 1: [M, D]
    int tile_tokens;         // set by the launcher
};

// Tokens per tile (a power of two up to 32) and CTAs per cluster (1, 2, 4 or 8) the launcher uses for a shape.
void add_rmsnorm_geometry(int M, int D, int row_major, int& tile_tokens, int& cluster);
cudaError_t launch_add_rmsnorm(const AddRmsNormParams& p, cudaStream_t stream);

} // namespace rkb200
