// moe_device.h -- device side of the routed-experts operator (rk_npu_moe_w8.h): parameter blocks and launchers.
//
// A run is a list of JOBS: up to 16 (token, slot) assignments that use the same expert.  Three launches work
// on the list: gate/up projection + SwiGLU (fp32 middle rows and their maxima), down projection (re-quantises
// the middle rows on the way into shared memory), and the weighted sum over each token's slots.
#pragma once
#include "w4a8_device.h"
#include <cuda_runtime.h>
#include <stdint.h>

namespace rkb200 {

constexpr int MOE_JOB_ROWS = 16;     // assignments per job: two 8-token halves of mma.m16n8k32
constexpr int MOE_KQ = 128;          // k extent of one packed weight record (four k-steps of 32)

// Packed int8 expert matrix W[K][N] (N a multiple of 16): records of 16 channels x 128 k in the register order
// of the m16n8k32 A operand, [channel block][k quarter-kilo][k-step 0..3][lane][16 B = a0 a1 a2 a3], zero beyond K.
inline size_t moe_packed_bytes(int K, int N) { return size_t((K + MOE_KQ - 1) / MOE_KQ) * MOE_KQ * size_t(N); }
// Int4 experts keep two codes per byte: [channel block][k quarter-kilo][half 0..1][lane][16 B], the 16 bytes being the
// words of k-steps 2 half and 2 half + 1 for channels g and g + 8; a word w holds the codes at k = 4t.. in its low
// nibbles and those at k = 16 + 4t.. in its high nibbles, so that (w << 4) & 0xF0F0F0F0 and w & 0xF0F0F0F0 are the two
// A registers of the channel with every code times 16 (the sums are shifted back, exactly).  Half the bytes.
inline size_t moe_packed_nibble_bytes(int K, int N) { return moe_packed_bytes(K, N) / 2; }
// A bank of experts: the first `nibble_experts` hold int4 records, the rest int8 records.  An immutable bank is one
// allocation (`base`, experts at fixed strides) with its scales in one array; a slot bank keeps every expert in an
// allocation of its own, which can change hands between banks, and gives the kernels two tables of pointers instead
// (`table`: each expert's records; `scale_table`: each expert's scales).
struct MoeBank {
    const uint8_t* base;
    size_t nibble_bytes, byte_bytes;   // one expert's records in either form
    int nibble_experts;
    const uint8_t* const* table;       // slot banks only, else null
    const float* const* scale_table;   // slot banks only, else null
    __host__ __device__ const uint8_t* expert(int e) const
    {
        if (table) return table[e];
        return e < nibble_experts ? base + size_t(e) * nibble_bytes
                                  : base + size_t(nibble_experts) * nibble_bytes + size_t(e - nibble_experts) * byte_bytes;
    }
    // the scales of expert e: `all` holds `stride` per expert where there is no table
    __host__ __device__ const float* scales(int e, const float* all, int stride) const
    {
        return scale_table ? scale_table[e] : all + size_t(e) * stride;
    }
    __host__ __device__ bool nibbles(int e) const { return e < nibble_experts; }
};

struct MoePackParams {
    const int8_t* W;      // [K][N] row-major, on the device
    uint8_t* packed;
    int K, N;
    int nibbles;          // 1: int4 codes, two per byte
};

struct MoeQuantParams {
    const float* X;       // [rows][H]
    int8_t* codes;        // [rows][H]
    float* scales;        // [rows]
    Status* status;       // bad_input: a non-finite element, or a scale whose reciprocal is not finite
    int rows, H;
};

struct MoeSchedule {
    const int* job_expert;     // [jobs]
    const int* job_first;      // [jobs] first assignment of the job
    const int* job_rows;       // [jobs] 1..16
    const int* assign_token;   // [assignments] source row of each assignment (assignments of a job are consecutive)
    int jobs;
};

struct MoeGateUpParams {
    MoeSchedule sched;
    MoeBank bank;                // experts' gate/up matrices
    const float* w_scales;       // [E][2I] (immutable banks; a slot bank's come from its table)
    const int8_t* codes;         // [rows][H]
    const float* in_scales;      // [rows]
    float* middle;               // [assignments][I]
    uint32_t* row_max;           // [assignments] bit patterns of max |middle|, zero before the launch
    int H, I;
};

struct MoeDownParams {
    MoeSchedule sched;
    MoeBank bank;                // experts' down matrices
    const float* w_scales;       // [E][H] (immutable banks)
    const float* middle;         // [assignments][I]
    const uint32_t* row_max;     // [assignments]
    float* expert_out;           // [assignments][H]
    int H, I;
};

struct MoeCombineParams {
    const float* expert_out;     // [assignments][H]
    const int* slot_assign;      // [rows][slots] assignment index, -1: the slot takes no part
    const float* coefficients;   // [rows][slots]
    float* out;                  // [rows][H]
    uint32_t* row_max;           // [assignments] cleared here for the next run
    int rows, slots, H;
};

cudaError_t launch_moe_pack(const MoePackParams& p, cudaStream_t stream);
cudaError_t launch_moe_quantize(const MoeQuantParams& p, cudaStream_t stream);
cudaError_t launch_moe_gate_up(const MoeGateUpParams& p, cudaStream_t stream);
cudaError_t launch_moe_down(const MoeDownParams& p, cudaStream_t stream);
cudaError_t launch_moe_combine(const MoeCombineParams& p, cudaStream_t stream);

} // namespace rkb200
