// w4a8_device.h -- data layouts in HBM and the launch interface between the host
// side of the library (w4a8_abi.cpp) and its CUDA kernels.
//
// Packed weights  Wp[g][c][r][16 B]
//   g : group of 32 output channels, 0 .. NG-1 (NG = ceil(N/32) rounded up to 4)
//   c : chunk of 32 reduction elements, 0 .. KC-1 (KC = Kp/32, Kp = K rounded up to 128)
//   r : channel inside the group
//   The 16 bytes are four 32-bit words j = 0..3; byte b of word j holds code(k = 32c+4j+b)
//   in its LOW nibble and code(k = 32c+16+4j+b) in its HIGH nibble (two's complement int4).
//   (w << 4) & 0xF0F0F0F0 and w & 0xF0F0F0F0 therefore give two words of four int8 values
//   equal to 16 x code, already in the k order both tensor-core paths want.  Sums are
//   16 x the true sum and are shifted right by four (exactly) before dequantisation.
//   Padding (k >= K, n >= N) holds zero codes.  Replaces the reference's
//   B[N/64, K/32, 64, 32] panel layout (src/rk_npu_i4_cpu.cpp:53-70).
//
// Activation codes  Xq[mt][kc][t][16 B]
//   mt : token tile (T tokens per tile), kc : chunk of 16 reduction elements (Kp/16 of
//   them), t : token inside the tile; the 16 bytes are the int8 codes k = 16kc .. 16kc+15.
//   A k-block (128 k) of one token tile is contiguous, and a group of eight tokens x 16
//   bytes is the 8x16-byte core matrix both mma.sync and tcgen05 (no-swizzle, K-major)
//   consume.  Replaces the reference's MSD-split A[K/32, 2*rows, 32] int4 layout
//   (src/rk_npu_w4a8_quant.cpp:87-135): int8 MMA is native here so no split is needed.
#pragma once
#include <atomic>
#include <cuda_runtime.h>
#include <stdint.h>

namespace rkb200 {

// A function attribute such as the dynamic shared-memory opt-in belongs to one device.  A process may
// open contexts on several GPUs, so "already set" is remembered per CUDA ordinal (one bit each; ordinals
// beyond 63 simply set the attribute on every launch).
struct PerDeviceOnce {
    std::atomic<unsigned long long> done{0};
    bool needed(int& device) const
    {
        if (cudaGetDevice(&device) != cudaSuccess) { device = -1; return true; }
        return device < 0 || device >= 64 || !(done.load(std::memory_order_acquire) & (1ull << device));
    }
    void mark(int device)
    {
        if (device >= 0 && device < 64) done.fetch_or(1ull << device, std::memory_order_release);
    }
};

constexpr int KBLOCK = 128;        // reduction elements per pipeline stage
constexpr int GROUP = 32;          // output channels per weight group
constexpr int TILE_N = 128;        // output channels per CTA (4 groups)

enum Epilogue : int { EPI_F32 = 0, EPI_F16 = 1, EPI_I32 = 2, EPI_SWIGLU = 3 };

// Device-side status block of a workspace (all int32).
struct Status {
    int bad_input;      // set by the quantise kernel: 1 = NaN/Inf activation, 2 = non-finite middle
    int bad_accum;      // scratch for the cross-CTA "any row bad" reduction
    unsigned done;      // scratch counter (wraps to 0 by itself)
    int device_error;   // 1 = a bounded wait inside a kernel ran out
};

struct QuantParams {
    const void* A;          // [M,K] fp32 or binary16
    uint8_t* Xq;            // activation codes, layout above
    float* scales;          // [M]
    float* inverse;         // [M]
    uint32_t* rowmax_zero;  // [M] cleared before a SwiGLU epilogue maxes into it (nullable)
    uint32_t* rowmax;       // [M] non-null: scales come from these magnitude bits (no scan); cleared after use
    Status* status;
    int* host_flag;         // mapped host word mirroring status->bad_input (nullable)
    int M, K, Kp, T;
    int half;
};

// Column-sharded FFN (w4a8_shard.cu): this GPU's slice of the SwiGLU output to int8 codes with the
// scale of the whole row.
struct SliceQuantParams {
    const float* X;         // [M, cols] fp32, compact
    int8_t* codes;          // [M, cols] int8, compact
    const uint32_t* rowmax; // [M] magnitude bits of max |middle[m, :]| over the whole row (read only)
    int M, cols;
};
// Column-sharded FFN: already quantised activations into the Xq layout.
struct CodesInParams {
    const int8_t* codes;    // [parts][M][K / parts] int8 (parts = 1: plain [M, K])
    uint8_t* Xq;
    float* scales;          // [M]
    float* inverse;         // [M]
    uint32_t* rowmax;       // [M] magnitude bits the scales come from; cleared after use
    Status* status;
    int M, K, Kp, T;
    int parts;
};

struct GemmParams {
    const uint8_t* Wp;
    const uint8_t* Xq;
    const float* sx;        // per-token scales
    const float* sw;        // per-channel scales (padded to 32*NG)
    void* out;              // [M,N] fp32 / fp16 / int32, or middle [M,F] fp32
    uint32_t* rowmax;       // SwiGLU: per-row max |middle| bit pattern (nullable)
    Status* status;
    int M, N, K;
    int KB;                 // k-blocks (Kp / 128)
    int NG;                 // weight groups (padded)
    int T;                  // token tile of Xq
    int F;                  // SwiGLU: N/2, else 0
    int epi;
    int split;              // split-K factor == cluster size along y (1, 2, 4, 8)
    int pair;               // tcgen05 path: 1 = two-CTA tiles (cta_group::2), T must be 128
    int w8;                 // tcgen05 per-tile kernel: Wp holds int8 codes in the W8 layout (w8a8_kernels.cu), sums are not scaled by 16
    unsigned long long timeout_ns;
    unsigned long long* trace;  // optional cycle stamps of CTA (0,0): [role 0..2][k-block 0..63][2] (nullable)
    int* partials;              // streaming kernel: [2 x CTAs][T / 4][128][4] int32 partial sums (two slots per CTA, never cleared)
    unsigned int* counts;       // streaming kernel: [tiles] stages accumulated so far, zero between launches
};

// Single-kernel linear for small batches: quantisation fused in front of the GEMM.
struct FusedParams {
    const uint8_t* Wp;
    const void* A;              // [M,K] fp32 or binary16 activations
    const float* sw;
    void* out;
    uint32_t* rowmax_out;       // SwiGLU: per-row max |middle| bits, atomically maxed (nullable)
    uint32_t* rowmax_in;        // non-null: row scales come from these bits (no scan); cleared after use
    float* scales_out;          // [M] per-token scales, written by the first CTA
    uint8_t* codes_out;         // activation codes in the Xq layout with T = tokens per CTA (nullable)
    Status* status;
    int M, N, K;
    int KB, NG, F, epi;
    int split;                  // cluster size along y == split-K factor
    int stages;                 // k-blocks of smem per CTA (>= ceil(KB / split))
    int tiles_per_cta;          // 1, or 2: a CTA runs two adjacent column tiles one after the other
    int half;                   // activations are binary16
    unsigned long long timeout_ns;
    unsigned long long* trace;  // optional [CTA][8] global-timer stamps of the kernel's phases (nullable)
};

// Single-kernel linear for up to eight tokens (w4a8_decode.cu): every CTA owns whole output channels over
// all of K; the CTAs of a cluster share the quantisation and exchange int8 codes.
struct DecodeParams {
    const uint8_t* Wp;
    const void* A;              // [M,K] fp32 or binary16 activations
    const float* sw;
    void* out;
    uint32_t* rowmax_out;       // SwiGLU: per-row max |middle| bits, atomically maxed (nullable)
    uint32_t* rowmax_in;        // non-null: row scales come from these bits (no scan); cleared after use
    float* scales_out;          // [M] per-token scales, written by the first cluster
    uint8_t* codes_out;         // activation codes in the Xq layout with T = 8 (nullable)
    Status* status;
    int M, N, K;
    int KB, NG, F, epi;
    int half;                   // activations are binary16
    int cluster;                // CTAs that share the quantisation: 1, 2, 4 or 8
    int ring;                   // 32 KB weight stages per CTA
    int ctas;                   // grid size, a multiple of `cluster`
    int starve;                 // test hook: the first weight barrier of every CTA expects 16 bytes that never arrive
    unsigned long long timeout_ns;
    unsigned long long* trace;  // optional [CTA][8] stamps of the kernel's phases (nullable)
};

// Column partition of a group of GPUs: contiguous runs of 64-column blocks, the first `blocks % world` ranks
// one block more (the reference's split over its cores, src/rk_npu_i4_plan.cpp:37-43).
__host__ __device__ inline void shard_range(int N, int world, int rank, int& n0, int& n1)
{
    const int blocks = (N + 63) / 64;
    const int even = blocks / world, extra = blocks % world;
    const int first = rank * even + (rank < extra ? rank : extra);
    const int count = even + (rank < extra ? 1 : 0);
    n0 = first * 64 < N ? first * 64 : N;
    n1 = (first + count) * 64 < N ? (first + count) * 64 : N;
}
// Reassembly of all-gathered column shards: slot r of `gathered` holds rank r's compact [M][its columns] block.
struct AssembleParams {
    const uint8_t* gathered;
    uint8_t* out;           // [M][N] row-major
    size_t slot_bytes;      // distance between two ranks' blocks
    int M, N, world;
    int elem;               // bytes per element (1, 2 or 4)
    int two_range;          // 1: a rank holds the same slice of both halves of N (gate | up packing)
};
cudaError_t launch_assemble_columns(const AssembleParams& p, cudaStream_t stream);

// Several independent decode linears in one launch (same token count, activation type, cluster size).
constexpr int DEC_MAX_BATCH = 4;
struct DecodeBatch {
    DecodeParams p[DEC_MAX_BATCH];
    int first_cta[DEC_MAX_BATCH + 1];   // grid piece of linear i: [first_cta[i], first_cta[i + 1])
    int count;
};

struct PackParams {
    const int8_t* B;        // [K,N] codes on the device
    uint8_t* Wp;
    int* error;             // set to 1 when a code lies outside [-8,7]
    int K, N, KC, NG;
};

// ---- W8A8 operators (w8a8_kernels.cu): int8 weights W8p[g][kb][c][r][16 B], activations in the same Xq layout
struct W8PackParams {
    const int8_t* B;        // [K,N] int8 on the device
    uint8_t* Wp;
    int K, N, KB, NG;
};
struct W8QuantParams {
    const void* A;              // [M,K] fp32, binary16 or int8
    const float* static_scale;  // [M] caller's per-token scales on the device, or NULL: scan the rows
    uint8_t* Xq;
    float* scales;              // [M] the scales used (1 for int8 input)
    int M, K, Kp, T;
    int kind;                   // 0 fp32, 1 binary16, 2 int8 as given
};
cudaError_t launch_w8_pack_weights(const W8PackParams& p, cudaStream_t stream);
cudaError_t launch_w8_quantize(const W8QuantParams& p, cudaStream_t stream);

// Launch wrappers (w4a8_kernels.cu / w4a8_gemm_tc.cu). All return the launch error.
cudaError_t launch_pack_weights(const PackParams& p, cudaStream_t stream);
cudaError_t launch_quantize(const QuantParams& p, cudaStream_t stream, bool pdl);
cudaError_t launch_quantize_slice(const SliceQuantParams& p, cudaStream_t stream);
cudaError_t launch_codes_in(const CodesInParams& p, cudaStream_t stream);
// tokens_per_cta: 8, 16 or 32 (must divide p.T)
cudaError_t launch_gemm_mma(const GemmParams& p, int tokens_per_cta, cudaStream_t stream, bool pdl);
size_t gemm_mma_smem_bytes(int tokens_per_cta);
// Persistent, evenly balanced small-batch tcgen05 GEMM (w4a8_stream.cu): p.T in {16, 32} >= p.M, K <= 131072,
// p.partials (2 x sm_count slots of p.T x 128 int32) and p.counts ([tiles], zeroed once at allocation).
cudaError_t launch_gemm_stream(const GemmParams& p, int sm_count, cudaStream_t stream, bool pdl);
// Fused small-batch kernel: tokens_per_cta 8, 16 or 32 (>= p.M); p.stages <= FUSED_MAX_STAGES.
constexpr int FUSED_MAX_STAGES = 16;
cudaError_t launch_gemm_fused(const FusedParams& p, int tokens_per_cta, cudaStream_t stream, bool pdl);
size_t gemm_fused_smem_bytes(int tokens_per_cta, int stages, int tiles_per_cta);
// Decode kernel (up to eight tokens).  The plan helpers pick the cluster size, the ring depth and the grid.
constexpr int DEC_MAX_RING = 12;
bool gemm_decode_supported(int M, int K);
size_t gemm_decode_smem_bytes(int M, int KB, bool swiglu, int ring);
int gemm_decode_ring(int M, int KB, bool swiglu);
int gemm_decode_cluster(int M, int KB);
int gemm_decode_ctas(int items, int cluster, int cap);
int gemm_decode_resident_ctas(int cluster, size_t smem, int sm_count);
cudaError_t launch_gemm_decode(const DecodeParams& p, cudaStream_t stream, bool pdl);
cudaError_t launch_gemm_decode_batch(const DecodeBatch& b, cudaStream_t stream, bool pdl);
// tcgen05 path: p.T is the token tile of the code layout (multiple of 16, <= 256; 128 when p.pair)
cudaError_t launch_gemm_tc(const GemmParams& p, cudaStream_t stream, bool pdl);
bool gemm_tc_supported(const GemmParams& p);
// persistent two-CTA form (binary16 output or fused SwiGLU); p.pair and p.T == 128 required
cudaError_t launch_gemm_tc_persist(const GemmParams& p, cudaStream_t stream, bool pdl);
bool gemm_tc_persist_supported(const GemmParams& p);
// Bytes of GemmParams.partials the persistent kernel uses to park accumulator chunks (NULL: chunks are finished one by
// one before the accumulator is handed back).  No initial contents needed.
size_t gemm_tc_persist_park_bytes(int sm_count);

} // namespace rkb200
