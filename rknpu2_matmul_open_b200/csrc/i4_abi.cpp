// i4_abi.cpp -- the exact int4 x int4 -> int32 operator of the original's include/rk_npu_matmul_i4.h on this library.
//
// The original packs A into int4 device tiles (directly or through a caller-supplied producer), runs int4 x int4 ->
// INT16 waves on its NPU and widens / sums the partials on the CPU (src/rk_npu_matmul_i4.cpp:8-71,
// src/rk_npu_i4_executor.cpp:54-126, src/rk_npu_i4_plan.cpp:126-242).  Here the int4 codes of A ride as int8 codes
// through the same tcgen05 per-tile kernel the W4A8 path uses (int4 weights unpacked into tensor memory, exact int32
// accumulation, the int32 epilogue), so there are no INT16 partials to saturate.  The producer protocol is kept: the
// callback is invoked serially on the calling thread, K wave by K wave and M panel by M panel, with a zeroed
// [padded_k / 32][rows][32] int4 tile (even element in the HIGH nibble) that the library then decodes.
// Validation, compatibility rules and return codes follow the original call for call.
#include "w4a8_host.h"
#include "../../include/rknpu_b200_quant.h"
#include <algorithm>
#include <chrono>
#include <climits>
#include <cstring>
#include <memory>
#include <new>
#include <vector>

using namespace rkb200;

namespace rkb200 {
int i4_memory(const rk_npu_i4_config& cfg, rk_npu_i4_memory_info& out);   // w4a8_abi.cpp: the original's accounting
}

struct rk_npu_i4i4i32_weights {
    rk_npu_iommu_domain* domain = nullptr;
    uint64_t ctx_id = 0;
    uint32_t domain_id = 0;
    rk_npu_i4_weight_config config{};
    uint8_t* packed = nullptr;
    float* ones = nullptr;          // channel scales the shared kernel reads; the int32 epilogue ignores them
    size_t packed_bytes = 0, scale_bytes = 0;
    int KB = 0, NG = 0;
};

struct rk_npu_i4_workspace {
    rk_npu_i4_config config{};
    rk_npu_iommu_domain* domain = nullptr;
    uint64_t ctx_id = 0;
    uint32_t domain_id = 0;
    std::atomic_flag busy = ATOMIC_FLAG_INIT;
    cudaStream_t stream = nullptr;
    int T = 0, KB = 0;
    uint8_t* codes = nullptr;
    float* scales = nullptr;
    Status* status = nullptr;
    int8_t* stage_in = nullptr;
    int32_t* stage_out = nullptr;
    size_t codes_bytes = 0, stage_in_bytes = 0, stage_out_bytes = 0;
    Status* host_status = nullptr;
    std::vector<int8_t> host_a;      // the decoded activations of a producer run
    std::vector<uint8_t> host_tile;  // one producer tile
};

namespace {
using Clock = std::chrono::steady_clock;
double since(Clock::time_point t) { return std::chrono::duration<double, std::micro>(Clock::now() - t).count(); }

bool weight_key_ok(const rk_npu_i4_weight_config& c)   // src/rk_npu_i4_plan.cpp:14-17
{
    return c.K > 0 && c.K <= INT32_MAX / 64 && c.N > 0 && c.N <= INT_MAX - 63 && c.k_tile >= 32 && c.k_tile <= 2048 && c.k_tile % 32 == 0;
}
bool runnable(int M, int N, int K) { return K <= 131072 && (int64_t)M * K <= INT32_MAX && (int64_t)M * N <= INT32_MAX; }

void weights_destroy(rk_npu_i4i4i32_weights* w)
{
    if (!w) return;
    if (w->domain) {
        cudaSetDevice(w->domain->ctx->device);
        if (w->packed) device_free(w->domain, w->packed, w->packed_bytes);
        if (w->ones) device_free(w->domain, w->ones, w->scale_bytes);
        domain_release(w->domain);
    }
    delete w;
}
void workspace_destroy(rk_npu_i4_workspace* ws)
{
    if (!ws) return;
    auto* d = ws->domain;
    if (d) cudaSetDevice(d->ctx->device);
    if (ws->stream) cudaStreamSynchronize(ws->stream);
    if (ws->codes) device_free(d, ws->codes, ws->codes_bytes);
    if (ws->scales) device_free(d, ws->scales, sizeof(float) * ws->config.M);
    if (ws->status) device_free(d, ws->status, sizeof(Status));
    if (ws->stage_in) device_free(d, ws->stage_in, ws->stage_in_bytes);
    if (ws->stage_out) device_free(d, ws->stage_out, ws->stage_out_bytes);
    if (ws->host_status) cudaFreeHost(ws->host_status);
    if (ws->stream) cudaStreamDestroy(ws->stream);
    if (d) domain_release(d);
    delete ws;
}

// One signed int4 code out of a packed byte: even elements sit in the high nibble
inline int8_t nibble(uint8_t byte, int j)
{
    const int v = (j & 1) ? (byte & 15) : (byte >> 4);
    return int8_t(v >= 8 ? v - 16 : v);
}

// The GPU part of a run: A (int8 codes, device) -> C (int32, device or staged)
int contract(rk_npu_i4_workspace* ws, const rk_npu_i4i4i32_weights* w, const int8_t* dA, int32_t* C, rk_npu_i4_timings& times)
{
    const auto& cfg = ws->config;
    cudaStream_t s = ws->stream;
    cudaPointerAttributes attr{};
    const bool c_dev = cudaPointerGetAttributes(&attr, C) == cudaSuccess && (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged);
    cudaGetLastError();
    int32_t* dC = c_dev ? C : ws->stage_out;
    W8QuantParams q{};
    q.A = dA;
    q.Xq = ws->codes;
    q.scales = ws->scales;
    q.M = cfg.M; q.K = cfg.K; q.Kp = ws->KB * KBLOCK; q.T = ws->T;
    q.kind = 2;                                   // int8 codes as given
    GemmParams g{};
    g.Wp = w->packed;
    g.Xq = ws->codes;
    g.sx = ws->scales;
    g.sw = w->ones;
    g.out = dC;
    g.status = ws->status;
    g.M = cfg.M; g.N = cfg.N; g.K = cfg.K;
    g.KB = ws->KB; g.NG = w->NG; g.T = ws->T;
    g.epi = EPI_I32;
    g.split = 1;
    g.pair = cfg.M > 128 ? 1 : 0;              // beyond 128 tokens: 128-token tiles, two per CTA pair of the persistent kernel
    g.timeout_ns = (unsigned long long)cfg.timeout_ms * 1000000ull;
    const auto t0 = Clock::now();
    const bool persistent = g.pair && gemm_tc_persist_supported(g);
    if (launch_w8_quantize(q, s) != cudaSuccess ||
        (persistent ? launch_gemm_tc_persist(g, s, false) : launch_gemm_tc(g, s, false)) != cudaSuccess) {
        cudaGetLastError();
        cudaStreamSynchronize(s);
        return RK_NPU_ERR_SUBMIT;
    }
    if (!c_dev) cudaMemcpyAsync(C, dC, ws->stage_out_bytes, cudaMemcpyDeviceToHost, s);
    cudaMemcpyAsync(ws->host_status, ws->status, sizeof(Status), cudaMemcpyDeviceToHost, s);
    if (cudaStreamSynchronize(s) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
    times.submit_us += since(t0);
    if (ws->host_status->device_error) {
        cudaMemsetAsync(&ws->status->device_error, 0, sizeof(int), s);
        cudaStreamSynchronize(s);
        return RK_NPU_ERR_SUBMIT;
    }
    return RK_NPU_OK;
}

struct Busy {
    explicit Busy(rk_npu_i4_workspace& ws) : flag(ws.busy), held(!flag.test_and_set(std::memory_order_acquire)) {}
    ~Busy() { if (held) flag.clear(std::memory_order_release); }
    std::atomic_flag& flag;
    bool held;
};
int bind_check(const rk_npu_i4_workspace* ws, const rk_npu_i4i4i32_weights* w)   // src/rk_npu_i4_plan.cpp:188-191
{
    if (w->ctx_id != ws->ctx_id || w->domain_id != ws->domain_id) return RK_NPU_ERR_DOMAIN;
    if (w->config.K != ws->config.K || w->config.N != ws->config.N || w->config.k_tile != ws->config.k_tile) return RK_NPU_ERR_PARAM;
    return RK_NPU_OK;
}
} // namespace

extern "C" int rk_npu_i4_memory_query(const rk_npu_i4_config* cfg, rk_npu_i4_memory_info* out)
{
    if (!cfg || !out) return RK_NPU_ERR_PARAM;
    return i4_memory(*cfg, *out);
}

extern "C" rk_npu_i4i4i32_weights* rk_npu_i4i4i32_weights_create(rk_npu_iommu_domain* domain, const rk_npu_i4_weight_config* cfg, const int8_t* B)
{
    if (!domain || !domain->ctx || !cfg || !B || !weight_key_ok(*cfg) || domain->ctx->world > 1 || !runnable(1, cfg->N, cfg->K)) return nullptr;
    uint64_t reference_bytes = 0;
    if (rk_npu_i4_weights_memory_query(cfg, &reference_bytes)) return nullptr;
    try {
        // an explicit tile above the universal 480 needs the proof that no INT16 partial of the original device could
        // saturate (src/rk_npu_i4_plan.cpp:95-99); the rule is part of the interface, so it is kept
        if (cfg->k_tile > 480) {
            WeightBound bound;
            if (bound_weights(cfg->K, cfg->N, B, cfg->k_tile, bound)) return nullptr;
        }
        rk_npu_ctx* ctx = domain->ctx;
        if (cudaSetDevice(ctx->device) != cudaSuccess) return nullptr;
        std::unique_ptr<rk_npu_i4i4i32_weights, void (*)(rk_npu_i4i4i32_weights*)> w(new rk_npu_i4i4i32_weights(), weights_destroy);
        w->config = *cfg;
        w->KB = (cfg->K + KBLOCK - 1) / KBLOCK;
        w->NG = align_up((cfg->N + GROUP - 1) / GROUP, 8) + 8;
        w->packed_bytes = size_t(w->NG) * (size_t(w->KB) * 4) * 512;
        w->scale_bytes = size_t(w->NG) * GROUP * sizeof(float);
        w->domain = domain;
        w->ctx_id = ctx->id;
        w->domain_id = domain->id;
        domain_retain(domain);
        if (device_alloc(domain, reinterpret_cast<void**>(&w->packed), w->packed_bytes) ||
            device_alloc(domain, reinterpret_cast<void**>(&w->ones), w->scale_bytes))
            return nullptr;
        int8_t* codes = nullptr;
        int* error = nullptr;
        const size_t code_bytes = size_t(cfg->K) * cfg->N;
        bool ok = cudaMalloc(reinterpret_cast<void**>(&codes), code_bytes) == cudaSuccess &&
                  cudaMalloc(reinterpret_cast<void**>(&error), sizeof(int)) == cudaSuccess;
        if (ok) {
            cudaStream_t s = ctx->stream;
            std::vector<float> ones(size_t(w->NG) * GROUP, 1.0f);
            ok = cudaMemcpyAsync(codes, B, code_bytes, cudaMemcpyHostToDevice, s) == cudaSuccess &&
                 cudaMemsetAsync(error, 0, sizeof(int), s) == cudaSuccess &&
                 cudaMemcpyAsync(w->ones, ones.data(), w->scale_bytes, cudaMemcpyHostToDevice, s) == cudaSuccess;
            if (ok) {
                PackParams p{codes, w->packed, error, cfg->K, cfg->N, w->KB * 4, w->NG};
                ok = launch_pack_weights(p, s) == cudaSuccess;
            }
            int host_error = 1;
            if (ok) ok = cudaMemcpyAsync(&host_error, error, sizeof(int), cudaMemcpyDeviceToHost, s) == cudaSuccess;
            ok = cudaStreamSynchronize(s) == cudaSuccess && ok && host_error == 0;   // a code outside [-8,7] fails creation
        }
        if (codes) cudaFree(codes);
        if (error) cudaFree(error);
        if (!ok) { cudaGetLastError(); return nullptr; }
        return w.release();
    } catch (...) { return nullptr; }
}
extern "C" void rk_npu_i4i4i32_weights_free(rk_npu_i4i4i32_weights* w) { weights_destroy(w); }

extern "C" rk_npu_i4_workspace* rk_npu_i4_workspace_create(rk_npu_iommu_domain* domain, const rk_npu_i4_config* cfg)
{
    if (!domain || !domain->ctx || !cfg || domain->ctx->world > 1) return nullptr;
    rk_npu_i4_memory_info info{};
    if (i4_memory(*cfg, info) || !runnable(cfg->M, cfg->N, cfg->K)) return nullptr;
    try {
        rk_npu_ctx* ctx = domain->ctx;
        if (cudaSetDevice(ctx->device) != cudaSuccess) return nullptr;
        std::unique_ptr<rk_npu_i4_workspace, void (*)(rk_npu_i4_workspace*)> ws(new rk_npu_i4_workspace(), workspace_destroy);
        ws->config = *cfg;
        ws->domain = domain;
        ws->ctx_id = ctx->id;
        ws->domain_id = domain->id;
        domain_retain(domain);
        ws->T = cfg->M > 128 ? 128 : align_up(cfg->M, 16);
        ws->KB = (cfg->K + KBLOCK - 1) / KBLOCK;
        ws->codes_bytes = size_t(align_up(cfg->M, cfg->M > 128 ? 256 : ws->T)) * size_t(ws->KB) * KBLOCK;
        ws->stage_in_bytes = size_t(cfg->M) * cfg->K;
        ws->stage_out_bytes = size_t(cfg->M) * cfg->N * sizeof(int32_t);
        bool ok = cudaStreamCreateWithFlags(&ws->stream, cudaStreamNonBlocking) == cudaSuccess &&
                  cudaMallocHost(reinterpret_cast<void**>(&ws->host_status), sizeof(Status)) == cudaSuccess;
        ok = ok && !device_alloc(domain, reinterpret_cast<void**>(&ws->codes), ws->codes_bytes) &&
             !device_alloc(domain, reinterpret_cast<void**>(&ws->scales), sizeof(float) * cfg->M) &&
             !device_alloc(domain, reinterpret_cast<void**>(&ws->status), sizeof(Status)) &&
             !device_alloc(domain, reinterpret_cast<void**>(&ws->stage_in), ws->stage_in_bytes) &&
             !device_alloc(domain, reinterpret_cast<void**>(&ws->stage_out), ws->stage_out_bytes);
        ok = ok && cudaMemsetAsync(ws->codes, 0, ws->codes_bytes, ws->stream) == cudaSuccess &&
             cudaMemsetAsync(ws->status, 0, sizeof(Status), ws->stream) == cudaSuccess && cudaStreamSynchronize(ws->stream) == cudaSuccess;
        if (!ok) { cudaGetLastError(); return nullptr; }
        return ws.release();
    } catch (...) { return nullptr; }
}
extern "C" void rk_npu_i4_workspace_free(rk_npu_i4_workspace* ws) { workspace_destroy(ws); }

extern "C" int rk_npu_i4_pack_a_tile(const rk_npu_i4_input_tile* t, const int8_t* A, int lda)   // src/rk_npu_i4_cpu.cpp:33-50
{
    if (!t || !A || !t->dst || t->m0 < 0 || t->rows <= 0 || t->rows > 128 || t->k0 < 0 || t->k <= 0 || t->padded_k < t->k ||
        t->padded_k > 2048 || t->padded_k % 32 || int64_t(t->k0) + t->k > lda || t->bytes < uint64_t(t->rows) * t->padded_k / 2)
        return RK_NPU_ERR_PARAM;
    std::memset(t->dst, 0, size_t(t->rows) * t->padded_k / 2);
    for (int kb = 0; kb < t->padded_k; kb += 32) {
        const int valid = std::min(32, std::max(0, t->k - kb));
        for (int m = 0; m < t->rows && valid; ++m) {
            const int8_t* src = A + (size_t(t->m0) + m) * lda + t->k0 + kb;
            uint8_t* dst = t->dst + (size_t(kb / 32) * t->rows + m) * 16;
            for (int j = 0; j < valid; ++j) {
                const int v = src[j];
                if (v < -8 || v > 7) return RK_NPU_ERR_PARAM;
                if (j & 1) dst[j / 2] |= uint8_t(v) & 15;
                else dst[j / 2] = uint8_t((uint8_t(v) & 15) << 4);
            }
        }
    }
    return RK_NPU_OK;
}

extern "C" int rk_npu_i4i4i32_run_with_producer(rk_npu_i4_workspace* ws, const rk_npu_i4i4i32_weights* w, rk_npu_i4_input_producer producer,
                                                void* user, int32_t* C, rk_npu_i4_timings* metrics)
{
    if (!ws || !w || !producer || !C) return RK_NPU_ERR_PARAM;
    Busy lock(*ws);
    if (!lock.held) return RK_NPU_ERR_BUSY;
    const auto start = Clock::now();
    rk_npu_i4_timings times{};
    if (const int rc = bind_check(ws, w)) return rc;
    const auto& cfg = ws->config;
    try {
        ws->host_a.assign(size_t(cfg.M) * cfg.K, 0);
        // K wave by K wave, M panel by M panel, serially on this thread (src/rk_npu_i4_plan.cpp:205-234)
        for (int k0 = 0; k0 < cfg.K; k0 += cfg.k_tile) {
            const int k = std::min(cfg.k_tile, cfg.K - k0), padded = align_up(k, 32);
            const auto t0 = Clock::now();
            for (int m0 = 0; m0 < cfg.M;) {
                const int rows = std::min(cfg.M - m0, cfg.m_tile);
                ws->host_tile.assign(size_t(rows) * padded / 2, 0);
                rk_npu_i4_input_tile tile{m0, rows, k0, k, padded, ws->host_tile.data(), uint64_t(rows) * padded / 2};
                int rc;
                try { rc = producer(user, &tile); } catch (...) { rc = RK_NPU_ERR_PARAM; }
                if (rc) return rc;
                for (int kb = 0; kb < padded; kb += 32)
                    for (int m = 0; m < rows; ++m) {
                        const uint8_t* src = ws->host_tile.data() + (size_t(kb / 32) * rows + m) * 16;
                        int8_t* dst = ws->host_a.data() + size_t(m0 + m) * cfg.K + k0 + kb;
                        for (int j = 0; j < std::min(32, k - kb); ++j) dst[j] = nibble(src[j / 2], j);
                    }
                m0 += rows;
            }
            times.pack_us += since(t0);
        }
    } catch (...) { return RK_NPU_ERR_NOMEM; }
    if (cudaSetDevice(ws->domain->ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    const auto t1 = Clock::now();
    if (cudaMemcpyAsync(ws->stage_in, ws->host_a.data(), ws->stage_in_bytes, cudaMemcpyHostToDevice, ws->stream) != cudaSuccess) {
        cudaGetLastError();
        return RK_NPU_ERR_SUBMIT;
    }
    times.sync_us += since(t1);
    const int rc = contract(ws, w, ws->stage_in, C, times);
    times.total_us = since(start);
    if (metrics) *metrics = times;
    return rc;
}

extern "C" int rk_npu_i4i4i32_run(rk_npu_i4_workspace* ws, const rk_npu_i4i4i32_weights* w, const int8_t* A, int32_t* C, rk_npu_i4_timings* metrics)
{
    if (!ws || !A) return RK_NPU_ERR_PARAM;
    if (!w || !C) return RK_NPU_ERR_PARAM;
    Busy lock(*ws);
    if (!lock.held) return RK_NPU_ERR_BUSY;
    const auto start = Clock::now();
    rk_npu_i4_timings times{};
    if (const int rc = bind_check(ws, w)) return rc;
    const auto& cfg = ws->config;
    if (cudaSetDevice(ws->domain->ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    // codes outside [-8,7] are an argument error, not masked (include/rk_npu_matmul_i4.h:73-74)
    const auto t0 = Clock::now();
    const size_t count = size_t(cfg.M) * cfg.K;
    int lowest = 0, highest = 0;
    for (size_t i = 0; i < count; ++i) { lowest = std::min<int>(lowest, A[i]); highest = std::max<int>(highest, A[i]); }
    if (lowest < -8 || highest > 7) return RK_NPU_ERR_PARAM;
    times.pack_us = since(t0);
    const auto t1 = Clock::now();
    if (cudaMemcpyAsync(ws->stage_in, A, ws->stage_in_bytes, cudaMemcpyHostToDevice, ws->stream) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
    times.sync_us = since(t1);
    const int rc = contract(ws, w, ws->stage_in, C, times);
    times.total_us = since(start);
    if (metrics) *metrics = times;
    return rc;
}
