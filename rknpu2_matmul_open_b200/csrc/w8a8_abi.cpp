// w8a8_abi.cpp -- the typed W8A8 operators of the original's second public header (include/rk_npu_quant_matmul.h:
// 296-421) on this library: raw int8 weight objects, workspaces made from a strategy, blocking runs.
//
// The original quantises A on the CPU into NPU tiles, runs int8 x int8 -> int32 waves on the NPU and reduces /
// dequantises on the CPU (src/rk_npu_quant_matmul.cpp:1758-1960, src/rk_npu_cpu_kernels.cpp).  Here a run is two
// launches on one stream: w8_quantize_kernel (scales and codes, or the caller's int8 codes re-laid) and the tcgen05
// per-tile kernel with int8 weights, whose epilogue dequantises.  Validation, compatibility rules and return codes
// follow the original call for call.
#include "w4a8_host.h"
#include "w4a8_tune.h"
#include "../../include/rknpu_b200_quant.h"
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <memory>
#include <new>

using namespace rkb200;

namespace {
constexpr int W8_N_TILE_MAX = 3072, W8_CHANNEL_TILE = 32;   // src/rk_npu_quant_matmul.cpp:50, src/rk_npu_internal.h:123
constexpr uint32_t W8_TIMEOUT_MS = 500;                      // the original's fixed plan timeout (src/rk_npu_quant_matmul.cpp:1709)

struct W8Weights {
    rk_npu_iommu_domain* domain = nullptr;
    uint64_t ctx_id = 0;
    uint32_t domain_id = 0;
    rk_npu_matmul_weight_config config{};
    uint8_t* packed = nullptr;
    float* scales = nullptr;      // padded to 32 * NG; ones for the int32 operator
    size_t packed_bytes = 0, scale_bytes = 0;
    int KB = 0, NG = 0;
};
}
struct rk_npu_i8i8i32_weights { W8Weights w; };
struct rk_npu_f16i8f16_weights { W8Weights w; };
struct rk_npu_f32i8f32_weights { W8Weights w; };

struct rk_npu_matmul_workspace {
    rk_npu_matmul_strategy strategy{};
    rk_npu_iommu_domain* domain = nullptr;
    uint64_t ctx_id = 0;
    uint32_t domain_id = 0;
    std::atomic_flag busy = ATOMIC_FLAG_INIT;
    cudaStream_t stream = nullptr;
    int T = 0, KB = 0;
    uint8_t* codes = nullptr;
    float* scales = nullptr;          // [M] used scales, then [M] the caller's static scales
    Status* status = nullptr;
    void* stage_in = nullptr;
    void* stage_out = nullptr;
    size_t codes_bytes = 0, scale_bytes = 0, stage_in_bytes = 0, stage_out_bytes = 0;
    Status* host_status = nullptr;    // pinned
    std::atomic<uint64_t> launches{0};
};

namespace {
bool finite_positive(float x) { return std::isfinite(x) && x > 0.0f; }
bool valid_scales(const float* s, int count)
{
    if (!s || count <= 0) return false;
    for (int i = 0; i < count; ++i)
        if (!finite_positive(s[i])) return false;
    return true;
}
bool valid_weight_config(const rk_npu_matmul_weight_config* c)   // src/rk_npu_quant_matmul.cpp:147-150
{
    return c && c->K > 0 && c->N > 0 && c->k_tile > 0 && c->k_tile <= c->K;
}
bool op_kind_ok(int kind) { return kind >= RK_NPU_MATMUL_I8I8I32 && kind <= RK_NPU_MATMUL_F32I8F32_STATIC; }
// src/rk_npu_quant_matmul.cpp:153-181.  Panel recipes change nothing here (they describe the original device's
// buffers) but are valid only where the original's device plan accepts them.
bool valid_strategy(const rk_npu_matmul_strategy* s)
{
    if (!s || !op_kind_ok(int(s->op_kind)) || s->M <= 0 || s->N <= 0 || s->K <= 0 || s->k_tile <= 0 || s->k_tile > s->K ||
        s->n_tile <= 0 || s->n_tile > W8_N_TILE_MAX || s->a_layout < RK_NPU_MATMUL_A_LAYOUT_NORMAL ||
        s->a_layout > RK_NPU_MATMUL_A_LAYOUT_PANEL16 || s->c_layout < RK_NPU_MATMUL_C_LAYOUT_NATIVE ||
        s->c_layout > RK_NPU_MATMUL_C_LAYOUT_PANEL16)
        return false;
    const uint32_t m = s->npu_core_mask;
    if (!(m == 1u || m == 2u || m == 4u || m == 3u || m == 7u) || s->cpu_core_mask == 0 || s->cpu_threads <= 0 ||
        s->cpu_threads != __builtin_popcountll(s->cpu_core_mask) || (s->cpu_core_mask & ~process_cpu_mask()))
        return false;
    if (!w8_panel_recipe_ok(s->M, s->N, s->k_tile, int(s->a_layout), int(s->c_layout))) return false;
    const int align_n = std::max(W8_CHANNEL_TILE, align_up(s->N, W8_CHANNEL_TILE));
    const int nt = std::min(align_n, align_up(s->n_tile, W8_CHANNEL_TILE));
    return (align_n + nt - 1) / nt >= __builtin_popcount(m);
}
// what the kernels need on top: K within the contraction kernel's range, sizes that fit
bool runnable_shape(int M, int N, int K) { return K <= 131072 && (int64_t)M * K <= INT32_MAX && (int64_t)M * N <= INT32_MAX; }
// Up to 128 tokens: one token tile per CTA of the per-tile kernel.  Beyond: 128-token tiles, two per CTA pair of the
// persistent kernel (the code buffer then covers whole pairs of tiles).
int token_tile(int M) { return M > 128 ? 128 : align_up(M, 16); }
int token_span(int M) { return M > 128 ? 256 : token_tile(M); }

struct Sizes {
    int T, KB, NG;
    size_t codes, scales, stage_in, stage_out, packed, wscales;
};
Sizes sizes_of(int M, int N, int K, int kind)
{
    Sizes z{};
    z.T = token_tile(M);
    z.KB = (K + KBLOCK - 1) / KBLOCK;
    z.NG = align_up((N + GROUP - 1) / GROUP, 8) + 8;   // zero groups behind the last tile, as for the int4 weights
    z.codes = size_t(align_up(M, token_span(M))) * size_t(z.KB) * KBLOCK;
    z.scales = sizeof(float) * 2 * size_t(M);
    const int in_elem = kind == RK_NPU_MATMUL_I8I8I32 ? 1 : (kind <= RK_NPU_MATMUL_F16I8F16_STATIC ? 2 : 4);
    const int out_elem = kind == RK_NPU_MATMUL_I8I8I32 ? 4 : (kind <= RK_NPU_MATMUL_F16I8F16_STATIC ? 2 : 4);
    z.stage_in = size_t(M) * K * in_elem;
    z.stage_out = size_t(M) * N * out_elem;
    z.packed = size_t(z.NG) * size_t(z.KB) * 4096;
    z.wscales = size_t(z.NG) * GROUP * sizeof(float);
    return z;
}

bool on_device(const void* p)
{
    cudaPointerAttributes a{};
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}

void weights_release(W8Weights& w)
{
    if (!w.domain) return;
    cudaSetDevice(w.domain->ctx->device);
    if (w.packed) device_free(w.domain, w.packed, w.packed_bytes);
    if (w.scales) device_free(w.domain, w.scales, w.scale_bytes);
    domain_release(w.domain);
    w = W8Weights{};
}

// B[K,N] int8 -> the W8 layout on the device; scales NULL: ones (the int32 operator's epilogue ignores them)
int weights_prepare(W8Weights& w, rk_npu_iommu_domain* domain, const rk_npu_matmul_weight_config* config, const int8_t* B,
                    const float* w_scale)
{
    if (!domain || !domain->ctx || !valid_weight_config(config) || !B) return RK_NPU_ERR_PARAM;
    rk_npu_ctx* ctx = domain->ctx;
    if (ctx->world > 1 || !runnable_shape(1, config->N, config->K)) return RK_NPU_ERR_PARAM;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    const Sizes z = sizes_of(1, config->N, config->K, RK_NPU_MATMUL_I8I8I32);
    w.config = *config;
    w.KB = z.KB;
    w.NG = z.NG;
    w.packed_bytes = z.packed;
    w.scale_bytes = z.wscales;
    w.domain = domain;
    w.ctx_id = ctx->id;
    w.domain_id = domain->id;
    domain_retain(domain);
    if (device_alloc(domain, reinterpret_cast<void**>(&w.packed), w.packed_bytes) ||
        device_alloc(domain, reinterpret_cast<void**>(&w.scales), w.scale_bytes)) {
        weights_release(w);
        return RK_NPU_ERR_NOMEM;
    }
    int8_t* dB = nullptr;
    const size_t b_bytes = size_t(config->K) * config->N;
    bool ok = cudaMalloc(reinterpret_cast<void**>(&dB), b_bytes) == cudaSuccess;
    if (ok) {
        cudaStream_t s = ctx->stream;
        std::unique_ptr<float[]> padded(new (std::nothrow) float[size_t(w.NG) * GROUP]);
        ok = padded != nullptr;
        if (ok) {
            for (int n = 0; n < w.NG * GROUP; ++n) padded[n] = n < config->N ? (w_scale ? w_scale[n] : 1.0f) : 0.0f;
            ok = cudaMemcpyAsync(dB, B, b_bytes, cudaMemcpyHostToDevice, s) == cudaSuccess &&
                 cudaMemcpyAsync(w.scales, padded.get(), w.scale_bytes, cudaMemcpyHostToDevice, s) == cudaSuccess;
        }
        if (ok) {
            const W8PackParams p{dB, w.packed, config->K, config->N, w.KB, w.NG};
            ok = launch_w8_pack_weights(p, s) == cudaSuccess;
        }
        ok = cudaStreamSynchronize(s) == cudaSuccess && ok;
    }
    if (dB) cudaFree(dB);
    if (!ok) { cudaGetLastError(); weights_release(w); return RK_NPU_ERR_NOMEM; }
    return RK_NPU_OK;
}

template <class Handle>
Handle* create_handle(rk_npu_iommu_domain* domain, const rk_npu_matmul_weight_config* config, const int8_t* B, const float* w_scale,
                      bool scaled)
{
    if (scaled && (!valid_weight_config(config) || !valid_scales(w_scale, config->N))) return nullptr;
    try {
        std::unique_ptr<Handle> h(new Handle());
        if (weights_prepare(h->w, domain, config, B, scaled ? w_scale : nullptr) != RK_NPU_OK) return nullptr;
        return h.release();
    } catch (...) { return nullptr; }
}
template <class Handle>
void free_handle(Handle* h)
{
    if (!h) return;
    weights_release(h->w);
    delete h;
}

void workspace_destroy(rk_npu_matmul_workspace* ws)
{
    if (!ws) return;
    auto* d = ws->domain;
    if (d) cudaSetDevice(d->ctx->device);
    if (ws->stream) cudaStreamSynchronize(ws->stream);
    if (ws->codes) device_free(d, ws->codes, ws->codes_bytes);
    if (ws->scales) device_free(d, ws->scales, ws->scale_bytes);
    if (ws->status) device_free(d, ws->status, sizeof(Status));
    if (ws->stage_in) device_free(d, ws->stage_in, ws->stage_in_bytes);
    if (ws->stage_out) device_free(d, ws->stage_out, ws->stage_out_bytes);
    if (ws->host_status) cudaFreeHost(ws->host_status);
    if (ws->stream) cudaStreamDestroy(ws->stream);
    if (d) domain_release(d);
    delete ws;
}

struct Lock {
    explicit Lock(rk_npu_matmul_workspace& ws) : flag(ws.busy), held(!flag.test_and_set(std::memory_order_acquire)) {}
    ~Lock() { if (held) flag.clear(std::memory_order_release); }
    std::atomic_flag& flag;
    bool held;
};

// One blocking run.  `kind_a` / `kind_b`: the operator kinds this entry point serves (dynamic or static is decided
// by the entry point, the workspace must have been made for exactly that one).
int run(rk_npu_matmul_workspace* ws, const W8Weights* w, int kind, const void* A, const float* a_scale, void* C)
{
    if (!ws || !w || !A || !C || int(ws->strategy.op_kind) != kind) return RK_NPU_ERR_PARAM;
    const auto& st = ws->strategy;
    const bool is_static = kind == RK_NPU_MATMUL_F16I8F16_STATIC || kind == RK_NPU_MATMUL_F32I8F32_STATIC;
    if (is_static && !valid_scales(a_scale, st.M)) return RK_NPU_ERR_PARAM;
    if (w->ctx_id != ws->ctx_id || w->domain_id != ws->domain_id) return RK_NPU_ERR_DOMAIN;
    if (w->config.K != st.K || w->config.N != st.N || w->config.k_tile != st.k_tile) return RK_NPU_ERR_PARAM;
    Lock lock(*ws);
    if (!lock.held) return RK_NPU_ERR_BUSY;
    if (cudaSetDevice(ws->domain->ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    cudaStream_t s = ws->stream;
    const void* dA = A;
    void* dC = C;
    const bool c_dev = on_device(C);
    if (!on_device(A)) {
        if (cudaMemcpyAsync(ws->stage_in, A, ws->stage_in_bytes, cudaMemcpyHostToDevice, s) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
        dA = ws->stage_in;
    }
    if (!c_dev) dC = ws->stage_out;
    float* static_dev = nullptr;
    if (is_static) {
        static_dev = ws->scales + st.M;
        if (cudaMemcpyAsync(static_dev, a_scale, sizeof(float) * st.M, cudaMemcpyHostToDevice, s) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
    }
    W8QuantParams q{};
    q.A = dA;
    q.static_scale = static_dev;
    q.Xq = ws->codes;
    q.scales = ws->scales;
    q.M = st.M; q.K = st.K; q.Kp = ws->KB * KBLOCK; q.T = ws->T;
    q.kind = kind == RK_NPU_MATMUL_I8I8I32 ? 2 : (kind <= RK_NPU_MATMUL_F16I8F16_STATIC ? 1 : 0);
    GemmParams g{};
    g.Wp = w->packed;
    g.Xq = ws->codes;
    g.sx = ws->scales;
    g.sw = w->scales;
    g.out = dC;
    g.status = ws->status;
    g.M = st.M; g.N = st.N; g.K = st.K;
    g.KB = ws->KB; g.NG = w->NG; g.T = ws->T;
    g.epi = kind == RK_NPU_MATMUL_I8I8I32 ? EPI_I32 : (kind <= RK_NPU_MATMUL_F16I8F16_STATIC ? EPI_F16 : EPI_F32);
    g.split = 1;
    g.w8 = 1;
    g.pair = st.M > 128 ? 1 : 0;
    g.timeout_ns = (unsigned long long)W8_TIMEOUT_MS * 1000000ull;
    const bool persistent = g.pair && gemm_tc_persist_supported(g);
    if (launch_w8_quantize(q, s) != cudaSuccess ||
        (persistent ? launch_gemm_tc_persist(g, s, false) : launch_gemm_tc(g, s, false)) != cudaSuccess) {
        cudaGetLastError();
        cudaStreamSynchronize(s);
        return RK_NPU_ERR_SUBMIT;
    }
    ws->launches.fetch_add(2, std::memory_order_relaxed);
    if (!c_dev) cudaMemcpyAsync(C, dC, ws->stage_out_bytes, cudaMemcpyDeviceToHost, s);
    cudaMemcpyAsync(ws->host_status, ws->status, sizeof(Status), cudaMemcpyDeviceToHost, s);
    if (cudaStreamSynchronize(s) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
    if (ws->host_status->device_error) {       // a bounded wait inside the kernel ran out: report, clear, stay usable
        cudaMemsetAsync(&ws->status->device_error, 0, sizeof(int), s);
        cudaStreamSynchronize(s);
        return RK_NPU_ERR_SUBMIT;
    }
    return RK_NPU_OK;
}

int weights_memory_query(const rk_npu_matmul_weight_config* config, bool with_scale, rk_npu_matmul_weight_requirements* out)
{
    if (!valid_weight_config(config) || !out || !runnable_shape(1, config->N, config->K)) return RK_NPU_ERR_PARAM;
    const Sizes z = sizes_of(1, config->N, config->K, RK_NPU_MATMUL_I8I8I32);
    std::memset(out, 0, sizeof(*out));
    out->packed_b_bytes = z.packed;
    out->scale_bytes = with_scale ? uint64_t(config->N) * sizeof(float) : 0;   // the logical payload, as the original counts it
    out->bytes = out->packed_b_bytes + out->scale_bytes;
    out->wave_count = uint32_t((config->K + config->k_tile - 1) / config->k_tile);
    out->buffer_count = 1;
    return RK_NPU_OK;
}
} // namespace

extern "C" int rk_npu_matmul_k_partition_query(int M, int K, int k_tile)
{
    if (M < 1 || K < 1 || k_tile < 1 || k_tile > K) return RK_NPU_ERR_PARAM;
    if (M <= 4) return RK_NPU_OK;
    if (K > k_tile && k_tile > 2048 && align_up(k_tile, W8_CHANNEL_TILE) % 1024) return RK_NPU_ERR_PARAM;
    for (int k0 = 0; k0 < K; k0 += k_tile) {
        const int k = align_up(std::min(k_tile, K - k0), W8_CHANNEL_TILE);
        if (k > 3072 && k < 4096) return RK_NPU_ERR_PARAM;
    }
    return RK_NPU_OK;
}

extern "C" int rk_npu_matmul_workspace_memory_query(const rk_npu_matmul_strategy* strategy, rk_npu_matmul_workspace_requirements* out)
{
    if (!strategy || !out || !valid_strategy(strategy) || !runnable_shape(strategy->M, strategy->N, strategy->K)) return RK_NPU_ERR_PARAM;
    const Sizes z = sizes_of(strategy->M, strategy->N, strategy->K, int(strategy->op_kind));
    std::memset(out, 0, sizeof(*out));
    out->input_bytes = z.codes + z.stage_in;
    out->output_bytes = z.stage_out;
    out->control_bytes = z.scales + sizeof(Status);
    out->bytes = out->input_bytes + out->output_bytes + out->control_bytes;
    out->wave_count = uint32_t((strategy->K + strategy->k_tile - 1) / strategy->k_tile);
    out->buffer_count = 5;
    return RK_NPU_OK;
}
extern "C" int rk_npu_i8i8i32_weights_memory_query(const rk_npu_matmul_weight_config* c, rk_npu_matmul_weight_requirements* out) { return weights_memory_query(c, false, out); }
extern "C" int rk_npu_f16i8f16_weights_memory_query(const rk_npu_matmul_weight_config* c, rk_npu_matmul_weight_requirements* out) { return weights_memory_query(c, true, out); }
extern "C" int rk_npu_f32i8f32_weights_memory_query(const rk_npu_matmul_weight_config* c, rk_npu_matmul_weight_requirements* out) { return weights_memory_query(c, true, out); }

extern "C" rk_npu_matmul_workspace* rk_npu_matmul_workspace_create(rk_npu_iommu_domain* domain, const rk_npu_matmul_strategy* strategy)
{
    if (!domain || !domain->ctx || !strategy || !valid_strategy(strategy) || !runnable_shape(strategy->M, strategy->N, strategy->K) ||
        domain->ctx->world > 1)
        return nullptr;
    rk_npu_ctx* ctx = domain->ctx;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return nullptr;
    rk_npu_matmul_workspace* ws = new (std::nothrow) rk_npu_matmul_workspace();
    if (!ws) return nullptr;
    const Sizes z = sizes_of(strategy->M, strategy->N, strategy->K, int(strategy->op_kind));
    ws->strategy = *strategy;
    ws->domain = domain;
    ws->ctx_id = ctx->id;
    ws->domain_id = domain->id;
    ws->T = z.T;
    ws->KB = z.KB;
    ws->codes_bytes = z.codes;
    ws->scale_bytes = z.scales;
    ws->stage_in_bytes = z.stage_in;
    ws->stage_out_bytes = z.stage_out;
    domain_retain(domain);
    bool ok = cudaStreamCreateWithFlags(&ws->stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaMallocHost(reinterpret_cast<void**>(&ws->host_status), sizeof(Status)) == cudaSuccess;
    ok = ok && !device_alloc(domain, reinterpret_cast<void**>(&ws->codes), ws->codes_bytes) &&
         !device_alloc(domain, reinterpret_cast<void**>(&ws->scales), ws->scale_bytes) &&
         !device_alloc(domain, reinterpret_cast<void**>(&ws->status), sizeof(Status)) &&
         !device_alloc(domain, &ws->stage_in, ws->stage_in_bytes) && !device_alloc(domain, &ws->stage_out, ws->stage_out_bytes);
    // codes of the tokens that pad the last tile stay zero for the life of the workspace
    ok = ok && cudaMemsetAsync(ws->codes, 0, ws->codes_bytes, ws->stream) == cudaSuccess &&
         cudaMemsetAsync(ws->status, 0, sizeof(Status), ws->stream) == cudaSuccess && cudaStreamSynchronize(ws->stream) == cudaSuccess;
    if (!ok) { cudaGetLastError(); workspace_destroy(ws); return nullptr; }
    return ws;
}
extern "C" void rk_npu_matmul_workspace_free(rk_npu_matmul_workspace* ws) { workspace_destroy(ws); }
extern "C" uint64_t rk_npu_b200_matmul_launch_count(const rk_npu_matmul_workspace* ws) { return ws ? ws->launches.load() : 0; }

extern "C" rk_npu_i8i8i32_weights* rk_npu_i8i8i32_weights_create(rk_npu_iommu_domain* d, const rk_npu_matmul_weight_config* c, const int8_t* B)
{
    return create_handle<rk_npu_i8i8i32_weights>(d, c, B, nullptr, false);
}
extern "C" void rk_npu_i8i8i32_weights_free(rk_npu_i8i8i32_weights* w) { free_handle(w); }
extern "C" int rk_npu_i8i8i32_run(rk_npu_matmul_workspace* ws, const rk_npu_i8i8i32_weights* w, const int8_t* A, int32_t* C)
{
    return run(ws, w ? &w->w : nullptr, RK_NPU_MATMUL_I8I8I32, A, nullptr, C);
}

extern "C" rk_npu_f16i8f16_weights* rk_npu_f16i8f16_weights_create(rk_npu_iommu_domain* d, const rk_npu_matmul_weight_config* c,
                                                                   const int8_t* B, const float* w_scale)
{
    return create_handle<rk_npu_f16i8f16_weights>(d, c, B, w_scale, true);
}
extern "C" void rk_npu_f16i8f16_weights_free(rk_npu_f16i8f16_weights* w) { free_handle(w); }
extern "C" int rk_npu_f16i8f16_run_dynamic(rk_npu_matmul_workspace* ws, const rk_npu_f16i8f16_weights* w, const uint16_t* A, uint16_t* C)
{
    return run(ws, w ? &w->w : nullptr, RK_NPU_MATMUL_F16I8F16_DYNAMIC, A, nullptr, C);
}
extern "C" int rk_npu_f16i8f16_run_static(rk_npu_matmul_workspace* ws, const rk_npu_f16i8f16_weights* w, const uint16_t* A,
                                          const float* a_scale, uint16_t* C)
{
    return run(ws, w ? &w->w : nullptr, RK_NPU_MATMUL_F16I8F16_STATIC, A, a_scale, C);
}

extern "C" rk_npu_f32i8f32_weights* rk_npu_f32i8f32_weights_create(rk_npu_iommu_domain* d, const rk_npu_matmul_weight_config* c,
                                                                   const int8_t* B, const float* w_scale)
{
    return create_handle<rk_npu_f32i8f32_weights>(d, c, B, w_scale, true);
}
extern "C" void rk_npu_f32i8f32_weights_free(rk_npu_f32i8f32_weights* w) { free_handle(w); }
extern "C" int rk_npu_f32i8f32_run_dynamic(rk_npu_matmul_workspace* ws, const rk_npu_f32i8f32_weights* w, const float* A, float* C)
{
    return run(ws, w ? &w->w : nullptr, RK_NPU_MATMUL_F32I8F32_DYNAMIC, A, nullptr, C);
}
extern "C" int rk_npu_f32i8f32_run_static(rk_npu_matmul_workspace* ws, const rk_npu_f32i8f32_weights* w, const float* A,
                                          const float* a_scale, float* C)
{
    return run(ws, w ? &w->w : nullptr, RK_NPU_MATMUL_F32I8F32_STATIC, A, a_scale, C);
}

// The original's *_weights_create_compress keep the same B in a lossless compressed form for its hardware decompressor
// (include/rk_npu_quant_matmul.h:321-330): same run and free functions, same results.  Here the codes are stored as they
// are -- HBM is not the scarce resource the original board's DRAM bandwidth is -- so these are the plain constructors.
extern "C" rk_npu_i8i8i32_weights* rk_npu_i8i8i32_weights_create_compress(rk_npu_iommu_domain* d, const rk_npu_matmul_weight_config* c, const int8_t* B)
{
    return rk_npu_i8i8i32_weights_create(d, c, B);
}
extern "C" rk_npu_f16i8f16_weights* rk_npu_f16i8f16_weights_create_compress(rk_npu_iommu_domain* d, const rk_npu_matmul_weight_config* c,
                                                                            const int8_t* B, const float* w_scale)
{
    return rk_npu_f16i8f16_weights_create(d, c, B, w_scale);
}
extern "C" rk_npu_f32i8f32_weights* rk_npu_f32i8f32_weights_create_compress(rk_npu_iommu_domain* d, const rk_npu_matmul_weight_config* c,
                                                                            const int8_t* B, const float* w_scale)
{
    return rk_npu_f32i8f32_weights_create(d, c, B, w_scale);
}
// include/rk_npu_quant_matmul.h:395-399: raw weights and NULL return zero
extern "C" uint64_t rk_npu_f32i8f32_weights_compressed_layout_generation(const rk_npu_f32i8f32_weights*) { return 0; }
