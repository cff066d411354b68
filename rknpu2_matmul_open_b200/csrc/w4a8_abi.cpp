// w4a8_abi.cpp -- the C ABI of the W4A8 path: context and domains, geometry
// validation and memory accounting, weight preparation, workspaces and the run entry
// points.  Host C++ only; every tensor operation is a CUDA kernel (w4a8_kernels.cu,
// w4a8_gemm_tc.cu).  There is no CPU compute path: without a GPU rk_npu_open fails.
//
// Behaviour mirrors the reference operator front-end src/rk_npu_w4a8.cpp (validation
// order :83-94, BUSY guard :70-81, run :98-159, accounting :169-207, FFN :354-380) and
// the backend geometry rules src/rk_npu_i4_plan.cpp:14-87.
#include "../../include/rknpu_b200_quant.h"
#include "w4a8_tune.h"
#include <algorithm>
#include <cerrno>
#include <chrono>
#include <climits>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <memory>
#include <new>
#include <vector>

using namespace rkb200;

namespace {
using Clock = std::chrono::steady_clock;
double elapsed_us(Clock::time_point t) { return std::chrono::duration<double, std::micro>(Clock::now() - t).count(); }

bool env_flag(const char* name, bool fallback)
{
    const char* v = std::getenv(name);
    if (!v || !*v) return fallback;
    return !(v[0] == '0' && v[1] == 0);
}

// ------------------------------------------------------------------ geometry rules
constexpr int K_TILE_MAX = 2048;
constexpr int N_TILE_MAX = 8128;
constexpr int COMMAND_WORDS = 112;   // register words per task of the original device
constexpr int TASK_BYTES = 40;
constexpr int REDUCE_COMMAND_WORDS = 68;

bool valid_shape(int K, int N) { return K > 0 && K <= INT32_MAX / 1024 && N > 0; }

bool weight_key_valid(int K, int N, int k_tile)
{
    const bool shape = K > 0 && K <= INT32_MAX / 64 && N > 0 && N <= INT_MAX - 63;
    return shape && k_tile >= 32 && k_tile <= K_TILE_MAX && k_tile % 32 == 0;
}

int weight_bytes_query(int K, int N, int k_tile, uint64_t& bytes)
{
    if (!weight_key_valid(K, N, k_tile)) return RK_NPU_ERR_PARAM;
    bytes = uint64_t(align_up(K, 32)) * align_up(N, 64) / 2;   // two codes per byte, K padded to 32, N to 64
    return bytes > UINT32_MAX ? RK_NPU_ERR_NOMEM : RK_NPU_OK;
}

// The problem as the original device saw it (two int4 rows per token), kept for one purpose: the memory
// queries and the constructors must accept exactly the geometries the original accepts and report the
// numbers it reports (include/rk_npu_w4a8.h:35-75; the arithmetic is that of src/rk_npu_i4_plan.cpp:14-87,
// src/rk_npu_w4a8_chain.cpp:49-58 and src/rk_npu_w4a8_npu_reduce.cpp:90-137).  Nothing here schedules work.
class DeviceGeometry {
public:
    int rows = 0, N = 0, K = 0;             // rows = 2 x tokens
    int row_tile = 0, k_tile = 0, n_tile = 0;
    uint32_t cores = 0, timeout_ms = 0;
    int pipeline = 0, threads = 0;
    bool panel8 = false;

    int core_count() const { return __builtin_popcount(cores); }
    int column_blocks() const { return align_up(N, 64) / 64; }
    // 64-column blocks of core `i`: an even share, the first `blocks % cores` cores take one more
    int core_columns(int i) const { return (column_blocks() / core_count() + (i < column_blocks() % core_count() ? 1 : 0)) * 64; }
    uint32_t waves() const { return uint32_t((K + k_tile - 1) / k_tile); }
    int wave_depth() const { return align_up(std::min(K, k_tile), 32); }

    // rows of the next activation panel when `remaining` rows are left: panel8 panels are whole groups of eight
    int panel_rows(int remaining) const
    {
        const int take = std::min(remaining, row_tile);
        return (panel8 && take >= 8) ? take - take % 8 : take;
    }
    // 32 KB buffer banks one panel8 activation panel occupies: 64 bytes per (group of eight rows, entry), where
    // a full 128-deep slice has 8 entries and a tail of up to 32 / 64 / 128 has 2 / 4 / 8
    static int panel_banks(int rows_in_panel, int depth)
    {
        const int tail = depth % 128;
        const int entries = depth / 128 * 8 + (tail == 0 ? 0 : tail <= 32 ? 2 : tail <= 64 ? 4 : 8);
        const long long bytes = (long long)(rows_in_panel / 8) * entries * 64;
        return int((bytes + 32767) / 32768);
    }

    bool valid() const
    {
        if (!weight_key_valid(K, N, k_tile) || rows < 1 || row_tile < 1) return false;
        if (panel8) {
            const bool tile_ok = row_tile >= 8 && row_tile <= 512 && row_tile % 8 == 0 && rows % 2 == 0;
            if (!tile_ok || panel_banks(panel_rows(rows), wave_depth()) > 8) return false;
        } else if (row_tile > 128) return false;
        const bool columns_ok = n_tile >= 64 && n_tile <= N_TILE_MAX && n_tile % 64 == 0;
        const bool cores_ok = (cores == 1 || cores == 2 || cores == 4 || cores == 3 || cores == 7) && column_blocks() >= core_count();
        const bool host_ok = timeout_ms > 0 && (pipeline == 0 || pipeline == 1) && threads >= 1 && threads <= 4;
        return columns_ok && cores_ok && host_ok;
    }

    // activation panels per column tile
    uint64_t panels() const
    {
        if (!panel8) return (uint64_t(rows) + row_tile - 1) / row_tile;
        const int rest = rows % row_tile;
        return uint64_t(rows) / row_tile + (rest >= 8 ? 1 : 0) + (rest % 8 ? 1 : 0);
    }
    uint64_t column_tiles() const
    {
        uint64_t tiles = 0;
        for (int i = 0; i < core_count(); ++i) tiles += uint64_t((core_columns(i) + n_tile - 1) / n_tile);
        return tiles;
    }

    int memory(rk_npu_i4_memory_info& out) const
    {
        if (!valid()) return RK_NPU_ERR_PARAM;
        out = {};
        if (const int rc = weight_bytes_query(K, N, k_tile, out.packed_weight_bytes)) return rc;
        out.wave_count = waves();
        const uint64_t buffers = std::min(out.wave_count, 2u);             // double-buffered across waves
        const uint64_t input_one = uint64_t(rows) * wave_depth() / 2, partial_one = uint64_t(rows) * align_up(N, 64) * 2;
        const uint64_t tasks = column_tiles() * panels();
        if (tasks > uint64_t(INT_MAX / COMMAND_WORDS) || input_one > UINT32_MAX || partial_one > UINT32_MAX) return RK_NPU_ERR_NOMEM;
        out.input_bytes = buffers * input_one;
        out.partial_bytes = buffers * partial_one;
        out.tasks_per_wave = uint32_t(tasks);
        out.control_bytes = uint64_t(out.wave_count) * tasks * (COMMAND_WORDS * 8 + TASK_BYTES);
        return RK_NPU_OK;
    }
    // all waves resident at once: the whole padded K of the activations, one partial buffer per wave
    int memory_chained(rk_npu_i4_memory_info& out) const
    {
        if (const int rc = memory(out)) return rc;
        const uint64_t all_tasks = uint64_t(out.tasks_per_wave) * out.wave_count;
        const uint64_t input = uint64_t(rows) * align_up(K, 32) / 2, per_wave = uint64_t(rows) * align_up(N, 64) * 2;
        if (all_tasks > uint64_t(INT_MAX / COMMAND_WORDS) || input > UINT32_MAX || per_wave > UINT32_MAX / out.wave_count) return RK_NPU_ERR_NOMEM;
        out.input_bytes = input;
        out.partial_bytes = per_wave * out.wave_count;
        return RK_NPU_OK;
    }
    // device-side reduction of retained partials: every (panel, column tile) is cut into parts of at most
    // `limit` 16-value rows, the limit halving until (waves + 1) input rows of 64 bytes fit eleven banks
    int memory_device_reduce(rk_npu_w4a8_memory_info_ex& info) const
    {
        const uint64_t wave_total = waves();
        if (wave_total > 31) return RK_NPU_ERR_PARAM;
        const uint64_t retained = uint64_t(rows) * align_up(N, 64) * 2 * wave_total;
        if (retained > UINT32_MAX) return RK_NPU_ERR_NOMEM;
        int limit = 512;
        while (uint64_t(limit) * 64 * (wave_total + 1) > 11ull * 32768) limit /= 2;
        uint64_t parts = 0, output = 0, largest = 256 * 1024;
        int column = 0;
        for (int core = 0; core < core_count(); ++core) {
            const int core_end = column + core_columns(core);
            for (; column < core_end;) {
                const int width = std::min(n_tile, core_end - column);
                for (int row = 0; row < rows;) {
                    const int height = panel_rows(rows - row);
                    if (height % 2 || row % 2 || width % 64) return RK_NPU_ERR_PARAM;
                    const int storage = height * width / 16;
                    if (storage > 4096) return RK_NPU_ERR_PARAM;
                    largest = std::max<uint64_t>(largest, uint64_t(height) * width * 2 * wave_total);
                    for (int done = 0; done < storage; done += limit, ++parts)
                        output += uint64_t(align_up(std::min(limit, storage - done), 4)) * 64;
                    row += height;
                }
                column += width;
            }
        }
        if (parts < uint64_t(core_count())) return RK_NPU_ERR_PARAM;
        if (parts > uint64_t(INT_MAX / REDUCE_COMMAND_WORDS)) return RK_NPU_ERR_NOMEM;
        info.base.backend.partial_bytes = retained + largest;
        info.reduction_output_bytes = output + 256 * 1024;
        info.reduction_weight_bytes = wave_total * 512;
        info.reduction_control_bytes = parts * (REDUCE_COMMAND_WORDS * 8 + TASK_BYTES);
        const bool fits = info.base.backend.partial_bytes <= UINT32_MAX && info.reduction_output_bytes <= UINT32_MAX &&
                          info.reduction_control_bytes <= UINT32_MAX;
        return fits ? RK_NPU_OK : RK_NPU_ERR_NOMEM;
    }
};

int options_decode(const rk_npu_w4a8_options* opt, int M, bool& panel8, bool& npu)
{
    panel8 = false;
    npu = false;
    if (!opt) return RK_NPU_OK;
    if (opt->struct_size != sizeof(*opt) ||
        (opt->input_layout != RK_NPU_W4A8_INPUT_NATIVE && opt->input_layout != RK_NPU_W4A8_INPUT_PANEL8) ||
        (opt->reduce_backend != RK_NPU_W4A8_REDUCE_CPU && opt->reduce_backend != RK_NPU_W4A8_REDUCE_NPU))
        return RK_NPU_ERR_PARAM;
    panel8 = opt->input_layout == RK_NPU_W4A8_INPUT_PANEL8;
    npu = opt->reduce_backend == RK_NPU_W4A8_REDUCE_NPU && M > 16;
    return RK_NPU_OK;
}

int geometry_from(const rk_npu_w4a8_config& cfg, bool panel8, DeviceGeometry& out)
{
    const bool tokens_ok = cfg.M >= 1 && cfg.M <= INT_MAX / 2 && cfg.m_tile >= 1 && cfg.m_tile <= (panel8 ? 256 : 64);
    const bool pipeline_ok = cfg.pipeline >= RK_NPU_W4A8_SERIAL && cfg.pipeline <= RK_NPU_W4A8_CHAIN;
    if (!valid_shape(cfg.K, cfg.N) || !tokens_ok || !pipeline_ok) return RK_NPU_ERR_PARAM;
    out = DeviceGeometry{};
    out.rows = cfg.M * 2;
    out.row_tile = cfg.m_tile * 2;
    out.N = cfg.N;
    out.K = cfg.K;
    out.k_tile = cfg.k_tile;
    out.n_tile = cfg.n_tile;
    out.cores = cfg.npu_core_mask;
    out.timeout_ms = cfg.timeout_ms;
    out.pipeline = cfg.pipeline == RK_NPU_W4A8_CHAIN ? 0 : cfg.pipeline;   // the chain mode submits like the serial one
    out.threads = cfg.cpu_threads;
    out.panel8 = panel8;
    return RK_NPU_OK;
}

} // namespace
// The original's accounting for the exact int4 operator (rows = tokens; src/rk_npu_i4_plan.cpp:19-87), for i4_abi.cpp.
namespace rkb200 {
int i4_memory(const rk_npu_i4_config& cfg, rk_npu_i4_memory_info& out)
{
    DeviceGeometry g;
    g.rows = cfg.M;
    g.row_tile = cfg.m_tile;
    g.N = cfg.N;
    g.K = cfg.K;
    g.k_tile = cfg.k_tile;
    g.n_tile = cfg.n_tile;
    g.cores = cfg.npu_core_mask;
    g.timeout_ms = cfg.timeout_ms;
    g.pipeline = cfg.pipeline;
    g.threads = cfg.cpu_threads;
    g.panel8 = false;
    return g.memory(out);
}
}
namespace {
// ------------------------------------------------------------------ locking
class WorkspaceLock {
public:
    explicit WorkspaceLock(rk_npu_w4a8_workspace& ws) : flag_(ws.busy), held_(!flag_.test_and_set(std::memory_order_acquire)) {}
    ~WorkspaceLock() { if (held_) flag_.clear(std::memory_order_release); }
    explicit operator bool() const { return held_; }
    WorkspaceLock(const WorkspaceLock&) = delete;
    WorkspaceLock& operator=(const WorkspaceLock&) = delete;
private:
    std::atomic_flag& flag_;
    bool held_;
};

int validate(const rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w, const void* A, const void* C, bool swiglu)
{
    if (!ws || !w || !A || !C || A == C || (swiglu && (ws->npu_reduce || ws->config.N % 64))) return RK_NPU_ERR_PARAM;
    if (swiglu && ws->domain->ctx->world > 1 && !ws->shard.two_range) return RK_NPU_ERR_PARAM;   // gate/up pairs must share a GPU
    if (w->ctx_id != ws->ctx_id || w->domain_id != ws->domain_id) return RK_NPU_ERR_DOMAIN;
    const auto& wc = w->info.config;
    if (wc.K != ws->config.K || wc.N != ws->config.N || wc.k_tile != ws->config.k_tile) return RK_NPU_ERR_PARAM;
    return RK_NPU_OK;
}

bool on_device(const void* p)
{
    cudaPointerAttributes a{};
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return false; }
    return a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged;
}
// Page-locked host memory that the GPU can address (cudaHostAlloc / cudaHostRegister): its device alias, else NULL.
void* mapped_alias(const void* p)
{
    cudaPointerAttributes a{};
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return a.type == cudaMemoryTypeHost ? a.devicePointer : nullptr;
}
// One query per tensor of a blocking call: is it device memory, and if it is page-locked host memory, its device alias.
struct Placement { bool device = false; void* alias = nullptr; };
Placement placement(const void* p)
{
    cudaPointerAttributes a{};
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) { cudaGetLastError(); return {}; }
    return {a.type == cudaMemoryTypeDevice || a.type == cudaMemoryTypeManaged, a.type == cudaMemoryTypeHost ? a.devicePointer : nullptr};
}

// ------------------------------------------------------------------ kernel sequencing
int pick_split_auto(const rk_npu_w4a8_workspace& ws, int tiles, int token_chunks)
{
    const int sms = ws.domain->ctx->sm_count;
    // The smallest split that gives every SM a CTA: more only adds reduction traffic and shortens
    // each CTA's stream (measured on 4096x11008: split 2 -> 13 us, split 4 -> 17 us).
    int split = 1;
    while (split < 8 && (long long)tiles * token_chunks * split < sms && ws.KB / (split * 2) >= 2) split *= 2;
    return split;
}
int pick_split(const rk_npu_w4a8_workspace& ws, int tiles, int token_chunks)
{
    return ws.split_override ? ws.split_override : pick_split_auto(ws, tiles, token_chunks);
}

struct Call {
    rk_npu_w4a8_workspace* ws;
    const rk_npu_w4a8_weights* w;
    const void* dA;        // device activations
    void* dOut;            // device output
    bool half;
    int epi;
    uint32_t* rowmax_out;  // SwiGLU row maxima to collect (device) or nullptr
    uint32_t* rowmax_in;   // scales come from these instead of a scan (cleared after use)
    cudaStream_t stream;
    cudaEvent_t* events;   // nullptr or three events: start, after quantise, after GEMM
    bool keep_codes = false;   // fused kernel: also store the activation codes (diagnostic entry only)
    const int8_t* codes_in = nullptr;   // activations arrive as int8 codes [parts][M][K/parts]; scales from rowmax_in
    int parts = 1;
    Status* status = nullptr;   // single-kernel families: where the launch reports (default: the workspace's device block)
};

// Split-K factor (= cluster size) of the single-kernel path: the largest split whose CTAs
// are all resident at once (each holds its whole weight slice in shared memory).
int fused_split(const rk_npu_w4a8_workspace& ws, int tiles)
{
    if (ws.split_override) return ws.split_override;
    const int sms = ws.domain->ctx->sm_count;
    const size_t smem_per_sm = 220 * 1024;
    int best = 0;
    for (int split = 1; split <= 8; ++split) {
        const int stages = (ws.KB + split - 1) / split;
        if (stages > FUSED_MAX_STAGES) continue;
        if (!best) best = split;
        const size_t bytes = gemm_fused_smem_bytes(ws.TC, stages, 1) + 1024;
        const long long slots = (long long)sms * std::min<long long>(8, (long long)(smem_per_sm / bytes));
        if ((long long)tiles * split <= slots) best = split;
    }
    if (!best) return 8;
    // ... but no finer than about eight k-blocks (1024 reduction elements) per CTA: below that the CTAs of a launch
    // outnumber the SMs by more than their short slices win back (decode ring at 8 tokens, K = 4096: split 4 against 8,
    // 1791 against 1709 GB/s; K = 11008 stays at 8, where 6 and 7 measured slower)
    const int want = std::max(1, std::min(8, (ws.KB + 4) / 8));
    if (want < best && (ws.KB + want - 1) / want <= FUSED_MAX_STAGES) best = want;
    return best;
}

// Column tiles per CTA of the single-kernel path.  Its CTAs hold their whole weight slice in shared memory
// from launch to exit, and a launch starts while the one in front still runs: when one launch alone would
// take more than half of the GPU's shared memory, part of its CTAs could only start once earlier CTAs leave,
// and they would then run the whole dependent chain a second time.  Such launches run two tiles per CTA.
int fused_tiles_per_cta(const rk_npu_w4a8_workspace& ws, int tiles, int split, int stages)
{
    if (tiles < 2 || gemm_fused_smem_bytes(ws.TC, stages, 2) > 227 * 1024) return 1;
    if (ws.tiles_per_cta_override) return ws.tiles_per_cta_override;
    const size_t all = size_t(tiles) * split * (gemm_fused_smem_bytes(ws.TC, stages, 1) + 1024);
    const size_t half_gpu = size_t(ws.domain->ctx->sm_count) * (220 * 1024) / 2;
    return all > half_gpu ? 2 : 1;
}

// Launch parameters of the decode kernel for one call (its workspace runs that family).
void decode_params(const Call& c, DecodeParams& d, int cluster_override = 0)
{
    auto& ws = *c.ws;
    const auto& cfg = ws.config;
    const int N = ws.shard_N;
    const bool swiglu = c.epi == EPI_SWIGLU;
    const int F = swiglu ? N / 2 : 0;
    d.Wp = c.w->packed;
    d.A = c.dA;
    d.sw = c.w->scales;
    d.out = c.dOut;
    d.rowmax_out = c.rowmax_out;
    d.rowmax_in = c.rowmax_in;
    d.scales_out = ws.scales;
    d.codes_out = c.keep_codes ? ws.codes : nullptr;
    d.status = c.status ? c.status : ws.status;
    d.M = cfg.M; d.N = N; d.K = cfg.K;
    d.KB = ws.KB; d.NG = c.w->NG; d.F = F; d.epi = c.epi;
    d.half = c.half ? 1 : 0;
    d.cluster = cluster_override ? cluster_override : ws.split_override ? ws.split_override : gemm_decode_cluster(cfg.M, ws.KB);
    d.ring = gemm_decode_ring(cfg.M, ws.KB, swiglu);
    const int slot = d.cluster == 1 ? 0 : d.cluster == 2 ? 1 : d.cluster == 4 ? 2 : 3;
    d.ctas = gemm_decode_ctas(swiglu ? F / GROUP : (N + GROUP - 1) / GROUP, d.cluster, ws.decode_cap[slot]);
    d.timeout_ns = (unsigned long long)cfg.timeout_ms * 1000000ull;
    d.trace = ws.trace;
    d.starve = ws.starve ? 1 : 0;
}

int enqueue(const Call& c)
{
    auto& ws = *c.ws;
    const auto& cfg = ws.config;
    const bool pdl = env_flag("RK_NPU_B200_PDL", true);
    if (c.events) cudaEventRecord(c.events[0], c.stream);
    const int N = ws.shard_N;                       // the columns this GPU computes (all of them outside a group)
    const int F = c.epi == EPI_SWIGLU ? N / 2 : 0;
    const int tiles = c.epi == EPI_SWIGLU ? (F + 63) / 64 : (N + TILE_N - 1) / TILE_N;
    const unsigned long long timeout_ns = (unsigned long long)cfg.timeout_ms * 1000000ull;
    if (ws.variant == 5 && !c.codes_in) {
        // One kernel, whole-K CTAs: scan + quantise (shared by a cluster) + GEMM + epilogue.
        DecodeParams d{};
        decode_params(c, d);
        if (c.events) cudaEventRecord(c.events[1], c.stream);
        if (launch_gemm_decode(d, c.stream, pdl) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
        if (c.events) cudaEventRecord(c.events[2], c.stream);
        ws.launches.fetch_add(1, std::memory_order_relaxed);
        return RK_NPU_OK;
    }
    if (ws.variant == 3 && !c.codes_in) {
        // One kernel: scan + quantise + GEMM + epilogue.
        FusedParams f{};
        f.Wp = c.w->packed;
        f.A = c.dA;
        f.sw = c.w->scales;
        f.out = c.dOut;
        f.rowmax_out = c.rowmax_out;
        f.rowmax_in = c.rowmax_in;
        f.scales_out = ws.scales;
        f.codes_out = c.keep_codes ? ws.codes : nullptr;
        f.status = c.status ? c.status : ws.status;
        f.M = cfg.M; f.N = N; f.K = cfg.K;
        f.KB = ws.KB; f.NG = c.w->NG; f.F = F; f.epi = c.epi;
        f.split = fused_split(ws, tiles);
        f.stages = (ws.KB + f.split - 1) / f.split;
        f.tiles_per_cta = fused_tiles_per_cta(ws, tiles, f.split, f.stages);
        f.half = c.half ? 1 : 0;
        f.timeout_ns = timeout_ns;
        f.trace = ws.trace;
        if (c.events) cudaEventRecord(c.events[1], c.stream);
        if (launch_gemm_fused(f, ws.TC, c.stream, pdl) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
        if (c.events) cudaEventRecord(c.events[2], c.stream);
        ws.launches.fetch_add(1, std::memory_order_relaxed);
        return RK_NPU_OK;
    }
    if (c.codes_in) {
        CodesInParams ci{};
        ci.codes = c.codes_in;
        ci.Xq = ws.codes;
        ci.scales = ws.scales;
        ci.inverse = ws.inverse;
        ci.rowmax = c.rowmax_in;
        ci.status = ws.status;
        ci.M = cfg.M; ci.K = cfg.K; ci.Kp = ws.KB * KBLOCK; ci.T = ws.T;
        ci.parts = c.parts;
        if (launch_codes_in(ci, c.stream) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
    } else {
    QuantParams q{};
    q.A = c.dA;
    q.Xq = ws.codes;
    q.scales = ws.scales;
    q.inverse = ws.inverse;
    q.rowmax_zero = nullptr;
    q.rowmax = c.rowmax_in;
    q.status = ws.status;
    q.host_flag = nullptr;
    q.M = cfg.M;
    q.K = cfg.K;
    q.Kp = ws.KB * KBLOCK;
    q.T = ws.T;
    q.half = c.half ? 1 : 0;
    if (launch_quantize(q, c.stream, pdl) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
    }
    if (c.events) cudaEventRecord(c.events[1], c.stream);

    GemmParams g{};
    g.Wp = c.w->packed;
    g.Xq = ws.codes;
    g.sx = ws.scales;
    g.sw = c.w->scales;
    g.out = c.dOut;
    g.rowmax = c.rowmax_out;
    g.status = ws.status;
    g.M = cfg.M;
    g.N = N;
    g.K = cfg.K;
    g.KB = ws.KB;
    g.NG = c.w->NG;
    g.T = ws.T;
    g.F = F;
    g.epi = c.epi;
    g.timeout_ns = timeout_ns;
    g.trace = ws.trace;
    cudaError_t err;
    if (ws.variant == 2) {
        g.split = 1;
        g.pair = ws.pair ? 1 : 0;
        // parking pays where finishing a chunk is expensive, i.e. for the SwiGLU epilogue (measured: the plain epilogues gain
        // nothing, the extra L2 traffic lengthens their MMA phase as much as the earlier hand-back saves);
        // RK_NPU_B200_PARK_ALL=1 parks for every epilogue (experiments)
        if (c.epi == EPI_SWIGLU || env_flag("RK_NPU_B200_PARK_ALL", false)) g.partials = ws.partials;
        if (gemm_tc_persist_supported(g) && !env_flag("RK_NPU_B200_NO_PERSIST", false)) err = launch_gemm_tc_persist(g, c.stream, pdl);
        else err = launch_gemm_tc(g, c.stream, pdl);
    } else if (ws.variant == 4) {
        g.split = 1;
        g.partials = ws.partials;
        g.counts = ws.counts;
        err = launch_gemm_stream(g, ws.domain->ctx->sm_count, c.stream, pdl);
    } else {
        // (a single-kernel workspace given codes runs the ring GEMM; its split override may be odd, so it is not used here)
        g.split = (ws.variant == 3 || ws.variant == 5) ? pick_split_auto(ws, tiles, (cfg.M + ws.TC - 1) / ws.TC)
                                  : pick_split(ws, tiles, (cfg.M + ws.TC - 1) / ws.TC);
        err = launch_gemm_mma(g, ws.TC, c.stream, pdl);
    }
    if (err != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
    if (c.events) cudaEventRecord(c.events[2], c.stream);
    ws.launches.fetch_add(2, std::memory_order_relaxed);
    return RK_NPU_OK;
}

float event_us(cudaEvent_t a, cudaEvent_t b)
{
    float ms = 0;
    if (cudaEventElapsedTime(&ms, a, b) != cudaSuccess) { cudaGetLastError(); return 0; }
    return ms * 1000.f;
}

int status_to_rc(rk_npu_w4a8_workspace& ws, cudaStream_t stream)
{
    const Status s = *ws.host_status;
    if (s.device_error) {
        cudaMemsetAsync(&ws.status->device_error, 0, sizeof(int), stream);
        // a streaming launch that gave up may have left partial sums behind
        if (ws.partials) cudaMemsetAsync(ws.partials, 0, ws.partials_bytes, stream);
        if (ws.counts) cudaMemsetAsync(ws.counts, 0, ws.counts_bytes, stream);
        cudaStreamSynchronize(stream);
        return RK_NPU_ERR_SUBMIT;
    }
    return s.bad_input ? RK_NPU_ERR_PARAM : RK_NPU_OK;
}

// Group of GPUs: the kernels have written this rank's compact [M][its columns] block into its slot of the
// workspace's gather buffer; one all-gather brings the other ranks' blocks and a copy kernel puts every row piece
// at its place in `dst` [M][cols] (elements of `elem` bytes).
int gather_output(rk_npu_w4a8_workspace& ws, void* dst, int cols, int elem, bool two_range, cudaStream_t stream)
{
    rk_npu_ctx* ctx = ws.domain->ctx;
    if (const int rc = group_all_gather(ctx, ws.gather, ws.gather_slot, stream)) return rc;
    AssembleParams a{};
    a.gathered = ws.gather;
    a.out = static_cast<uint8_t*>(dst);
    a.slot_bytes = ws.gather_slot;
    a.M = ws.config.M;
    a.N = cols;
    a.world = ctx->world;
    a.elem = elem;
    a.two_range = two_range ? 1 : 0;
    if (launch_assemble_columns(a, stream) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
    ws.launches.fetch_add(1, std::memory_order_relaxed);
    return RK_NPU_OK;
}
bool grouped(const rk_npu_w4a8_workspace& ws) { return ws.domain->ctx->world > 1; }
void* own_slot(const rk_npu_w4a8_workspace& ws) { return ws.gather + size_t(ws.domain->ctx->rank) * ws.gather_slot; }
int element_bytes(int epi) { return epi == EPI_F16 ? 2 : 4; }

// One linear queued on `stream`: outside a group straight into dOut; in a group into this rank's slot, then the
// exchange that leaves the whole [M][columns] tensor in dOut on every rank.
int enqueue_linear(Call call, void* dOut)
{
    auto& ws = *call.ws;
    call.dOut = grouped(ws) ? own_slot(ws) : dOut;
    if (const int rc = enqueue(call)) return rc;
    if (!grouped(ws)) return RK_NPU_OK;
    const bool swiglu = call.epi == EPI_SWIGLU;
    const int rc = gather_output(ws, dOut, swiglu ? ws.config.N / 2 : ws.config.N, element_bytes(call.epi), !swiglu && ws.shard.two_range, call.stream);
    if (call.events) cudaEventRecord(call.events[3], call.stream);   // the exchange between GPUs ends here
    return rc;
}

// One blocking projection; the caller holds the workspace.
int run_locked(rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w, const void* A, void* C, bool half, int epi,
               rk_npu_w4a8_timings* metrics)
{
    const auto start = Clock::now();
    const auto& cfg = ws->config;
    rk_npu_w4a8_timings t{};
    if (cudaSetDevice(ws->domain->ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    const size_t in_bytes = size_t(cfg.M) * cfg.K * (half ? 2 : 4);
    const int out_cols = epi == EPI_SWIGLU ? cfg.N / 2 : cfg.N;
    const size_t out_bytes = size_t(cfg.M) * out_cols * (epi == EPI_F16 ? 2 : 4);
    const Placement a_at = placement(A), c_at = placement(C);
    const bool a_dev = a_at.device, c_dev = c_at.device;
    cudaStream_t s = ws->stream;
    const void* dA = A;
    void* dC = C;
    auto copy_start = Clock::now();
    if (!a_dev) {
        // ordinary (pageable) host memory: a small tensor is copied into the workspace's page-locked piece first -- the
        // host copy is cheaper than the staging the driver does for pageable memory
        const void* from = A;
        if (!a_at.alias && ws->bounce_in && in_bytes <= ws->bounce_bytes) { std::memcpy(ws->bounce_in, A, in_bytes); from = ws->bounce_in; }
        if (cudaMemcpyAsync(ws->stage_in, from, in_bytes, cudaMemcpyHostToDevice, s) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
        dA = ws->stage_in;
    }
    // A small batch through one of the single-kernel families writes every output element once and reports through two
    // plain stores, so a host caller is served without the two copies behind the kernel: the kernel stores straight
    // into the caller's tensor when that is page-locked memory the GPU can address, and reports into the workspace's
    // own page-locked status block.  (The activations are still copied in: every CTA reads them.)
    // (Not when the caller asks for stage timings: the device part of a call must not contain stores that cross the bus,
    // or the figures of different kernel families -- which the search tuner ranks -- stop being comparable.)
    const bool single_kernel = (ws->variant == 3 || ws->variant == 5) && !grouped(*ws) && epi != EPI_SWIGLU && !metrics;
    void* c_alias = (!c_dev && single_kernel && out_bytes <= (size_t(1) << 20)) ? c_at.alias : nullptr;
    // ... and an ordinary host result of a small batch lands in the workspace's page-locked piece and is copied out by the host
    const bool bounce_out = !c_dev && !c_alias && single_kernel && ws->bounce_out_alias && out_bytes <= ws->bounce_bytes;
    if (bounce_out) c_alias = ws->bounce_out_alias;
    if (c_alias) dC = c_alias;
    else if (!c_dev) dC = ws->stage_out;
    Status* status_alias = single_kernel ? ws->host_status_alias : nullptr;
    if (status_alias) *ws->host_status = Status{};
    t.sync_us += elapsed_us(copy_start);
    Call call{ws, w, dA, dC, half, epi, nullptr, nullptr, s, metrics ? ws->events : nullptr, epi == EPI_I32};
    call.status = status_alias;
    int rc = enqueue_linear(call, dC);
    if (rc) { cudaStreamSynchronize(s); return rc; }
    copy_start = Clock::now();
    // Other host tensors are copied straight from and to the caller's memory.
    if (!c_dev && !c_alias) cudaMemcpyAsync(C, dC, out_bytes, cudaMemcpyDeviceToHost, s);
    if (!status_alias) cudaMemcpyAsync(ws->host_status, ws->status, sizeof(Status), cudaMemcpyDeviceToHost, s);
    if (cudaStreamSynchronize(s) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
    rc = status_to_rc(*ws, s);
    if (bounce_out && rc == RK_NPU_OK) std::memcpy(C, ws->bounce_out, out_bytes);
    t.sync_us += elapsed_us(copy_start);
    if (metrics) {
        t.activation_scan_us = event_us(ws->events[0], ws->events[1]);
        t.submit_us = rc ? 0.0 : event_us(ws->events[1], ws->events[2]);   // a rejected input did no GEMM work
        if (grouped(*ws)) t.reduce_us = event_us(ws->events[2], ws->events[3]);   // all-gather + reassembly of the column shards
        t.total_us = elapsed_us(start);
        *metrics = t;
    }
    return rc;
}

int run(rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w, const void* A, void* C, bool half, int epi,
        rk_npu_w4a8_timings* metrics)
{
    const int rc = validate(ws, w, A, C, epi == EPI_SWIGLU);
    if (rc) return rc;
    WorkspaceLock lock(*ws);
    if (!lock) return RK_NPU_ERR_BUSY;
    try { return run_locked(ws, w, A, C, half, epi, metrics); } catch (...) { return RK_NPU_ERR_PARAM; }
}

void workspace_destroy(rk_npu_w4a8_workspace* ws)
{
    if (!ws) return;
    auto* d = ws->domain;
    if (d) cudaSetDevice(d->ctx->device);
    if (ws->stream) cudaStreamSynchronize(ws->stream);
    if (ws->codes) device_free(d, ws->codes, ws->codes_bytes);
    if (ws->scales) device_free(d, ws->scales, sizeof(float) * 2 * ws->config.M);
    if (ws->rowmax) device_free(d, ws->rowmax, sizeof(uint32_t) * ws->config.M);
    if (ws->status) device_free(d, ws->status, sizeof(Status));
    if (ws->stage_in) device_free(d, ws->stage_in, ws->stage_in_bytes);
    if (ws->stage_out) device_free(d, ws->stage_out, ws->stage_out_bytes);
    if (ws->bounce_in) cudaFreeHost(ws->bounce_in);
    if (ws->bounce_out) cudaFreeHost(ws->bounce_out);
    if (ws->trace) device_free(d, ws->trace, ws->trace_bytes);
    if (ws->partials) device_free(d, ws->partials, ws->partials_bytes);
    if (ws->counts) device_free(d, ws->counts, ws->counts_bytes);
    if (ws->gather) device_free(d, ws->gather, ws->gather_bytes);
    if (ws->code_gather) device_free(d, ws->code_gather, ws->code_gather_bytes);
    if (ws->host_status) cudaFreeHost(ws->host_status);
    for (auto& e : ws->events) if (e) cudaEventDestroy(e);
    if (ws->stream) cudaStreamDestroy(ws->stream);
    if (d) domain_release(d);
    delete ws;
}
} // namespace

// ================================================================== domains, context
namespace rkb200 {
void domain_retain(rk_npu_iommu_domain* d) { if (d) d->refs.fetch_add(1, std::memory_order_relaxed); }
void domain_release(rk_npu_iommu_domain* d)
{
    if (d && d->refs.fetch_sub(1, std::memory_order_acq_rel) == 1) delete d;
}
// Test hook: the allocation that brings this counter to zero fails as if the device were out of memory.
static std::atomic<long long> g_allocations_until_failure{-1};
int device_alloc(rk_npu_iommu_domain* d, void** ptr, size_t bytes)
{
    *ptr = nullptr;
    if (!bytes) bytes = 16;
    if (g_allocations_until_failure.load(std::memory_order_relaxed) >= 0 &&
        g_allocations_until_failure.fetch_sub(1, std::memory_order_relaxed) == 0)
        return RK_NPU_ERR_NOMEM;
    if (cudaMalloc(ptr, bytes) != cudaSuccess) { cudaGetLastError(); *ptr = nullptr; return RK_NPU_ERR_NOMEM; }
    std::lock_guard<std::mutex> g(d->lock);
    d->stats.live_bytes += bytes;
    d->stats.peak_bytes = std::max(d->stats.peak_bytes, d->stats.live_bytes);
    ++d->stats.creates;
    return RK_NPU_OK;
}
void device_free(rk_npu_iommu_domain* d, void* ptr, size_t bytes)
{
    if (!ptr) return;
    if (!bytes) bytes = 16;
    cudaFree(ptr);
    std::lock_guard<std::mutex> g(d->lock);
    d->stats.live_bytes -= std::min<uint64_t>(bytes, d->stats.live_bytes);
    ++d->stats.destroys;
}
} // namespace rkb200

extern "C" void rk_npu_b200_test_fail_allocation(long long after)
{
    rkb200::g_allocations_until_failure.store(after, std::memory_order_relaxed);
}

extern "C" rk_npu_ctx* rk_npu_open(const char* dev)
{
    int device = -1;
    const char* spec = (dev && *dev) ? dev : std::getenv("RK_NPU_CUDA_DEVICE");
    if (spec && *spec) {
        const char* digits = std::strncmp(spec, "cuda:", 5) == 0 ? spec + 5 : spec;
        char* end = nullptr;
        errno = 0;
        const long v = std::strtol(digits, &end, 10);
        if (errno || end == digits || *end || v < 0 || v > 1023) { errno = ENODEV; return nullptr; }
        device = int(v);
    }
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count < 1) { cudaGetLastError(); errno = ENODEV; return nullptr; }
    if (device < 0 && cudaGetDevice(&device) != cudaSuccess) { cudaGetLastError(); errno = ENODEV; return nullptr; }
    if (device >= count) { errno = ENODEV; return nullptr; }
    cudaDeviceProp prop{};
    if (cudaSetDevice(device) != cudaSuccess || cudaGetDeviceProperties(&prop, device) != cudaSuccess) {
        cudaGetLastError();
        errno = ENODEV;
        return nullptr;
    }
    if (prop.major != 10) { errno = ENODEV; return nullptr; }   // kernels are built for sm_100a only
    auto* ctx = new (std::nothrow) rk_npu_ctx;
    if (!ctx) { errno = ENOMEM; return nullptr; }
    ctx->device = device;
    ctx->id = uint64_t(reinterpret_cast<uintptr_t>(ctx));
    int driver = 0;
    cudaDriverGetVersion(&driver);
    ctx->driver_version = uint32_t(driver);
    ctx->sm_count = prop.multiProcessorCount;
    if (cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking) != cudaSuccess) {
        cudaGetLastError();
        delete ctx;
        errno = ENODEV;
        return nullptr;
    }
    return ctx;
}

extern "C" rk_npu_ctx* rk_npu_b200_open_offline(uint32_t driver_version)
{
    auto* ctx = new (std::nothrow) rk_npu_ctx;
    if (!ctx) { errno = ENOMEM; return nullptr; }
    ctx->device = -1;
    ctx->id = uint64_t(reinterpret_cast<uintptr_t>(ctx));
    ctx->driver_version = driver_version;
    return ctx;
}

extern "C" void rk_npu_close(rk_npu_ctx* ctx)
{
    if (!ctx) return;
    if (ctx->device < 0) { delete ctx; return; }
    cudaSetDevice(ctx->device);
    if (ctx->stream) { cudaStreamSynchronize(ctx->stream); cudaStreamDestroy(ctx->stream); }
    group_close(ctx);
    delete ctx;
}

extern "C" int rk_npu_b200_device(const rk_npu_ctx* ctx) { return ctx ? ctx->device : -1; }
extern "C" uint32_t rk_npu_b200_driver_version(const rk_npu_ctx* ctx) { return ctx ? ctx->driver_version : 0; }

extern "C" rk_npu_iommu_domain* rk_npu_iommu_domain_create(rk_npu_ctx* ctx, uint32_t domain_id)
{
    if (!ctx || ctx->device < 0 || domain_id >= RK_NPU_IOMMU_DOMAIN_COUNT) { errno = EINVAL; return nullptr; }
    auto* d = new (std::nothrow) rk_npu_iommu_domain;
    if (!d) { errno = ENOMEM; return nullptr; }
    d->ctx = ctx;
    d->id = domain_id;
    return d;
}
extern "C" void rk_npu_iommu_domain_free(rk_npu_iommu_domain* domain) { domain_release(domain); }
extern "C" uint32_t rk_npu_iommu_domain_id(const rk_npu_iommu_domain* domain) { return domain ? domain->id : 0; }
extern "C" int rk_npu_iommu_domain_memory_stats(const rk_npu_iommu_domain* domain, rk_npu_domain_memory_stats* stats)
{
    if (!domain || !stats) return RK_NPU_ERR_PARAM;
    auto* d = const_cast<rk_npu_iommu_domain*>(domain);
    std::lock_guard<std::mutex> g(d->lock);
    *stats = d->stats;
    return RK_NPU_OK;
}

extern "C" const char* rk_npu_strerror(int code)
{
    switch (code) {
    case RK_NPU_OK: return "ok";
    case RK_NPU_ERR_OPEN: return "could not open the device";
    case RK_NPU_ERR_IOCTL: return "device runtime call failed";
    case RK_NPU_ERR_PARAM: return "bad argument";
    case RK_NPU_ERR_NOMEM: return "buffer too small or allocation failed";
    case RK_NPU_ERR_SUBMIT: return "device job failed or timed out";
    case RK_NPU_ERR_BUSY: return "workspace is already running";
    case RK_NPU_ERR_DOMAIN: return "context or domain mismatch";
    case RK_NPU_ERR_IO: return "file I/O failed";
    case RK_NPU_ERR_CACHE_MISS: return "tuning cache miss";
    default: return "unknown error";
    }
}

// ================================================================== configuration and accounting
extern "C" void rk_npu_w4a8_config_init(rk_npu_w4a8_config* cfg, int M, int N, int K)
{
    if (!cfg) return;
    *cfg = {};
    cfg->M = M; cfg->N = N; cfg->K = K;
    cfg->m_tile = 64; cfg->k_tile = 480; cfg->n_tile = 1024;
    cfg->npu_core_mask = 1; cfg->timeout_ms = 500;
    cfg->pipeline = RK_NPU_W4A8_PIPELINED; cfg->cpu_threads = 1;
}
extern "C" void rk_npu_w4a8_options_init(rk_npu_w4a8_options* options)
{
    if (options) *options = {uint32_t(sizeof(*options)), RK_NPU_W4A8_INPUT_NATIVE, RK_NPU_W4A8_REDUCE_CPU};
}
extern "C" int rk_npu_i4_weights_memory_query(const rk_npu_i4_weight_config* cfg, uint64_t* bytes)
{
    if (!cfg || !bytes) return RK_NPU_ERR_PARAM;
    return weight_bytes_query(cfg->K, cfg->N, cfg->k_tile, *bytes);
}
extern "C" int rk_npu_w4a8_memory_query_ex(const rk_npu_w4a8_config* cfg, const rk_npu_w4a8_options* options,
                                           rk_npu_w4a8_memory_info_ex* out)
{
    if (!cfg || !out) return RK_NPU_ERR_PARAM;
    bool panel8, npu;
    int rc = options_decode(options, cfg->M, panel8, npu);
    if (rc) return rc;
    DeviceGeometry device;
    rc = geometry_from(*cfg, panel8, device);
    if (rc) return rc;
    rk_npu_w4a8_memory_info_ex info{};
    info.effective_reduce_backend = npu ? RK_NPU_W4A8_REDUCE_NPU : RK_NPU_W4A8_REDUCE_CPU;
    const bool chained = cfg->pipeline == RK_NPU_W4A8_CHAIN;
    if (chained && npu) return RK_NPU_ERR_PARAM;
    rc = chained ? device.memory_chained(info.base.backend) : device.memory(info.base.backend);
    if (rc) return rc;
    // host side of a call: 8 bytes of channel metadata per column; per token a scale and its inverse, and with
    // the host reduction an int32 accumulator row (plus per-thread row maxima when a SwiGLU epilogue is possible)
    info.base.weight_metadata_bytes = uint64_t(cfg->N) * 8;
    info.base.cpu_scratch_bytes = uint64_t(cfg->M) * 8;
    if (npu) {
        rc = device.memory_device_reduce(info);
        if (rc) return rc;
    } else {
        info.base.cpu_scratch_bytes += uint64_t(cfg->M) * uint64_t(align_up64(cfg->N, 64)) * 4;
        if (cfg->N % 64 == 0) info.base.cpu_scratch_bytes += (uint64_t(cfg->M) + 16) * cfg->cpu_threads * 4;
    }
    info.workspace_bytes = info.base.backend.input_bytes + info.base.backend.partial_bytes +
                           info.base.backend.control_bytes + info.base.cpu_scratch_bytes +
                           info.reduction_output_bytes + info.reduction_weight_bytes + info.reduction_control_bytes;
    *out = info;
    return RK_NPU_OK;
}
extern "C" int rk_npu_w4a8_memory_query(const rk_npu_w4a8_config* cfg, rk_npu_w4a8_memory_info* out)
{
    if (!out) return RK_NPU_ERR_PARAM;
    rk_npu_w4a8_memory_info_ex info{};
    const int rc = rk_npu_w4a8_memory_query_ex(cfg, nullptr, &info);
    if (!rc) *out = info.base;
    return rc;
}

// ================================================================== weights
rk_npu_w4a8_weights* rkb200::create_weights(rk_npu_iommu_domain* domain, const rk_npu_w4a8_weight_info& info,
                                            const int8_t* B, const float* scales, const Profile* profile)
{
    const auto& key = info.config;
    if (!domain || !domain->ctx || !B || !scales || !valid_shape(key.K, key.N)) return nullptr;
    uint64_t reference_bytes = 0;
    if (weight_bytes_query(key.K, key.N, key.k_tile, reference_bytes)) return nullptr;
    std::unique_ptr<rk_npu_w4a8_weights> w(new (std::nothrow) rk_npu_w4a8_weights);
    if (!w) return nullptr;
    if (profile) {
        w->profile = *profile;
    } else {
        // Explicit-k_tile factories still capture the full proof and the identity.
        rk_npu_w4a8_autotune_config c;
        rk_npu_w4a8_autotune_config_init(&c, 1, key.N, key.K);
        c.required_k_tile = 0;
        c.k_tile_multiplier = info.multiplier;
        if (make_profile(c, B, scales, w->profile)) return nullptr;
    }
    for (int n = 0; n < key.N; ++n)
        if (!std::isfinite(scales[n]) || !(scales[n] > 0)) return nullptr;
    // An explicit tile above the universal 480 must be certified by the weights
    // unless the caller's policy relaxed the bound (src/rk_npu_i4_plan.cpp:95-99).
    if (key.k_tile > 480 && !info.bound_relaxed && !w->profile.certified(key.k_tile)) {
        WeightBound b;
        if (bound_weights(key.K, key.N, B, key.k_tile, b)) return nullptr;
    }
    auto* ctx = domain->ctx;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return nullptr;
    w->info = info;
    // In a group of GPUs this object holds its rank's columns only; identity (profile, fingerprint, the checks
    // above) is that of the whole matrix, so every rank agrees on it.
    w->shard = shard_plan(key.N, ctx->world, ctx->rank);
    w->shard_N = w->shard.columns();
    const int local_N = std::max(w->shard_N, 1);            // a rank beyond the last block still builds valid (empty) tensors
    std::vector<int8_t> local_B;
    std::vector<float> local_scales;
    if (ctx->world > 1) {
        local_B.assign(size_t(key.K) * local_N, 0);
        local_scales.assign(size_t(local_N), 1.0f);
        const int width = w->shard.n1 - w->shard.n0, pieces = w->shard.two_range ? 2 : 1;
        for (int piece = 0; piece < pieces; ++piece) {
            const int from = piece * (key.N / 2) + w->shard.n0, to = piece * width;
            for (int k = 0; k < key.K; ++k)
                std::memcpy(local_B.data() + size_t(k) * local_N + to, B + size_t(k) * key.N + from, size_t(width));
            std::memcpy(local_scales.data() + to, scales + from, sizeof(float) * size_t(width));
        }
        B = local_B.data();
        scales = local_scales.data();
    }
    w->KB = (key.K + KBLOCK - 1) / KBLOCK;
    w->NG = align_up((local_N + GROUP - 1) / GROUP, 8) + 8;   // zero groups: odd tile counts of CTA pairs, SwiGLU tails
    w->packed_bytes = size_t(w->NG) * (size_t(w->KB) * 4) * 512;
    w->scale_bytes = size_t(w->NG) * GROUP * sizeof(float);
    w->domain = domain;
    w->ctx_id = ctx->id;
    w->domain_id = domain->id;
    domain_retain(domain);
    auto fail = [&]() -> rk_npu_w4a8_weights* {
        if (w->packed) device_free(domain, w->packed, w->packed_bytes);
        if (w->scales) device_free(domain, w->scales, w->scale_bytes);
        domain_release(domain);
        return nullptr;
    };
    if (device_alloc(domain, reinterpret_cast<void**>(&w->packed), w->packed_bytes)) return fail();
    if (device_alloc(domain, reinterpret_cast<void**>(&w->scales), w->scale_bytes)) return fail();
    int8_t* codes = nullptr;
    int* error = nullptr;
    const size_t code_bytes = size_t(key.K) * local_N;
    bool ok = cudaMalloc(reinterpret_cast<void**>(&codes), code_bytes) == cudaSuccess &&
              cudaMalloc(reinterpret_cast<void**>(&error), sizeof(int)) == cudaSuccess;
    if (ok) {
        cudaStream_t s = ctx->stream;
        ok = cudaMemcpyAsync(codes, B, code_bytes, cudaMemcpyHostToDevice, s) == cudaSuccess &&
             cudaMemsetAsync(error, 0, sizeof(int), s) == cudaSuccess &&
             cudaMemsetAsync(w->scales, 0, w->scale_bytes, s) == cudaSuccess &&
             cudaMemcpyAsync(w->scales, scales, sizeof(float) * local_N, cudaMemcpyHostToDevice, s) == cudaSuccess;
        if (ok) {
            PackParams p{codes, w->packed, error, key.K, local_N, w->KB * 4, w->NG};
            ok = launch_pack_weights(p, s) == cudaSuccess;
        }
        int host_error = 1;
        if (ok) ok = cudaMemcpyAsync(&host_error, error, sizeof(int), cudaMemcpyDeviceToHost, s) == cudaSuccess;
        ok = cudaStreamSynchronize(s) == cudaSuccess && ok && host_error == 0;   // a code outside [-8,7] fails creation
    }
    if (codes) cudaFree(codes);
    if (error) cudaFree(error);
    if (!ok) { cudaGetLastError(); return fail(); }
    return w.release();
}

const Profile& rkb200::weights_profile(const rk_npu_w4a8_weights* w) { return w->profile; }

extern "C" rk_npu_w4a8_weights* rk_npu_w4a8_weights_create(rk_npu_iommu_domain* domain, const rk_npu_i4_weight_config* cfg,
                                                           const int8_t* B, const float* scales)
{
    if (!domain || !cfg || !B || !scales || !valid_shape(cfg->K, cfg->N)) return nullptr;
    try {
        rk_npu_i4_weight_config actual = *cfg;
        int safe = cfg->k_tile;
        double factor = 1;
        Profile profile;
        if (cfg->k_tile == 0) {
            WeightBound bound;
            if (bound_weights(cfg->K, cfg->N, B, 0, bound)) return nullptr;
            safe = bound.k_tile;
            if (const char* text = std::getenv("RK_NPU_W4A8_K_TILE_MULTIPLIER")) {
                errno = 0;
                char* end = nullptr;
                factor = std::strtod(text, &end);
                if (errno || end == text || *end || !std::isfinite(factor) || factor < 1) return nullptr;
            }
            const int cap = std::min(K_TILE_MAX, align_up(cfg->K, 32));
            actual.k_tile = int(std::min(double(cap), safe * factor) / 32) * 32;
            profile.K = cfg->K;
            profile.N = cfg->N;
            profile.safe = safe;
            profile.safe_tiles = bound.safe_tiles;
            profile.multiplier = factor;
            profile.limit = actual.k_tile;
            profile.fingerprint = weight_fingerprint(cfg->K, cfg->N, B, scales);
        }
        const rk_npu_w4a8_weight_info info{actual, safe, factor, actual.k_tile > safe};
        return create_weights(domain, info, B, scales, cfg->k_tile == 0 ? &profile : nullptr);
    } catch (...) { return nullptr; }
}

extern "C" void rk_npu_w4a8_weights_free(rk_npu_w4a8_weights* w)
{
    if (!w) return;
    cudaSetDevice(w->domain->ctx->device);
    device_free(w->domain, w->packed, w->packed_bytes);
    device_free(w->domain, w->scales, w->scale_bytes);
    domain_release(w->domain);
    delete w;
}
extern "C" int rk_npu_w4a8_weights_query(const rk_npu_w4a8_weights* w, rk_npu_w4a8_weight_info* out)
{
    if (!w || !out) return RK_NPU_ERR_PARAM;
    *out = w->info;
    return RK_NPU_OK;
}

// ================================================================== workspaces
rk_npu_w4a8_workspace* rkb200::create_workspace_scheduled(rk_npu_iommu_domain* domain, const rk_npu_w4a8_config* cfg,
                                                          const rk_npu_w4a8_options* options, const Schedule& schedule)
{
    if (!domain || !domain->ctx || !cfg) return nullptr;
    rk_npu_w4a8_memory_info_ex info{};
    if (rk_npu_w4a8_memory_query_ex(cfg, options, &info)) return nullptr;
    auto* ctx = domain->ctx;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return nullptr;
    rk_npu_w4a8_workspace* ws = new (std::nothrow) rk_npu_w4a8_workspace;
    if (!ws) return nullptr;
    bool panel8 = false;
    options_decode(options, cfg->M, panel8, ws->npu_reduce);
    ws->input_layout = panel8;
    ws->config = *cfg;
    ws->domain = domain;
    ws->ctx_id = ctx->id;
    ws->domain_id = domain->id;
    domain_retain(domain);
    ws->KB = (cfg->K + KBLOCK - 1) / KBLOCK;
    ws->shard = shard_plan(cfg->N, ctx->world, ctx->rank);
    ws->shard_N = ws->shard.columns();
    if (ws->shard_N < 1) { workspace_destroy(ws); return nullptr; }   // fewer 64-column blocks than GPUs in the group
    const int local_N = ws->shard_N;      // what this GPU's kernels compute; schedules are chosen for it
    // Schedule: the mma.sync kernel serves up to 32 tokens per CTA pass; larger batches
    // go to the tcgen05 kernel when it can run this geometry.
    GemmParams probe{};
    probe.M = cfg->M; probe.N = local_N; probe.K = cfg->K; probe.KB = ws->KB;
    // an explicit schedule (a tuned strategy) wins over the environment override, which wins over the rules below
    const int forced = schedule.family ? schedule.family : std::getenv("RK_NPU_B200_VARIANT") ? std::atoi(std::getenv("RK_NPU_B200_VARIANT")) : 0;
    const bool tc_ok = gemm_tc_supported(probe);
    const bool fused_ok = cfg->M <= 32 && ws->KB <= 8 * FUSED_MAX_STAGES;
    const bool stream_ok = cfg->M <= 128 && (long long)ws->KB * KBLOCK <= 131072;
    // Small batches: the single-kernel path wins while all of the weights fit in the SMs' shared
    // memory at once (one wave, up to about 24 MB) and the batch is a single 8-token MMA column
    // block; beyond that the two-kernel ring (quantise + mma.sync GEMM) streams better.  Up to 32
    // tokens the tcgen05 streaming kernel (4) is opt-in: its time does not depend on the batch
    // size, but it only overtakes the ring at 32 tokens.
    long long fused_limit_mb = 24;
    if (const char* e = std::getenv("RK_NPU_B200_FUSED_MAX_MB")) fused_limit_mb = std::max(0, std::atoi(e));   // experiments
    const bool fused_best = fused_ok && cfg->M <= 8 && (long long)cfg->K * local_N / 2 <= (fused_limit_mb << 20);
    // Up to eight tokens: the decode kernel (5), whose CTAs own whole output channels over all of K.  Up to four
    // tokens (at most one 16-element unit to quantise per thread of a four-CTA cluster, or none to exchange at all)
    // it beats the split-K kernel (3) on 7B-class shapes (4 tokens: 1783 against 1718 GB/s on the decode ring);
    // from five tokens on its exchange of int8 codes costs more than the split-K kernel's exchange of row maxima
    // and partial sums (8 tokens: 1479 against 1669 GB/s), so the split-K kernel keeps those where it applies.
    const bool decode_ok = gemm_decode_supported(cfg->M, cfg->K);
    const bool decode_best = decode_ok && (cfg->M <= 4 || !fused_best);
    // 33..128 tokens: the per-tile tcgen05 kernel has one CTA per 128 output channels; when that is less than
    // half the SMs and K is long, the streaming kernel (all SMs, K split between CTAs) is faster.
    const bool stream_best = stream_ok && cfg->M > 32 && cfg->K >= 8192 &&
                             (local_N + TILE_N - 1) / TILE_N * 2 <= ctx->sm_count;
    // 33..128 tokens with so few tiles that tiles x 32-token chunks fit the SMs in one wave (N = 4096: 32 x 4): the
    // mma.sync ring, one CTA per (tile, chunk, K split), fills the GPU where the tcgen05 kernels leave SMs idle or
    // pay for combining partial tiles (11008 -> 4096 at 128 tokens: 33 us against 44 and 47 us).
    const bool ring_best = cfg->M > 32 && cfg->M <= 128 &&
                           (long long)((local_N + TILE_N - 1) / TILE_N) * ((cfg->M + 31) / 32) <= ctx->sm_count;
    int variant = decode_best ? 5 : ring_best ? 1 : (cfg->M > 32 && stream_best) ? 4 : (cfg->M > 32 && tc_ok) ? 2 : fused_best ? 3 : 1;
    if (forced == 1 || (forced == 2 && tc_ok) || (forced == 3 && fused_ok) || (forced == 4 && stream_ok) || (forced == 5 && decode_ok))
        variant = forced;
    ws->variant = variant;
    if (const char* e = std::getenv("RK_NPU_B200_TILES_PER_CTA")) {   // experiments and tests: 1 or 2, else automatic
        const int v = std::atoi(e);
        ws->tiles_per_cta_override = (v == 1 || v == 2) ? v : 0;
    }
    if (variant == 2) {
        // Two-CTA tiles (128-token code tiles, two per MMA tile) on the persistent kernel.  Also for 33..128 tokens,
        // where half of every MMA multiplies zero tokens: its resident CTA pairs still beat one launch-and-leave CTA
        // per tile (FFN 4096 -> 2 x 14336 -> 4096 at 128 tokens 129 -> 104 us, the 128 x 4096 x 28672 linear 49 -> 41 us).
        ws->TC = 0;
        int pair_min = 33;
        if (const char* e = std::getenv("RK_NPU_B200_PAIR_MIN")) pair_min = std::max(1, std::atoi(e));   // experiments
        ws->pair = cfg->M >= pair_min && !env_flag("RK_NPU_B200_NO_PAIR", false);
        ws->T = ws->pair ? 128 : (cfg->M >= 256 ? 256 : align_up(cfg->M, 16));
    } else if (variant == 4) {
        ws->TC = ws->T = cfg->M <= 16 ? 16 : cfg->M <= 32 ? 32 : cfg->M <= 64 ? 64 : 128;   // tcgen05 N
    } else {
        ws->TC = cfg->M <= 8 ? 8 : cfg->M <= 16 ? 16 : 32;
        ws->T = ws->TC;
    }
    if (decode_ok)   // (also when another family is the default: rk_npu_b200_w4a8_set_schedule may switch to the decode kernel)
        for (int i = 0; i < 4; ++i)   // one CTA per SM at most, fewer where whole clusters do not fit
            ws->decode_cap[i] = gemm_decode_resident_ctas(1 << i, gemm_decode_smem_bytes(cfg->M, ws->KB, true, gemm_decode_ring(cfg->M, ws->KB, true)), ctx->sm_count);
    // cooperating CTAs per column tile: split-K factor of the ring and of the split-K single kernel, cluster size of the
    // decode kernel; ignored where the family balances by itself or the reduction is too short to split
    if (schedule.cluster && (variant == 1 || variant == 5 || (variant == 3 && (ws->KB + schedule.cluster - 1) / schedule.cluster <= FUSED_MAX_STAGES)) &&
        (variant == 5 || ws->KB >= schedule.cluster))
        ws->split_override = schedule.cluster;
    const size_t Mp = size_t(align_up(cfg->M, ws->pair ? 256 : ws->T));
    ws->codes_bytes = Mp * size_t(ws->KB) * KBLOCK;
    const int out_cols = cfg->N;
    ws->stage_in_bytes = size_t(cfg->M) * cfg->K * 4;
    ws->stage_out_bytes = size_t(cfg->M) * out_cols * 4;
    bool ok = !device_alloc(domain, reinterpret_cast<void**>(&ws->codes), ws->codes_bytes);
    ok = ok && !device_alloc(domain, reinterpret_cast<void**>(&ws->scales), sizeof(float) * 2 * cfg->M);
    ok = ok && !device_alloc(domain, reinterpret_cast<void**>(&ws->rowmax), sizeof(uint32_t) * cfg->M);
    ok = ok && !device_alloc(domain, reinterpret_cast<void**>(&ws->status), sizeof(Status));
    if (variant == 4) {
        const size_t tiles = size_t(local_N + TILE_N - 1) / TILE_N;
        ws->partials_bytes = 2 * size_t(ctx->sm_count) * 128 * size_t(ws->TC) * sizeof(int);   // two slots per CTA
        ws->counts_bytes = tiles * sizeof(unsigned int);
        ok = ok && !device_alloc(domain, reinterpret_cast<void**>(&ws->partials), ws->partials_bytes);
        ok = ok && !device_alloc(domain, reinterpret_cast<void**>(&ws->counts), ws->counts_bytes);
    }
    if (variant == 2 && ws->pair && env_flag("RK_NPU_B200_PARK", true)) {
        // the persistent kernel parks accumulator chunks here between reading them out of tensor memory and finishing them
        ws->partials_bytes = gemm_tc_persist_park_bytes(ctx->sm_count);
        ok = ok && !device_alloc(domain, reinterpret_cast<void**>(&ws->partials), ws->partials_bytes);
    }
    if (ctx->world > 1) {
        ws->gather_slot = size_t(cfg->M) * size_t(shard_plan(cfg->N, ctx->world, 0).columns()) * 4;   // rank 0's share is the widest
        ws->gather_bytes = ws->gather_slot * size_t(ctx->world);
        ok = ok && !device_alloc(domain, reinterpret_cast<void**>(&ws->gather), ws->gather_bytes);
        // a down projection of a group FFN may receive its activations as all-gathered int8 codes [world][M][K / world]
        ws->code_gather_bytes = size_t(cfg->M) * size_t(align_up(cfg->K, 64));
        ok = ok && !device_alloc(domain, reinterpret_cast<void**>(&ws->code_gather), ws->code_gather_bytes);
    }
    ok = ok && !device_alloc(domain, &ws->stage_in, ws->stage_in_bytes);
    ok = ok && !device_alloc(domain, &ws->stage_out, ws->stage_out_bytes);
    if (ok) {
        ws->inverse = ws->scales + cfg->M;
        ok = cudaHostAlloc(reinterpret_cast<void**>(&ws->host_status), sizeof(Status), cudaHostAllocDefault) == cudaSuccess &&
             cudaStreamCreateWithFlags(&ws->stream, cudaStreamNonBlocking) == cudaSuccess;
    }
    for (auto& e : ws->events) ok = ok && cudaEventCreate(&e) == cudaSuccess;
    if (ok) {
        // Token and K padding of the code buffer stays zero for the life of the workspace.
        ok = cudaMemsetAsync(ws->codes, 0, ws->codes_bytes, ws->stream) == cudaSuccess &&
             cudaMemsetAsync(ws->status, 0, sizeof(Status), ws->stream) == cudaSuccess &&
             cudaMemsetAsync(ws->rowmax, 0, sizeof(uint32_t) * cfg->M, ws->stream) == cudaSuccess &&
             (!ws->partials || cudaMemsetAsync(ws->partials, 0, ws->partials_bytes, ws->stream) == cudaSuccess) &&
             (!ws->counts || cudaMemsetAsync(ws->counts, 0, ws->counts_bytes, ws->stream) == cudaSuccess) &&
             cudaStreamSynchronize(ws->stream) == cudaSuccess;
        std::memset(ws->host_status, 0, sizeof(Status));
        ws->host_status_alias = static_cast<Status*>(mapped_alias(ws->host_status));
        // page-locked pieces for small host tensors of the blocking calls (optional: without them the calls copy directly)
        const size_t most = std::max(ws->stage_in_bytes, ws->stage_out_bytes);
        if ((variant == 3 || variant == 5) && ctx->world == 1 && most <= (size_t(1) << 20)) {
            if (cudaHostAlloc(&ws->bounce_in, most, cudaHostAllocDefault) == cudaSuccess &&
                cudaHostAlloc(&ws->bounce_out, most, cudaHostAllocMapped) == cudaSuccess) {
                ws->bounce_bytes = most;
                ws->bounce_out_alias = mapped_alias(ws->bounce_out);
            } else {
                cudaGetLastError();
                if (ws->bounce_in) cudaFreeHost(ws->bounce_in);
                if (ws->bounce_out) cudaFreeHost(ws->bounce_out);
                ws->bounce_in = ws->bounce_out = nullptr;
            }
        }
    }
    if (!ok) { cudaGetLastError(); workspace_destroy(ws); return nullptr; }
    return ws;
}
extern "C" rk_npu_w4a8_workspace* rk_npu_w4a8_workspace_create_ex(rk_npu_iommu_domain* domain, const rk_npu_w4a8_config* cfg,
                                                                  const rk_npu_w4a8_options* options)
{
    return create_workspace_scheduled(domain, cfg, options, Schedule{});
}
extern "C" rk_npu_w4a8_workspace* rk_npu_w4a8_workspace_create(rk_npu_iommu_domain* domain, const rk_npu_w4a8_config* cfg)
{
    return create_workspace_scheduled(domain, cfg, nullptr, Schedule{});
}
extern "C" void rk_npu_w4a8_workspace_free(rk_npu_w4a8_workspace* ws) { workspace_destroy(ws); }

// ================================================================== blocking runs
extern "C" int rk_npu_w4a8_run_f32(rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w, const float* A, float* C,
                                   rk_npu_w4a8_timings* t)
{
    return run(ws, w, A, C, false, EPI_F32, t);
}
extern "C" int rk_npu_w4a8_run_f16(rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w, const uint16_t* A,
                                   uint16_t* C, rk_npu_w4a8_timings* t)
{
    return run(ws, w, A, C, true, EPI_F16, t);
}
extern "C" int rk_npu_w4a8_run_swiglu_f32(rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w, const float* A,
                                          float* middle, rk_npu_w4a8_timings* t)
{
    return run(ws, w, A, middle, false, EPI_SWIGLU, t);
}
extern "C" int rk_npu_b200_w4a8_run_acc_i32(rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w, const void* A,
                                            int activation_is_f16, int32_t* acc)
{
    return run(ws, w, A, acc, activation_is_f16 != 0, EPI_I32, nullptr);
}

extern "C" int rk_npu_w4a8_run_ffn_f32(rk_npu_w4a8_workspace* gate_up, const rk_npu_w4a8_weights* gate_up_weights,
                                       rk_npu_w4a8_workspace* down, const rk_npu_w4a8_weights* down_weights,
                                       const float* A, float* middle, float* C, rk_npu_w4a8_ffn_timings* metrics)
{
    if (metrics) *metrics = {};
    if (gate_up == down || middle == C || A == C) return RK_NPU_ERR_PARAM;
    int rc = validate(gate_up, gate_up_weights, A, middle, true);
    if (rc) return rc;
    rc = validate(down, down_weights, middle, C, false);
    if (rc) return rc;
    if (gate_up->config.M != down->config.M || gate_up->config.N / 2 != down->config.K) return RK_NPU_ERR_PARAM;
    if (gate_up->ctx_id != down->ctx_id || gate_up->domain_id != down->domain_id) return RK_NPU_ERR_DOMAIN;
    WorkspaceLock gate_lock(*gate_up);
    if (!gate_lock) return RK_NPU_ERR_BUSY;
    WorkspaceLock down_lock(*down);
    if (!down_lock) return RK_NPU_ERR_BUSY;
    try {
        const auto begin = Clock::now();
        rk_npu_w4a8_ffn_timings t{};
        const int M = gate_up->config.M, K = gate_up->config.K, F = gate_up->config.N / 2, N = down->config.N;
        if (cudaSetDevice(gate_up->domain->ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
        cudaStream_t s = gate_up->stream;
        const bool a_dev = on_device(A), m_dev = on_device(middle), c_dev = on_device(C);
        const void* dA = A;
        float* dMiddle = m_dev ? middle : static_cast<float*>(gate_up->stage_out);
        float* dC = c_dev ? C : static_cast<float*>(down->stage_out);
        auto mark = Clock::now();
        if (!a_dev) {
            if (cudaMemcpyAsync(gate_up->stage_in, A, size_t(M) * K * 4, cudaMemcpyHostToDevice, s) != cudaSuccess)
                return RK_NPU_ERR_SUBMIT;
            dA = gate_up->stage_in;
        }
        t.gate_up.sync_us += elapsed_us(mark);
        cudaEvent_t* ev = metrics ? gate_up->events : nullptr;
        Call first{gate_up, gate_up_weights, dA, dMiddle, false, EPI_SWIGLU, gate_up->rowmax, nullptr, s, ev};
        rc = enqueue_linear(first, dMiddle);
        // in a group every GPU has collected the maxima of its feature slice: the row maximum is their maximum
        if (!rc && grouped(*gate_up)) rc = group_all_reduce_max_u32(gate_up->domain->ctx, gate_up->rowmax, size_t(M), s);
        if (!rc) {
            // Down quantises `middle` with scales finished from the collected row maxima:
            // no rescan (src/rk_npu_w4a8.cpp:112-121,376); a non-finite maximum makes the
            // down kernels return without work.
            Call second{down, down_weights, dMiddle, dC, false, EPI_F32, nullptr, gate_up->rowmax, s, metrics ? down->events : nullptr};
            rc = enqueue_linear(second, dC);
        }
        if (rc) { cudaStreamSynchronize(s); return rc; }
        mark = Clock::now();
        if (!m_dev) cudaMemcpyAsync(middle, dMiddle, size_t(M) * F * 4, cudaMemcpyDeviceToHost, s);
        if (!c_dev) cudaMemcpyAsync(C, dC, size_t(M) * N * 4, cudaMemcpyDeviceToHost, s);
        cudaMemcpyAsync(gate_up->host_status, gate_up->status, sizeof(Status), cudaMemcpyDeviceToHost, s);
        cudaMemcpyAsync(down->host_status, down->status, sizeof(Status), cudaMemcpyDeviceToHost, s);
        if (cudaStreamSynchronize(s) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
        t.down.sync_us += elapsed_us(mark);
        rc = status_to_rc(*gate_up, s);
        const int rc_down = status_to_rc(*down, s);
        if (!rc) rc = rc_down;
        if (metrics) {
            t.gate_up.activation_scan_us = event_us(gate_up->events[0], gate_up->events[1]);
            t.gate_up.submit_us = event_us(gate_up->events[1], gate_up->events[2]);
            t.gate_up.total_us = event_us(gate_up->events[0], gate_up->events[2]);
            t.down.quant_pack_us = event_us(down->events[0], down->events[1]);
            t.down.submit_us = rc_down ? 0.0 : event_us(down->events[1], down->events[2]);
            t.down.total_us = event_us(down->events[0], down->events[2]);
            t.total_us = elapsed_us(begin);
            *metrics = t;
        }
        return rc;
    } catch (...) { return RK_NPU_ERR_PARAM; }
}

// ================================================================== enqueue forms
namespace {
int enqueue_public(rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w, const void* dA, void* dC, bool half, int epi,
                   void* stream)
{
    const int rc = validate(ws, w, dA, dC, epi == EPI_SWIGLU);
    if (rc) return rc;
    WorkspaceLock lock(*ws);
    if (!lock) return RK_NPU_ERR_BUSY;
    Call call{ws, w, dA, dC, half, epi, nullptr, nullptr, static_cast<cudaStream_t>(stream), nullptr};
    return enqueue_linear(call, dC);
}
}
extern "C" int rk_npu_b200_w4a8_enqueue_f32(rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w, const float* dA,
                                            float* dC, void* stream)
{
    return enqueue_public(ws, w, dA, dC, false, EPI_F32, stream);
}
extern "C" int rk_npu_b200_w4a8_enqueue_f16(rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w, const uint16_t* dA,
                                            uint16_t* dC, void* stream)
{
    return enqueue_public(ws, w, dA, dC, true, EPI_F16, stream);
}
// ---- several independent linears in one launch
extern "C" int rk_npu_b200_w4a8_enqueue_batch_f16(int count, rk_npu_w4a8_workspace* const* workspaces,
                                                  const rk_npu_w4a8_weights* const* weights, const uint16_t* const* dA,
                                                  uint16_t* const* dLocal, void* stream)
{
    if (count < 1 || count > DEC_MAX_BATCH || !workspaces || !weights || !dA || !dLocal) return RK_NPU_ERR_PARAM;
    for (int i = 0; i < count; ++i) {
        const int rc = validate(workspaces[i], weights[i], dA[i], dLocal[i], false);
        if (rc) return rc;
        for (int j = 0; j < i; ++j)
            if (workspaces[j] == workspaces[i] || dLocal[j] == dLocal[i]) return RK_NPU_ERR_PARAM;
        const auto* ws = workspaces[i];
        if (ws->variant != 5 || ws->config.M != workspaces[0]->config.M || ws->ctx_id != workspaces[0]->ctx_id) return RK_NPU_ERR_PARAM;
    }
    // one cluster size for the launch: the one the longest reduction asks for
    int cluster = 1;
    for (int i = 0; i < count; ++i) cluster = std::max(cluster, gemm_decode_cluster(workspaces[i]->config.M, workspaces[i]->KB));
    std::unique_ptr<WorkspaceLock> locks[DEC_MAX_BATCH];
    for (int i = 0; i < count; ++i) {
        locks[i].reset(new WorkspaceLock(*workspaces[i]));
        if (!*locks[i]) return RK_NPU_ERR_BUSY;
    }
    if (cudaSetDevice(workspaces[0]->domain->ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    DecodeBatch batch{};
    batch.count = count;
    batch.first_cta[0] = 0;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    for (int i = 0; i < count; ++i) {
        Call call{workspaces[i], weights[i], dA[i], dLocal[i], true, EPI_F16, nullptr, nullptr, s, nullptr};
        decode_params(call, batch.p[i], cluster);
        batch.p[i].trace = nullptr;
        batch.first_cta[i + 1] = batch.first_cta[i] + batch.p[i].ctas;
    }
    if (launch_gemm_decode_batch(batch, s, env_flag("RK_NPU_B200_PDL", true)) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
    workspaces[0]->launches.fetch_add(1, std::memory_order_relaxed);
    return RK_NPU_OK;
}

// ---- group of GPUs without the exchange: this rank's columns only, compact [M][columns]
extern "C" int rk_npu_b200_w4a8_workspace_shard(const rk_npu_w4a8_workspace* ws, int* two_range, int* n0, int* n1, int* columns)
{
    if (!ws) return RK_NPU_ERR_PARAM;
    if (two_range) *two_range = ws->shard.two_range ? 1 : 0;
    if (n0) *n0 = ws->shard.n0;
    if (n1) *n1 = ws->shard.n1;
    if (columns) *columns = ws->shard_N;
    return RK_NPU_OK;
}
namespace {
int enqueue_local(rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w, const void* dA, void* dLocal, bool half, int epi, void* stream)
{
    const int rc = validate(ws, w, dA, dLocal, false);
    if (rc) return rc;
    WorkspaceLock lock(*ws);
    if (!lock) return RK_NPU_ERR_BUSY;
    Call call{ws, w, dA, dLocal, half, epi, nullptr, nullptr, static_cast<cudaStream_t>(stream), nullptr};
    return enqueue(call);
}
}
extern "C" int rk_npu_b200_w4a8_enqueue_local_f16(rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w, const uint16_t* dA,
                                                  uint16_t* dLocal, void* stream)
{
    return enqueue_local(ws, w, dA, dLocal, true, EPI_F16, stream);
}
extern "C" int rk_npu_b200_w4a8_enqueue_local_f32(rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w, const float* dA,
                                                  float* dLocal, void* stream)
{
    return enqueue_local(ws, w, dA, dLocal, false, EPI_F32, stream);
}
extern "C" int rk_npu_b200_group_all_gather(rk_npu_ctx* ctx, void* dBuffer, size_t bytes_per_rank, void* stream)
{
    if (!ctx || !dBuffer || !bytes_per_rank || ctx->world < 2) return RK_NPU_ERR_PARAM;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    return group_all_gather(ctx, dBuffer, bytes_per_rank, static_cast<cudaStream_t>(stream));
}

extern "C" int rk_npu_b200_w4a8_enqueue_swiglu_f32(rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w,
                                                   const float* dA, float* dMiddle, void* stream)
{
    return enqueue_public(ws, w, dA, dMiddle, false, EPI_SWIGLU, stream);
}
extern "C" int rk_npu_b200_w4a8_enqueue_ffn_f32(rk_npu_w4a8_workspace* gate_up, const rk_npu_w4a8_weights* gate_up_weights,
                                                rk_npu_w4a8_workspace* down, const rk_npu_w4a8_weights* down_weights,
                                                const float* dA, float* dMiddle, float* dC, void* stream)
{
    if (!gate_up || !down || gate_up == down || !dC || (dMiddle && dMiddle == dC) || dA == dC) return RK_NPU_ERR_PARAM;
    // In a group a NULL dMiddle says the caller does not need the middle tensor: the GPUs then exchange int8 codes
    // (a quarter of the fp32 middle's bytes) instead of gathering it.
    const bool codes_only = dMiddle == nullptr;
    if (codes_only && !(grouped(*gate_up) && down->code_gather && gate_up->config.N / 2 == down->config.K &&
                        (down->config.K / 64) % gate_up->domain->ctx->world == 0 && down->config.K % 64 == 0))
        return RK_NPU_ERR_PARAM;
    float* local_middle = codes_only ? static_cast<float*>(own_slot(*gate_up)) : dMiddle;
    int rc = validate(gate_up, gate_up_weights, dA, local_middle, true);
    if (rc) return rc;
    rc = validate(down, down_weights, local_middle, dC, false);
    if (rc) return rc;
    if (gate_up->config.M != down->config.M || gate_up->config.N / 2 != down->config.K) return RK_NPU_ERR_PARAM;
    if (gate_up->ctx_id != down->ctx_id || gate_up->domain_id != down->domain_id) return RK_NPU_ERR_DOMAIN;
    WorkspaceLock gate_lock(*gate_up);
    if (!gate_lock) return RK_NPU_ERR_BUSY;
    WorkspaceLock down_lock(*down);
    if (!down_lock) return RK_NPU_ERR_BUSY;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int M = gate_up->config.M;
    if (codes_only) {
        rk_npu_ctx* ctx = gate_up->domain->ctx;
        const int slice = gate_up->shard.n1 - gate_up->shard.n0;          // features of this GPU
        Call first{gate_up, gate_up_weights, dA, local_middle, false, EPI_SWIGLU, gate_up->rowmax, nullptr, s, nullptr};
        rc = enqueue(first);                                              // middle slice stays local
        if (!rc) rc = group_all_reduce_max_u32(ctx, gate_up->rowmax, size_t(M), s);
        if (rc) return rc;
        const size_t piece = size_t(M) * slice;                            // int8 codes of one GPU's slice
        SliceQuantParams q{local_middle, reinterpret_cast<int8_t*>(down->code_gather) + size_t(ctx->rank) * piece, gate_up->rowmax, M, slice};
        if (launch_quantize_slice(q, s) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
        gate_up->launches.fetch_add(1, std::memory_order_relaxed);
        rc = group_all_gather(ctx, down->code_gather, piece, s);
        if (rc) return rc;
        Call second{down, down_weights, nullptr, dC, false, EPI_F32, nullptr, gate_up->rowmax, s, nullptr};
        second.codes_in = reinterpret_cast<const int8_t*>(down->code_gather);
        second.parts = ctx->world;
        return enqueue_linear(second, dC);
    }
    Call first{gate_up, gate_up_weights, dA, dMiddle, false, EPI_SWIGLU, gate_up->rowmax, nullptr, s, nullptr};
    rc = enqueue_linear(first, dMiddle);
    if (!rc && grouped(*gate_up)) rc = group_all_reduce_max_u32(gate_up->domain->ctx, gate_up->rowmax, size_t(M), s);
    if (rc) return rc;
    Call second{down, down_weights, dMiddle, dC, false, EPI_F32, nullptr, gate_up->rowmax, s, nullptr};
    return enqueue_linear(second, dC);
}

// ---- column-sharded FFN: the pieces around the exchange between GPUs
extern "C" int rk_npu_b200_w4a8_enqueue_swiglu_collect_f32(rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w,
                                                           const float* dA, float* dMiddle, uint32_t* dRowMaxima, void* stream)
{
    if (!dRowMaxima) return RK_NPU_ERR_PARAM;
    const int rc = validate(ws, w, dA, dMiddle, true);
    if (rc) return rc;
    if (grouped(*ws)) return RK_NPU_ERR_PARAM;   // a group context shards by itself; these pieces are for callers that shard by hand
    WorkspaceLock lock(*ws);
    if (!lock) return RK_NPU_ERR_BUSY;
    Call call{ws, w, dA, dMiddle, false, EPI_SWIGLU, dRowMaxima, nullptr, static_cast<cudaStream_t>(stream), nullptr};
    return enqueue(call);
}
extern "C" int rk_npu_b200_w4a8_enqueue_quantize_slice(rk_npu_w4a8_workspace* gate_up, const float* dMiddle,
                                                       const uint32_t* dRowMaxima, int8_t* dCodes, void* stream)
{
    if (!gate_up || !dMiddle || !dRowMaxima || !dCodes || gate_up->config.N % 2 || grouped(*gate_up)) return RK_NPU_ERR_PARAM;
    WorkspaceLock lock(*gate_up);
    if (!lock) return RK_NPU_ERR_BUSY;
    if (cudaSetDevice(gate_up->domain->ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    SliceQuantParams q{dMiddle, dCodes, dRowMaxima, gate_up->config.M, gate_up->config.N / 2};
    if (launch_quantize_slice(q, static_cast<cudaStream_t>(stream)) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
    gate_up->launches.fetch_add(1, std::memory_order_relaxed);
    return RK_NPU_OK;
}
extern "C" int rk_npu_b200_w4a8_enqueue_codes_f32(rk_npu_w4a8_workspace* down, const rk_npu_w4a8_weights* w,
                                                  const int8_t* dCodes, int parts, uint32_t* dRowMaxima, float* dC, void* stream)
{
    if (!dRowMaxima) return RK_NPU_ERR_PARAM;
    const int rc = validate(down, w, dCodes, dC, false);
    if (rc) return rc;
    const int K = down->config.K;
    if (parts < 1 || K % parts || (parts > 1 && (K / parts) % 16) || grouped(*down)) return RK_NPU_ERR_PARAM;
    WorkspaceLock lock(*down);
    if (!lock) return RK_NPU_ERR_BUSY;
    Call call{down, w, nullptr, dC, false, EPI_F32, nullptr, dRowMaxima, static_cast<cudaStream_t>(stream), nullptr};
    call.codes_in = dCodes;
    call.parts = parts;
    return enqueue(call);
}

extern "C" int rk_npu_b200_w4a8_finish(rk_npu_w4a8_workspace* ws)
{
    if (!ws) return RK_NPU_ERR_PARAM;
    WorkspaceLock lock(*ws);
    if (!lock) return RK_NPU_ERR_BUSY;
    if (cudaSetDevice(ws->domain->ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    if (cudaMemcpy(ws->host_status, ws->status, sizeof(Status), cudaMemcpyDeviceToHost) != cudaSuccess) {
        cudaGetLastError();
        return RK_NPU_ERR_SUBMIT;
    }
    return status_to_rc(*ws, ws->stream);
}

extern "C" int rk_npu_b200_w4a8_last_quant(rk_npu_w4a8_workspace* ws, float* scales, int8_t* codes)
{
    if (!ws) return RK_NPU_ERR_PARAM;
    WorkspaceLock lock(*ws);
    if (!lock) return RK_NPU_ERR_BUSY;
    if (cudaSetDevice(ws->domain->ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    const int M = ws->config.M, K = ws->config.K, T = ws->T;
    if (scales && cudaMemcpy(scales, ws->scales, sizeof(float) * M, cudaMemcpyDeviceToHost) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    if (codes) {
        std::vector<uint8_t> raw(ws->codes_bytes);
        if (cudaMemcpy(raw.data(), ws->codes, ws->codes_bytes, cudaMemcpyDeviceToHost) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
        const size_t chunks = size_t(ws->KB) * 8;
        for (int m = 0; m < M; ++m)
            for (int k = 0; k < K; ++k)
                codes[size_t(m) * K + k] = int8_t(raw[((size_t(m / T) * chunks + k / 16) * T + m % T) * 16 + k % 16]);
    }
    return RK_NPU_OK;
}

extern "C" int rk_npu_b200_w4a8_set_schedule(rk_npu_w4a8_workspace* ws, int variant, int split_k)
{
    if (!ws || variant < 0 || variant > 5 || split_k < 0 || split_k > 8) return RK_NPU_ERR_PARAM;
    int target = variant ? variant : ws->variant;
    if (target != ws->variant) {
        // The code layout is fixed at creation.  The two single-kernel families for up to eight tokens share it
        // (eight-token code tiles), so a workspace may move between them where the geometry allows both.
        const bool single = (ws->variant == 3 || ws->variant == 5) && ws->config.M <= 8;
        const bool to_decode = target == 5 && gemm_decode_supported(ws->config.M, ws->config.K) && ws->decode_cap[0] > 0;
        const bool to_split = target == 3 && ws->KB <= 8 * FUSED_MAX_STAGES;
        if (!single || !(to_decode || to_split)) return RK_NPU_ERR_PARAM;
    }
    if (target != 3 && split_k != 0 && split_k != 1 && split_k != 2 && split_k != 4 && split_k != 8) return RK_NPU_ERR_PARAM;
    if (target == 3 && split_k && (ws->KB + split_k - 1) / split_k > FUSED_MAX_STAGES) return RK_NPU_ERR_PARAM;
    WorkspaceLock lock(*ws);
    if (!lock) return RK_NPU_ERR_BUSY;
    ws->variant = target;
    ws->split_override = split_k;
    return RK_NPU_OK;
}
extern "C" int rk_npu_b200_w4a8_schedule(const rk_npu_w4a8_workspace* ws, int* variant, int* split_k)
{
    if (!ws) return RK_NPU_ERR_PARAM;
    if (variant) *variant = ws->variant;
    if (split_k) *split_k = ws->split_override;
    return RK_NPU_OK;
}
extern "C" int rk_npu_b200_w4a8_test_starve(rk_npu_w4a8_workspace* ws, int on)
{
    if (!ws || ws->variant != 5) return RK_NPU_ERR_PARAM;
    WorkspaceLock lock(*ws);
    if (!lock) return RK_NPU_ERR_BUSY;
    ws->starve = on != 0;
    return RK_NPU_OK;
}
extern "C" int rk_npu_b200_w4a8_test_device_error(rk_npu_w4a8_workspace* ws)
{
    if (!ws) return RK_NPU_ERR_PARAM;
    WorkspaceLock lock(*ws);
    if (!lock) return RK_NPU_ERR_BUSY;
    if (cudaSetDevice(ws->domain->ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    const int one = 1;
    return cudaMemcpy(&ws->status->device_error, &one, sizeof(int), cudaMemcpyHostToDevice) == cudaSuccess ? RK_NPU_OK : RK_NPU_ERR_SUBMIT;
}
extern "C" uint64_t rk_npu_b200_w4a8_launch_count(const rk_npu_w4a8_workspace* ws)
{
    return ws ? ws->launches.load(std::memory_order_relaxed) : 0;
}

// ================================================================== phase stamps (diagnostics)
extern "C" int rk_npu_b200_w4a8_trace_enable(rk_npu_w4a8_workspace* ws, int enable)
{
    if (!ws) return RK_NPU_ERR_PARAM;
    WorkspaceLock lock(*ws);
    if (!lock) return RK_NPU_ERR_BUSY;
    if (cudaSetDevice(ws->domain->ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    if (enable && !ws->trace) {
        ws->trace_bytes = size_t(1) << 20;
        if (device_alloc(ws->domain, reinterpret_cast<void**>(&ws->trace), ws->trace_bytes)) return RK_NPU_ERR_NOMEM;
        cudaMemset(ws->trace, 0, ws->trace_bytes);
    } else if (!enable && ws->trace) {
        cudaStreamSynchronize(ws->stream);
        device_free(ws->domain, ws->trace, ws->trace_bytes);
        ws->trace = nullptr;
    }
    return RK_NPU_OK;
}
extern "C" int rk_npu_b200_w4a8_trace_read(rk_npu_w4a8_workspace* ws, unsigned long long* stamps, int ctas)
{
    if (!ws || !stamps || ctas < 1 || !ws->trace || size_t(ctas) * 64 > ws->trace_bytes) return RK_NPU_ERR_PARAM;
    if (cudaSetDevice(ws->domain->ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    return cudaMemcpy(stamps, ws->trace, size_t(ctas) * 64, cudaMemcpyDeviceToHost) == cudaSuccess ? RK_NPU_OK : RK_NPU_ERR_SUBMIT;
}
