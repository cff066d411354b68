// moe_abi.cpp -- the routed-experts operator of the original's include/rk_npu_moe_w8.h on this library: immutable expert
// weight objects (int8, int4, or int4 routed experts with an int8 shared one), mutable slot banks of int4 experts with
// the cache records they import and export, workspaces, the two blocking run calls.
//
// The original (src/rk_npu_moe_w8.cpp:570-817) quantises the input rows on the CPU, groups the (token, slot)
// assignments by expert, gathers and multiplies on the NPU, runs the middle stage and the weighted combine on the
// CPU.  Here the host only validates and groups (the ids and coefficients are host arrays); quantisation, both
// projections, the middle stage and the combine are four launches on the workspace's stream (moe_kernels.cu).
// Validation order and return codes follow the original's moe_run (src/rk_npu_moe_w8.cpp:845-875) and
// Workspace::run (:582-595).
#include "w4a8_host.h"
#include "moe_device.h"
#include "../../include/rknpu_b200_moe.h"
#include <algorithm>
#include <chrono>
#include <cmath>
#include <cstring>
#include <memory>
#include <mutex>
#include <new>
#include <vector>

using namespace rkb200;

namespace {
using Clock = std::chrono::steady_clock;
double since_us(Clock::time_point t) { return std::chrono::duration<double, std::micro>(Clock::now() - t).count(); }
constexpr int MOE_HIDDEN_MAX = 8192;   // 16 gathered rows of codes must fit one CTA's shared memory

bool valid_weights(const rk_npu_moe_w8_weight_config& c)   // src/rk_npu_moe_w8.cpp:293-298
{
    return c.hidden >= 64 && c.hidden % 32 == 0 && c.hidden <= MOE_HIDDEN_MAX && c.intermediate >= 32 && c.intermediate <= 512 &&
           c.intermediate % 32 == 0 && c.routed_experts >= 1 && (c.shared_expert == 0 || c.shared_expert == 1);
}
bool same_weights(const rk_npu_moe_w8_weight_config& a, const rk_npu_moe_w8_weight_config& b)
{
    return a.hidden == b.hidden && a.intermediate == b.intermediate && a.routed_experts == b.routed_experts &&
           a.shared_expert == b.shared_expert;
}
bool valid_config(const rk_npu_moe_w8_config& c)           // src/rk_npu_moe_w8.cpp:303-310; the table-lookup middle is not built
{
    return c.struct_size == sizeof(c) && valid_weights(c.weights) && c.max_rows >= 1 && c.max_rows <= 256 && c.top_k >= 1 &&
           c.top_k <= std::min(c.weights.routed_experts, 8) && c.npu_cores >= 1 && c.npu_cores <= 3 && c.cpu_threads >= 1 &&
           c.cpu_threads <= 4 && (c.native_input == 0 || c.native_input == 1) && c.timeout_ms >= 1 && c.timeout_ms <= 60000 &&
           c.middle == RK_NPU_MOE_MIDDLE_CPU;
}
// src/rk_npu_moe_w8.cpp:368-389: which experts hold int4 codes.  Int4 experts are checked like the dense W4A8 weights
// (codes in [-8, 7]; the K tile the original would run must be certified against its INT16 partial sums) and then
// stored two codes per byte; the sums are the same integers as with int8 storage.
enum class Mode { W8 = 0, RoutedW4SharedW8 = 1, W4 = 2 };
bool expert_is_w4(Mode mode, int expert, int routed) { return mode == Mode::W4 || (mode == Mode::RoutedW4SharedW8 && expert < routed); }
bool can_use_full_gate(int hidden) { return hidden > 512 && hidden <= 2048; }
// Cache records (src/rk_npu_moe_w8.cpp:383): the last 32-bit word of a record carries, in its low three bits, whether
// the original device would run the gate/up projection over the whole of K or in slices.  Nothing here depends on it
// (the sums are exact either way); it is kept, checked and handed on so that a record says what it was certified for.
constexpr int32_t record_tag_mask = 7, record_sliced = 1, record_full_k = 2;
constexpr uint32_t record_magic = 0x34424b52u;      // "RKB4": an int4 expert in this library's record layout
struct RecordTrailer {                               // the last 16 bytes of a record
    uint32_t magic;
    int32_t hidden, intermediate;
    int32_t tag;
};
bool valid_w4(const rk_npu_moe_w8_weight_config& c)
{
    return valid_weights(c) && c.hidden % 64 == 0 && c.intermediate % 64 == 0 && c.hidden <= 8128;
}
bool finite_positive(float x) { return std::isfinite(x) && x > 0.0f; }
bool overlap(const void* a, size_t na, const void* b, size_t nb)
{
    const auto x = reinterpret_cast<uintptr_t>(a), y = reinterpret_cast<uintptr_t>(b);
    return x <= y ? y - x < na : x - y < nb;
}
float event_us(cudaEvent_t a, cudaEvent_t b)
{
    float ms = 0;
    if (cudaEventElapsedTime(&ms, a, b) != cudaSuccess) { cudaGetLastError(); return 0; }
    return ms * 1000.f;
}
} // namespace

struct rk_npu_moe_w8_weights {
    rk_npu_iommu_domain* domain = nullptr;
    uint64_t ctx_id = 0;
    uint32_t domain_id = 0;
    rk_npu_moe_w8_weight_config config{};
    Mode mode = Mode::W8;
    uint8_t* gate_up = nullptr;   // [E] records of the [H, 2I] matrices: the int4 experts first (two codes per byte), then int8
    uint8_t* down = nullptr;      // [E] records of the [I, H] matrices
    float* gate_up_scales = nullptr, *down_scales = nullptr;
    int nibble_experts = 0;
    MoeBank gate_up_bank() const { return MoeBank{gate_up, moe_packed_nibble_bytes(config.hidden, 2 * config.intermediate), moe_packed_bytes(config.hidden, 2 * config.intermediate), nibble_experts}; }
    MoeBank down_bank() const { return MoeBank{down, moe_packed_nibble_bytes(config.intermediate, config.hidden), moe_packed_bytes(config.intermediate, config.hidden), nibble_experts}; }
    size_t gate_up_bytes = 0, down_bytes = 0, gate_up_scale_bytes = 0, down_scale_bytes = 0;
    std::vector<int32_t> tags;    // per int4 expert: record_sliced or record_full_k
    // A slot bank (rk_npu_moe_*_slots_create) keeps every expert in an allocation of its own, laid out like a cache
    // record: [gate/up records | down records | gate/up scales | down scales].  Slots change hands between banks by
    // exchanging these structs; the four arrays above stay null.
    struct Slot {
        uint8_t* storage = nullptr;
        size_t bytes = 0;
    };
    bool slotted = false;
    std::vector<Slot> slots;
    cudaStream_t stream = nullptr;   // imports and exports
    std::mutex transfer;             // one of them at a time on `stream`
    int experts() const { return config.routed_experts + config.shared_expert; }
    size_t gate_up_record_bytes(int e) const { return e < nibble_experts ? moe_packed_nibble_bytes(config.hidden, 2 * config.intermediate) : moe_packed_bytes(config.hidden, 2 * config.intermediate); }
    size_t down_record_bytes(int e) const { return e < nibble_experts ? moe_packed_nibble_bytes(config.intermediate, config.hidden) : moe_packed_bytes(config.intermediate, config.hidden); }
    size_t slot_bytes(int e) const { return gate_up_record_bytes(e) + down_record_bytes(e) + sizeof(float) * (2 * size_t(config.intermediate) + size_t(config.hidden)); }
    // where expert e's four pieces are, in either representation
    uint8_t* gate_up_at(int e) const { return slotted ? slots[e].storage : const_cast<uint8_t*>(gate_up_bank().expert(e)); }
    uint8_t* down_at(int e) const { return slotted ? slots[e].storage + gate_up_record_bytes(e) : const_cast<uint8_t*>(down_bank().expert(e)); }
    float* gate_up_scales_at(int e) const
    {
        return slotted ? reinterpret_cast<float*>(slots[e].storage + gate_up_record_bytes(e) + down_record_bytes(e))
                       : gate_up_scales + size_t(e) * 2 * config.intermediate;
    }
    float* down_scales_at(int e) const { return slotted ? gate_up_scales_at(e) + 2 * config.intermediate : down_scales + size_t(e) * config.hidden; }
    uint64_t record_bytes() const      // one int4 expert as a cache record; 0 for banks without int4 experts
    {
        return nibble_experts ? uint64_t(slot_bytes(0) + sizeof(RecordTrailer)) : 0;
    }
};

struct rk_npu_moe_w8_workspace {
    rk_npu_iommu_domain* domain = nullptr;
    uint64_t ctx_id = 0;
    uint32_t domain_id = 0;
    rk_npu_moe_w8_config config{};
    Mode mode = Mode::W8;
    std::atomic_flag busy = ATOMIC_FLAG_INIT;
    cudaStream_t stream = nullptr;
    cudaEvent_t events[5] = {};
    int slots = 0, assignments_max = 0;
    int8_t* codes = nullptr;       // [max_rows][H] codes made by the quantise kernel (run_f32)
    float* in_scales = nullptr;    // [max_rows] and their scales
    float* middle = nullptr;       // [assignments][I]
    uint32_t* row_max = nullptr;   // [assignments]
    float* expert_out = nullptr;   // [assignments][H]
    float* out = nullptr;          // [max_rows][H]
    uint8_t* upload = nullptr;     // one run's host arrays in one piece (see Upload)
    Status* status = nullptr;
    size_t codes_bytes = 0, in_scale_bytes = 0, middle_bytes = 0, row_max_bytes = 0, expert_out_bytes = 0, out_bytes = 0,
           upload_bytes = 0;
    uint8_t* host_upload = nullptr;   // pinned mirror of `upload`
    Status* host_status = nullptr; // pinned; the quantise kernel reports into it through its device alias
    Status* host_status_alias = nullptr;
    float* host_out = nullptr;     // pinned landing place of small results, written by the combine kernel through its alias
    float* host_out_alias = nullptr;
    size_t host_out_bytes = 0;
    std::vector<std::vector<int>> groups;   // per expert: token * slots + slot of its assignments
};

namespace {
void weights_destroy(rk_npu_moe_w8_weights* w)
{
    if (!w) return;
    auto* d = w->domain;
    if (d) {
        cudaSetDevice(d->ctx->device);
        if (w->gate_up) device_free(d, w->gate_up, w->gate_up_bytes);
        if (w->down) device_free(d, w->down, w->down_bytes);
        if (w->gate_up_scales) device_free(d, w->gate_up_scales, w->gate_up_scale_bytes);
        if (w->down_scales) device_free(d, w->down_scales, w->down_scale_bytes);
        for (auto& slot : w->slots)
            if (slot.storage) device_free(d, slot.storage, slot.bytes);
        if (w->stream) { cudaStreamSynchronize(w->stream); cudaStreamDestroy(w->stream); }
        domain_release(d);
    }
    delete w;
}

void workspace_destroy(rk_npu_moe_w8_workspace* ws)
{
    if (!ws) return;
    auto* d = ws->domain;
    if (d) cudaSetDevice(d->ctx->device);
    if (ws->stream) cudaStreamSynchronize(ws->stream);
    if (ws->codes) device_free(d, ws->codes, ws->codes_bytes);
    if (ws->in_scales) device_free(d, ws->in_scales, ws->in_scale_bytes);
    if (ws->middle) device_free(d, ws->middle, ws->middle_bytes);
    if (ws->row_max) device_free(d, ws->row_max, ws->row_max_bytes);
    if (ws->expert_out) device_free(d, ws->expert_out, ws->expert_out_bytes);
    if (ws->out) device_free(d, ws->out, ws->out_bytes);
    if (ws->upload) device_free(d, ws->upload, ws->upload_bytes);
    if (ws->status) device_free(d, ws->status, sizeof(Status));
    if (ws->host_upload) cudaFreeHost(ws->host_upload);
    if (ws->host_status) cudaFreeHost(ws->host_status);
    if (ws->host_out) cudaFreeHost(ws->host_out);
    for (auto& e : ws->events)
        if (e) cudaEventDestroy(e);
    if (ws->stream) cudaStreamDestroy(ws->stream);
    if (d) domain_release(d);
    delete ws;
}

struct Lock {
    explicit Lock(rk_npu_moe_w8_workspace& ws) : flag(ws.busy), held(!flag.test_and_set(std::memory_order_acquire)) {}
    ~Lock() { if (held) flag.clear(std::memory_order_release); }
    std::atomic_flag& flag;
    bool held;
};

// What one run sends to the device, packed into one page-locked piece so that it travels as ONE copy: the
// schedule (jobs and assignments, grouped by expert), each token's slots, the coefficients, and the input rows
// (int8 codes with their scales, or fp32 rows).  Offsets in bytes from the start of the piece.
struct Upload {
    size_t job_expert, job_first, job_rows, assign_token, slot_assign, coefficients, scales, rows_data, bytes;
    int jobs, assignments;
};
size_t upload_capacity(int max_rows, int slots, int H, int experts)
{
    const size_t A = size_t(max_rows) * slots;
    return (4 * A + 2 * A + size_t(max_rows)) * 4 + 16 + size_t(max_rows) * H * 4 + 16 + 4 * sizeof(void*) * size_t(experts);   // + a slot bank's tables
}

// Groups the assignments by expert, cuts the groups into jobs of at most 16 and writes everything into the mirror.
Upload build_upload(rk_npu_moe_w8_workspace& ws, int rows, const void* input, bool f32, const float* scales, const int32_t* ids,
                    const float* routes)
{
    const auto& c = ws.config;
    const int R = c.weights.routed_experts, top = c.top_k, S = ws.slots, H = c.weights.hidden;
    for (auto& g : ws.groups) g.clear();
    int assignments = 0, jobs = 0;
    for (int r = 0; r < rows; ++r) {
        for (int slot = 0; slot < top; ++slot)
            if (routes[r * top + slot] != 0.0f) ws.groups[ids[r * top + slot]].push_back(r * S + slot);   // a zero coefficient leaves the route out
        if (c.weights.shared_expert) ws.groups[R].push_back(r * S + top);
    }
    for (const auto& g : ws.groups) { assignments += int(g.size()); jobs += int((g.size() + MOE_JOB_ROWS - 1) / MOE_JOB_ROWS); }
    Upload u{};
    u.jobs = jobs;
    u.assignments = assignments;
    u.job_expert = 0;
    u.job_first = u.job_expert + size_t(jobs) * 4;
    u.job_rows = u.job_first + size_t(jobs) * 4;
    u.assign_token = u.job_rows + size_t(jobs) * 4;
    u.slot_assign = u.assign_token + size_t(assignments) * 4;
    u.coefficients = u.slot_assign + size_t(rows) * S * 4;
    u.scales = u.coefficients + size_t(rows) * S * 4;
    u.rows_data = (u.scales + size_t(rows) * 4 + 15) / 16 * 16;
    u.bytes = u.rows_data + size_t(rows) * H * (f32 ? 4 : 1);
    uint8_t* base = ws.host_upload;
    int* job_expert = reinterpret_cast<int*>(base + u.job_expert), *job_first = reinterpret_cast<int*>(base + u.job_first);
    int* job_rows = reinterpret_cast<int*>(base + u.job_rows), *assign_token = reinterpret_cast<int*>(base + u.assign_token);
    int* slot_assign = reinterpret_cast<int*>(base + u.slot_assign);
    float* coefficients = reinterpret_cast<float*>(base + u.coefficients);
    std::fill(slot_assign, slot_assign + size_t(rows) * S, -1);
    int a = 0, j = 0;
    for (int e = 0; e < int(ws.groups.size()); ++e) {
        const auto& g = ws.groups[e];
        for (size_t first = 0; first < g.size(); first += MOE_JOB_ROWS, ++j) {
            const int n = int(std::min<size_t>(MOE_JOB_ROWS, g.size() - first));
            job_expert[j] = e;
            job_first[j] = a;
            job_rows[j] = n;
            for (int i = 0; i < n; ++i, ++a) {
                const int key = g[first + i];
                assign_token[a] = key / S;
                slot_assign[key] = a;
            }
        }
    }
    for (int r = 0; r < rows; ++r)
        for (int slot = 0; slot < S; ++slot) coefficients[r * S + slot] = slot < top ? routes[r * top + slot] : 1.0f;
    if (!f32) std::memcpy(base + u.scales, scales, size_t(rows) * 4);
    std::memcpy(base + u.rows_data, input, size_t(rows) * H * (f32 ? 4 : 1));
    return u;
}

int moe_run(rk_npu_moe_w8_workspace* ws, const rk_npu_moe_w8_weights* w, int rows, const void* input, bool f32, const float* scales,
            const int32_t* ids, const float* routes, float* output, rk_npu_moe_w8_timings* timings)
{
    if (timings) *timings = rk_npu_moe_w8_timings{};
    if (!ws || !w || !input || !ids || !routes || !output || (!f32 && !scales) || rows < 1 || rows > ws->config.max_rows)
        return RK_NPU_ERR_PARAM;
    const auto& c = ws->config;
    const int H = c.weights.hidden, I = c.weights.intermediate, R = c.weights.routed_experts, top = c.top_k, S = ws->slots;
    const size_t values = size_t(rows) * H, routed = size_t(rows) * top;
    if (overlap(input, values * (f32 ? 4 : 1), output, values * 4) || overlap(ids, routed * 4, output, values * 4) ||
        overlap(routes, routed * 4, output, values * 4) || (!f32 && overlap(scales, size_t(rows) * 4, output, values * 4)))
        return RK_NPU_ERR_PARAM;
    Lock lock(*ws);
    if (!lock.held) return RK_NPU_ERR_BUSY;
    const auto begin = Clock::now();
    if (ws->mode != w->mode || !same_weights(c.weights, w->config)) return RK_NPU_ERR_PARAM;
    if (w->ctx_id != ws->ctx_id || w->domain_id != ws->domain_id) return RK_NPU_ERR_DOMAIN;
    for (size_t i = 0; i < routed; ++i)
        if (ids[i] < 0 || ids[i] >= R || !std::isfinite(routes[i]) || routes[i] < 0.0f) return RK_NPU_ERR_PARAM;
    if (!f32)
        for (int r = 0; r < rows; ++r)
            if (!finite_positive(scales[r])) return RK_NPU_ERR_PARAM;
    if (cudaSetDevice(ws->domain->ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    cudaStream_t s = ws->stream;
    rk_npu_moe_w8_timings t{};
    try {
        // ---- the routes grouped by expert, the input rows: one piece, one copy
        auto at = Clock::now();
        Upload u = build_upload(*ws, rows, input, f32, scales, ids, routes);
        const int assignments = u.assignments, jobs = u.jobs;
        MoeBank gate_up_bank = w->gate_up_bank(), down_bank = w->down_bank();
        if (w->slotted) {      // where every expert lives right now travels with the run: records and scales of both projections
            const int E = w->experts();
            const size_t tables = (u.bytes + 15) / 16 * 16;
            const void** host = reinterpret_cast<const void**>(ws->host_upload + tables);
            for (int e = 0; e < E; ++e) {
                host[e] = w->gate_up_at(e);
                host[E + e] = w->down_at(e);
                host[2 * E + e] = w->gate_up_scales_at(e);
                host[3 * E + e] = w->down_scales_at(e);
            }
            const uint8_t* device = ws->upload + tables;
            gate_up_bank.table = reinterpret_cast<const uint8_t* const*>(device);
            down_bank.table = reinterpret_cast<const uint8_t* const*>(device + sizeof(void*) * E);
            gate_up_bank.scale_table = reinterpret_cast<const float* const*>(device + 2 * sizeof(void*) * E);
            down_bank.scale_table = reinterpret_cast<const float* const*>(device + 3 * sizeof(void*) * E);
            u.bytes = tables + 4 * sizeof(void*) * E;
        }
        t.schedule_us = since_us(at);
        at = Clock::now();
        if (timings) cudaEventRecord(ws->events[0], s);
        bool ok = true;
        if (assignments || f32) ok = cudaMemcpyAsync(ws->upload, ws->host_upload, u.bytes, cudaMemcpyHostToDevice, s) == cudaSuccess;
        const int8_t* codes = reinterpret_cast<const int8_t*>(ws->upload + u.rows_data);
        const float* in_scales = reinterpret_cast<const float*>(ws->upload + u.scales);
        if (f32) {
            // the kernel's verdict lands in page-locked memory by itself: no copy, no second wait
            *ws->host_status = Status{};
            const MoeQuantParams q{reinterpret_cast<const float*>(ws->upload + u.rows_data), ws->codes, ws->in_scales, ws->host_status_alias, rows, H};
            ok = ok && launch_moe_quantize(q, s) == cudaSuccess;
            codes = ws->codes;
            in_scales = ws->in_scales;
        }
        if (!ok) { cudaGetLastError(); cudaStreamSynchronize(s); return RK_NPU_ERR_SUBMIT; }
        t.input_us = since_us(at);
        if (!assignments) {                    // nothing routed: the output is zero and no device work is issued for it
            if (f32) {                         // (the rows are still judged)
                if (cudaStreamSynchronize(s) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
                if (ws->host_status->bad_input) return RK_NPU_ERR_PARAM;
            }
            at = Clock::now();
            std::fill_n(output, values, 0.0f);
            t.combine_us = since_us(at);
            t.total_us = since_us(begin);
            if (timings) *timings = t;
            return RK_NPU_OK;
        }
        if (timings) cudaEventRecord(ws->events[1], s);
        // A small result is stored by the combine kernel straight into page-locked host memory and copied to the caller's
        // array by the host after the wait (a rejected call must not touch that array); a large one takes the copy engine.
        const bool direct = values * 4 <= ws->host_out_bytes;
        float* const landing = direct ? ws->host_out_alias : ws->out;
        const MoeSchedule sched{reinterpret_cast<const int*>(ws->upload + u.job_expert), reinterpret_cast<const int*>(ws->upload + u.job_first),
                                reinterpret_cast<const int*>(ws->upload + u.job_rows), reinterpret_cast<const int*>(ws->upload + u.assign_token), jobs};
        const MoeGateUpParams gu{sched, gate_up_bank, w->gate_up_scales, codes, in_scales, ws->middle, ws->row_max, H, I};
        ok = launch_moe_gate_up(gu, s) == cudaSuccess;
        if (timings) cudaEventRecord(ws->events[2], s);
        const MoeDownParams dn{sched, down_bank, w->down_scales, ws->middle, ws->row_max, ws->expert_out, H, I};
        ok = ok && launch_moe_down(dn, s) == cudaSuccess;
        if (timings) cudaEventRecord(ws->events[3], s);
        const MoeCombineParams cb{ws->expert_out, reinterpret_cast<const int*>(ws->upload + u.slot_assign),
                                  reinterpret_cast<const float*>(ws->upload + u.coefficients), landing, ws->row_max, rows, S, H};
        ok = ok && launch_moe_combine(cb, s) == cudaSuccess;
        if (timings) cudaEventRecord(ws->events[4], s);
        if (!ok) {      // a launch failed part-way: the row maxima may be left behind
            cudaGetLastError();
            cudaMemsetAsync(ws->row_max, 0, ws->row_max_bytes, s);
            cudaStreamSynchronize(s);
            return RK_NPU_ERR_SUBMIT;
        }
        at = Clock::now();
        if (!direct && !f32 && cudaMemcpyAsync(output, ws->out, values * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess) ok = false;
        if (!ok || cudaStreamSynchronize(s) != cudaSuccess) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
        if (f32 && ws->host_status->bad_input) return RK_NPU_ERR_PARAM;      // a rejected row: the output is not written
        if (direct) std::memcpy(output, ws->host_out, values * 4);
        else if (f32 && (cudaMemcpyAsync(output, ws->out, values * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
                         cudaStreamSynchronize(s) != cudaSuccess)) {
            cudaGetLastError();
            return RK_NPU_ERR_SUBMIT;
        }
        t.sync_us = since_us(at);
        if (timings) {
            t.input_us = event_us(ws->events[0], ws->events[1]);
            t.gate_us = event_us(ws->events[1], ws->events[2]);
            t.down_us = event_us(ws->events[2], ws->events[3]);
            t.combine_us = event_us(ws->events[3], ws->events[4]);
            t.gather_tasks = t.middle_tasks = uint32_t(assignments);
            t.gemm_tasks = uint32_t(2 * jobs);
            t.total_us = since_us(begin);
            *timings = t;
        }
        return RK_NPU_OK;
    } catch (const std::bad_alloc&) {
        return RK_NPU_ERR_NOMEM;
    } catch (...) {
        return RK_NPU_ERR_PARAM;
    }
}
} // namespace

// ================================================================== C ABI
extern "C" void rk_npu_moe_w8_config_init(rk_npu_moe_w8_config* c, int hidden, int intermediate, int routed_experts, int shared_expert,
                                          int top_k, int max_rows)
{
    // src/rk_npu_moe_w8.cpp:824-826: three cores, four threads, normal input, fp32 middle stage, one second
    if (c) *c = rk_npu_moe_w8_config{uint32_t(sizeof(*c)), {hidden, intermediate, routed_experts, shared_expert}, max_rows, top_k, 3, 4, 0,
                                     RK_NPU_MOE_MIDDLE_CPU, 1000};
}

namespace {
// src/rk_npu_moe_w8.cpp:453-474: one expert as the caller gives it.  Int4 experts: gate/up is certified over the whole
// of K where the original would try that (with its 512 slices as the fallback), else over slices of at most 512; down
// over the whole of K = intermediate.  `tag` says which gate/up certification held.
bool valid_expert(const rk_npu_moe_w8_expert& x, int H, int I, bool int4, bool try_full, int32_t& tag)
{
    tag = record_sliced;
    if (!x.gate_up || !x.down || !x.gate_up_scales || !x.down_scales) return false;
    for (int n = 0; n < 2 * I; ++n)
        if (!finite_positive(x.gate_up_scales[n])) return false;
    for (int n = 0; n < H; ++n)
        if (!finite_positive(x.down_scales[n])) return false;
    if (!int4) return true;
    WeightBound gate, down;
    const int slice = std::min(H, 512);
    try {
        if (bound_weights(H, 2 * I, x.gate_up, try_full ? H : slice, gate, try_full ? slice : 0) != RK_NPU_OK ||
            bound_weights(I, H, x.down, I, down) != RK_NPU_OK)
            return false;
    } catch (...) { return false; }
    if (try_full && gate.k_tile > slice) tag = record_full_k;
    return true;
}

// Uploads one expert's matrices through `raw` (room for both), packs them into records and copies its scales.
bool place_expert(const rk_npu_moe_w8_weights& w, int e, const rk_npu_moe_w8_expert& x, int8_t* raw, cudaStream_t s)
{
    const int H = w.config.hidden, I = w.config.intermediate;
    const size_t gu_raw = size_t(H) * 2 * I, dn_raw = size_t(I) * H;
    const bool nib = e < w.nibble_experts;
    return cudaMemcpyAsync(raw, x.gate_up, gu_raw, cudaMemcpyHostToDevice, s) == cudaSuccess &&
           cudaMemcpyAsync(raw + gu_raw, x.down, dn_raw, cudaMemcpyHostToDevice, s) == cudaSuccess &&
           cudaMemcpyAsync(w.gate_up_scales_at(e), x.gate_up_scales, sizeof(float) * 2 * I, cudaMemcpyHostToDevice, s) == cudaSuccess &&
           cudaMemcpyAsync(w.down_scales_at(e), x.down_scales, sizeof(float) * H, cudaMemcpyHostToDevice, s) == cudaSuccess &&
           launch_moe_pack(MoePackParams{raw, w.gate_up_at(e), H, 2 * I, nib}, s) == cudaSuccess &&
           launch_moe_pack(MoePackParams{raw + gu_raw, w.down_at(e), I, H, nib}, s) == cudaSuccess &&
           cudaStreamSynchronize(s) == cudaSuccess;     // the caller's arrays and `raw` are reused by the next expert
}

// experts != null: an immutable bank of all E experts.  experts == null: a slot bank -- E zeroed slots (an expert that
// was never imported contributes zero), plus the int8 shared expert `shared` packed into the last one where the
// configuration has it.
rk_npu_moe_w8_weights* weights_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_weight_config* config,
                                      const rk_npu_moe_w8_expert* experts, Mode mode, bool certify_full_k,
                                      const rk_npu_moe_w8_expert* shared = nullptr)
{
    const bool slotted = experts == nullptr;
    if (!domain || !domain->ctx || !config || !(mode == Mode::W8 ? valid_weights(*config) : valid_w4(*config)) || domain->ctx->world > 1)
        return nullptr;
    if (slotted && (mode == Mode::W8 || (mode == Mode::W4) != (config->shared_expert == 0) || (config->shared_expert && !shared))) return nullptr;
    const int H = config->hidden, I = config->intermediate, R = config->routed_experts, E = R + config->shared_expert;
    std::vector<int32_t> tags;
    try { tags.assign(size_t(E), record_sliced); } catch (...) { return nullptr; }
    const bool try_full = (certify_full_k || mode == Mode::RoutedW4SharedW8) && can_use_full_gate(H);
    if (!slotted) {
        for (int e = 0; e < E; ++e)
            if (!valid_expert(experts[e], H, I, expert_is_w4(mode, e, R), try_full, tags[size_t(e)])) return nullptr;
    } else if (shared && !valid_expert(*shared, H, I, false, false, tags[size_t(R)])) {
        return nullptr;
    }
    rk_npu_ctx* ctx = domain->ctx;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return nullptr;
    rk_npu_moe_w8_weights* w = nullptr;
    try { w = new rk_npu_moe_w8_weights(); } catch (...) { return nullptr; }
    w->domain = domain;
    w->ctx_id = ctx->id;
    w->domain_id = domain->id;
    w->config = *config;
    w->mode = mode;
    w->tags.swap(tags);
    w->slotted = slotted;
    domain_retain(domain);
    w->nibble_experts = mode == Mode::W4 ? E : (mode == Mode::RoutedW4SharedW8 ? R : 0);
    bool ok = cudaStreamCreateWithFlags(&w->stream, cudaStreamNonBlocking) == cudaSuccess;
    if (slotted) {
        try { w->slots.resize(size_t(E)); } catch (...) { ok = false; }
        for (int e = 0; ok && e < E; ++e) {
            auto& slot = w->slots[size_t(e)];
            slot.bytes = w->slot_bytes(e);
            ok = !device_alloc(domain, reinterpret_cast<void**>(&slot.storage), slot.bytes) &&
                 cudaMemsetAsync(slot.storage, 0, slot.bytes, w->stream) == cudaSuccess;
        }
        ok = ok && cudaStreamSynchronize(w->stream) == cudaSuccess;
    } else {
        const MoeBank gb = w->gate_up_bank(), db = w->down_bank();
        w->gate_up_bytes = size_t(w->nibble_experts) * gb.nibble_bytes + size_t(E - w->nibble_experts) * gb.byte_bytes;
        w->down_bytes = size_t(w->nibble_experts) * db.nibble_bytes + size_t(E - w->nibble_experts) * db.byte_bytes;
        w->gate_up_scale_bytes = sizeof(float) * 2 * size_t(I) * E;
        w->down_scale_bytes = sizeof(float) * size_t(H) * E;
        ok = ok && !device_alloc(domain, reinterpret_cast<void**>(&w->gate_up), w->gate_up_bytes) &&
             !device_alloc(domain, reinterpret_cast<void**>(&w->down), w->down_bytes) &&
             !device_alloc(domain, reinterpret_cast<void**>(&w->gate_up_scales), w->gate_up_scale_bytes) &&
             !device_alloc(domain, reinterpret_cast<void**>(&w->down_scales), w->down_scale_bytes);
    }
    int8_t* raw = nullptr;     // one expert's matrices as given, on their way into records
    if (!slotted || shared) ok = ok && cudaMalloc(reinterpret_cast<void**>(&raw), size_t(H) * 2 * I + size_t(I) * H) == cudaSuccess;
    for (int e = 0; ok && !slotted && e < E; ++e) ok = place_expert(*w, e, experts[e], raw, ctx->stream);
    if (ok && slotted && shared) ok = place_expert(*w, R, *shared, raw, ctx->stream);
    if (raw) cudaFree(raw);
    if (!ok) { cudaGetLastError(); weights_destroy(w); return nullptr; }
    return w;
}
} // namespace

extern "C" rk_npu_moe_w8_weights* rk_npu_moe_w8_weights_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_weight_config* config,
                                                               const rk_npu_moe_w8_expert* experts)
{
    return weights_create(domain, config, experts, Mode::W8, false);
}
extern "C" void rk_npu_moe_w8_weights_free(rk_npu_moe_w8_weights* w) { weights_destroy(w); }

namespace {
rk_npu_moe_w8_workspace* workspace_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_config* config, Mode mode)
{
    if (!domain || !domain->ctx || !config || !valid_config(*config) || domain->ctx->world > 1) return nullptr;
    if (mode != Mode::W8 && (!valid_w4(config->weights) || config->native_input)) return nullptr;   // src/rk_npu_moe_w8.cpp:892-893
    rk_npu_ctx* ctx = domain->ctx;
    if (cudaSetDevice(ctx->device) != cudaSuccess) return nullptr;
    rk_npu_moe_w8_workspace* ws = nullptr;
    try { ws = new rk_npu_moe_w8_workspace(); } catch (...) { return nullptr; }
    ws->domain = domain;
    ws->ctx_id = ctx->id;
    ws->domain_id = domain->id;
    ws->config = *config;
    ws->mode = mode;
    domain_retain(domain);
    const int H = config->weights.hidden, I = config->weights.intermediate, rows = config->max_rows;
    ws->slots = config->top_k + config->weights.shared_expert;
    ws->assignments_max = rows * ws->slots;
    const size_t A = size_t(ws->assignments_max);
    ws->codes_bytes = size_t(rows) * H;
    ws->in_scale_bytes = size_t(rows) * 4;
    ws->middle_bytes = A * I * 4;
    ws->row_max_bytes = A * 4;
    ws->expert_out_bytes = A * H * 4;
    ws->out_bytes = size_t(rows) * H * 4;
    ws->upload_bytes = upload_capacity(rows, ws->slots, H, config->weights.routed_experts + config->weights.shared_expert);
    bool ok = true;
    try { ws->groups.resize(size_t(config->weights.routed_experts + config->weights.shared_expert)); } catch (...) { ok = false; }
    ok = ok && !device_alloc(domain, reinterpret_cast<void**>(&ws->codes), ws->codes_bytes) &&
         !device_alloc(domain, reinterpret_cast<void**>(&ws->in_scales), ws->in_scale_bytes) &&
         !device_alloc(domain, reinterpret_cast<void**>(&ws->middle), ws->middle_bytes) &&
         !device_alloc(domain, reinterpret_cast<void**>(&ws->row_max), ws->row_max_bytes) &&
         !device_alloc(domain, reinterpret_cast<void**>(&ws->expert_out), ws->expert_out_bytes) &&
         !device_alloc(domain, reinterpret_cast<void**>(&ws->out), ws->out_bytes) &&
         !device_alloc(domain, reinterpret_cast<void**>(&ws->upload), ws->upload_bytes) &&
         !device_alloc(domain, reinterpret_cast<void**>(&ws->status), sizeof(Status));
    ok = ok && cudaStreamCreateWithFlags(&ws->stream, cudaStreamNonBlocking) == cudaSuccess &&
         cudaMallocHost(reinterpret_cast<void**>(&ws->host_upload), ws->upload_bytes) == cudaSuccess &&
         cudaHostAlloc(reinterpret_cast<void**>(&ws->host_status), sizeof(Status), cudaHostAllocMapped) == cudaSuccess &&
         cudaHostGetDevicePointer(reinterpret_cast<void**>(&ws->host_status_alias), ws->host_status, 0) == cudaSuccess;
    ws->host_out_bytes = std::min<size_t>(ws->out_bytes, size_t(256) << 10);
    ok = ok && cudaHostAlloc(reinterpret_cast<void**>(&ws->host_out), ws->host_out_bytes, cudaHostAllocMapped) == cudaSuccess &&
         cudaHostGetDevicePointer(reinterpret_cast<void**>(&ws->host_out_alias), ws->host_out, 0) == cudaSuccess;
    for (auto& e : ws->events) ok = ok && cudaEventCreate(&e) == cudaSuccess;
    ok = ok && cudaMemsetAsync(ws->status, 0, sizeof(Status), ws->stream) == cudaSuccess &&
         cudaMemsetAsync(ws->row_max, 0, ws->row_max_bytes, ws->stream) == cudaSuccess &&     // every run leaves them zero again
         cudaStreamSynchronize(ws->stream) == cudaSuccess;
    if (!ok) { cudaGetLastError(); workspace_destroy(ws); return nullptr; }
    return ws;
}
} // namespace

extern "C" rk_npu_moe_w8_workspace* rk_npu_moe_w8_workspace_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_config* config)
{
    return workspace_create(domain, config, Mode::W8);
}
extern "C" void rk_npu_moe_w8_workspace_free(rk_npu_moe_w8_workspace* ws) { workspace_destroy(ws); }

extern "C" uint64_t rk_npu_moe_w8_weights_device_bytes(const rk_npu_moe_w8_weights* w)
{
    if (!w) return 0;
    uint64_t bytes = uint64_t(w->gate_up_bytes + w->down_bytes + w->gate_up_scale_bytes + w->down_scale_bytes);
    for (const auto& slot : w->slots) bytes += slot.bytes;      // what the bank holds now; exchanged slots count where they are
    return bytes;
}
extern "C" uint64_t rk_npu_moe_w8_workspace_device_bytes(const rk_npu_moe_w8_workspace* ws)
{
    return ws ? uint64_t(ws->codes_bytes + ws->in_scale_bytes + ws->middle_bytes + ws->row_max_bytes + ws->expert_out_bytes +
                         ws->out_bytes + ws->upload_bytes + sizeof(Status))
              : 0;
}

extern "C" int rk_npu_moe_w8_run_quantized(rk_npu_moe_w8_workspace* ws, const rk_npu_moe_w8_weights* w, int rows, const int8_t* input,
                                           const float* row_scales, const int32_t* expert_ids, const float* route_weights, float* output,
                                           rk_npu_moe_w8_timings* timings)
{
    return moe_run(ws, w, rows, input, false, row_scales, expert_ids, route_weights, output, timings);
}
extern "C" int rk_npu_moe_w8_run_f32(rk_npu_moe_w8_workspace* ws, const rk_npu_moe_w8_weights* w, int rows, const float* input,
                                     const int32_t* expert_ids, const float* route_weights, float* output, rk_npu_moe_w8_timings* timings)
{
    return moe_run(ws, w, rows, input, true, nullptr, expert_ids, route_weights, output, timings);
}

// ---- int4 experts (include/rk_npu_moe_w8.h:87-111): all experts int4, or routed int4 with an int8 shared expert.
// The handles work with the same run / free / byte-query functions; a workspace runs weights of its own form only.
extern "C" rk_npu_moe_w8_weights* rk_npu_moe_quant_weights_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_weight_config* config,
                                                                  const rk_npu_moe_w8_expert* experts)
{
    return weights_create(domain, config, experts, Mode::W4, false);
}
extern "C" rk_npu_moe_w8_weights* rk_npu_moe_quant_weights_create_full_k(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_weight_config* config,
                                                                         const rk_npu_moe_w8_expert* experts)
{
    return weights_create(domain, config, experts, Mode::W4, true);
}
extern "C" rk_npu_moe_w8_workspace* rk_npu_moe_quant_workspace_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_config* config)
{
    return workspace_create(domain, config, Mode::W4);
}
extern "C" rk_npu_moe_w8_weights* rk_npu_moe_w4_weights_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_weight_config* config,
                                                               const rk_npu_moe_w8_expert* experts)
{
    return weights_create(domain, config, experts, Mode::RoutedW4SharedW8, false);
}
extern "C" rk_npu_moe_w8_workspace* rk_npu_moe_w4_workspace_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_config* config)
{
    return workspace_create(domain, config, Mode::RoutedW4SharedW8);
}

// ---- mutable slot banks and their cache records (include/rk_npu_moe_w8.h:113-146, src/rk_npu_moe_w8.cpp:915-1000)
// A record is one int4 expert exactly as a slot stores it -- gate/up records, down records, gate/up scales, down scales
// -- followed by a 16-byte trailer (magic, hidden, intermediate, tag).  Records made by an immutable bank, a slot bank or
// the mixed form are the same bytes for the same expert; import is one copy into the slot.
extern "C" rk_npu_moe_w8_weights* rk_npu_moe_quant_slots_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_weight_config* config)
{
    return weights_create(domain, config, nullptr, Mode::W4, false);
}
extern "C" rk_npu_moe_w8_weights* rk_npu_moe_w4_slots_create(rk_npu_iommu_domain* domain, const rk_npu_moe_w8_weight_config* config,
                                                             const rk_npu_moe_w8_expert* shared)
{
    if (!shared) return nullptr;
    return weights_create(domain, config, nullptr, Mode::RoutedW4SharedW8, false, shared);
}
extern "C" uint64_t rk_npu_moe_quant_expert_blob_bytes(const rk_npu_moe_w8_weights* w) { return w ? w->record_bytes() : 0; }

namespace {
bool record_expert(const rk_npu_moe_w8_weights* w, int e)
{
    return w && w->record_bytes() && e >= 0 && e < w->experts() && expert_is_w4(w->mode, e, w->config.routed_experts);
}
} // namespace

extern "C" int rk_npu_moe_quant_export_expert(const rk_npu_moe_w8_weights* w, int expert, void* data, uint64_t bytes)
{
    if (!record_expert(w, expert) || !data || bytes < w->record_bytes()) return RK_NPU_ERR_PARAM;
    auto* self = const_cast<rk_npu_moe_w8_weights*>(w);      // the transfer stream and its lock are not part of the value
    if (cudaSetDevice(w->domain->ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    const int H = w->config.hidden, I = w->config.intermediate;
    const size_t gu = w->gate_up_record_bytes(expert), dn = w->down_record_bytes(expert);
    uint8_t* out = static_cast<uint8_t*>(data);
    std::lock_guard<std::mutex> guard(self->transfer);
    cudaStream_t s = w->stream;
    const bool ok = cudaMemcpyAsync(out, w->gate_up_at(expert), gu, cudaMemcpyDeviceToHost, s) == cudaSuccess &&
                    cudaMemcpyAsync(out + gu, w->down_at(expert), dn, cudaMemcpyDeviceToHost, s) == cudaSuccess &&
                    cudaMemcpyAsync(out + gu + dn, w->gate_up_scales_at(expert), sizeof(float) * 2 * I, cudaMemcpyDeviceToHost, s) == cudaSuccess &&
                    cudaMemcpyAsync(out + gu + dn + sizeof(float) * 2 * I, w->down_scales_at(expert), sizeof(float) * H, cudaMemcpyDeviceToHost, s) == cudaSuccess &&
                    cudaStreamSynchronize(s) == cudaSuccess;
    if (!ok) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
    const RecordTrailer trailer{record_magic, H, I, w->tags[size_t(expert)]};
    std::memcpy(out + w->slot_bytes(expert), &trailer, sizeof(trailer));
    return RK_NPU_OK;
}

// Import only between blocking runs that use the bank (the original's rule).  The record is checked BEFORE anything is
// copied -- length, trailer, tag, every scale positive and finite -- so a refused record leaves the slot as it was.
extern "C" int rk_npu_moe_quant_import_expert_timed(rk_npu_moe_w8_weights* w, int slot, const void* data, uint64_t bytes,
                                                    rk_npu_moe_import_timings* timings)
{
    if (!record_expert(w, slot) || !data || bytes < w->record_bytes()) return RK_NPU_ERR_PARAM;
    if (timings) *timings = rk_npu_moe_import_timings{};
    const auto begin = Clock::now();
    const int H = w->config.hidden, I = w->config.intermediate;
    const size_t gu = w->gate_up_record_bytes(slot), dn = w->down_record_bytes(slot), payload = w->slot_bytes(slot);
    const uint8_t* in = static_cast<const uint8_t*>(data);
    RecordTrailer trailer;
    std::memcpy(&trailer, in + payload, sizeof(trailer));
    const int32_t tag = trailer.tag & record_tag_mask;
    if (trailer.magic != record_magic || trailer.hidden != H || trailer.intermediate != I ||
        (tag != record_sliced && !(tag == record_full_k && can_use_full_gate(H))))
        return RK_NPU_ERR_PARAM;
    const float* scales = reinterpret_cast<const float*>(in + gu + dn);
    for (int n = 0; n < 2 * I + H; ++n) {
        float value;
        std::memcpy(&value, scales + n, sizeof(value));
        if (!finite_positive(value)) return RK_NPU_ERR_PARAM;
    }
    const double validate_us = since_us(begin);
    if (cudaSetDevice(w->domain->ctx->device) != cudaSuccess) return RK_NPU_ERR_SUBMIT;
    auto at = Clock::now();
    double gate_us = 0, down_us = 0;
    {
        std::lock_guard<std::mutex> guard(w->transfer);
        cudaStream_t s = w->stream;
        bool ok;
        if (w->slotted) {      // the slot is laid out like the record: one copy
            ok = cudaMemcpyAsync(w->slots[size_t(slot)].storage, in, payload, cudaMemcpyHostToDevice, s) == cudaSuccess &&
                 cudaStreamSynchronize(s) == cudaSuccess;
            gate_us = since_us(at);
        } else {
            ok = cudaMemcpyAsync(w->gate_up_at(slot), in, gu, cudaMemcpyHostToDevice, s) == cudaSuccess &&
                 cudaMemcpyAsync(w->gate_up_scales_at(slot), in + gu + dn, sizeof(float) * 2 * I, cudaMemcpyHostToDevice, s) == cudaSuccess &&
                 cudaStreamSynchronize(s) == cudaSuccess;
            gate_us = since_us(at);
            at = Clock::now();
            ok = ok && cudaMemcpyAsync(w->down_at(slot), in + gu, dn, cudaMemcpyHostToDevice, s) == cudaSuccess &&
                 cudaMemcpyAsync(w->down_scales_at(slot), in + gu + dn + sizeof(float) * 2 * I, sizeof(float) * H, cudaMemcpyHostToDevice, s) == cudaSuccess &&
                 cudaStreamSynchronize(s) == cudaSuccess;
            down_us = since_us(at);
        }
        if (!ok) { cudaGetLastError(); return RK_NPU_ERR_SUBMIT; }
        w->tags[size_t(slot)] = tag;
    }
    if (timings) {      // copy_us: host-side staging in the original, nothing here; the two sync fields: the transfers
        timings->validate_us = validate_us;
        timings->gate_sync_us = gate_us;
        timings->down_sync_us = down_us;
        timings->total_us = since_us(begin);
    }
    return RK_NPU_OK;
}
extern "C" int rk_npu_moe_quant_import_expert(rk_npu_moe_w8_weights* w, int slot, const void* data, uint64_t bytes)
{
    return rk_npu_moe_quant_import_expert_timed(w, slot, data, bytes, nullptr);
}

// Exchanges two slots' storage and tags: no copy, no wait.  Both banks are all-int4 slot banks of one geometry, context
// and domain (the original accepts its immutable all-int4 banks too, whose experts are separate allocations there; here
// an immutable bank is one allocation and cannot give a piece away).  The caller keeps the two slots idle meanwhile;
// other slots of either bank may be imported at the same time.
extern "C" int rk_npu_moe_quant_swap_slots(rk_npu_moe_w8_weights* a, int ai, rk_npu_moe_w8_weights* b, int bi)
{
    if (!a || !b || a->mode != Mode::W4 || b->mode != Mode::W4 || !a->slotted || !b->slotted || a->config.hidden != b->config.hidden ||
        a->config.intermediate != b->config.intermediate || a->ctx_id != b->ctx_id || a->domain_id != b->domain_id || ai < 0 || bi < 0 ||
        ai >= a->experts() || bi >= b->experts())
        return RK_NPU_ERR_PARAM;
    std::swap(a->slots[size_t(ai)], b->slots[size_t(bi)]);
    std::swap(a->tags[size_t(ai)], b->tags[size_t(bi)]);
    return RK_NPU_OK;
}
