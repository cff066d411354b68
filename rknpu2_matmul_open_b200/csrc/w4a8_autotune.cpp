// w4a8_autotune.cpp -- the search tuner of the W4A8 path (include/rk_npu_w4a8_tune.h:62-167) for B200.
//
// The original searches K/N/M tiles, host teams and pipeline modes of its three-core device
// (candidates: src/rk_npu_w4a8_tune_policy.cpp:81-122; loop: src/rk_npu_w4a8_tune.cpp:26-100; score:
// src/rk_npu_autotune_common.cpp:14-38).  Here the search space is this library's own: which kernel
// family runs the shape and how many CTAs cooperate on a column tile (split-K factor / cluster size).
// The protocol is the original's: complete blocking calls on a deterministic calibration tensor, every
// candidate's output compared with an anchor result that was itself checked against the int64 formula,
// warm-up + loops x repeats, median over the repeats, jitter = range / median, robust = median + half
// the range.  What RANKS the candidates is measured the way the kernels are used in a model: `loops`
// launches queued back to back on one stream over device tensors, timed by two events (a blocking
// call's own device window is a few microseconds of kernel inside tens of microseconds of launch
// latency and cannot tell the families apart on small shapes).  The winner is written into the
// strategy's existing fields (w4a8_tune.h: schedule_of), so cache files keep their format and a tuned
// workspace honours the choice.
#include "w4a8_tune.h"
#include <algorithm>
#include <cfloat>
#include <climits>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <memory>
#include <set>
#include <type_traits>
#include <vector>

namespace rkb200 {

std::vector<Schedule> schedule_candidates(int M, int N, int K, int sm_count)
{
    (void)N;
    (void)sm_count;
    std::vector<Schedule> out;
    out.push_back(Schedule{});                                  // the library's own rule comes first and wins ties
    const int clusters[] = {1, 2, 4, 8};
    if (M <= 8 && gemm_decode_supported(M, K))
        for (int c : clusters) out.push_back(Schedule{5, c});
    if (M <= 128) {
        const int kb = (K + KBLOCK - 1) / KBLOCK;
        for (int c : clusters)
            if (kb >= 2 * c || c == 1) out.push_back(Schedule{1, c});
        if ((long long)kb * KBLOCK <= 131072) out.push_back(Schedule{4, 0});
    }
    if (M > 32 && M <= 128) out.push_back(Schedule{2, 0});
    return out;
}

namespace {
// ---- calibration tensor and the anchor result ------------------------------------------------------------
// Values are small multiples of 1/64, exactly representable in binary16 and fp32 alike, so both activation
// types quantise the same numbers; row 0 of a batch of three or more is zero (scale 1, exact zero outputs).
struct Calibration {
    int M, K, N;
    bool half;
    std::vector<float> a32;
    std::vector<uint16_t> a16;
    std::vector<uint8_t> out, anchor;      // raw output bytes of the last run / of the anchor run
    void* dA = nullptr;                    // the same tensor and an output on the device, for the queued timing
    void* dC = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;

    Calibration(const Calibration&) = delete;
    Calibration& operator=(const Calibration&) = delete;
    ~Calibration()
    {
        if (dA) cudaFree(dA);
        if (dC) cudaFree(dC);
        if (e0) cudaEventDestroy(e0);
        if (e1) cudaEventDestroy(e1);
    }
    // device copies, made on first use (the CUDA device of the search is current)
    bool on_device()
    {
        if (dA) return true;
        const size_t a_bytes = half ? a16.size() * 2 : a32.size() * 4;
        const bool ok = cudaMalloc(&dA, a_bytes) == cudaSuccess && cudaMalloc(&dC, out.size()) == cudaSuccess &&
                        cudaMemcpy(dA, half ? static_cast<const void*>(a16.data()) : static_cast<const void*>(a32.data()), a_bytes,
                                   cudaMemcpyHostToDevice) == cudaSuccess &&
                        cudaEventCreate(&e0) == cudaSuccess && cudaEventCreate(&e1) == cudaSuccess;
        if (!ok) cudaGetLastError();
        return ok;
    }
    // `loops` launches queued back to back on the workspace's stream: microseconds per launch, < 0 on failure
    double queued_us(rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w, int loops)
    {
        if (!on_device()) return -1;
        cudaStream_t s = ws->stream;
        cudaEventRecord(e0, s);
        for (int l = 0; l < loops; ++l) {
            const int rc = half ? rk_npu_b200_w4a8_enqueue_f16(ws, w, static_cast<const uint16_t*>(dA), static_cast<uint16_t*>(dC), s)
                                : rk_npu_b200_w4a8_enqueue_f32(ws, w, static_cast<const float*>(dA), static_cast<float*>(dC), s);
            if (rc) { cudaStreamSynchronize(s); return -1; }
        }
        cudaEventRecord(e1, s);
        if (cudaStreamSynchronize(s) != cudaSuccess) { cudaGetLastError(); return -1; }
        if (rk_npu_b200_w4a8_finish(ws) != RK_NPU_OK) return -1;
        float ms = 0;
        if (cudaEventElapsedTime(&ms, e0, e1) != cudaSuccess) { cudaGetLastError(); return -1; }
        return double(ms) * 1000.0 / loops;
    }

    explicit Calibration(const rk_npu_w4a8_autotune_config& c)
        : M(c.M), K(c.K), N(c.N), half(c.activation_type == RK_NPU_W4A8_F16), a32(size_t(c.M) * c.K),
          out(size_t(c.M) * c.N * (c.activation_type == RK_NPU_W4A8_F16 ? 2 : 4))
    {
        uint64_t x = 0x9E3779B97F4A7C15ull;
        for (size_t i = 0; i < a32.size(); ++i) {
            x ^= x << 13; x ^= x >> 7; x ^= x << 17;          // xorshift64
            const int step = int((x >> 24) % 401) - 200;      // -200 .. 200
            a32[i] = (M >= 3 && i < size_t(K)) ? 0.f : float(step) * 0.015625f;
        }
        if (half) {
            a16.resize(a32.size());
            for (size_t i = 0; i < a32.size(); ++i) a16[i] = exact_half(a32[i]);
        }
    }
    // binary16 pattern of a multiple of 1/64 with magnitude below 4: always exact
    static uint16_t exact_half(float v)
    {
        if (v == 0.f) return 0;
        const uint16_t sign = v < 0 ? 0x8000u : 0u;
        int e = 0;
        const float m = std::frexp(std::fabs(v), &e);         // |v| = m * 2^e, m in [0.5, 1)
        const int mant = int(m * 2048.f) - 1024;              // 10 fraction bits of 2m - 1
        return uint16_t(sign | uint16_t((e + 14) << 10) | uint16_t(mant));
    }
    int run(rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w, rk_npu_w4a8_timings& t)
    {
        return half ? rk_npu_w4a8_run_f16(ws, w, a16.data(), reinterpret_cast<uint16_t*>(out.data()), &t)
                    : rk_npu_w4a8_run_f32(ws, w, a32.data(), reinterpret_cast<float*>(out.data()), &t);
    }
    bool matches_anchor() const { return out == anchor; }

    // The anchor against the defining formula, in integers: codes by round-half-away of a * (1 / scale),
    // int64 dot product, (float(sum) * scale) * w_scale.  All columns of a small problem, 17 evenly spaced
    // ones of a large one (the original's sampling).
    bool anchor_is_correct(const int8_t* B, const float* w_scale) const
    {
        std::vector<int> columns;
        if (int64_t(M) * K <= 16000000 / int64_t(N)) for (int n = 0; n < N; ++n) columns.push_back(n);
        else for (int i = 0; i < 17; ++i) columns.push_back(int(int64_t(i) * (N - 1) / 16));
        std::vector<int> code(static_cast<size_t>(K), 0);
        for (int m = 0; m < M; ++m) {
            const float* row = a32.data() + size_t(m) * K;
            float top = 0;
            for (int k = 0; k < K; ++k) top = std::max(top, std::fabs(row[k]));
            const float scale = top == 0 ? 1.f : std::max(top / 127.f, FLT_MIN), inverse = 1.f / scale;
            for (int k = 0; k < K; ++k) code[size_t(k)] = int(std::clamp(std::round(row[k] * inverse), -127.f, 127.f));
            for (int n : columns) {
                int64_t sum = 0;
                for (int k = 0; k < K; ++k) sum += int64_t(code[size_t(k)]) * B[size_t(k) * N + n];
                const float expected = (float(sum) * scale) * w_scale[n];
                const size_t i = size_t(m) * N + n;
                if (half) {
                    uint16_t got;
                    std::memcpy(&got, anchor.data() + 2 * i, 2);
                    if (got != round_to_half(expected)) return false;
                } else {
                    float got;
                    std::memcpy(&got, anchor.data() + 4 * i, 4);
                    if (std::memcmp(&got, &expected, 4) != 0) return false;
                }
            }
        }
        return true;
    }
    // fp32 -> binary16, round to nearest even, overflow to infinity (src/rk_npu_half_bits.h:29-53 defines the result)
    static uint16_t round_to_half(float f)
    {
        uint32_t x;
        std::memcpy(&x, &f, 4);
        const uint32_t sign = (x >> 16) & 0x8000u, mag = x & 0x7fffffffu;
        if (mag >= 0x7f800000u) return uint16_t(sign | 0x7c00u | (mag > 0x7f800000u ? 0x200u | ((mag >> 13) & 0x3ffu) : 0u));
        if (mag >= 0x477ff000u) return uint16_t(sign | 0x7c00u);                      // rounds to or beyond 65520
        if (mag < 0x33000001u) return uint16_t(sign);                                 // below half the smallest subnormal
        int exponent = int(mag >> 23) - 127;
        uint32_t mant = (mag & 0x7fffffu) | 0x800000u;
        int shift = 13;
        if (exponent < -14) { shift += -14 - exponent; exponent = -15; }
        const uint32_t kept = mant >> shift, rest = mant & ((1u << shift) - 1u), halfway = 1u << (shift - 1);
        uint32_t value = (exponent == -15 ? kept : ((uint32_t(exponent + 15) << 10) + (kept - 0x400u)));
        if (rest > halfway || (rest == halfway && (value & 1u))) ++value;
        return uint16_t(sign | value);
    }
};

// ---- timing ----------------------------------------------------------------------------------------------
struct Score {
    double input_us = 0, device_us = 0, sync_us = 0, output_us = 0, total_us = 0;   // medians over the repeats
    double jitter_pct = 0, robust_us = 0;
    double work_us = 0, work_robust_us = 0;   // the device part (what ranks candidates) and its robust form
};
double median_of(std::vector<double> v)
{
    if (v.empty()) return 0;
    const size_t mid = v.size() / 2;
    std::nth_element(v.begin(), v.begin() + mid, v.end());
    const double upper = v[mid];
    if (v.size() % 2) return upper;
    return (*std::max_element(v.begin(), v.begin() + mid) + upper) / 2;
}
double spread_of(const std::vector<double>& v)
{
    const auto ends = std::minmax_element(v.begin(), v.end());
    return *ends.second - *ends.first;
}

struct Deleter {
    void operator()(rk_npu_iommu_domain* d) const { rk_npu_iommu_domain_free(d); }
    void operator()(rk_npu_w4a8_weights* w) const { rk_npu_w4a8_weights_free(w); }
    void operator()(rk_npu_w4a8_workspace* w) const { rk_npu_w4a8_workspace_free(w); }
};
template <class T> using Owned = std::unique_ptr<T, Deleter>;

// K tile every candidate carries: the one the request demands, else the widest permitted tile up to the
// universally certified 480 (on this library the tile is part of a weight's identity, nothing more).
int tile_for(const rk_npu_w4a8_autotune_config& request, const Profile& profile)
{
    if (request.required_k_tile) return request.required_k_tile;
    for (int k = std::min(480, profile.limit) / 32 * 32; k >= 32; k -= 32)
        if (profile.permits(k)) return k;
    return 0;
}

int measure(Calibration& data, rk_npu_w4a8_workspace* ws, const rk_npu_w4a8_weights* w, const rk_npu_w4a8_autotune_config& request,
            Score& score)
{
    rk_npu_w4a8_timings t{};
    for (int i = 0; i < request.warmup; ++i)
        if (const int rc = data.run(ws, w, t)) return rc;
    std::vector<double> total, input, device, sync, output, work;
    for (int r = 0; r < request.repeats; ++r) {
        double s_total = 0, s_input = 0, s_device = 0, s_sync = 0, s_output = 0;
        for (int l = 0; l < request.loops; ++l) {
            if (const int rc = data.run(ws, w, t)) return rc;
            if (!data.matches_anchor()) return RK_NPU_ERR_PARAM;        // every timed output is checked
            s_total += t.total_us;
            s_input += t.activation_scan_us + t.quant_pack_us;
            s_device += t.submit_us;
            s_sync += t.sync_us;
            s_output += t.reduce_us + t.dequant_us;
        }
        const double n = request.loops;
        total.push_back(s_total / n); input.push_back(s_input / n); device.push_back(s_device / n);
        sync.push_back(s_sync / n); output.push_back(s_output / n);
        // what ranks the candidate: launches queued back to back (at least eight, so that launch latency is hidden)
        const double queued = data.queued_us(ws, w, std::max(8, request.loops));
        work.push_back(queued >= 0 ? queued : (s_input + s_device + s_output) / n);
    }
    score.total_us = median_of(total);
    score.input_us = median_of(input);
    score.device_us = median_of(device);
    score.sync_us = median_of(sync);
    score.output_us = median_of(output);
    score.jitter_pct = score.total_us > 0 ? spread_of(total) * 100.0 / score.total_us : 0;
    score.robust_us = score.total_us + spread_of(total) / 2;
    score.work_us = median_of(work);
    score.work_robust_us = score.work_us + spread_of(work) / 2;
    return RK_NPU_OK;
}

// One search: every candidate schedule timed on complete calls; `fastest` has the least device time,
// `stable` the least device time plus half its range.  The complete call is dominated by host copies that
// are the same for every candidate, which is why the device part ranks them; the strategy still records
// the complete call's figures in total_us / robust_us as the original does.
int search(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config& request, const int8_t* B, const float* scales, const Profile& profile,
           const HostResources& res, bool extended, Strategy& fastest, Strategy& stable)
{
    if (!ctx || ctx->device < 0) return RK_NPU_ERR_PARAM;
    const int kt = tile_for(request, profile);
    if (!kt) return RK_NPU_ERR_PARAM;
    Owned<rk_npu_iommu_domain> domain(rk_npu_iommu_domain_create(ctx, 0));
    if (!domain) return RK_NPU_ERR_DOMAIN;
    Owned<rk_npu_w4a8_weights> weights(create_weights(domain.get(), profile.info(kt), B, scales, &profile));
    if (!weights) return RK_NPU_ERR_NOMEM;
    Calibration data(request);
    rk_npu_w4a8_options execution;
    rk_npu_w4a8_options_init(&execution);

    auto config_for = [&](const Schedule& schedule) {
        rk_npu_w4a8_config c;
        rk_npu_w4a8_config_init(&c, request.M, request.N, request.K);
        c.k_tile = kt;
        c.npu_core_mask = res.device_cores;
        c.timeout_ms = request.timeout_ms;
        c.cpu_threads = res.threads;
        schedule_into(schedule, c);
        return c;
    };
    auto as_strategy = [&](const rk_npu_w4a8_config& c, const Score& score) {
        Strategy s{};
        s.execution = execution;
        s.base.config = c;
        s.base.activation_type = request.activation_type;
        s.base.cpu_core_mask = res.cpus;
        s.base.weights = profile.info(kt);
        s.base.weight_fingerprint = profile.fingerprint;
        s.base.tuning_revision = TUNING_REVISION;
        s.base.input_us = score.input_us; s.base.npu_us = score.device_us; s.base.sync_us = score.sync_us;
        s.base.output_us = score.output_us; s.base.total_us = score.total_us;
        s.base.jitter_pct = score.jitter_pct; s.base.robust_us = score.robust_us;
        return s;
    };

    bool found = false;
    double best_work = 0, best_robust = 0;
    for (const Schedule& schedule : schedule_candidates(request.M, request.N, request.K, ctx->sm_count)) {
        const rk_npu_w4a8_config c = config_for(schedule);
        Strategy probe = as_strategy(c, Score{});
        if (!strategy_acceptable(probe, request, profile, res, extended)) continue;      // e.g. the chain value above its token limit
        const Schedule decoded = schedule_of(c);
        if (decoded.family != schedule.family || decoded.cluster != schedule.cluster) continue;
        Owned<rk_npu_w4a8_workspace> ws(create_workspace_scheduled(domain.get(), &c, &execution, schedule));
        if (!ws) return RK_NPU_ERR_NOMEM;
        if (schedule.family && ws->variant != schedule.family) continue;                   // the geometry cannot run this family
        rk_npu_w4a8_timings t{};
        if (data.anchor.empty()) {
            // first candidate (the automatic schedule): its output becomes the anchor once the formula confirms it
            if (const int rc = data.run(ws.get(), weights.get(), t)) return rc;
            data.anchor = data.out;
            if (!data.anchor_is_correct(B, scales)) return RK_NPU_ERR_PARAM;
        }
        bool agrees = true;
        for (int trial = 0; trial < 2 && agrees; ++trial) {
            if (const int rc = data.run(ws.get(), weights.get(), t)) return rc;
            agrees = data.matches_anchor();
        }
        if (!agrees) {
            if (request.verbose) std::fprintf(stderr, "w4a8 autotune: family %d cluster %d rejected: output differs\n", schedule.family, schedule.cluster);
            continue;
        }
        Score score;
        const int rc = measure(data, ws.get(), weights.get(), request, score);
        if (rc == RK_NPU_ERR_SUBMIT) return rc;       // a device failure ends the search at once
        if (rc) continue;
        if (request.verbose)
            std::fprintf(stderr, "w4a8 autotune: M=%d N=%d K=%d family %d cluster %d: device %.2f us (robust %.2f), call %.2f us\n", request.M,
                         request.N, request.K, ws->variant, schedule.cluster, score.work_us, score.work_robust_us, score.total_us);
        const Strategy candidate = as_strategy(c, score);
        if (!found || score.work_us < best_work) { fastest = candidate; best_work = score.work_us; }
        if (!found || score.work_robust_us < best_robust) { stable = candidate; best_robust = score.work_robust_us; }
        found = true;
    }
    return found ? RK_NPU_OK : RK_NPU_ERR_PARAM;
}

void hand_out(rk_npu_w4a8_strategy* to, const Strategy& from) { if (to) *to = from.base; }
void hand_out(rk_npu_w4a8_strategy_ex* to, const Strategy& from) { if (to) *to = from; }

struct Request {
    Profile profile;
    HostResources res;
};
int prepare(const rk_npu_w4a8_autotune_config& request, const int8_t* B, const float* scales, Request& out)
{
    if (const int rc = make_profile(request, B, scales, out.profile)) return rc;
    out.res = host_resources(request);
    return out.res.usable() ? RK_NPU_OK : RK_NPU_ERR_PARAM;
}

// Cached search: a valid file answers without device work unless `refresh`; otherwise search, then try to
// save (a failed save leaves the strategies valid).
int search_cached(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config& request, const int8_t* B, const float* scales, const Request& rq,
                  const std::string& file, int refresh, bool extended, Strategy& fastest, Strategy& stable, int* hit)
{
    if (hit) *hit = 0;
    const std::string key = cache_key_line(ctx, request, rq.profile, rq.res, extended);
    const std::string path = file.empty() ? cache_file_for(key) : file;
    if (!refresh && cache_read(path, key, request, rq.profile, rq.res, extended, fastest, stable) == RK_NPU_OK) {
        if (hit) *hit = 1;
        return RK_NPU_OK;
    }
    if (const int rc = search(ctx, request, B, scales, rq.profile, rq.res, extended, fastest, stable)) return rc;
    const int saved = cache_write(path, key, fastest, stable);
    if (saved && request.verbose) std::fprintf(stderr, "w4a8 autotune: could not save %s (%d); the strategies stay valid\n", path.c_str(), saved);
    return RK_NPU_OK;
}

template <class Public>
int tune_entry(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* request, const int8_t* B, const float* scales, const char* path,
               int refresh, Public* fastest, Public* stable, int* hit, bool cached)
{
    constexpr bool extended = std::is_same<Public, rk_npu_w4a8_strategy_ex>::value;
    if (hit) *hit = 0;
    if (!ctx || !request || (!fastest && !stable) || (path && *path == 0)) return RK_NPU_ERR_PARAM;
    try {
        Request rq;
        if (const int rc = prepare(*request, B, scales, rq)) return rc;
        Strategy f{}, s{};
        const int rc = cached ? search_cached(ctx, *request, B, scales, rq, path ? std::string(path) : std::string(), refresh, extended, f, s, hit)
                              : search(ctx, *request, B, scales, rq.profile, rq.res, extended, f, s);
        if (rc == RK_NPU_OK) { hand_out(fastest, f); hand_out(stable, s); }
        return rc;
    } catch (const std::bad_alloc&) { return RK_NPU_ERR_NOMEM; } catch (...) { return RK_NPU_ERR_PARAM; }
}

// A family: several batch sizes of one weight, tuned one by one with a shared K tile (one weight object serves
// them all); the summaries weight each batch size's figures by its stated call frequency.
template <class Public>
int family_entry(rk_npu_ctx* ctx, const rk_npu_w4a8_family_config* family, const int8_t* B, const float* scales, const char* directory,
                 int refresh, rk_npu_w4a8_family_summary* fast_summary, Public* fast, rk_npu_w4a8_family_summary* stable_summary,
                 Public* stable, int* hits, int* misses, bool cached)
{
    constexpr bool extended = std::is_same<Public, rk_npu_w4a8_strategy_ex>::value;
    if (hits) *hits = 0;
    if (misses) *misses = 0;
    const bool outputs_ok = (fast_summary || stable_summary) && bool(fast_summary) == bool(fast) && bool(stable_summary) == bool(stable);
    if (!ctx || !family || family->m_count < 1 || !family->m_values || !outputs_ok || (directory && *directory == 0)) return RK_NPU_ERR_PARAM;
    try {
        std::set<int> seen;
        double weight_sum = 0;
        std::vector<double> share(size_t(family->m_count), 1.0);
        for (int i = 0; i < family->m_count; ++i) {
            const int m = family->m_values[i];
            if (family->frequencies) share[size_t(i)] = family->frequencies[i];
            if (m < 1 || m > INT_MAX / 2 || !seen.insert(m).second || !std::isfinite(share[size_t(i)]) || share[size_t(i)] <= 0) return RK_NPU_ERR_PARAM;
            weight_sum += share[size_t(i)];
        }
        if (!std::isfinite(weight_sum)) return RK_NPU_ERR_PARAM;
        rk_npu_w4a8_autotune_config base = family->base;
        base.M = 1;
        Request rq;
        if (const int rc = prepare(base, B, scales, rq)) return rc;
        base.required_k_tile = tile_for(base, rq.profile);            // one K partition for the whole family
        if (!base.required_k_tile) return RK_NPU_ERR_PARAM;
        std::vector<Strategy> f(size_t(family->m_count)), s(size_t(family->m_count));
        int hit_count = 0, miss_count = 0;
        for (int i = 0; i < family->m_count; ++i) {
            rk_npu_w4a8_autotune_config one = base;
            one.M = family->m_values[i];
            int rc, hit = 0;
            if (cached) {
                const std::string key = cache_key_line(ctx, one, rq.profile, rq.res, extended);
                rc = search_cached(ctx, one, B, scales, rq, cache_file_for(key, directory), refresh, extended, f[size_t(i)], s[size_t(i)], &hit);
                if (rc == RK_NPU_OK) { hit_count += hit; miss_count += !hit; }
            } else {
                rc = search(ctx, one, B, scales, rq.profile, rq.res, extended, f[size_t(i)], s[size_t(i)]);
            }
            if (rc) return rc;
        }
        if (hits) *hits = hit_count;
        if (misses) *misses = miss_count;
        auto publish = [&](rk_npu_w4a8_family_summary* summary, Public* strategies, const std::vector<Strategy>& chosen) {
            if (!summary) return;
            *summary = {chosen[0].base.weights, rq.profile.fingerprint, 0, 0};
            for (int i = 0; i < family->m_count; ++i) {
                hand_out(strategies + i, chosen[size_t(i)]);
                summary->weighted_total_us += share[size_t(i)] / weight_sum * chosen[size_t(i)].base.total_us;
                summary->weighted_robust_us += share[size_t(i)] / weight_sum * chosen[size_t(i)].base.robust_us;
            }
        };
        publish(fast_summary, fast, f);
        publish(stable_summary, stable, s);
        return RK_NPU_OK;
    } catch (const std::bad_alloc&) { return RK_NPU_ERR_NOMEM; } catch (...) { return RK_NPU_ERR_PARAM; }
}
} // namespace
} // namespace rkb200

using namespace rkb200;

extern "C" int rk_npu_w4a8_autotune(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* c, const int8_t* B, const float* scale,
                                    rk_npu_w4a8_strategy* fastest, rk_npu_w4a8_strategy* stable)
{
    return tune_entry(ctx, c, B, scale, nullptr, 0, fastest, stable, nullptr, false);
}
extern "C" int rk_npu_w4a8_autotune_cached(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* c, const int8_t* B, const float* scale,
                                           const char* path, int refresh, rk_npu_w4a8_strategy* fastest, rk_npu_w4a8_strategy* stable,
                                           int* cache_hit)
{
    return tune_entry(ctx, c, B, scale, path, refresh, fastest, stable, cache_hit, true);
}
extern "C" int rk_npu_w4a8_autotune_ex(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* c, const int8_t* B, const float* scale,
                                       rk_npu_w4a8_strategy_ex* fastest, rk_npu_w4a8_strategy_ex* stable)
{
    return tune_entry(ctx, c, B, scale, nullptr, 0, fastest, stable, nullptr, false);
}
extern "C" int rk_npu_w4a8_autotune_cached_ex(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* c, const int8_t* B, const float* scale,
                                              const char* path, int refresh, rk_npu_w4a8_strategy_ex* fastest,
                                              rk_npu_w4a8_strategy_ex* stable, int* cache_hit)
{
    return tune_entry(ctx, c, B, scale, path, refresh, fastest, stable, cache_hit, true);
}
extern "C" int rk_npu_w4a8_autotune_family(rk_npu_ctx* ctx, const rk_npu_w4a8_family_config* c, const int8_t* B, const float* scale,
                                           rk_npu_w4a8_family_summary* f, rk_npu_w4a8_strategy* fs, rk_npu_w4a8_family_summary* s,
                                           rk_npu_w4a8_strategy* ss)
{
    return family_entry(ctx, c, B, scale, nullptr, 0, f, fs, s, ss, nullptr, nullptr, false);
}
extern "C" int rk_npu_w4a8_autotune_family_cached(rk_npu_ctx* ctx, const rk_npu_w4a8_family_config* c, const int8_t* B,
                                                  const float* scale, const char* directory, int refresh, rk_npu_w4a8_family_summary* f,
                                                  rk_npu_w4a8_strategy* fs, rk_npu_w4a8_family_summary* s, rk_npu_w4a8_strategy* ss,
                                                  int* hits, int* misses)
{
    return family_entry(ctx, c, B, scale, directory, refresh, f, fs, s, ss, hits, misses, true);
}
extern "C" int rk_npu_w4a8_autotune_family_ex(rk_npu_ctx* ctx, const rk_npu_w4a8_family_config* c, const int8_t* B, const float* scale,
                                              rk_npu_w4a8_family_summary* f, rk_npu_w4a8_strategy_ex* fs, rk_npu_w4a8_family_summary* s,
                                              rk_npu_w4a8_strategy_ex* ss)
{
    return family_entry(ctx, c, B, scale, nullptr, 0, f, fs, s, ss, nullptr, nullptr, false);
}
extern "C" int rk_npu_w4a8_autotune_family_cached_ex(rk_npu_ctx* ctx, const rk_npu_w4a8_family_config* c, const int8_t* B,
                                                     const float* scale, const char* directory, int refresh,
                                                     rk_npu_w4a8_family_summary* f, rk_npu_w4a8_strategy_ex* fs,
                                                     rk_npu_w4a8_family_summary* s, rk_npu_w4a8_strategy_ex* ss, int* hits, int* misses)
{
    return family_entry(ctx, c, B, scale, directory, refresh, f, fs, s, ss, hits, misses, true);
}
