// w4a8_tune.cpp -- weight certification, weight identity and the tuning cache.
// Pure host code: nothing here touches the GPU, so a cache lookup costs file I/O only
// (the reference's contract, include/rk_npu_w4a8_tune.h:46-49).
//
// What is contract here, and where the original defines it:
//   certified K tiles       src/rk_npu_i4_bounds.cpp:9-69
//   weight fingerprint      src/rk_npu_autotune_common.cpp:83-89, src/rk_npu_w4a8.cpp:275-277 (FNV-1a over K, N, codes, scales)
//   profile of a weight     src/rk_npu_w4a8_tune_policy.cpp:41-62
//   request resources, key line, strategy rules   src/rk_npu_w4a8_tune_policy.cpp:14-33,63-71,123-155
//   cache text              src/rk_npu_w4a8_tune_cache.cpp:7-60, default location src/rk_npu_autotune_cache.cpp:15-30
// Cache files are interchangeable with the original's: same magic line, same key line (the
// driver-version field holds the CUDA driver version here), same two records.  The code that
// produces and checks that text is this library's own: one field table drives both the record
// reader and the writer, the key is assembled from a typed field list, the rules are named
// predicates.
#include "w4a8_tune.h"
#include "../../include/rknpu_b200_quant.h"
#include <algorithm>
#include <atomic>
#include <cerrno>
#include <climits>
#include <cmath>
#include <cstdlib>
#include <cstdio>
#include <cstring>
#include <fcntl.h>
#include <filesystem>
#include <fstream>
#include <iomanip>
#include <locale>
#include <sched.h>
#include <sstream>
#include <sys/stat.h>
#include <thread>
#include <type_traits>
#include <unistd.h>
#include <vector>

namespace rkb200 {
namespace {
constexpr const char* CACHE_MAGIC = "rk_npu_w4a8_tuning_cache_v2";

struct Fnv {
    uint64_t value = 1469598103934665603ull;
    void bytes(const void* p, size_t n)
    {
        const auto* b = static_cast<const uint8_t*>(p);
        uint64_t h = value;
        for (size_t i = 0; i < n; ++i) { h ^= b[i]; h *= 1099511628211ull; }
        value = h;
    }
    void mix(uint64_t v)
    {
        uint8_t le[8];
        for (int i = 0; i < 8; ++i) le[i] = uint8_t(v >> (8 * i));
        bytes(le, 8);
    }
};
uint64_t double_bits(double d) { uint64_t b; std::memcpy(&b, &d, 8); return b; }
double bits_double(uint64_t b) { double d; std::memcpy(&d, &b, 8); return d; }

// One slab of up to 128 columns: prefix sums of the two worst-case magnitudes per
// 32-row block, then the per-tile check.  Returns false on an out-of-range code.
struct SlabResult {
    bool codes_ok = true;
    // per tile size t (1..64): unsafe flag and maxima seen before the first unsafe column
    bool unsafe[65] = {};
    int64_t max_pos[65] = {}, max_neg[65] = {};
};

void scan_slab(int K, int N, const int8_t* B, int n0, int width, int blocks, int limit, const bool* wanted, SlabResult& out)
{
    std::vector<int64_t> pos(size_t(blocks + 1) * width, 0), neg(size_t(blocks + 1) * width, 0);
    for (int b = 0; b < blocks; ++b) {
        int64_t* p = pos.data() + size_t(b + 1) * width;
        int64_t* q = neg.data() + size_t(b + 1) * width;
        std::copy(p - width, p, p);
        std::copy(q - width, q, q);
        const int kend = std::min(K, (b + 1) * 32);
        for (int k = b * 32; k < kend; ++k) {
            const int8_t* row = B + size_t(k) * N + n0;
            for (int n = 0; n < width; ++n) {
                const int w = row[n];
                if (w < -8 || w > 7) { out.codes_ok = false; return; }
                p[n] += w >= 0 ? 7 * w : -8 * w;
                q[n] += w >= 0 ? 8 * w : -7 * w;
            }
        }
    }
    for (int t = 1; t <= limit; ++t) {
        if (!wanted[t]) continue;
        for (int b = 0; b < blocks && !out.unsafe[t]; b += t) {
            const int e = std::min(blocks, b + t);
            for (int n = 0; n < width; ++n) {
                const int64_t hi = pos[size_t(e) * width + n] - pos[size_t(b) * width + n];
                const int64_t lo = neg[size_t(e) * width + n] - neg[size_t(b) * width + n];
                out.max_pos[t] = std::max(out.max_pos[t], hi);
                out.max_neg[t] = std::max(out.max_neg[t], lo);
                if (hi > 32767 || lo > 32768) { out.unsafe[t] = true; break; }
            }
        }
    }
}
} // namespace

// A tile size is certified when no column of any tile of that fixed partition can push
// an int4 x int4 partial sum outside INT16.  The B200 kernels accumulate in int32 and
// need no such proof; it is kept because the weight info, the tuning profile, the cache
// key and the "explicit k_tile above 480 must be certified" rule all expose it.
// Slabs are independent, so they are scanned by several host threads; the merge
// replays them in column order, which gives the sequential algorithm's maxima exactly.
int bound_weights(int K, int N, const int8_t* B, int requested, WeightBound& out, int fallback)
{
    if (!B || K < 1 || K > INT32_MAX / 64 || N < 1 || N > INT_MAX - 63 || requested < 0 || requested > 2048 ||
        requested % 32 || fallback < 0 || fallback % 32 || (fallback && fallback >= requested))
        return RK_NPU_ERR_PARAM;
    const int blocks = (K + 31) / 32;
    const int limit = requested ? requested / 32 : std::min(64, blocks);
    bool wanted[65] = {};
    for (int t = 1; t <= limit; ++t) wanted[t] = !requested || t == limit || t * 32 == fallback;
    const int slab = 128, slabs = (N + slab - 1) / slab;
    std::vector<SlabResult> results(slabs);
    const int workers = int(std::max(1u, std::min<unsigned>({std::thread::hardware_concurrency(), 16u, unsigned(slabs)})));
    std::atomic<int> next{0};
    auto work = [&]() {
        for (int s = next.fetch_add(1); s < slabs; s = next.fetch_add(1))
            scan_slab(K, N, B, s * slab, std::min(slab, N - s * slab), blocks, limit, wanted, results[s]);
    };
    if (workers > 1 && size_t(K) * N > (1u << 20)) {
        std::vector<std::thread> pool;
        for (int i = 0; i < workers; ++i) pool.emplace_back(work);
        for (auto& t : pool) t.join();
    } else {
        work();
    }
    bool safe[65];
    int64_t max_pos[65] = {}, max_neg[65] = {};
    for (int t = 0; t <= 64; ++t) safe[t] = wanted[t];
    for (const auto& r : results) {
        if (!r.codes_ok) return RK_NPU_ERR_PARAM;
        for (int t = 1; t <= limit; ++t) {
            if (!safe[t]) continue;   // the sequential scan stops looking at a tile once it failed
            max_pos[t] = std::max(max_pos[t], r.max_pos[t]);
            max_neg[t] = std::max(max_neg[t], r.max_neg[t]);
            if (r.unsafe[t]) safe[t] = false;
        }
    }
    uint64_t mask = 0;
    for (int t = 1; t <= limit; ++t) if (safe[t]) mask |= uint64_t(1) << (t - 1);
    for (int t = limit; t >= 1; --t)
        if (safe[t]) {
            out = {t * 32, max_pos[t], max_neg[t], mask};
            return RK_NPU_OK;
        }
    return RK_NPU_ERR_PARAM;
}


uint64_t weight_fingerprint(int K, int N, const int8_t* B, const float* scales)
{
    Fnv h;
    h.mix(uint64_t(int64_t(K)));
    h.mix(uint64_t(int64_t(N)));
    h.bytes(B, size_t(K) * N);
    h.bytes(scales, size_t(N) * sizeof(float));
    return h.value;
}

// ================================================================== requests and profiles
namespace {
int widest_tile(int K) { return std::min(2048, align_up(K, 32)); }

// RK_NPU_W4A8_K_TILE_MULTIPLIER: a complete, finite number >= 1; 1 when unset.  false = malformed.
bool multiplier_from_environment(double& factor)
{
    factor = 1;
    const char* text = std::getenv("RK_NPU_W4A8_K_TILE_MULTIPLIER");
    if (!text) return true;
    char* end = nullptr;
    errno = 0;
    const double parsed = std::strtod(text, &end);
    const bool whole = end != text && *end == 0 && errno == 0;
    if (!whole || !std::isfinite(parsed) || parsed < 1) return false;
    factor = parsed;
    return true;
}
bool scales_usable(const float* scale, int N)
{
    return std::all_of(scale, scale + N, [](float s) { return std::isfinite(s) && s > 0; });
}
} // namespace

bool valid_autotune_config(const rk_npu_w4a8_autotune_config& c)
{
    const bool shape = c.M > 0 && c.M <= INT_MAX / 2 && c.K > 0 && c.K <= INT32_MAX / 1024 && c.N > 0 && c.N <= INT_MAX - 63;
    const bool type = c.activation_type == RK_NPU_W4A8_F32 || c.activation_type == RK_NPU_W4A8_F16;
    const bool timing = c.warmup >= 0 && c.loops > 0 && c.repeats > 0 && c.timeout_ms != 0;
    if (!shape || !type || !timing || (c.allowed_npu_core_mask & ~7u)) return false;
    const bool tile = c.required_k_tile >= 0 && c.required_k_tile % 32 == 0 && c.required_k_tile <= widest_tile(c.K);
    const bool factor = std::isfinite(c.k_tile_multiplier) && (c.k_tile_multiplier == 0 || c.k_tile_multiplier >= 1);
    return tile && factor;
}

int make_profile(const rk_npu_w4a8_autotune_config& c, const int8_t* B, const float* scale, Profile& out)
{
    if (!B || !scale || !valid_autotune_config(c)) return RK_NPU_ERR_PARAM;
    // the packed size of the original layout must be representable, as for any weight object
    uint64_t packed = 0;
    const rk_npu_i4_weight_config smallest{c.K, c.N, 32};
    if (const int rc = rk_npu_i4_weights_memory_query(&smallest, &packed)) return rc;
    Profile p;
    p.K = c.K;
    p.N = c.N;
    p.multiplier = c.k_tile_multiplier;
    if (p.multiplier == 0 && !multiplier_from_environment(p.multiplier)) return RK_NPU_ERR_PARAM;
    if (!scales_usable(scale, c.N)) return RK_NPU_ERR_PARAM;
    WeightBound bound;
    if (const int rc = bound_weights(c.K, c.N, B, 0, bound)) return rc;
    p.safe = bound.k_tile;
    p.safe_tiles = bound.safe_tiles;
    const double relaxed = std::min(double(widest_tile(c.K)), double(bound.k_tile) * p.multiplier);
    p.limit = int(relaxed / 32) * 32;
    p.fingerprint = weight_fingerprint(c.K, c.N, B, scale);
    if (c.required_k_tile != 0 && !p.permits(c.required_k_tile)) return RK_NPU_ERR_PARAM;
    out = p;
    return RK_NPU_OK;
}

// ================================================================== host resources of a request
namespace {
uint64_t affinity_mask()
{
    cpu_set_t cpus;
    CPU_ZERO(&cpus);
    uint64_t mask = 0;
    if (::sched_getaffinity(0, sizeof(cpus), &cpus) == 0)
        for (int cpu = 0; cpu < 64 && cpu < CPU_SETSIZE; ++cpu)
            mask |= uint64_t(CPU_ISSET(cpu, &cpus) ? 1 : 0) << cpu;
    return mask ? mask : 1;   // an unreadable or empty affinity counts as CPU 0
}
} // namespace
uint64_t process_cpu_mask() { return affinity_mask(); }
namespace {
// Up to `want` CPUs out of `allowed`, CPUs 4..7 before the others (the fast cores of the SoC the cache
// format was designed on; the resulting mask is a key field, so the order is kept).
uint64_t pick_cpus(uint64_t allowed, int want, int& picked)
{
    std::vector<int> order;
    for (int cpu = 0; cpu < 64; ++cpu)
        if (allowed >> cpu & 1) order.push_back(cpu);
    std::stable_partition(order.begin(), order.end(), [](int cpu) { return cpu >= 4 && cpu <= 7; });
    picked = std::min<int>(want, int(order.size()));
    uint64_t mask = 0;
    for (int i = 0; i < picked; ++i) mask |= uint64_t(1) << order[size_t(i)];
    return mask;
}
// The widest core set, in the original's order of preference, that the request allows and that leaves every
// core at least one 64-column block.
uint32_t pick_device_cores(uint32_t allowed, int N)
{
    if (N < 1) return 0;
    const int64_t blocks = (int64_t(N) + 63) / 64;
    static const uint32_t preference[] = {7u, 3u, 1u, 2u, 4u};
    for (uint32_t mask : preference)
        if ((allowed & mask) == mask && __builtin_popcount(mask) <= blocks) return mask;
    return 0;
}
} // namespace

int chain_token_limit()
{
    const char* text = std::getenv("RK_NPU_W4A8_CHAIN_MAX_M");
    if (!text) return SMALL_BATCH_TOKENS;
    const size_t length = std::strlen(text);
    if (length == 0 || length > 2 || std::strspn(text, "0123456789") != length) return -1;   // digits only, at most 64
    const int value = std::atoi(text);
    return value <= 64 ? value : -1;
}

HostResources host_resources(const rk_npu_w4a8_autotune_config& request)
{
    HostResources r;
    r.chain_tokens = chain_token_limit();
    if (r.chain_tokens < 0) return r;
    const uint64_t affinity = affinity_mask();
    r.cpus_allowed = affinity & (request.allowed_cpu_core_mask ? request.allowed_cpu_core_mask : affinity);
    r.cpus = pick_cpus(r.cpus_allowed, 4, r.threads);
    r.device_cores = pick_device_cores(request.allowed_npu_core_mask ? request.allowed_npu_core_mask : 7u, request.N);
    return r;
}

Strategy widen(const rk_npu_w4a8_strategy& s)
{
    Strategy out{};
    out.base = s;
    rk_npu_w4a8_options_init(&out.execution);
    return out;
}

// ================================================================== rules
namespace {
// Host-thread and pipeline values a strategy may carry for `tokens`: all of the request's threads (one is
// also fine for a small batch); the chain value only up to the chain limit and with more than one K tile;
// the serial value only for a small batch.
bool team_and_pipeline_allowed(const rk_npu_w4a8_config& c, int request_threads, int chain_tokens)
{
    if (request_threads < 1 || request_threads > 4 || chain_tokens < 0) return false;
    const bool small_batch = c.M <= std::max(SMALL_BATCH_TOKENS, chain_tokens);
    const bool team_ok = c.cpu_threads == request_threads || (small_batch && c.cpu_threads == 1);
    bool pipeline_ok = false;
    switch (c.pipeline) {
    case RK_NPU_W4A8_PIPELINED: pipeline_ok = true; break;
    case RK_NPU_W4A8_SERIAL: pipeline_ok = small_batch; break;
    case RK_NPU_W4A8_CHAIN: pipeline_ok = c.M <= chain_tokens && c.K > c.k_tile; break;
    default: break;
    }
    return team_ok && pipeline_ok;
}
bool timings_plausible(const rk_npu_w4a8_strategy& s)
{
    const double values[] = {s.input_us, s.npu_us, s.sync_us, s.output_us, s.total_us, s.jitter_pct, s.robust_us};
    return std::all_of(std::begin(values), std::end(values), [](double v) { return std::isfinite(v) && v >= 0; });
}

struct RuleInput {
    const Strategy& strategy;
    const rk_npu_w4a8_autotune_config& request;
    const Profile& profile;
    const HostResources& res;
    bool extended;
};
struct Rule {
    const char* what;
    bool (*holds)(const RuleInput&);
};
const Rule REQUEST_RULES[] = {
    {"the strategy can run", [](const RuleInput& in) { return strategy_executable(in.strategy, in.extended); }},
    {"same revision and activation type", [](const RuleInput& in) {
         return in.strategy.base.tuning_revision == TUNING_REVISION && in.strategy.base.activation_type == in.request.activation_type; }},
    {"made for these weights", [](const RuleInput& in) { return in.strategy.base.weight_fingerprint == in.profile.fingerprint; }},
    {"made for this shape", [](const RuleInput& in) {
         const auto& c = in.strategy.base.config;
         return c.M == in.request.M && c.N == in.request.N && c.K == in.request.K; }},
    {"carries the request's device cores, CPUs and time limit", [](const RuleInput& in) {
         const auto& s = in.strategy.base;
         return s.config.npu_core_mask == in.res.device_cores && s.cpu_core_mask == in.res.cpus &&
                s.config.timeout_ms == in.request.timeout_ms; }},
    {"team and pipeline fit the request", [](const RuleInput& in) {
         return team_and_pipeline_allowed(in.strategy.base.config, in.res.threads, in.res.chain_tokens); }},
    {"K tile permitted by the weights (and the one the request demands)", [](const RuleInput& in) {
         const int kt = in.strategy.base.config.k_tile;
         return in.profile.permits(kt) && (in.request.required_k_tile == 0 || kt == in.request.required_k_tile); }},
    {"weight block agrees with the profile", [](const RuleInput& in) {
         const auto& s = in.strategy.base;
         const auto& w = s.weights;
         return w.config.K == in.request.K && w.config.N == in.request.N && w.config.k_tile == s.config.k_tile &&
                w.safe_k_tile == in.profile.safe && w.multiplier == in.profile.multiplier &&
                (w.bound_relaxed != 0) == !in.profile.certified(s.config.k_tile); }},
    {"timings are finite and non-negative", [](const RuleInput& in) { return timings_plausible(in.strategy.base); }},
};
} // namespace

bool strategy_executable(const Strategy& s, bool extended)
{
    const auto& o = s.execution;
    if (o.struct_size != sizeof(o) || o.reduce_backend != RK_NPU_W4A8_REDUCE_CPU) return false;
    const bool layout_ok = o.input_layout == RK_NPU_W4A8_INPUT_NATIVE || (extended && o.input_layout == RK_NPU_W4A8_INPUT_PANEL8);
    if (!layout_ok) return false;
    if (!team_and_pipeline_allowed(s.base.config, __builtin_popcountll(s.base.cpu_core_mask), chain_token_limit())) return false;
    rk_npu_w4a8_memory_info_ex unused{};
    return rk_npu_w4a8_memory_query_ex(&s.base.config, &o, &unused) == RK_NPU_OK;
}

bool strategy_acceptable(const Strategy& s, const rk_npu_w4a8_autotune_config& request, const Profile& profile,
                         const HostResources& res, bool extended)
{
    const RuleInput in{s, request, profile, res, extended};
    for (const Rule& rule : REQUEST_RULES)
        if (!rule.holds(in)) return false;
    return true;
}

// ================================================================== cache text
namespace {
// A line of the file is a run of blank-separated tokens.  Each token of a strategy record is described once:
// its wire type and where it lives in the strategy; the writer and the reader both walk this table.
enum class Wire { Int, U32, U64, DoubleBits, Choice };
struct Slot {
    Wire wire;
    size_t offset;
    int lowest, highest;   // Choice: accepted values
};
#define RKB200_SLOT(wire, member) {Wire::wire, offsetof(Strategy, member), 0, 0}
#define RKB200_CHOICE(member, lo, hi) {Wire::Choice, offsetof(Strategy, member), lo, hi}
const Slot RECORD_SLOTS[] = {
    RKB200_SLOT(Int, base.config.M), RKB200_SLOT(Int, base.config.N), RKB200_SLOT(Int, base.config.K),
    RKB200_SLOT(Int, base.config.m_tile), RKB200_SLOT(Int, base.config.k_tile), RKB200_SLOT(Int, base.config.n_tile),
    RKB200_SLOT(U32, base.config.npu_core_mask), RKB200_SLOT(U32, base.config.timeout_ms),
    RKB200_SLOT(Int, base.config.pipeline), RKB200_SLOT(Int, base.config.cpu_threads),
    RKB200_CHOICE(base.activation_type, RK_NPU_W4A8_F32, RK_NPU_W4A8_F16),
    RKB200_SLOT(U64, base.cpu_core_mask),
    RKB200_SLOT(Int, base.weights.config.K), RKB200_SLOT(Int, base.weights.config.N), RKB200_SLOT(Int, base.weights.config.k_tile),
    RKB200_SLOT(Int, base.weights.safe_k_tile), RKB200_SLOT(DoubleBits, base.weights.multiplier),
    RKB200_SLOT(Int, base.weights.bound_relaxed),
    RKB200_SLOT(U64, base.weight_fingerprint), RKB200_SLOT(U32, base.tuning_revision),
    RKB200_SLOT(DoubleBits, base.input_us), RKB200_SLOT(DoubleBits, base.npu_us), RKB200_SLOT(DoubleBits, base.sync_us),
    RKB200_SLOT(DoubleBits, base.output_us), RKB200_SLOT(DoubleBits, base.total_us), RKB200_SLOT(DoubleBits, base.jitter_pct),
    RKB200_SLOT(DoubleBits, base.robust_us),
    RKB200_SLOT(U32, execution.struct_size),
    RKB200_CHOICE(execution.input_layout, RK_NPU_W4A8_INPUT_NATIVE, RK_NPU_W4A8_INPUT_PANEL8),
    RKB200_CHOICE(execution.reduce_backend, RK_NPU_W4A8_REDUCE_CPU, RK_NPU_W4A8_REDUCE_CPU),
};
#undef RKB200_SLOT
#undef RKB200_CHOICE
static_assert(sizeof(rk_npu_w4a8_activation_type) == sizeof(int) && sizeof(rk_npu_w4a8_input_layout) == sizeof(int),
              "enumerations travel as int");

template <class T> T& field(Strategy& s, size_t offset) { return *reinterpret_cast<T*>(reinterpret_cast<char*>(&s) + offset); }
template <class T> const T& field(const Strategy& s, size_t offset)
{
    return *reinterpret_cast<const T*>(reinterpret_cast<const char*>(&s) + offset);
}

std::string record_text(const char* label, const Strategy& s)
{
    std::ostringstream line;
    line.imbue(std::locale::classic());
    line << label;
    for (const Slot& slot : RECORD_SLOTS) {
        line << ' ';
        switch (slot.wire) {
        case Wire::Int: case Wire::Choice: line << field<int>(s, slot.offset); break;
        case Wire::U32: line << field<uint32_t>(s, slot.offset); break;
        case Wire::U64: line << field<uint64_t>(s, slot.offset); break;
        case Wire::DoubleBits: line << double_bits(field<double>(s, slot.offset)); break;
        }
    }
    line << '\n';
    return line.str();
}
template <class T> bool take(std::istream& in, T& value) { return bool(in >> value); }
bool record_parse(std::istream& in, const char* label, Strategy& s)
{
    std::string word;
    if (!take(in, word) || word != label) return false;
    s = Strategy{};
    for (const Slot& slot : RECORD_SLOTS) {
        bool ok = false;
        switch (slot.wire) {
        case Wire::Int: ok = take(in, field<int>(s, slot.offset)); break;
        case Wire::U32: ok = take(in, field<uint32_t>(s, slot.offset)); break;
        case Wire::U64: ok = take(in, field<uint64_t>(s, slot.offset)); break;
        case Wire::DoubleBits: {
            uint64_t bits = 0;
            ok = take(in, bits);
            field<double>(s, slot.offset) = bits_double(bits);
            break;
        }
        case Wire::Choice: {
            int value = 0;
            ok = take(in, value) && value >= slot.lowest && value <= slot.highest;
            field<int>(s, slot.offset) = value;
            break;
        }
        }
        if (!ok) return false;
    }
    return true;
}

// Key line: typed values joined by single blanks, in the order the format fixes.
class KeyLine {
public:
    KeyLine() { text_.imbue(std::locale::classic()); }
    template <class T> KeyLine& add(T value)
    {
        if (!first_) text_ << ' ';
        first_ = false;
        text_ << value;
        return *this;
    }
    std::string str() const { return text_.str(); }
private:
    std::ostringstream text_;
    bool first_ = true;
};
} // namespace

std::string cache_key_line(const rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config& request, const Profile& profile,
                           const HostResources& res, bool extended)
{
    KeyLine key;
    key.add(TUNING_REVISION).add(extended ? 3 : 1)                       // revision, search-space id
        .add(ctx->driver_version)
        .add(request.M).add(request.N).add(request.K).add(int(request.activation_type))
        .add(request.allowed_npu_core_mask ? request.allowed_npu_core_mask : 7u).add(res.cpus_allowed)
        .add(res.device_cores).add(res.cpus)
        .add(request.warmup).add(request.loops).add(request.repeats).add(request.timeout_ms)
        .add(request.required_k_tile)
        .add(profile.fingerprint).add(profile.safe).add(profile.safe_tiles).add(profile.limit)
        .add(double_bits(profile.multiplier))
        .add(res.chain_tokens);
    return key.str();
}

std::string cache_file_for(const std::string& key, const char* directory)
{
    namespace fs = std::filesystem;
    fs::path folder;
    if (directory) {
        folder = directory;
    } else {
        const char* xdg = std::getenv("XDG_CACHE_HOME");
        const char* home = std::getenv("HOME");
        if (xdg && *xdg) folder = xdg;
        else if (home && *home) folder = fs::path(home) / ".cache";
        else return {};
        folder /= "rk_npu_w4a8";
    }
    Fnv h;
    h.bytes(key.data(), key.size());
    char name[32];
    std::snprintf(name, sizeof(name), "%016llx.tune", static_cast<unsigned long long>(h.value));
    return (folder / name).string();
}

int cache_read(const std::string& path, const std::string& key, const rk_npu_w4a8_autotune_config& request,
               const Profile& profile, const HostResources& res, bool extended, Strategy& fastest, Strategy& stable)
{
    std::ifstream file(path, std::ios::binary);
    if (!file) return RK_NPU_ERR_CACHE_MISS;
    file.imbue(std::locale::classic());
    std::string magic, stored_key;
    if (!std::getline(file, magic) || magic != CACHE_MAGIC) return RK_NPU_ERR_CACHE_MISS;
    if (!std::getline(file, stored_key) || stored_key != key) return RK_NPU_ERR_CACHE_MISS;
    Strategy first, second;
    if (!record_parse(file, "fastest", first) || !record_parse(file, "stable", second)) return RK_NPU_ERR_CACHE_MISS;
    // nothing but white space may follow the two records
    char extra = 0;
    if (file >> extra) return RK_NPU_ERR_CACHE_MISS;
    if (!strategy_acceptable(first, request, profile, res, extended) || !strategy_acceptable(second, request, profile, res, extended))
        return RK_NPU_ERR_CACHE_MISS;
    fastest = first;
    stable = second;
    return RK_NPU_OK;
}

// The file appears under its final name only complete: it is written next to it under a name no other
// writer uses (O_EXCL), flushed to the device, and renamed over the target.
int write_file_whole(const std::string& path, const std::string& text);
int cache_write(const std::string& path, const std::string& key, const Strategy& fastest, const Strategy& stable)
{
    return write_file_whole(path, std::string(CACHE_MAGIC) + "\n" + key + "\n" + record_text("fastest", fastest) + record_text("stable", stable));
}
int write_file_whole(const std::string& path, const std::string& text)
{
    namespace fs = std::filesystem;
    if (path.empty()) return RK_NPU_ERR_IO;
    std::error_code ec;
    const fs::path target(path);
    if (target.has_parent_path()) {
        fs::create_directories(target.parent_path(), ec);
        if (ec && !fs::is_directory(target.parent_path())) return RK_NPU_ERR_IO;
    }
    static std::atomic<unsigned> attempt{0};
    std::string scratch;
    int fd = -1;
    for (int tries = 0; tries < 16 && fd < 0; ++tries) {
        char suffix[48];
        std::snprintf(suffix, sizeof(suffix), ".%lx-%x.partial", static_cast<unsigned long>(::getpid()), attempt.fetch_add(1));
        scratch = path + suffix;
        fd = ::open(scratch.c_str(), O_WRONLY | O_CREAT | O_EXCL | O_CLOEXEC, 0600);
        if (fd < 0 && errno != EEXIST) return RK_NPU_ERR_IO;
    }
    if (fd < 0) return RK_NPU_ERR_IO;
    size_t written = 0;
    bool ok = true;
    while (ok && written < text.size()) {
        const ssize_t n = ::write(fd, text.data() + written, text.size() - written);
        if (n < 0 && errno == EINTR) continue;
        ok = n > 0;
        if (ok) written += size_t(n);
    }
    ok = ok && ::fsync(fd) == 0;
    ok = (::close(fd) == 0) && ok;
    ok = ok && ::rename(scratch.c_str(), path.c_str()) == 0;
    if (!ok) ::unlink(scratch.c_str());
    return ok ? RK_NPU_OK : RK_NPU_ERR_IO;
}

// ================================================================== what a strategy selects on this library
Schedule schedule_of(const rk_npu_w4a8_config& c)
{
    Schedule s;
    if (c.pipeline == RK_NPU_W4A8_CHAIN) s.family = 5;
    else if (c.pipeline == RK_NPU_W4A8_SERIAL) s.family = 1;
    else if (c.m_tile == 32) s.family = 1;
    else if (c.m_tile == 48) s.family = 4;
    else if (c.m_tile == 56) s.family = 2;
    if (c.n_tile == 128 || c.n_tile == 256 || c.n_tile == 512 || c.n_tile == 1024) s.cluster = c.n_tile / 128;
    return s;
}
void schedule_into(const Schedule& s, rk_npu_w4a8_config& c)
{
    c.pipeline = RK_NPU_W4A8_PIPELINED;
    c.m_tile = 64;
    c.n_tile = 2048;                              // a value without a cluster meaning: automatic
    switch (s.family) {
    case 5: c.pipeline = RK_NPU_W4A8_CHAIN; break;
    case 1: c.m_tile = 32; break;
    case 4: c.m_tile = 48; break;
    case 2: c.m_tile = 56; break;
    default: break;
    }
    if (s.cluster == 1 || s.cluster == 2 || s.cluster == 4 || s.cluster == 8) c.n_tile = 128 * s.cluster;
    c.n_tile = std::min(c.n_tile, 8128);
}

// ================================================================== cache entry points
namespace {
struct Prepared {
    Profile profile;
    HostResources res;
    std::string key;
};
// Profile from a fresh weight scan, resources, key; the common front of the scanning entry points.
int prepare(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config& request, const int8_t* B, const float* scales, bool extended,
            Prepared& out)
{
    if (const int rc = make_profile(request, B, scales, out.profile)) return rc;
    out.res = host_resources(request);
    if (!out.res.usable()) return RK_NPU_ERR_PARAM;
    out.key = cache_key_line(ctx, request, out.profile, out.res, extended);
    return RK_NPU_OK;
}
void hand_out(rk_npu_w4a8_strategy* to, const Strategy& from) { if (to) *to = from.base; }
void hand_out(rk_npu_w4a8_strategy_ex* to, const Strategy& from) { if (to) *to = from; }
Strategy take_in(const rk_npu_w4a8_strategy& s) { return widen(s); }
Strategy take_in(const rk_npu_w4a8_strategy_ex& s) { return s; }

template <class Public>
int load_scanning(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* request, const int8_t* B, const float* scales,
                  const char* path, Public* fastest, Public* stable)
{
    constexpr bool extended = std::is_same<Public, rk_npu_w4a8_strategy_ex>::value;
    if (!ctx || !request || !fastest || !stable || (path && *path == 0)) return RK_NPU_ERR_PARAM;
    try {
        Prepared p;
        if (const int rc = prepare(ctx, *request, B, scales, extended, p)) return rc;
        Strategy f{}, s{};
        const int rc = cache_read(path ? std::string(path) : cache_file_for(p.key), p.key, *request, p.profile, p.res, extended, f, s);
        if (rc == RK_NPU_OK) { hand_out(fastest, f); hand_out(stable, s); }
        return rc;
    } catch (const std::bad_alloc&) { return RK_NPU_ERR_NOMEM; } catch (...) { return RK_NPU_ERR_PARAM; }
}
template <class Public>
int save_scanning(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* request, const int8_t* B, const float* scales,
                  const char* path, const Public* fastest, const Public* stable)
{
    constexpr bool extended = std::is_same<Public, rk_npu_w4a8_strategy_ex>::value;
    if (!ctx || !request || !fastest || !stable || (path && *path == 0)) return RK_NPU_ERR_PARAM;
    try {
        Prepared p;
        if (const int rc = prepare(ctx, *request, B, scales, extended, p)) return rc;
        const Strategy f = take_in(*fastest), s = take_in(*stable);
        if (!strategy_acceptable(f, *request, p.profile, p.res, extended) || !strategy_acceptable(s, *request, p.profile, p.res, extended))
            return RK_NPU_ERR_PARAM;
        return cache_write(path ? std::string(path) : cache_file_for(p.key), p.key, f, s);
    } catch (const std::bad_alloc&) { return RK_NPU_ERR_NOMEM; } catch (...) { return RK_NPU_ERR_PARAM; }
}

// Weights for a strategy: the weights are scanned again and the strategy has to pass every rule against
// a request rebuilt from its own fields (its masks stand for the resources) before anything is created.
rk_npu_w4a8_weights* weights_for(rk_npu_iommu_domain* domain, const Strategy& strategy, const int8_t* B, const float* scale,
                                 bool extended)
{
    if (!domain || !B || !scale) return nullptr;
    try {
        const auto& s = strategy.base;
        rk_npu_w4a8_autotune_config request;
        rk_npu_w4a8_autotune_config_init(&request, s.config.M, s.config.N, s.config.K);
        request.activation_type = s.activation_type;
        request.timeout_ms = s.config.timeout_ms;
        request.required_k_tile = s.config.k_tile;
        request.k_tile_multiplier = s.weights.multiplier;
        Profile profile;
        if (make_profile(request, B, scale, profile)) return nullptr;
        HostResources res;
        res.device_cores = s.config.npu_core_mask;
        res.cpus = res.cpus_allowed = s.cpu_core_mask;
        res.threads = __builtin_popcountll(s.cpu_core_mask);
        res.chain_tokens = chain_token_limit();
        if (!strategy_acceptable(strategy, request, profile, res, extended)) return nullptr;
        return create_weights(domain, profile.info(request.required_k_tile), B, scale, &profile);
    } catch (...) { return nullptr; }
}
} // namespace
} // namespace rkb200

using namespace rkb200;

struct rk_npu_w4a8_tuning_profile {
    Profile value;
};

extern "C" rk_npu_w4a8_tuning_profile* rk_npu_w4a8_tuning_profile_from_weights(const rk_npu_w4a8_weights* w)
{
    if (!w) return nullptr;
    auto* p = new (std::nothrow) rk_npu_w4a8_tuning_profile;
    if (p) p->value = weights_profile(w);
    return p;
}
extern "C" void rk_npu_w4a8_tuning_profile_free(rk_npu_w4a8_tuning_profile* p) { delete p; }
extern "C" uint64_t rk_npu_w4a8_tuning_profile_fingerprint(const rk_npu_w4a8_tuning_profile* p)
{
    return p ? p->value.fingerprint : 0;
}
extern "C" void rk_npu_w4a8_autotune_config_init(rk_npu_w4a8_autotune_config* c, int M, int N, int K)
{
    if (!c) return;
    *c = {};
    c->M = M; c->N = N; c->K = K;
    c->activation_type = RK_NPU_W4A8_F32;
    c->allowed_npu_core_mask = 7;
    c->warmup = 2; c->loops = 8; c->repeats = 3;
    c->timeout_ms = 500;
}
// Lookup from a captured profile: no weight scan, no device work (include/rk_npu_w4a8_tune.h:46-60).
// The caller states the multiplier policy; a captured profile never adopts a changed environment silently.
extern "C" int rk_npu_w4a8_autotune_cache_load_profile_ex(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* request,
                                                          const rk_npu_w4a8_tuning_profile* profile, const char* path,
                                                          rk_npu_w4a8_strategy_ex* fastest, rk_npu_w4a8_strategy_ex* stable)
{
    if (!ctx || !request || !profile || !fastest || !stable || (path && *path == 0) || !valid_autotune_config(*request))
        return RK_NPU_ERR_PARAM;
    try {
        const Profile& p = profile->value;
        const bool same_weights = p.K == request->K && p.N == request->N && request->k_tile_multiplier == p.multiplier;
        if (!same_weights || (request->required_k_tile != 0 && !p.permits(request->required_k_tile))) return RK_NPU_ERR_PARAM;
        const HostResources res = host_resources(*request);
        if (!res.usable()) return RK_NPU_ERR_PARAM;
        const std::string key = cache_key_line(ctx, *request, p, res, true);
        return cache_read(path ? std::string(path) : cache_file_for(key), key, *request, p, res, true, *fastest, *stable);
    } catch (const std::bad_alloc&) { return RK_NPU_ERR_NOMEM; } catch (...) { return RK_NPU_ERR_PARAM; }
}
extern "C" int rk_npu_w4a8_autotune_cache_load(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* cfg, const int8_t* B,
                                               const float* s, const char* path, rk_npu_w4a8_strategy* fast,
                                               rk_npu_w4a8_strategy* stable)
{
    return load_scanning(ctx, cfg, B, s, path, fast, stable);
}
extern "C" int rk_npu_w4a8_autotune_cache_save(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* cfg, const int8_t* B,
                                               const float* s, const char* path, const rk_npu_w4a8_strategy* fast,
                                               const rk_npu_w4a8_strategy* stable)
{
    return save_scanning(ctx, cfg, B, s, path, fast, stable);
}
extern "C" int rk_npu_w4a8_autotune_cache_load_ex(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* cfg, const int8_t* B,
                                                  const float* s, const char* path, rk_npu_w4a8_strategy_ex* fast,
                                                  rk_npu_w4a8_strategy_ex* stable)
{
    return load_scanning(ctx, cfg, B, s, path, fast, stable);
}
extern "C" int rk_npu_w4a8_autotune_cache_save_ex(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* cfg, const int8_t* B,
                                                  const float* s, const char* path, const rk_npu_w4a8_strategy_ex* fast,
                                                  const rk_npu_w4a8_strategy_ex* stable)
{
    return save_scanning(ctx, cfg, B, s, path, fast, stable);
}
extern "C" rk_npu_w4a8_weights* rk_npu_w4a8_weights_create_tuned(rk_npu_iommu_domain* domain, const rk_npu_w4a8_strategy* s,
                                                                 const int8_t* B, const float* scale)
{
    return s ? weights_for(domain, widen(*s), B, scale, false) : nullptr;
}
extern "C" rk_npu_w4a8_weights* rk_npu_w4a8_weights_create_tuned_ex(rk_npu_iommu_domain* domain,
                                                                    const rk_npu_w4a8_strategy_ex* s, const int8_t* B,
                                                                    const float* scale)
{
    return s ? weights_for(domain, *s, B, scale, true) : nullptr;
}
// A workspace that runs the schedule the strategy's fields select (see schedule_of in w4a8_tune.h).
extern "C" rk_npu_w4a8_workspace* rk_npu_w4a8_workspace_create_tuned_ex(rk_npu_iommu_domain* domain,
                                                                        const rk_npu_w4a8_strategy_ex* s)
{
    if (!s || s->base.tuning_revision != TUNING_REVISION || !strategy_executable(*s, true)) return nullptr;
    const auto& c = s->base.config;
    const auto& w = s->base.weights.config;
    if (c.K != w.K || c.N != w.N || c.k_tile != w.k_tile) return nullptr;
    return create_workspace_scheduled(domain, &c, &s->execution, schedule_of(c));
}

// ================================================================== W8 load-only tuning cache
// The second public header's cache reader, restated from src/rk_npu_quant_matmul.cpp:183-349
// (key fields, record fields, validity rules) and :1522-1563 (defaults, entry point).  The
// records describe executions of the original device; this library only has to answer the
// question "is there a valid, current record for this request" the way the original does.
namespace rkb200 {
namespace {
constexpr const char* W8_CACHE_MAGIC = "rk_npu_matmul_tuning_cache_v2";
constexpr uint32_t W8_CACHE_FORMAT = 2, W8_TUNING_REVISION = 6;
constexpr int W8_N_TILE_MAX = 3072, W8_CHANNEL_TILE = 32;

struct W8Key {
    uint32_t format = W8_CACHE_FORMAT, revision = W8_TUNING_REVISION, driver = 0;
    int op = 0, M = 0, N = 0, K = 0;
    uint32_t npu = 0;
    uint64_t cpu = 0;
    int warmup = 0, loops = 0, repeats = 0;
    uint32_t timeout_ms = 0;
    int required_k_tile = 0;
    bool operator==(const W8Key& o) const
    {
        return format == o.format && revision == o.revision && driver == o.driver && op == o.op && M == o.M && N == o.N &&
               K == o.K && npu == o.npu && cpu == o.cpu && warmup == o.warmup && loops == o.loops && repeats == o.repeats &&
               timeout_ms == o.timeout_ms && required_k_tile == o.required_k_tile;
    }
};
bool w8_kind_ok(int kind) { return kind >= RK_NPU_MATMUL_I8I8I32 && kind <= RK_NPU_MATMUL_F32I8F32_STATIC; }
// bit 0: reduction on the device, bit 1: dequantisation on the device; both chosen by the
// original's environment switches and part of a record's identity
uint32_t w8_execution_mode(int kind)
{
    auto on = [](const char* name) { const char* v = std::getenv(name); return v && std::strcmp(v, "1") == 0; };
    const bool dequant = kind != RK_NPU_MATMUL_I8I8I32 && on("RK_NPU_W8A8_NPU_DEQUANT");
    return ((on("RK_NPU_I8_NPU_REDUCE") || dequant) ? 1u : 0u) | (dequant ? 2u : 0u);
}
bool w8_config_ok(const rk_npu_matmul_autotune_config* c)
{
    return c && c->M > 0 && c->N > 0 && c->K > 0 && (c->allowed_npu_core_mask & ~7u) == 0 && c->warmup >= 0 && c->loops > 0 &&
           c->repeats > 0 && c->timeout_ms > 0 && c->required_k_tile >= 0 && c->required_k_tile <= c->K;
}
bool w8_make_key(const rk_npu_ctx* ctx, const rk_npu_matmul_autotune_config* c, int kind, W8Key& key)
{
    if (!ctx || !w8_config_ok(c) || !w8_kind_ok(kind)) return false;
    const uint64_t affinity = affinity_mask();
    key.driver = ctx->driver_version;
    key.revision |= w8_execution_mode(kind) << 16;
    key.op = kind;
    key.M = c->M; key.N = c->N; key.K = c->K;
    key.npu = c->allowed_npu_core_mask ? c->allowed_npu_core_mask : 7u;
    key.cpu = (c->allowed_cpu_core_mask ? c->allowed_cpu_core_mask : affinity) & affinity;
    key.warmup = c->warmup; key.loops = c->loops; key.repeats = c->repeats;
    key.timeout_ms = c->timeout_ms;
    key.required_k_tile = c->required_k_tile;
    return key.cpu != 0 && key.npu != 0;
}
bool w8_read_record(std::istream& in, const char* label, rk_npu_matmul_strategy& s)
{
    std::string word;
    int op = 0, a = 0, c = 0;
    uint64_t t[7] = {};
    if (!(in >> word >> op >> s.M >> s.N >> s.K >> s.k_tile >> s.n_tile >> a >> c >> s.wave_count >> s.n_groups >>
          s.npu_core_mask >> s.cpu_core_mask >> s.cpu_threads >> t[0] >> t[1] >> t[2] >> t[3] >> t[4] >> t[5] >> t[6]) ||
        word != label)
        return false;
    s.op_kind = static_cast<rk_npu_matmul_op_kind>(op);
    s.a_layout = static_cast<rk_npu_matmul_a_layout>(a);
    s.c_layout = static_cast<rk_npu_matmul_c_layout>(c);
    s.input_us = bits_double(t[0]); s.npu_us = bits_double(t[1]); s.sync_us = bits_double(t[2]);
    s.output_us = bits_double(t[3]); s.total_us = bits_double(t[4]); s.jitter_pct = bits_double(t[5]);
    s.robust_us = bits_double(t[6]);
    return true;
}
bool w8_record_ok(const rk_npu_matmul_strategy& s, const W8Key& key)
{
    const uint32_t m = s.npu_core_mask;
    if (int(s.op_kind) != key.op || s.M <= 0 || s.N <= 0 || s.K <= 0 || s.k_tile <= 0 || s.k_tile > s.K || s.n_tile <= 0 ||
        s.n_tile > W8_N_TILE_MAX || s.a_layout < RK_NPU_MATMUL_A_LAYOUT_NORMAL || s.a_layout > RK_NPU_MATMUL_A_LAYOUT_PANEL16 ||
        s.c_layout < RK_NPU_MATMUL_C_LAYOUT_NATIVE || s.c_layout > RK_NPU_MATMUL_C_LAYOUT_PANEL16 ||
        !(m == 1u || m == 2u || m == 4u || m == 3u || m == 7u) || s.cpu_core_mask == 0 || s.cpu_threads <= 0 ||
        s.cpu_threads != __builtin_popcountll(s.cpu_core_mask) || (s.cpu_core_mask & ~affinity_mask()))
        return false;
    // Panel recipes describe the original device's buffers and change nothing here, but a record is a hit only where
    // the original would accept it.
    if (!rkb200::w8_panel_recipe_ok(s.M, s.N, s.k_tile, int(s.a_layout), int(s.c_layout))) return false;
    const int align_n = std::max(W8_CHANNEL_TILE, rkb200::align_up(s.N, W8_CHANNEL_TILE));
    const int nt = std::min(align_n, rkb200::align_up(s.n_tile, W8_CHANNEL_TILE));
    if ((align_n + nt - 1) / nt < __builtin_popcount(m)) return false;
    if (s.M != key.M || s.N != key.N || s.K != key.K || (m & ~key.npu) || (s.cpu_core_mask & ~key.cpu) ||
        s.n_tile != rkb200::align_up(s.n_tile, W8_CHANNEL_TILE) || (key.required_k_tile > 0 && s.k_tile != key.required_k_tile) ||
        s.wave_count != (s.K + s.k_tile - 1) / s.k_tile || s.n_groups != (align_n + s.n_tile - 1) / s.n_tile)
        return false;
    for (double v : {s.input_us, s.npu_us, s.sync_us, s.output_us, s.total_us, s.jitter_pct, s.robust_us})
        if (!std::isfinite(v) || v < 0) return false;
    return true;
}
} // namespace

bool w8_panel_recipe_ok(int M, int N, int k_tile, int a_layout, int c_layout)
{
    const int a_width = a_layout == RK_NPU_MATMUL_A_LAYOUT_PANEL8 ? 8 : a_layout == RK_NPU_MATMUL_A_LAYOUT_PANEL16 ? 16 : 0;
    const int c_width = c_layout == RK_NPU_MATMUL_C_LAYOUT_PANEL8 ? 8 : c_layout == RK_NPU_MATMUL_C_LAYOUT_PANEL16 ? 16 : 0;
    if (a_width && c_width && c_width != a_width) return false;                 // a panel input writes a native output or panels of its own width
    if (!a_width && c_width && !(a_layout == RK_NPU_MATMUL_A_LAYOUT_NORMAL && c_width == 8)) return false;
    const int width = std::max(a_width, c_width);
    if (!width) return true;
    // every K wave is checked by the original; the widest is k_tile and every bound falls with K
    if (M % width || k_tile > 8192 || (a_width == 8 && k_tile > 2048) || (a_width == 16 && k_tile > 4096)) return false;
    if (c_width && int64_t(rkb200::align_up(N, 32) / 4 - 1) * c_width > 8191) return false;
    return true;
}
} // namespace rkb200

extern "C" void rk_npu_matmul_autotune_config_init(rk_npu_matmul_autotune_config* c, int M, int N, int K)
{
    if (!c) return;
    *c = {};
    c->M = M; c->N = N; c->K = K;
    c->allowed_npu_core_mask = 7;
    c->warmup = 2; c->loops = 8; c->repeats = 3;
    c->timeout_ms = 500;
}
extern "C" void rk_npu_matmul_family_autotune_config_init(rk_npu_matmul_family_autotune_config* c, int N, int K, int m_count,
                                                          const int* m_values)
{
    if (!c) return;
    *c = {};
    c->K = K; c->N = N;
    c->m_count = m_count;
    c->m_values = m_values;
    c->allowed_npu_core_mask = 7;
    c->warmup = 2; c->loops = 8; c->repeats = 3;
    c->timeout_ms = 500;
}
extern "C" int rk_npu_matmul_autotune_cache_load(rk_npu_ctx* ctx, const char* path, rk_npu_matmul_op_kind kind,
                                                 const rk_npu_matmul_autotune_config* cfg, rk_npu_matmul_strategy* fastest,
                                                 rk_npu_matmul_strategy* stable)
{
    using namespace rkb200;
    try {
        if (!path || !*path || !fastest || !stable) return RK_NPU_ERR_PARAM;
        W8Key expected;
        if (!w8_make_key(ctx, cfg, int(kind), expected)) return RK_NPU_ERR_PARAM;
        std::ifstream in(path, std::ios::binary);
        if (!in) return RK_NPU_ERR_CACHE_MISS;
        in.imbue(std::locale::classic());
        std::string magic, label;
        W8Key stored;
        rk_npu_matmul_strategy f{}, s{};
        if (!(in >> magic >> label >> stored.format >> stored.revision >> stored.driver >> stored.op >> stored.M >> stored.N >>
              stored.K >> stored.npu >> stored.cpu >> stored.warmup >> stored.loops >> stored.repeats >> stored.timeout_ms >>
              stored.required_k_tile) ||
            magic != W8_CACHE_MAGIC || label != "key" || !(stored == expected) || !w8_read_record(in, "fastest", f) ||
            !w8_read_record(in, "stable", s) || !w8_record_ok(f, expected) || !w8_record_ok(s, expected))
            return RK_NPU_ERR_CACHE_MISS;
        in >> std::ws;
        if (!in.eof()) return RK_NPU_ERR_CACHE_MISS;
        *fastest = f;
        *stable = s;
        return RK_NPU_OK;
    } catch (...) { return RK_NPU_ERR_PARAM; }
}
// src/rk_npu_quant_matmul.cpp:1565-1579 (checks), :266-277,336-349 (text): the same bytes the original writes.
extern "C" int rk_npu_matmul_autotune_cache_save(rk_npu_ctx* ctx, const char* path, rk_npu_matmul_op_kind kind,
                                                 const rk_npu_matmul_autotune_config* cfg, const rk_npu_matmul_strategy* fastest,
                                                 const rk_npu_matmul_strategy* stable)
{
    using namespace rkb200;
    try {
        if (!path || !*path || !fastest || !stable) return RK_NPU_ERR_PARAM;
        W8Key key;
        if (!w8_make_key(ctx, cfg, int(kind), key) || !w8_record_ok(*fastest, key) || !w8_record_ok(*stable, key)) return RK_NPU_ERR_PARAM;
        std::ostringstream out;
        out.imbue(std::locale::classic());
        out << W8_CACHE_MAGIC << '\n'
            << "key " << key.format << ' ' << key.revision << ' ' << key.driver << ' ' << key.op << ' ' << key.M << ' ' << key.N << ' '
            << key.K << ' ' << key.npu << ' ' << key.cpu << ' ' << key.warmup << ' ' << key.loops << ' ' << key.repeats << ' '
            << key.timeout_ms << ' ' << key.required_k_tile << '\n';
        auto record = [&](const char* label, const rk_npu_matmul_strategy& s) {
            out << label << ' ' << int(s.op_kind) << ' ' << s.M << ' ' << s.N << ' ' << s.K << ' ' << s.k_tile << ' ' << s.n_tile << ' '
                << int(s.a_layout) << ' ' << int(s.c_layout) << ' ' << s.wave_count << ' ' << s.n_groups << ' ' << s.npu_core_mask << ' '
                << s.cpu_core_mask << ' ' << s.cpu_threads;
            for (double v : {s.input_us, s.npu_us, s.sync_us, s.output_us, s.total_us, s.jitter_pct, s.robust_us}) out << ' ' << double_bits(v);
            out << '\n';
        };
        record("fastest", *fastest);
        record("stable", *stable);
        return write_file_whole(path, out.str());
    } catch (...) { return RK_NPU_ERR_PARAM; }
}
extern "C" void rk_npu_i4_config_init(rk_npu_i4_config* c, int M, int N, int K)
{
    if (c) *c = {M, N, K, 128, 480, 1024, 1, 500, 1, 1};
}
extern "C" void rk_npu_w4a8_family_config_init(rk_npu_w4a8_family_config* c, int N, int K, int m_count, const int* m_values)
{
    if (!c) return;
    *c = {};
    rk_npu_w4a8_autotune_config_init(&c->base, 1, N, K);
    c->m_count = m_count;
    c->m_values = m_values;
}
