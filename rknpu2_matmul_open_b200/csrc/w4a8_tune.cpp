// w4a8_tune.cpp -- weight certification, weight identity and the tuning cache.
// Pure host code: nothing here touches the GPU, so a cache lookup costs file I/O only
// (the reference's contract, include/rk_npu_w4a8_tune.h:46-49).
//
// Restates, for this library's handles:
//   bound_weights      src/rk_npu_i4_bounds.cpp:9-69
//   weight_fingerprint src/rk_npu_autotune_common.cpp:83-89, src/rk_npu_w4a8.cpp:275-277
//   make_profile       src/rk_npu_w4a8_tune_policy.cpp:41-62
//   resources / key / strategy validity   src/rk_npu_w4a8_tune_policy.cpp:14-33,63-71,123-155
//   cache text format  src/rk_npu_w4a8_tune_cache.cpp:7-60, src/rk_npu_autotune_cache.cpp:15-63
// The cache files are interchangeable with the reference's: same magic line, same key
// line (the driver-version field holds the CUDA driver version here), same records.
#include "w4a8_host.h"
#include "../../include/rknpu_b200_quant.h"
#include <algorithm>
#include <atomic>
#include <cerrno>
#include <climits>
#include <cmath>
#include <cstdlib>
#include <cstring>
#include <fstream>
#include <iomanip>
#include <locale>
#include <sched.h>
#include <sstream>
#include <sys/stat.h>
#include <thread>
#include <unistd.h>
#include <vector>

namespace rkb200 {
namespace {
constexpr uint32_t TUNING_REVISION = 5;
constexpr int SMALL_BATCH_LIMIT = 8;
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

bool valid_autotune_config(const rk_npu_w4a8_autotune_config& c)
{
    return c.M > 0 && c.M <= INT_MAX / 2 && c.K > 0 && c.K <= INT32_MAX / 1024 && c.N > 0 && c.N <= INT_MAX - 63 &&
           (c.activation_type == RK_NPU_W4A8_F32 || c.activation_type == RK_NPU_W4A8_F16) &&
           !(c.allowed_npu_core_mask & ~7u) && c.warmup >= 0 && c.loops > 0 && c.repeats > 0 && c.timeout_ms &&
           c.required_k_tile >= 0 && c.required_k_tile <= std::min(2048, align_up(c.K, 32)) && c.required_k_tile % 32 == 0 &&
           std::isfinite(c.k_tile_multiplier) && (c.k_tile_multiplier == 0 || c.k_tile_multiplier >= 1);
}

int make_profile(const rk_npu_w4a8_autotune_config& c, const int8_t* B, const float* scale, Profile& out)
{
    if (!valid_autotune_config(c) || !B || !scale) return RK_NPU_ERR_PARAM;
    uint64_t bytes = 0;
    const rk_npu_i4_weight_config key{c.K, c.N, 32};
    int rc = rk_npu_i4_weights_memory_query(&key, &bytes);
    if (rc) return rc;
    double factor = c.k_tile_multiplier;
    if (factor == 0) {
        factor = 1;
        if (const char* text = std::getenv("RK_NPU_W4A8_K_TILE_MULTIPLIER")) {
            errno = 0;
            char* end = nullptr;
            factor = std::strtod(text, &end);
            if (errno || end == text || *end || !std::isfinite(factor) || factor < 1) return RK_NPU_ERR_PARAM;
        }
    }
    for (int n = 0; n < c.N; ++n)
        if (!std::isfinite(scale[n]) || scale[n] <= 0) return RK_NPU_ERR_PARAM;
    WeightBound b;
    rc = bound_weights(c.K, c.N, B, 0, b);
    if (rc) return rc;
    Profile p;
    p.K = c.K;
    p.N = c.N;
    p.safe = b.k_tile;
    p.safe_tiles = b.safe_tiles;
    p.multiplier = factor;
    p.limit = int(std::min(double(std::min(2048, align_up(c.K, 32))), b.k_tile * factor) / 32) * 32;
    p.fingerprint = weight_fingerprint(c.K, c.N, B, scale);
    if (c.required_k_tile && !p.permits(c.required_k_tile)) return RK_NPU_ERR_PARAM;
    out = p;
    return RK_NPU_OK;
}

namespace {
// ------------------------------------------------------------------ resources
struct Resources {
    uint32_t npu = 0;
    uint64_t cpu = 0, allowed_cpu = 0;
    int threads = 0;
    int chain_max_m = 8;
};

int chain_max_m()   // RK_NPU_W4A8_CHAIN_MAX_M: integer 0..64, default 8, -1 when malformed
{
    const char* text = std::getenv("RK_NPU_W4A8_CHAIN_MAX_M");
    if (!text) return 8;
    if (!*text) return -1;
    int value = 0;
    for (const char* p = text; *p; ++p) {
        if (*p < '0' || *p > '9') return -1;
        value = value * 10 + (*p - '0');
        if (value > 64) return -1;
    }
    return value;
}
uint64_t process_cpu_mask()
{
    cpu_set_t set;
    CPU_ZERO(&set);
    if (::sched_getaffinity(0, sizeof(set), &set) != 0) return 1;
    uint64_t mask = 0;
    for (int c = 0; c < 64 && c < CPU_SETSIZE; ++c) if (CPU_ISSET(c, &set)) mask |= 1ull << c;
    return mask ? mask : 1;
}
// CPUs 4..7 first (the big cores of the original SoC), then the rest in order; kept so
// that the masks written into cache keys and strategies mean the same thing.
std::vector<int> preferred_cpus(uint64_t allowed)
{
    std::vector<int> cpus;
    for (int c = 4; c <= 7; ++c) if (allowed & (1ull << c)) cpus.push_back(c);
    for (int c = 0; c < 64; ++c) if ((c < 4 || c > 7) && (allowed & (1ull << c))) cpus.push_back(c);
    return cpus;
}
uint64_t first_cpu_mask(const std::vector<int>& cpus, int count)
{
    uint64_t mask = 0;
    for (int i = 0; i < count && i < int(cpus.size()); ++i) mask |= 1ull << cpus[size_t(i)];
    return mask;
}
uint32_t fixed_npu_mask(uint32_t allowed, int N, int alignment)
{
    if (N < 1 || alignment < 1) return 0;
    const int groups = int((int64_t(N) + alignment - 1) / alignment);
    for (uint32_t mask : {7u, 3u, 1u, 2u, 4u})
        if ((mask & allowed) == mask && __builtin_popcount(mask) <= groups) return mask;
    return 0;
}
Resources resolve_resources(const rk_npu_w4a8_autotune_config& c)
{
    Resources r;
    const uint64_t affinity = process_cpu_mask();
    r.chain_max_m = chain_max_m();
    if (r.chain_max_m < 0) return r;
    r.allowed_cpu = (c.allowed_cpu_core_mask ? c.allowed_cpu_core_mask : affinity) & affinity;
    const auto cpus = preferred_cpus(r.allowed_cpu);
    r.threads = std::min(4, int(cpus.size()));
    r.cpu = first_cpu_mask(cpus, r.threads);
    r.npu = fixed_npu_mask(c.allowed_npu_core_mask ? c.allowed_npu_core_mask : 7, c.N, 64);
    return r;
}

// ------------------------------------------------------------------ strategy validity
using Strategy = rk_npu_w4a8_strategy_ex;
Strategy extend(const rk_npu_w4a8_strategy& s)
{
    return {s, {uint32_t(sizeof(rk_npu_w4a8_options)), RK_NPU_W4A8_INPUT_NATIVE, RK_NPU_W4A8_REDUCE_CPU}};
}
bool cpu_policy_ok(const rk_npu_w4a8_config& c, int maximum_threads, int chain_limit)
{
    if (maximum_threads < 1 || maximum_threads > 4 || chain_limit < 0) return false;
    const bool small = c.M <= std::max(SMALL_BATCH_LIMIT, chain_limit);
    if (c.cpu_threads != maximum_threads && !(small && c.cpu_threads == 1)) return false;
    if (c.pipeline == RK_NPU_W4A8_CHAIN) return c.M <= chain_limit && c.K > c.k_tile;
    return c.pipeline == RK_NPU_W4A8_PIPELINED || (small && c.pipeline == RK_NPU_W4A8_SERIAL);
}
bool execution_ok(const Strategy& s, bool panel8)
{
    const auto& o = s.execution;
    if (!cpu_policy_ok(s.base.config, __builtin_popcountll(s.base.cpu_core_mask), chain_max_m()) ||
        o.struct_size != sizeof(o) || o.reduce_backend != RK_NPU_W4A8_REDUCE_CPU ||
        (o.input_layout != RK_NPU_W4A8_INPUT_NATIVE && (!panel8 || o.input_layout != RK_NPU_W4A8_INPUT_PANEL8)))
        return false;
    rk_npu_w4a8_memory_info_ex info{};
    return !rk_npu_w4a8_memory_query_ex(&s.base.config, &o, &info);
}
bool strategy_ok(const Strategy& strategy, const rk_npu_w4a8_autotune_config& c, const Profile& p, const Resources& r,
                 bool panel8)
{
    const auto& s = strategy.base;
    if (!execution_ok(strategy, panel8)) return false;
    const auto& a = s.config;
    const auto& w = s.weights;
    if (s.tuning_revision != TUNING_REVISION || s.activation_type != c.activation_type ||
        s.weight_fingerprint != p.fingerprint || a.M != c.M || a.N != c.N || a.K != c.K || a.npu_core_mask != r.npu ||
        !cpu_policy_ok(a, r.threads, r.chain_max_m) || s.cpu_core_mask != r.cpu || a.timeout_ms != c.timeout_ms ||
        !p.permits(a.k_tile) || (c.required_k_tile && a.k_tile != c.required_k_tile) || w.config.K != c.K ||
        w.config.N != c.N || w.config.k_tile != a.k_tile || w.safe_k_tile != p.safe || w.multiplier != p.multiplier ||
        w.bound_relaxed != !p.certified(a.k_tile))
        return false;
    for (double t : {s.input_us, s.npu_us, s.sync_us, s.output_us, s.total_us, s.jitter_pct, s.robust_us})
        if (!std::isfinite(t) || t < 0) return false;
    return true;
}

// ------------------------------------------------------------------ cache text
std::string cache_key(const rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config& c, const Profile& p, const Resources& r,
                      bool panel8)
{
    std::ostringstream out;
    out.imbue(std::locale::classic());
    out << TUNING_REVISION << ' ' << (panel8 ? 3 : 1) << ' ' << ctx->driver_version << ' ' << c.M << ' ' << c.N << ' '
        << c.K << ' ' << int(c.activation_type) << ' ' << (c.allowed_npu_core_mask ? c.allowed_npu_core_mask : 7) << ' '
        << r.allowed_cpu << ' ' << r.npu << ' ' << r.cpu << ' ' << c.warmup << ' ' << c.loops << ' ' << c.repeats << ' '
        << c.timeout_ms << ' ' << c.required_k_tile << ' ' << p.fingerprint << ' ' << p.safe << ' ' << p.safe_tiles
        << ' ' << p.limit << ' ' << double_bits(p.multiplier) << ' ' << r.chain_max_m;
    return out.str();
}
std::string default_cache_path(const std::string& key)
{
    Fnv h;
    h.bytes(key.data(), key.size());
    std::string base;
    const char* xdg = std::getenv("XDG_CACHE_HOME");
    const char* home = std::getenv("HOME");
    if (xdg && *xdg) base = xdg;
    else if (home && *home) base = std::string(home) + "/.cache";
    else return {};
    base += "/rk_npu_w4a8";
    std::ostringstream path;
    path.imbue(std::locale::classic());
    path << base << '/' << std::hex << std::setfill('0') << std::setw(16) << h.value << ".tune";
    return path.str();
}
void write_record(std::ostream& out, const char* label, const Strategy& strategy)
{
    const auto& s = strategy.base;
    const auto& c = s.config;
    const auto& w = s.weights;
    out << label << ' ' << c.M << ' ' << c.N << ' ' << c.K << ' ' << c.m_tile << ' ' << c.k_tile << ' ' << c.n_tile << ' '
        << c.npu_core_mask << ' ' << c.timeout_ms << ' ' << c.pipeline << ' ' << c.cpu_threads << ' '
        << int(s.activation_type) << ' ' << s.cpu_core_mask << ' ' << w.config.K << ' ' << w.config.N << ' '
        << w.config.k_tile << ' ' << w.safe_k_tile << ' ' << double_bits(w.multiplier) << ' ' << w.bound_relaxed << ' '
        << s.weight_fingerprint << ' ' << s.tuning_revision;
    for (double d : {s.input_us, s.npu_us, s.sync_us, s.output_us, s.total_us, s.jitter_pct, s.robust_us})
        out << ' ' << double_bits(d);
    out << ' ' << strategy.execution.struct_size << ' ' << int(strategy.execution.input_layout) << ' '
        << int(strategy.execution.reduce_backend) << '\n';
}
bool read_record(std::istream& in, const char* label, Strategy& strategy)
{
    auto& s = strategy.base;
    auto& c = s.config;
    auto& w = s.weights;
    std::string name;
    int dtype = 0;
    uint64_t factor = 0;
    if (!(in >> name >> c.M >> c.N >> c.K >> c.m_tile >> c.k_tile >> c.n_tile >> c.npu_core_mask >> c.timeout_ms >>
          c.pipeline >> c.cpu_threads >> dtype >> s.cpu_core_mask >> w.config.K >> w.config.N >> w.config.k_tile >>
          w.safe_k_tile >> factor >> w.bound_relaxed >> s.weight_fingerprint >> s.tuning_revision) ||
        name != label || (dtype != RK_NPU_W4A8_F32 && dtype != RK_NPU_W4A8_F16))
        return false;
    s.activation_type = static_cast<rk_npu_w4a8_activation_type>(dtype);
    w.multiplier = bits_double(factor);
    for (double* d : {&s.input_us, &s.npu_us, &s.sync_us, &s.output_us, &s.total_us, &s.jitter_pct, &s.robust_us}) {
        uint64_t bits;
        if (!(in >> bits)) return false;
        *d = bits_double(bits);
    }
    int layout = 0, reduce = 0;
    if (!(in >> strategy.execution.struct_size >> layout >> reduce) ||
        (layout != RK_NPU_W4A8_INPUT_NATIVE && layout != RK_NPU_W4A8_INPUT_PANEL8) || reduce != RK_NPU_W4A8_REDUCE_CPU)
        return false;
    strategy.execution.input_layout = static_cast<rk_npu_w4a8_input_layout>(layout);
    strategy.execution.reduce_backend = static_cast<rk_npu_w4a8_reduce_backend>(reduce);
    return true;
}
int load_file(const std::string& path, const std::string& expected, const rk_npu_w4a8_autotune_config& cfg,
              const Profile& profile, const Resources& res, Strategy& fast, Strategy& stable, bool panel8)
{
    std::ifstream in(path, std::ios::binary);
    if (!in) return RK_NPU_ERR_CACHE_MISS;
    in.imbue(std::locale::classic());
    std::string header, key;
    Strategy f{}, s{};
    if (!std::getline(in, header) || header != CACHE_MAGIC || !std::getline(in, key) || key != expected ||
        !read_record(in, "fastest", f) || !read_record(in, "stable", s) || !strategy_ok(f, cfg, profile, res, panel8) ||
        !strategy_ok(s, cfg, profile, res, panel8))
        return RK_NPU_ERR_CACHE_MISS;
    in >> std::ws;
    if (!in.eof()) return RK_NPU_ERR_CACHE_MISS;   // trailing bytes make the file invalid
    fast = f;
    stable = s;
    return RK_NPU_OK;
}
bool make_parents(const std::string& path)
{
    const size_t slash = path.find_last_of('/');
    if (slash == std::string::npos) return true;
    const std::string parent = path.substr(0, slash);
    if (parent.empty()) return true;
    for (size_t pos = parent[0] == '/' ? 1 : 0;;) {
        pos = parent.find('/', pos);
        const auto part = parent.substr(0, pos);
        if (!part.empty() && ::mkdir(part.c_str(), 0700) != 0 && errno != EEXIST) return false;
        if (pos == std::string::npos) break;
        ++pos;
    }
    return true;
}
int save_file(const std::string& path, const std::string& key, const Strategy& fast, const Strategy& stable)
{
    if (path.empty() || !make_parents(path)) return RK_NPU_ERR_IO;
    static std::atomic<uint64_t> serial{0};
    const std::string tmp = path + ".tmp." + std::to_string((long long)::getpid()) + "." +
                            std::to_string(serial.fetch_add(1, std::memory_order_relaxed));
    {
        std::ofstream out(tmp, std::ios::binary | std::ios::trunc);
        if (!out) return RK_NPU_ERR_IO;
        out.imbue(std::locale::classic());
        out << CACHE_MAGIC << '\n' << key << '\n';
        write_record(out, "fastest", fast);
        write_record(out, "stable", stable);
        out.close();
        if (!out) { ::unlink(tmp.c_str()); return RK_NPU_ERR_IO; }
    }
    if (::rename(tmp.c_str(), path.c_str()) != 0) { ::unlink(tmp.c_str()); return RK_NPU_ERR_IO; }
    return RK_NPU_OK;
}

template <bool EX, class S>
int load_entry(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* cfg, const int8_t* B, const float* scales,
               const char* path, S* fast, S* stable)
{
    if (!ctx || !cfg || !fast || !stable || (path && !*path)) return RK_NPU_ERR_PARAM;
    try {
        Profile p;
        int rc = make_profile(*cfg, B, scales, p);
        if (rc) return rc;
        const Resources r = resolve_resources(*cfg);
        if (!r.npu || !r.threads) return RK_NPU_ERR_PARAM;
        const std::string key = cache_key(ctx, *cfg, p, r, EX);
        Strategy f{}, s{};
        rc = load_file(path ? std::string(path) : default_cache_path(key), key, *cfg, p, r, f, s, EX);
        if (!rc) {
            if constexpr (EX) { *fast = f; *stable = s; }
            else { *fast = f.base; *stable = s.base; }
        }
        return rc;
    } catch (const std::bad_alloc&) { return RK_NPU_ERR_NOMEM; } catch (...) { return RK_NPU_ERR_PARAM; }
}
template <bool EX, class S>
int save_entry(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* cfg, const int8_t* B, const float* scales,
               const char* path, const S* fast, const S* stable)
{
    if (!ctx || !cfg || !fast || !stable || (path && !*path)) return RK_NPU_ERR_PARAM;
    try {
        Profile p;
        int rc = make_profile(*cfg, B, scales, p);
        if (rc) return rc;
        const Resources r = resolve_resources(*cfg);
        if (!r.npu || !r.threads) return RK_NPU_ERR_PARAM;
        Strategy f, s;
        if constexpr (EX) { f = *fast; s = *stable; }
        else { f = extend(*fast); s = extend(*stable); }
        if (!strategy_ok(f, *cfg, p, r, EX) || !strategy_ok(s, *cfg, p, r, EX)) return RK_NPU_ERR_PARAM;
        const std::string key = cache_key(ctx, *cfg, p, r, EX);
        return save_file(path ? std::string(path) : default_cache_path(key), key, f, s);
    } catch (const std::bad_alloc&) { return RK_NPU_ERR_NOMEM; } catch (...) { return RK_NPU_ERR_PARAM; }
}

rk_npu_w4a8_weights* create_tuned(rk_npu_iommu_domain* domain, const Strategy& strategy, const int8_t* B,
                                  const float* scale, bool panel8)
{
    const auto& s = strategy.base;
    if (!domain || !B || !scale) return nullptr;
    try {
        rk_npu_w4a8_autotune_config c;
        rk_npu_w4a8_autotune_config_init(&c, s.config.M, s.config.N, s.config.K);
        c.activation_type = s.activation_type;
        c.required_k_tile = s.config.k_tile;
        c.k_tile_multiplier = s.weights.multiplier;
        c.timeout_ms = s.config.timeout_ms;
        Profile p;
        if (make_profile(c, B, scale, p)) return nullptr;
        const Resources r{s.config.npu_core_mask, s.cpu_core_mask, s.cpu_core_mask, __builtin_popcountll(s.cpu_core_mask),
                          chain_max_m()};
        if (!strategy_ok(strategy, c, p, r, panel8)) return nullptr;
        return create_weights(domain, p.info(c.required_k_tile), B, scale, &p);
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
extern "C" int rk_npu_w4a8_autotune_cache_load_profile_ex(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* cfg,
                                                          const rk_npu_w4a8_tuning_profile* profile, const char* path,
                                                          rk_npu_w4a8_strategy_ex* fast, rk_npu_w4a8_strategy_ex* stable)
{
    if (!ctx || !cfg || !profile || !fast || !stable || (path && !*path) || !valid_autotune_config(*cfg))
        return RK_NPU_ERR_PARAM;
    try {
        const Profile& p = profile->value;
        // The caller states the multiplier policy explicitly; a captured profile never
        // adopts a changed environment silently.
        if (p.K != cfg->K || p.N != cfg->N || cfg->k_tile_multiplier != p.multiplier ||
            (cfg->required_k_tile && !p.permits(cfg->required_k_tile)))
            return RK_NPU_ERR_PARAM;
        const Resources r = resolve_resources(*cfg);
        if (!r.npu || !r.threads) return RK_NPU_ERR_PARAM;
        const std::string key = cache_key(ctx, *cfg, p, r, true);
        return load_file(path ? std::string(path) : default_cache_path(key), key, *cfg, p, r, *fast, *stable, true);
    } catch (const std::bad_alloc&) { return RK_NPU_ERR_NOMEM; } catch (...) { return RK_NPU_ERR_PARAM; }
}
extern "C" int rk_npu_w4a8_autotune_cache_load(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* cfg, const int8_t* B,
                                               const float* s, const char* path, rk_npu_w4a8_strategy* fast,
                                               rk_npu_w4a8_strategy* stable)
{
    return load_entry<false>(ctx, cfg, B, s, path, fast, stable);
}
extern "C" int rk_npu_w4a8_autotune_cache_save(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* cfg, const int8_t* B,
                                               const float* s, const char* path, const rk_npu_w4a8_strategy* fast,
                                               const rk_npu_w4a8_strategy* stable)
{
    return save_entry<false>(ctx, cfg, B, s, path, fast, stable);
}
extern "C" int rk_npu_w4a8_autotune_cache_load_ex(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* cfg, const int8_t* B,
                                                  const float* s, const char* path, rk_npu_w4a8_strategy_ex* fast,
                                                  rk_npu_w4a8_strategy_ex* stable)
{
    return load_entry<true>(ctx, cfg, B, s, path, fast, stable);
}
extern "C" int rk_npu_w4a8_autotune_cache_save_ex(rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config* cfg, const int8_t* B,
                                                  const float* s, const char* path, const rk_npu_w4a8_strategy_ex* fast,
                                                  const rk_npu_w4a8_strategy_ex* stable)
{
    return save_entry<true>(ctx, cfg, B, s, path, fast, stable);
}
extern "C" rk_npu_w4a8_weights* rk_npu_w4a8_weights_create_tuned(rk_npu_iommu_domain* domain, const rk_npu_w4a8_strategy* s,
                                                                 const int8_t* B, const float* scale)
{
    return s ? create_tuned(domain, extend(*s), B, scale, false) : nullptr;
}
extern "C" rk_npu_w4a8_weights* rk_npu_w4a8_weights_create_tuned_ex(rk_npu_iommu_domain* domain,
                                                                    const rk_npu_w4a8_strategy_ex* s, const int8_t* B,
                                                                    const float* scale)
{
    return s ? create_tuned(domain, *s, B, scale, true) : nullptr;
}
extern "C" rk_npu_w4a8_workspace* rk_npu_w4a8_workspace_create_tuned_ex(rk_npu_iommu_domain* domain,
                                                                        const rk_npu_w4a8_strategy_ex* s)
{
    if (!s || s->base.tuning_revision != TUNING_REVISION || !execution_ok(*s, true) ||
        s->base.config.K != s->base.weights.config.K || s->base.config.N != s->base.weights.config.N ||
        s->base.config.k_tile != s->base.weights.config.k_tile)
        return nullptr;
    return rk_npu_w4a8_workspace_create_ex(domain, &s->base.config, &s->execution);
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
    const uint64_t affinity = process_cpu_mask();
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
        s.cpu_threads != __builtin_popcountll(s.cpu_core_mask) || (s.cpu_core_mask & ~process_cpu_mask()))
        return false;
    // Panel recipes are checked by the original against its device plan; they have no meaning
    // here and their rules are not restated: such a record is treated as not usable.
    if (s.a_layout >= RK_NPU_MATMUL_A_LAYOUT_PANEL8 || s.c_layout != RK_NPU_MATMUL_C_LAYOUT_NATIVE) return false;
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
