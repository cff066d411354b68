// w4a8_tune.h -- internal interface between the tuning-cache code (w4a8_tune.cpp), the search tuner
// (w4a8_autotune.cpp) and the operator front-end (w4a8_abi.cpp).  Host code only.
#pragma once
#include "w4a8_host.h"
#include <string>
#include <vector>

namespace rkb200 {

using Strategy = rk_npu_w4a8_strategy_ex;

constexpr uint32_t TUNING_REVISION = 5;   // the text format's revision field; files of another revision are a miss
constexpr int SMALL_BATCH_TOKENS = 8;     // batches up to this size may use one host thread / the serial pipeline value

// What a tuning request may use of the host and of the (three-core) device the file format was made for.
// The masks are part of the cache key and of every stored strategy, so they are derived exactly as the
// original derives them; on this library they select nothing.
struct HostResources {
    uint32_t device_cores = 0;       // core mask every strategy of this request must carry
    uint64_t cpus = 0;               // CPU mask every strategy must carry (at most four CPUs)
    uint64_t cpus_allowed = 0;       // request mask intersected with the process affinity
    int threads = 0;                 // popcount(cpus)
    int chain_tokens = SMALL_BATCH_TOKENS;   // RK_NPU_W4A8_CHAIN_MAX_M (0..64), -1 when malformed
    bool usable() const { return device_cores != 0 && threads > 0 && chain_tokens >= 0; }
};
HostResources host_resources(const rk_npu_w4a8_autotune_config& request);
int chain_token_limit();   // the environment value alone
uint64_t process_cpu_mask();   // CPUs 0..63 of the process affinity (CPU 0 when it cannot be read)

// A strategy as the legacy (non-_ex) entry points see it.
Strategy widen(const rk_npu_w4a8_strategy& s);

// Every rule a stored or caller-supplied strategy has to satisfy for `request`; `extended` selects the
// search space of the _ex entry points (panel8 layouts allowed).
bool strategy_acceptable(const Strategy& s, const rk_npu_w4a8_autotune_config& request, const Profile& profile,
                         const HostResources& res, bool extended);
// The subset that needs no request: revision, execution options, geometry accepted by the memory query.
bool strategy_executable(const Strategy& s, bool extended);

std::string cache_key_line(const rk_npu_ctx* ctx, const rk_npu_w4a8_autotune_config& request, const Profile& profile,
                           const HostResources& res, bool extended);
// Default location: $XDG_CACHE_HOME or $HOME/.cache, then rk_npu_w4a8/<16 hex digits of FNV-1a(key)>.tune;
// `directory` non-null replaces everything in front of the file name.  Empty when no base directory exists.
std::string cache_file_for(const std::string& key, const char* directory = nullptr);
int cache_read(const std::string& path, const std::string& key, const rk_npu_w4a8_autotune_config& request,
               const Profile& profile, const HostResources& res, bool extended, Strategy& fastest, Strategy& stable);
int cache_write(const std::string& path, const std::string& key, const Strategy& fastest, const Strategy& stable);

// ---- what a strategy means on this library ------------------------------------------------------------
// The strategy's fields keep the original's names, ranges and validity rules (files written by either
// library load in the other); on B200 they select among this library's kernels:
//   pipeline  CHAIN      one launch per linear: the decode kernel (whole-K CTAs, cluster code exchange)
//             SERIAL     two launches: quantise, then the mma.sync split-K ring
//             PIPELINED  see m_tile
//   m_tile    64         (the original's default) automatic choice
//             32         two launches, mma.sync ring in 32-token chunks
//             48         two launches, persistent tcgen05 streaming kernel (up to 128 tokens)
//             56         two launches, per-tile / persistent two-CTA tcgen05 kernel (more than 32 tokens)
//             other      automatic
//   n_tile    128, 256, 512, 1024   CTAs that cooperate on one column tile: 1, 2, 4, 8 -- the split-K factor
//             of the ring / the cluster size of the decode kernel; other values: automatic
// A choice the geometry cannot run (e.g. the decode kernel above eight tokens) falls back to automatic.
struct Schedule {
    int family = 0;    // 0 automatic, else the workspace's kernel family (1, 2, 4, 5)
    int cluster = 0;   // 0 automatic, else 1, 2, 4, 8
};
Schedule schedule_of(const rk_npu_w4a8_config& config);
void schedule_into(const Schedule& s, rk_npu_w4a8_config& config);
// Families that can run `M` tokens with reduction length `K` (the candidate set of the search tuner).
std::vector<Schedule> schedule_candidates(int M, int N, int K, int sm_count);

// W8 strategies that name a panel layout (a_layout PANEL8 / PANEL16, or c_layout other than NATIVE) are accepted by
// the original only when its device plan can be built for them.  Those rules (src/rk_npu_matmul_i8.cpp:65-92, reached
// through src/rk_npu_kn_plan.cpp:43-70 from src/rk_npu_quant_matmul.cpp:167-177) restated on the strategy's own fields;
// the layouts are the integer values of rk_npu_matmul_a_layout / rk_npu_matmul_c_layout.  True for non-panel recipes.
bool w8_panel_recipe_ok(int M, int N, int k_tile, int a_layout, int c_layout);

// Workspace creation with an explicit schedule (w4a8_abi.cpp).
rk_npu_w4a8_workspace* create_workspace_scheduled(rk_npu_iommu_domain* domain, const rk_npu_w4a8_config* cfg,
                                                  const rk_npu_w4a8_options* options, const Schedule& schedule);

} // namespace rkb200
