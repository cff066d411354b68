// rmsnorm_abi.cpp -- C entry points of the caller-owned buffers (rk_npu_mem_*, include/rk_npu_common.h:160-190) and
// of the residual add + RMSNorm operator that works on them (include/rk_npu_add_rmsnorm_f16.h).
//
// A buffer is page-locked host memory mapped into the GPU's address space: the host writes through vaddr, the kernel
// reads and writes the same bytes through dma_addr, and the blocking run has returned before the host looks again,
// so no copies and no cache maintenance are needed (the original's uncached DMA buffers behave the same way).
#include "../../include/rknpu_b200_ext.h"
#include "rmsnorm_device.h"
#include "w4a8_host.h"
#include <atomic>
#include <cmath>
#include <cstring>
#include <new>
#include <unordered_map>

using namespace rkb200;

namespace {

// live base allocations by handle: the domain they are accounted to (retained while they live) and their bytes
struct Allocation {
    rk_npu_iommu_domain* domain;
    void* host;
    uint64_t bytes;
};
std::mutex g_allocations_lock;
std::unordered_map<uint32_t, Allocation> g_allocations;
uint32_t g_next_handle = 1;

bool same_ctx(const rk_npu_ctx* ctx, const rk_npu_mem* mem) { return mem->ctx_id == ctx->id; }

bool valid_config(const rk_npu_add_rmsnorm_f16_config* c)
{
    return c && c->M >= 1 && c->M <= 65536 && c->D >= 8 && c->D <= 32768 && c->D % 8 == 0 && std::isfinite(c->eps) && c->eps >= 0.f;
}

// src/rk_npu_add_rmsnorm_f16.cpp:73-77, on device addresses
bool overlaps(uint64_t a, uint64_t b, uint64_t bytes) { return a < b + bytes && b < a + bytes; }

} // namespace

struct rk_npu_add_rmsnorm_f16_plan {
    rk_npu_ctx* ctx = nullptr;
    rk_npu_iommu_domain* domain = nullptr;
    rk_npu_add_rmsnorm_f16_config cfg{};
    void* gamma = nullptr;           // [D] fp16, device
    cudaStream_t stream = nullptr;   // the blocking call's
    std::atomic_flag busy = ATOMIC_FLAG_INIT;
};

// ------------------------------------------------------------------------------------------------ buffers
// src/rk_npu_core.cpp:214-262
extern "C" int rk_npu_mem_alloc(rk_npu_iommu_domain* domain, uint64_t size, uint32_t alloc_flags, rk_npu_mem* out)
{
    if (!domain || !domain->ctx || !out || size == 0) return RK_NPU_ERR_PARAM;
    rk_npu_ctx* ctx = domain->ctx;
    std::memset(out, 0, sizeof(*out));
    if (cudaSetDevice(ctx->device) != cudaSuccess) return RK_NPU_ERR_IOCTL;
    void* host = nullptr;
    void* device = nullptr;
    if (cudaHostAlloc(&host, size, cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
        cudaGetLastError();
        return RK_NPU_ERR_NOMEM;
    }
    if (cudaHostGetDevicePointer(&device, host, 0) != cudaSuccess) {
        cudaGetLastError();
        cudaFreeHost(host);
        return RK_NPU_ERR_IOCTL;
    }
    {
        std::lock_guard<std::mutex> g(g_allocations_lock);
        while (!g_next_handle || g_allocations.count(g_next_handle)) ++g_next_handle;
        out->handle = g_next_handle++;
        g_allocations[out->handle] = {domain, host, size};
    }
    domain_retain(domain);
    out->flags = RK_NPU_MEM_F_OWN_RKNPU | RK_NPU_MEM_F_MAPPED;
    if (alloc_flags & RK_NPU_MEM_CACHEABLE) out->flags |= RK_NPU_MEM_F_CACHEABLE;
    out->obj_addr = out->dma_addr = uint64_t(reinterpret_cast<uintptr_t>(device));
    out->vaddr = host;
    out->size = out->capacity = size;
    out->ctx_id = ctx->id;
    out->iommu_domain_id = domain->id;
    std::lock_guard<std::mutex> g(domain->lock);
    domain->stats.live_bytes += size;
    domain->stats.peak_bytes = std::max(domain->stats.peak_bytes, domain->stats.live_bytes);
    ++domain->stats.creates;
    return RK_NPU_OK;
}

// A view is the base struct narrowed to [offset, offset + size): both addresses and the offset from the base object
// move by `offset`, the capacity still names the base object, and of the state bits only the ones that describe the
// mapping survive -- a view owns nothing.  Semantics of src/rk_npu_core.cpp:318-331.
extern "C" int rk_npu_mem_view(const rk_npu_mem* base, uint64_t offset, uint64_t size, rk_npu_mem* out_view)
{
    const bool usable = base && out_view && base->capacity != 0;
    const bool inside = usable && size != 0 && offset <= base->size && size <= base->size - offset;
    if (!inside) return RK_NPU_ERR_PARAM;
    constexpr uint32_t inherited = RK_NPU_MEM_F_IMPORTED | RK_NPU_MEM_F_MAPPED | RK_NPU_MEM_F_CACHEABLE;
    rk_npu_mem view = *base;
    view.flags = (base->flags & inherited) | RK_NPU_MEM_F_VIEW;
    view.size = size;
    view.offset += offset;
    view.dma_addr += offset;
    if (view.vaddr) view.vaddr = static_cast<uint8_t*>(view.vaddr) + offset;
    *out_view = view;
    return RK_NPU_OK;
}

// src/rk_npu_core.cpp:333-344: mapped page-locked memory needs no maintenance; only the arguments are checked
extern "C" int rk_npu_mem_sync(rk_npu_ctx* ctx, const rk_npu_mem* mem, rk_npu_sync_dir dir)
{
    if (!ctx || !mem || !same_ctx(ctx, mem) || !(dir == RK_NPU_SYNC_TO_DEVICE || dir == RK_NPU_SYNC_FROM_DEVICE))
        return RK_NPU_ERR_PARAM;
    return RK_NPU_OK;
}

// src/rk_npu_core.cpp:346-373.  A struct that does not describe a live allocation of this library (a stale copy, a
// second free) is refused instead of being handed to the allocator.
extern "C" int rk_npu_mem_free(rk_npu_ctx* ctx, rk_npu_mem* mem)
{
    if (!ctx || !mem) return RK_NPU_ERR_PARAM;
    if (mem->flags & RK_NPU_MEM_F_VIEW) {
        std::memset(mem, 0, sizeof(*mem));
        return RK_NPU_OK;
    }
    if (!same_ctx(ctx, mem)) return RK_NPU_ERR_PARAM;
    Allocation found{};
    {
        std::lock_guard<std::mutex> g(g_allocations_lock);
        auto it = g_allocations.find(mem->handle);
        if (!(mem->flags & RK_NPU_MEM_F_OWN_RKNPU) || it == g_allocations.end() || it->second.host != mem->vaddr) return RK_NPU_ERR_PARAM;
        found = it->second;
        g_allocations.erase(it);
    }
    int rc = RK_NPU_OK;
    cudaSetDevice(ctx->device);
    if (cudaFreeHost(found.host) != cudaSuccess) {
        cudaGetLastError();
        rc = RK_NPU_ERR_IOCTL;
    }
    {
        std::lock_guard<std::mutex> g(found.domain->lock);
        found.domain->stats.live_bytes -= std::min<uint64_t>(found.bytes, found.domain->stats.live_bytes);
        ++found.domain->stats.destroys;
    }
    domain_release(found.domain);
    std::memset(mem, 0, sizeof(*mem));
    return rc;
}

// no dmabuf on this platform
extern "C" int rk_npu_mem_import_dmabuf(rk_npu_iommu_domain*, int, void*, uint64_t, uint32_t, rk_npu_mem*) { return RK_NPU_ERR_PARAM; }
extern "C" int rk_npu_mem_export_dmabuf(rk_npu_ctx*, const rk_npu_mem*, int*) { return RK_NPU_ERR_PARAM; }

// ------------------------------------------------------------------------------------------------ operator
// src/rk_npu_add_rmsnorm_f16.cpp:211-219
extern "C" void rk_npu_add_rmsnorm_f16_config_init(rk_npu_add_rmsnorm_f16_config* cfg, int M, int D)
{
    if (!cfg) return;
    std::memset(cfg, 0, sizeof(*cfg));
    cfg->M = M;
    cfg->D = D;
    cfg->eps = 1.0e-5f;
    cfg->timeout_ms = 6000;
}

// src/rk_npu_add_rmsnorm_f16.cpp:221-236
extern "C" int rk_npu_add_rmsnorm_f16_query(const rk_npu_add_rmsnorm_f16_config* cfg, rk_npu_add_rmsnorm_f16_sizes* out)
{
    if (!valid_config(cfg) || !out) return RK_NPU_ERR_PARAM;
    std::memset(out, 0, sizeof(*out));
    out->tensor_bytes = uint64_t(cfg->M) * uint64_t(cfg->D) * sizeof(uint16_t);
    out->weight_bytes = uint64_t(cfg->D) * sizeof(uint16_t);
    out->num_tasks = 1;
    return RK_NPU_OK;
}

// src/rk_npu_add_rmsnorm_f16.cpp:238-268
extern "C" rk_npu_add_rmsnorm_f16_plan* rk_npu_add_rmsnorm_f16_plan_create(rk_npu_iommu_domain* domain,
                                                                           const rk_npu_add_rmsnorm_f16_config* cfg,
                                                                           const uint16_t* gamma)
{
    if (!domain || !domain->ctx || !valid_config(cfg) || !gamma) return nullptr;
    if (cudaSetDevice(domain->ctx->device) != cudaSuccess) return nullptr;
    auto* plan = new (std::nothrow) rk_npu_add_rmsnorm_f16_plan();
    if (!plan) return nullptr;
    plan->ctx = domain->ctx;
    plan->domain = domain;
    plan->cfg = *cfg;
    domain_retain(domain);
    const size_t bytes = size_t(cfg->D) * sizeof(uint16_t);
    bool ok = device_alloc(domain, &plan->gamma, bytes) == RK_NPU_OK &&
              cudaStreamCreateWithFlags(&plan->stream, cudaStreamNonBlocking) == cudaSuccess &&
              cudaMemcpyAsync(plan->gamma, gamma, bytes, cudaMemcpyHostToDevice, plan->stream) == cudaSuccess &&
              cudaStreamSynchronize(plan->stream) == cudaSuccess;
    if (!ok) {
        cudaGetLastError();
        rk_npu_add_rmsnorm_f16_plan_free(plan);
        return nullptr;
    }
    return plan;
}

extern "C" void rk_npu_add_rmsnorm_f16_plan_free(rk_npu_add_rmsnorm_f16_plan* plan)
{
    if (!plan) return;
    cudaSetDevice(plan->ctx->device);
    if (plan->stream) {
        cudaStreamSynchronize(plan->stream);
        cudaStreamDestroy(plan->stream);
    }
    device_free(plan->domain, plan->gamma, size_t(plan->cfg.D) * sizeof(uint16_t));
    domain_release(plan->domain);
    delete plan;
}

namespace {
int launch(rk_npu_add_rmsnorm_f16_plan* plan, int rows, int row_major, uint64_t x, uint64_t r, uint64_t ro, uint64_t no,
           cudaStream_t stream)
{
    AddRmsNormParams p{};
    p.x = reinterpret_cast<const uint4*>(uintptr_t(x));
    p.residual = reinterpret_cast<const uint4*>(uintptr_t(r));
    p.residual_out = reinterpret_cast<uint4*>(uintptr_t(ro));
    p.norm_out = reinterpret_cast<uint4*>(uintptr_t(no));
    p.gamma = static_cast<const uint4*>(plan->gamma);
    p.M = rows;
    p.D = plan->cfg.D;
    p.eps = plan->cfg.eps;
    p.row_major = row_major;
    if (launch_add_rmsnorm(p, stream) != cudaSuccess) {
        cudaGetLastError();
        return RK_NPU_ERR_SUBMIT;
    }
    return RK_NPU_OK;
}
} // namespace

// The original's blocking call (src/rk_npu_add_rmsnorm_f16.cpp:270-304) answers, in this order: missing arguments or a
// plan of another context (PARAM); per tensor in argument order, a buffer of another context or too small (NOMEM) before
// one of another domain (DOMAIN); an output lying on an input or on the other output (PARAM); a plan in use (BUSY).
// The two inputs may be the same tensor.  Here a view at an address the kernel's 16-byte chunks cannot start at is PARAM too.
extern "C" int rk_npu_add_rmsnorm_f16_run(rk_npu_ctx* ctx, rk_npu_add_rmsnorm_f16_plan* plan, const rk_npu_mem* x,
                                          const rk_npu_mem* residual, rk_npu_mem* residual_out, rk_npu_mem* norm_out)
{
    const rk_npu_mem* const tensors[4] = {x, residual, residual_out, norm_out};      // inputs first, outputs last
    if (!ctx || !plan || plan->ctx != ctx) return RK_NPU_ERR_PARAM;
    for (const rk_npu_mem* t : tensors)
        if (!t) return RK_NPU_ERR_PARAM;
    const uint64_t bytes = uint64_t(plan->cfg.M) * uint64_t(plan->cfg.D) * sizeof(uint16_t);
    for (const rk_npu_mem* t : tensors) {
        if (t->ctx_id != ctx->id || t->size < bytes) return RK_NPU_ERR_NOMEM;
        if (t->iommu_domain_id != plan->domain->id) return RK_NPU_ERR_DOMAIN;
    }
    for (int out = 2; out < 4; ++out)              // each output against everything in front of it
        for (int other = 0; other < out; ++other)
            if (overlaps(tensors[other]->dma_addr, tensors[out]->dma_addr, bytes)) return RK_NPU_ERR_PARAM;
    for (const rk_npu_mem* t : tensors)
        if (t->dma_addr % 16) return RK_NPU_ERR_PARAM;
    if (plan->busy.test_and_set(std::memory_order_acquire)) return RK_NPU_ERR_BUSY;
    int rc = cudaSetDevice(ctx->device) == cudaSuccess ? RK_NPU_OK : RK_NPU_ERR_SUBMIT;
    if (rc == RK_NPU_OK)
        rc = launch(plan, plan->cfg.M, 0, x->dma_addr, residual->dma_addr, residual_out->dma_addr, norm_out->dma_addr, plan->stream);
    if (rc == RK_NPU_OK && cudaStreamSynchronize(plan->stream) != cudaSuccess) {
        cudaGetLastError();
        rc = RK_NPU_ERR_SUBMIT;
    }
    plan->busy.clear(std::memory_order_release);
    return rc;
}

extern "C" int rk_npu_b200_add_rmsnorm_f16_enqueue(rk_npu_add_rmsnorm_f16_plan* plan, int rows, int row_major, const uint16_t* dX,
                                                   const uint16_t* dResidual, uint16_t* dResidualOut, uint16_t* dNormOut,
                                                   void* cuda_stream)
{
    if (!plan || rows < 1 || rows > plan->cfg.M || (row_major != 0 && row_major != 1) || !dX || !dResidual || !dResidualOut ||
        !dNormOut)
        return RK_NPU_ERR_PARAM;
    const uint64_t bytes = uint64_t(rows) * uint64_t(plan->cfg.D) * 2;
    const uint64_t x = uint64_t(reinterpret_cast<uintptr_t>(dX)), r = uint64_t(reinterpret_cast<uintptr_t>(dResidual)),
                   ro = uint64_t(reinterpret_cast<uintptr_t>(dResidualOut)), no = uint64_t(reinterpret_cast<uintptr_t>(dNormOut));
    if ((x | r | ro | no) % 16) return RK_NPU_ERR_PARAM;
    if (overlaps(x, ro, bytes) || overlaps(x, no, bytes) || overlaps(r, ro, bytes) || overlaps(r, no, bytes) || overlaps(ro, no, bytes))
        return RK_NPU_ERR_PARAM;
    int current = -1;
    if (cudaGetDevice(&current) != cudaSuccess || current != plan->ctx->device) return RK_NPU_ERR_PARAM;
    return launch(plan, rows, row_major, x, r, ro, no, static_cast<cudaStream_t>(cuda_stream));
}
