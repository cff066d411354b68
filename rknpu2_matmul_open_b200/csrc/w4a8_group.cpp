// w4a8_group.cpp -- a context that is one rank of a group of GPUs: column sharding inside the library.
//
// The reference splits the output columns of a GEMM over its NPU cores in contiguous runs of 64-column
// blocks, the first `blocks % cores` cores taking one block more (src/rk_npu_i4_plan.cpp:37-43), all inside
// one submit.  Here the same partition runs over the GPUs of a box, one process (rank) per GPU: a group
// context shards every weight object at creation, every run computes this rank's columns of C, and one NCCL
// all-gather over NVLink reassembles the rows on every rank.  Per-column arithmetic is untouched, so results
// are bit-identical for any group size.  NCCL is used through its C API, loaded on first use (a process that
// never opens a group needs no NCCL at all).
#include "w4a8_host.h"
#include <nccl.h>
#include <cerrno>
#include <cstdlib>
#include <cstring>
#include <dlfcn.h>
#include <mutex>
#include <new>

namespace rkb200 {

// ------------------------------------------------------------------ NCCL, loaded on first use
namespace {
struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    bool ok = false;
};
const NcclApi& nccl()
{
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        void* lib = nullptr;
        for (const char* name : {"libnccl.so.2", "libnccl.so"}) {
            lib = ::dlopen(name, RTLD_NOW | RTLD_LOCAL);
            if (lib) break;
        }
        if (!lib) return;
        auto find = [&](const char* symbol) { return ::dlsym(lib, symbol); };
        api.GetUniqueId = reinterpret_cast<decltype(api.GetUniqueId)>(find("ncclGetUniqueId"));
        api.CommInitRank = reinterpret_cast<decltype(api.CommInitRank)>(find("ncclCommInitRank"));
        api.CommDestroy = reinterpret_cast<decltype(api.CommDestroy)>(find("ncclCommDestroy"));
        api.AllGather = reinterpret_cast<decltype(api.AllGather)>(find("ncclAllGather"));
        api.AllReduce = reinterpret_cast<decltype(api.AllReduce)>(find("ncclAllReduce"));
        api.ok = api.GetUniqueId && api.CommInitRank && api.CommDestroy && api.AllGather && api.AllReduce;
    });
    return api;
}
static_assert(sizeof(ncclUniqueId) == RK_NPU_B200_GROUP_ID_BYTES, "the group id is an NCCL unique id");
} // namespace

void group_close(rk_npu_ctx* ctx)
{
    if (ctx && ctx->comm) {
        nccl().CommDestroy(static_cast<ncclComm_t>(ctx->comm));
        ctx->comm = nullptr;
    }
}

// All-gather of `bytes_per_rank` bytes: this rank's piece already sits at its slot of `buffer` (in place).
int group_all_gather(rk_npu_ctx* ctx, void* buffer, size_t bytes_per_rank, cudaStream_t stream)
{
    if (!ctx || !ctx->comm) return RK_NPU_ERR_PARAM;
    const char* mine = static_cast<const char*>(buffer) + size_t(ctx->rank) * bytes_per_rank;
    const ncclResult_t r = nccl().AllGather(mine, buffer, bytes_per_rank, ncclInt8, static_cast<ncclComm_t>(ctx->comm), stream);
    return r == ncclSuccess ? RK_NPU_OK : RK_NPU_ERR_SUBMIT;
}
// Element-wise maximum of `count` non-negative 32-bit patterns across the group (row maxima of an FFN's middle:
// the bit patterns of non-negative floats order like integers, and a maximum is exact under any grouping).
int group_all_reduce_max_u32(rk_npu_ctx* ctx, uint32_t* values, size_t count, cudaStream_t stream)
{
    if (!ctx || !ctx->comm) return RK_NPU_ERR_PARAM;
    const ncclResult_t r = nccl().AllReduce(values, values, count, ncclUint32, ncclMax, static_cast<ncclComm_t>(ctx->comm), stream);
    return r == ncclSuccess ? RK_NPU_OK : RK_NPU_ERR_SUBMIT;
}

} // namespace rkb200

using namespace rkb200;

extern "C" int rk_npu_b200_group_id(unsigned char* id)
{
    if (!id) return RK_NPU_ERR_PARAM;
    if (!nccl().ok) return RK_NPU_ERR_OPEN;
    ncclUniqueId unique;
    if (nccl().GetUniqueId(&unique) != ncclSuccess) return RK_NPU_ERR_IOCTL;
    std::memcpy(id, &unique, sizeof(unique));
    return RK_NPU_OK;
}

extern "C" rk_npu_ctx* rk_npu_b200_open_group(const char* dev, int rank, int world, const unsigned char* id)
{
    if (!id || world < 1 || world > 64 || rank < 0 || rank >= world) { errno = EINVAL; return nullptr; }
    // A rank whose communicator cannot be created fails here, on the host, before any GPU work: the switch
    // below lets a test stand in for a lost peer or a failed bootstrap.
    if (const char* refuse = std::getenv("RK_NPU_B200_REFUSE_GROUP"))
        if (refuse[0] == '1' && refuse[1] == 0) { errno = ECONNREFUSED; return nullptr; }
    if (!nccl().ok) { errno = ENOSYS; return nullptr; }
    rk_npu_ctx* ctx = rk_npu_open(dev);
    if (!ctx) return nullptr;
    ncclUniqueId unique;
    std::memcpy(&unique, id, sizeof(unique));
    ncclComm_t comm = nullptr;
    if (cudaSetDevice(ctx->device) != cudaSuccess || nccl().CommInitRank(&comm, world, unique, rank) != ncclSuccess) {
        cudaGetLastError();
        rk_npu_close(ctx);
        errno = ECONNREFUSED;
        return nullptr;
    }
    ctx->comm = comm;
    ctx->rank = rank;
    ctx->world = world;
    return ctx;
}

extern "C" int rk_npu_b200_group_rank(const rk_npu_ctx* ctx) { return ctx ? ctx->rank : -1; }
extern "C" int rk_npu_b200_group_size(const rk_npu_ctx* ctx) { return ctx ? ctx->world : 0; }
extern "C" int rk_npu_b200_shard_columns(int N, int world, int rank, int* n0, int* n1)
{
    if (N < 1 || world < 1 || rank < 0 || rank >= world || !n0 || !n1) return RK_NPU_ERR_PARAM;
    shard_range(N, world, rank, *n0, *n1);
    return RK_NPU_OK;
}
