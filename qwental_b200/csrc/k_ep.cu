// Expert-parallel exchange step of the MoE layer (no counterpart in the reference, which is one device):
// after the down projection each rank holds the (token, rank) rows of the experts it owns and zeros elsewhere;
// summing the buffers over ranks gives every rank all rows, bit-identical to the one-GPU layer, because each
// row has exactly one non-zero contributor.  The sum is an NCCL all-reduce over NVLink/NVSwitch enqueued on the
// batch's stream like any other dispatch, so it is ordered with the kernels around it and can be captured in a
// CUDA graph.  NCCL is loaded at run time (dlopen), so single-GPU use needs no NCCL at all.
#include "../../include/qw_engine.h"
#include "qw_kern.h"

#include <dlfcn.h>
#include <cstdio>
#include <cstdlib>

namespace {
typedef struct ncclComm *ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
struct Nccl {
    void *h = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t *, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*AllReduce)(const void *, void *, size_t, int, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    ncclComm_t comm = nullptr;
    int rank = 0, size = 1;
} N;

bool load_nccl() {
    if (N.h) return true;
    const char *names[] = {getenv("QW_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
    for (const char *n : names) {
        if (!n) continue;
        N.h = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
        if (N.h) break;
    }
    if (!N.h) return false;
    N.GetUniqueId = (decltype(N.GetUniqueId))dlsym(N.h, "ncclGetUniqueId");
    N.CommInitRank = (decltype(N.CommInitRank))dlsym(N.h, "ncclCommInitRank");
    N.AllReduce = (decltype(N.AllReduce))dlsym(N.h, "ncclAllReduce");
    N.CommDestroy = (decltype(N.CommDestroy))dlsym(N.h, "ncclCommDestroy");
    N.GetErrorString = (decltype(N.GetErrorString))dlsym(N.h, "ncclGetErrorString");
    return N.GetUniqueId && N.CommInitRank && N.AllReduce;
}
}  // namespace

extern "C" int qw_ep_unique_id(void *id128) {
    if (!id128 || !load_nccl()) return -1;
    ncclUniqueId id;
    if (N.GetUniqueId(&id) != 0) return -1;
    memcpy(id128, &id, sizeof id);
    return 0;
}

// Called by qw_engine_ep_init (engine.cpp) with the engine's rank and size.
extern "C" int qw_ep_comm_init(int rank, int size, const void *id128) {
    if (!id128 || size < 1 || rank < 0 || rank >= size || !load_nccl()) return -1;
    if (N.comm) return N.rank == rank && N.size == size ? 0 : -1;
    ncclUniqueId id;
    memcpy(&id, id128, sizeof id);
    const ncclResult_t r = N.CommInitRank(&N.comm, size, id, rank);
    if (r != 0) {
        fprintf(stderr, "[qw_ep] ncclCommInitRank failed: %s\n", N.GetErrorString ? N.GetErrorString(r) : "?");
        N.comm = nullptr;
        return -1;
    }
    N.rank = rank;
    N.size = size;
    return 0;
}

// binds: 0 = fp32 buffer summed in place over the ranks, 1 = {uint64 count}
static cudaError_t launch_ep_allreduce(const QwLaunch &L) {
    const uint64_t cnt = L.bytes<uint64_t>(1);
    QW_CHECK_ARG(L.buf<float>(0) && cnt >= 1 && L.avail(0) >= cnt * 4 && N.comm);
    const ncclResult_t r = N.AllReduce(L.buf<float>(0), L.buf<float>(0), (size_t)cnt, /*ncclFloat32*/ 7, /*ncclSum*/ 0, N.comm, L.stream);
    return r == 0 ? cudaSuccess : cudaErrorUnknown;
}
QW_FAMILY(ep_allreduce, launch_ep_allreduce, 1)
