// C ABI: the per-context NCCL communicator used by sharded sumchecks.
//
// One process per GPU.  The library does not link NCCL: libnccl.so.2 is opened
// on first use, so single-GPU users carry no dependency and a process that has
// already loaded an NCCL (e.g. through torch) shares that copy.  The exchange
// per round is tiny (d+1 field elements per rank): one ncclAllGather over
// NVLink, then each rank adds the partial sums mod p on the host, where the
// transcript lives anyway (NCCL has no modular sum).
#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <thread>

#include "comm.cuh"

namespace dpb {

NcclApi& nccl_api() {
    static NcclApi api;
    return api;
}

int nccl_load() {
    NcclApi& a = nccl_api();
    if (a.handle) return DPB_OK;
    void* h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return fail(DPB_ENCCL, "cannot open libnccl.so.2: %s", dlerror());
#define DPB_SYM(name)                                                                  \
    a.name = (decltype(a.name))dlsym(h, #name);                                        \
    if (!a.name) return fail(DPB_ENCCL, "libnccl.so.2 lacks the symbol %s", #name);
    DPB_SYM(ncclGetUniqueId)
    DPB_SYM(ncclCommInitRank)
    DPB_SYM(ncclCommDestroy)
    DPB_SYM(ncclCommAbort)
    DPB_SYM(ncclAllGather)
    DPB_SYM(ncclGetErrorString)
    DPB_SYM(ncclCommGetAsyncError)
#undef DPB_SYM
    a.handle = h;
    return DPB_OK;
}

// Waits for the stream with a time limit instead of blocking forever on a peer
// that never joins its collective.
int sync_bounded(dpb_ctx* ctx, double seconds) {
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
        cudaError_t e = cudaStreamQuery(ctx->stream);
        if (e == cudaSuccess) return DPB_OK;
        if (e != cudaErrorNotReady) return fail(DPB_ECUDA, "stream: %s", cudaGetErrorString(e));
        if (ctx->nccl_comm) {
            ncclResult_t ar = ncclSuccess;
            if (nccl_api().ncclCommGetAsyncError((ncclComm_t)ctx->nccl_comm, &ar) == ncclSuccess && ar != ncclSuccess &&
                ar != ncclInProgress)
                return fail(DPB_ENCCL, "collective failed: %s", nccl_api().ncclGetErrorString(ar));
        }
        const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
        if (dt > seconds) return fail(DPB_ETIMEOUT, "waited %.1f s for a collective; a peer rank is missing", dt);
        if (dt > 2e-4) std::this_thread::yield();
    }
}

}  // namespace dpb

using namespace dpb;

extern "C" {

int dpb_comm_unique_id(void* out_id) {
    if (!out_id) return fail(DPB_EINVAL, "null argument");
    DPB_TRY(nccl_load());
    ncclUniqueId id;
    ncclResult_t r = nccl_api().ncclGetUniqueId(&id);
    if (r != ncclSuccess) return fail(DPB_ENCCL, "ncclGetUniqueId: %s", nccl_api().ncclGetErrorString(r));
    memcpy(out_id, &id, sizeof id);
    return DPB_OK;
}

int dpb_comm_init(dpb_ctx* ctx, const void* id, int rank, int nranks) {
    if (!ctx || !id) return fail(DPB_EINVAL, "null argument");
    if (nranks < 1 || (nranks & (nranks - 1))) return fail(DPB_EINVAL, "rank count %d is not a power of two", nranks);
    if (rank < 0 || rank >= nranks) return fail(DPB_EINVAL, "rank %d outside 0..%d", rank, nranks - 1);
    if (ctx->nccl_comm) return fail(DPB_ESTATE, "the context already has a communicator");
    DPB_TRY(nccl_load());
    DPB_CUDA(cudaSetDevice(ctx->device));
    ncclUniqueId uid;
    memcpy(&uid, id, sizeof uid);
    ncclComm_t comm = nullptr;
    ncclResult_t r = nccl_api().ncclCommInitRank(&comm, nranks, uid, rank);
    if (r != ncclSuccess) return fail(DPB_ENCCL, "ncclCommInitRank: %s", nccl_api().ncclGetErrorString(r));
    ctx->nccl_comm = comm;
    ctx->rank = rank;
    ctx->nranks = nranks;
    ctx->gather_bytes = 64 * 1024;
    DPB_CUDA(cudaMalloc(&ctx->gather_dev, 2 * ctx->gather_bytes));
    DPB_CUDA(cudaHostAlloc(&ctx->gather_host, ctx->gather_bytes, cudaHostAllocDefault));
    return DPB_OK;
}

int dpb_comm_rank(const dpb_ctx* ctx) { return ctx ? ctx->rank : -1; }
int dpb_comm_size(const dpb_ctx* ctx) { return ctx ? ctx->nranks : 0; }

int dpb_comm_free(dpb_ctx* ctx) {
    if (!ctx || !ctx->nccl_comm) return DPB_OK;
    cudaStreamSynchronize(ctx->stream);
    nccl_api().ncclCommDestroy((ncclComm_t)ctx->nccl_comm);
    ctx->nccl_comm = nullptr;
    ctx->nranks = 1;
    ctx->rank = 0;
    cudaFree(ctx->gather_dev);
    cudaFreeHost(ctx->gather_host);
    ctx->gather_dev = ctx->gather_host = nullptr;
    return DPB_OK;
}

}  // extern "C"
