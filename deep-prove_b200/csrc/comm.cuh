// NCCL entry points resolved at run time (see api_comm.cu).
#pragma once
#include <nccl.h>

#include "common.cuh"

namespace dpb {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*ncclGetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*ncclCommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*ncclCommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*ncclCommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*ncclAllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char* (*ncclGetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*ncclCommGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;
};

// Layout of the shared exchange segment: a header line, then per rank two slots (used in turn, so that a rank may
// publish round s + 1 while a slower host still reads round s).  A slot holds up to kMaxAcc elements as 16-byte
// chunks {8 bytes of data, sequence number, pad} (see ReduceScratch::chunk_out).
constexpr size_t kXchHeader = 256;
constexpr size_t kXchSlot = (size_t)kMaxAcc * 4 * 16;
inline size_t xch_slot_offset(int rank, unsigned int seq) { return kXchHeader + ((size_t)rank * 2 + (seq & 1)) * kXchSlot; }
inline size_t xch_bytes_for(int nranks) { return kXchHeader + (size_t)nranks * 2 * kXchSlot; }
// Waits until every rank's slot of exchange `seq` is published, then copies the messages to out[rank][msg_bytes].
int xch_collect(dpb_ctx* ctx, unsigned int seq, size_t msg_bytes, void* out, double seconds);

NcclApi& nccl_api();
int nccl_load();
int sync_bounded(dpb_ctx* ctx, double seconds);

// All ranks contribute `bytes` from `send_dev`; every rank receives nranks * bytes
// at ctx->gather_dev and, after the bounded wait, in ctx->gather_host.
inline int allgather_to_host(dpb_ctx* ctx, const void* send_dev, size_t bytes) {
    if ((size_t)ctx->nranks * bytes > ctx->gather_bytes)
        return fail(DPB_EINVAL, "exchange of %zu bytes per rank exceeds the gather buffer", bytes);
    ncclResult_t r = nccl_api().ncclAllGather(send_dev, ctx->gather_dev, bytes, ncclUint8, (ncclComm_t)ctx->nccl_comm,
                                              ctx->stream);
    if (r != ncclSuccess) return fail(DPB_ENCCL, "ncclAllGather: %s", nccl_api().ncclGetErrorString(r));
    DPB_CUDA(cudaMemcpyAsync(ctx->gather_host, ctx->gather_dev, (size_t)ctx->nranks * bytes, cudaMemcpyDeviceToHost,
                             ctx->stream));
    return sync_bounded(ctx, 60.0);
}

}  // namespace dpb
