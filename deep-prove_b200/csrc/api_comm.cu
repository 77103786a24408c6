// C ABI: the per-context NCCL communicator used by sharded sumchecks.
//
// One process per GPU.  The library does not link NCCL: libnccl.so.2 is opened
// on first use, so single-GPU users carry no dependency and a process that has
// already loaded an NCCL (e.g. through torch) shares that copy.  The exchange
// per round is tiny (d+1 field elements per rank) and its readers are the
// HOSTS (each adds the partial sums mod p and runs the transcript; NCCL has no
// modular sum).  On one node the ranks therefore share a small POSIX
// shared-memory segment that each process registers with CUDA: a rank's round
// kernel writes its sums and a sequence number straight into it and every host
// polls it — no collective and no device-to-host copy on the per-round path.
// When the ranks are not on one host, or the set-up fails anywhere, the
// exchange is one ncclAllGather over NVLink followed by a copy to the host.
// NCCL also carries the once-per-proof gather of the one-entry shards.
#include <dlfcn.h>
#include <fcntl.h>
#include <nccl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <random>
#include <thread>

#include <algorithm>

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

int xch_collect(dpb_ctx* ctx, unsigned int seq, size_t msg_bytes, void* out, double seconds) {
    const auto t0 = std::chrono::steady_clock::now();
    uint64_t spins = 0;
    const size_t words = msg_bytes / 8;
    for (int q = 0; q < ctx->nranks; q++) {
        const volatile TailChunk* c = (const volatile TailChunk*)((const char*)ctx->xch_host + xch_slot_offset(q, seq));
        uint64_t* dst = (uint64_t*)((char*)out + (size_t)q * msg_bytes);
        for (size_t w = 0; w < words; w++) {
            while (c[w].seq != seq) {
                if ((++spins & 0xFFF) == 0) {
                    cudaError_t e = cudaStreamQuery(ctx->stream);  // our own launch may have failed
                    if (e != cudaSuccess && e != cudaErrorNotReady)
                        return fail(DPB_ECUDA, "round kernel: %s", cudaGetErrorString(e));
                    const double dt = std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count();
                    if (dt > seconds) return fail(DPB_ETIMEOUT, "waited %.1f s for the partial sums of rank %d", dt, q);
                }
            }
            std::atomic_thread_fence(std::memory_order_acquire);
            dst[w] = c[w].data;
        }
    }
    return DPB_OK;
}

// FNV-1a over the host name and the boot id: equal on two ranks exactly when they share a host
static uint64_t host_fingerprint() {
    char buf[512];
    memset(buf, 0, sizeof buf);
    gethostname(buf, 255);
    if (FILE* f = fopen("/proc/sys/kernel/random/boot_id", "r")) {
        const size_t used = strlen(buf);
        if (!fgets(buf + used, (int)(sizeof buf - used - 1), f)) buf[used] = 0;
        fclose(f);
    }
    uint64_t h = 1469598103934665603ull;
    for (const char* p = buf; *p; p++) h = (h ^ (unsigned char)*p) * 1099511628211ull;
    return h;
}

// every rank contributes one 64-bit word; true when all are equal to ours
static int all_ranks_agree(dpb_ctx* ctx, uint64_t mine, bool* agree) {
    uint64_t* slot = (uint64_t*)((char*)ctx->gather_dev + (size_t)ctx->rank * 8);
    DPB_CUDA(cudaMemcpyAsync(slot, &mine, 8, cudaMemcpyHostToDevice, ctx->stream));
    DPB_TRY(allgather_to_host(ctx, slot, 8));
    *agree = true;
    for (int q = 0; q < ctx->nranks; q++)
        if (((const uint64_t*)ctx->gather_host)[q] != mine) *agree = false;
    return DPB_OK;
}

// Tries to set the shared exchange segment up; leaves ctx->xch_host null when it cannot.  Every rank ends with
// the same answer (the last step is an agreement over NCCL).
static int xch_setup(dpb_ctx* ctx, const void* unique_id) {
    bool same_host = false;
    DPB_TRY(all_ranks_agree(ctx, host_fingerprint(), &same_host));
    bool ok = same_host;
    void* map = MAP_FAILED;
    // the slots, then one 64-byte line that holds a nonce rank 0 draws for this segment
    const size_t nonce_off = (xch_bytes_for(ctx->nranks) + 63) & ~(size_t)63;
    const size_t bytes = (nonce_off + 64 + 4095) & ~(size_t)4095;
    uint64_t nonce = 0;
    char name[64];
    {
        uint64_t h = 1469598103934665603ull;
        for (size_t i = 0; i < sizeof(ncclUniqueId); i++) h = (h ^ ((const unsigned char*)unique_id)[i]) * 1099511628211ull;
        snprintf(name, sizeof name, "/dpb-xch-%016llx", (unsigned long long)h);
    }
    if (ok) {
        int fd = -1;
        if (ctx->rank == 0) {
            shm_unlink(name);  // a leftover of a crashed run with the same id
            fd = shm_open(name, O_CREAT | O_EXCL | O_RDWR, 0600);
            if (fd >= 0 && ftruncate(fd, (off_t)bytes) != 0) {
                close(fd);
                fd = -1;
            }
        } else {
            const auto t0 = std::chrono::steady_clock::now();
            while (std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() < 10.0) {
                fd = shm_open(name, O_RDWR, 0600);
                struct stat st;
                if (fd >= 0 && fstat(fd, &st) == 0 && (size_t)st.st_size >= bytes) break;
                if (fd >= 0) close(fd);
                fd = -1;
                std::this_thread::sleep_for(std::chrono::milliseconds(1));
            }
        }
        if (fd >= 0) {
            map = mmap(nullptr, bytes, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
            close(fd);
        }
        ok = map != MAP_FAILED;
        if (ok) {
            // Which segment did this rank map?  Rank 0 marks the one it created with a random non-zero word; the
            // others wait (bounded) for a mark to appear.  A rank that opened a leftover segment of the same name
            // before rank 0 unlinked it reads another value, and the agreement below then fails for everybody.
            volatile uint64_t* mark = (volatile uint64_t*)((char*)map + nonce_off);
            if (ctx->rank == 0) {
                std::random_device rd;
                do nonce = ((uint64_t)rd() << 32) ^ rd() ^ (uint64_t)std::chrono::steady_clock::now().time_since_epoch().count();
                while (nonce == 0);
                *mark = nonce;
                std::atomic_thread_fence(std::memory_order_seq_cst);
            } else {
                const auto t0 = std::chrono::steady_clock::now();
                while ((nonce = *mark) == 0 &&
                       std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count() < 10.0)
                    std::this_thread::sleep_for(std::chrono::milliseconds(1));
                ok = nonce != 0;
            }
        }
    }
    bool registered = false;
    void* dev = nullptr;
    if (ok) {
        // rank 0 created the segment zero-filled (ftruncate); nobody writes before the agreement below
        registered = cudaHostRegister(map, bytes, cudaHostRegisterMapped | cudaHostRegisterPortable) == cudaSuccess;
        ok = registered && cudaHostGetDevicePointer(&dev, map, 0) == cudaSuccess;
        if (!ok) cudaGetLastError();  // clear the sticky-free error of a refused registration
    }
    // every rank reports the mark of the segment it mapped (0: it has none): equal non-zero marks = one segment
    bool all_ok = false;
    int rc = all_ranks_agree(ctx, ok ? nonce : 0, &all_ok);
    if (ctx->rank == 0 && same_host) shm_unlink(name);  // every rank that could has mapped it by now
    if (rc == DPB_OK && ok && all_ok) {
        ctx->xch_host = map;
        ctx->xch_dev = dev;
        ctx->xch_bytes = bytes;
        ctx->xseq = 0;
        return DPB_OK;
    }
    if (registered) cudaHostUnregister(map);
    if (map != MAP_FAILED) munmap(map, bytes);
    return rc;
}

int comm_allgather_host(dpb_ctx* ctx, const void* in, size_t bytes, void* out) {
    if (ctx->nranks <= 1) {
        memcpy(out, in, bytes);
        return DPB_OK;
    }
    if (!ctx->nccl_comm) return fail(DPB_ESTATE, "the context has no communicator (dpb_comm_init)");
    // in pieces that fit the exchange buffer
    const size_t piece_max = ctx->gather_bytes / (size_t)ctx->nranks / 16 * 16;
    for (size_t done = 0; done < bytes; done += piece_max) {
        const size_t piece = std::min(piece_max, bytes - done);
        char* slot = (char*)ctx->gather_dev + (size_t)ctx->rank * piece;
        DPB_CUDA(cudaMemcpyAsync(slot, (const char*)in + done, piece, cudaMemcpyHostToDevice, ctx->stream));
        DPB_TRY(allgather_to_host(ctx, slot, piece));
        for (int q = 0; q < ctx->nranks; q++)
            memcpy((char*)out + (size_t)q * bytes + done, (const char*)ctx->gather_host + (size_t)q * piece, piece);
    }
    return DPB_OK;
}

}  // namespace dpb

using namespace dpb;

// eq(x, point) restricted to this rank's shard of the hypercube: x = (x_low, rank bits).  The shard is the eq table
// of the low coordinates times prod_b eq(rank_b, point[m - c + b]).
template <class F>
static int eq_table_shard_impl(dpb_ctx* ctx, const void* point, uint32_t m, uint32_t c, dpb_mle** out) {
    typedef typename F::E E;
    const E* pt = (const E*)point;
    E scale = F::one();
    for (uint32_t b = 0; b < c; b++) {
        const E q = pt[m - c + b];
        scale = F::mul(scale, ((ctx->rank >> b) & 1) ? q : F::sub(F::one(), q));
    }
    dpb_mle* low = nullptr;
    DPB_TRY(dpb_eq_table(ctx, F::kChalDtype, point, m - c, &low));
    dpb_mle* one_tab[1] = {low};
    const int rc = dpb_linear_combination(ctx, one_tab, &scale, 1, out);
    dpb_mle_free(low);
    return rc;
}

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
    if (nranks > 1 && !getenv("DPB_NO_SHARED_EXCHANGE")) DPB_TRY(xch_setup(ctx, id));
    return DPB_OK;
}

int dpb_eq_table_shard(dpb_ctx* ctx, int family_dtype, const void* point, uint32_t m, dpb_mle** out) {
    if (!ctx || !out || (!point && m)) return fail(DPB_EINVAL, "null argument");
    if (!valid_dtype(family_dtype)) return fail(DPB_EINVAL, "unknown dtype %d", family_dtype);
    uint32_t c = 0;
    while ((1 << c) < ctx->nranks) c++;
    if (m < c) return fail(DPB_EINVAL, "a point of %u coordinates cannot be sharded over %d ranks", m, ctx->nranks);
    return is_gl(family_dtype) ? eq_table_shard_impl<GlFam>(ctx, point, m, c, out)
                               : eq_table_shard_impl<FrFam>(ctx, point, m, c, out);
}

int dpb_comm_shared_exchange(const dpb_ctx* ctx) { return ctx && ctx->xch_host ? 1 : 0; }

int dpb_comm_rank(const dpb_ctx* ctx) { return ctx ? ctx->rank : -1; }
int dpb_comm_size(const dpb_ctx* ctx) { return ctx ? ctx->nranks : 0; }

int dpb_comm_free(dpb_ctx* ctx) {
    if (!ctx || !ctx->nccl_comm) return DPB_OK;
    cudaStreamSynchronize(ctx->stream);
    if (ctx->xch_host) {
        cudaHostUnregister(ctx->xch_host);
        munmap(ctx->xch_host, ctx->xch_bytes);
        ctx->xch_host = ctx->xch_dev = nullptr;
    }
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
