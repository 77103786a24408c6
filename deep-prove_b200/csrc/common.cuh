// Host-side plumbing shared by the C-ABI translation units: error reporting,
// the context, table handles and launch-size helpers.
#pragma once
#include <cuda_runtime.h>

#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>
#include <map>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "family.cuh"
#include "sumcheck_kernels.cuh"

namespace dpb {

// Message of the last failing call on this host thread.
std::string& last_error_slot();
int fail(int code, const char* fmt, ...);

#define DPB_CUDA(call)                                                                  \
    do {                                                                                \
        cudaError_t e__ = (call);                                                       \
        if (e__ != cudaSuccess)                                                         \
            return ::dpb::fail(e__ == cudaErrorMemoryAllocation ? DPB_ENOMEM : DPB_ECUDA, \
                               "%s: %s", #call, cudaGetErrorString(e__));               \
    } while (0)

#define DPB_TRY(call)            \
    do {                         \
        int rc__ = (call);       \
        if (rc__ != DPB_OK) return rc__; \
    } while (0)

inline bool is_gl(int dtype) {
    return dtype == DPB_GL_BASE || dtype == DPB_GL_EXT || dtype == DPB_GL_I64 || dtype == DPB_GL_I32;
}
inline bool valid_dtype(int dtype) { return dtype >= DPB_GL_BASE && dtype <= DPB_FR_I32; }
inline bool is_int_dtype(int dtype) { return dtype >= DPB_GL_I64 && dtype <= DPB_FR_I32; }
inline size_t dtype_size(int dtype) {
    switch (dtype) {
        case DPB_GL_BASE: case DPB_GL_I64: case DPB_FR_I64: return 8;
        case DPB_GL_EXT: return 16;
        case DPB_GL_I32: case DPB_FR_I32: return 4;
        default: return 32;
    }
}
inline int chal_dtype(int dtype) { return is_gl(dtype) ? DPB_GL_EXT : DPB_FR; }
inline bool is_pow2(uint64_t x) { return x && !(x & (x - 1)); }
inline uint32_t log2u(uint64_t x) {
    uint32_t l = 0;
    while ((1ull << l) < x) l++;
    return l;
}

constexpr int kMaxAcc = 8;  // round-polynomial evaluations per launch (degree <= 7)

// Opt-in host-side phase timers (dpb_trace_enable): wall time per named phase of the whole-protocol entry points,
// summed over calls -- where a logup batch or a sumcheck spends its host time (the counterpart of the reference's
// timed_instrument spans, zkml/src/layers/activation.rs:620).  Off: one relaxed load per phase.
bool trace_on();
void trace_add(const char* phase, double seconds);
struct TracePhase {
    const char* name;
    bool on;
    std::chrono::steady_clock::time_point t0;
    explicit TracePhase(const char* n) : name(n), on(trace_on()) {
        if (on) t0 = std::chrono::steady_clock::now();
    }
    void stop() {
        if (on) trace_add(name, std::chrono::duration<double>(std::chrono::steady_clock::now() - t0).count());
        on = false;
    }
    ~TracePhase() { stop(); }
};

}  // namespace dpb

struct dpb_ctx {
    int device = 0;
    int sm_count = 0;
    cudaStream_t stream = nullptr;
    // per-launch reduction scratch (partials are sized for the widest element)
    void* partials = nullptr;
    unsigned int* counter = nullptr;
    uint32_t max_blocks = 0;
    // mapped pinned buffer the last block of a round writes its sums to, as sequence-numbered 16-byte chunks
    // that the host polls (ReduceScratch::chunk_out)
    void* result_host = nullptr;
    void* result_dev = nullptr;
    size_t result_bytes = 0;
    // where the next launch publishes for the host: result_dev, this rank's slot of the shared exchange segment,
    // or null when the round is followed by a collective on the stream (the sums then go to round_out)
    void* chunk_out_dev = nullptr;
    unsigned int done_seq = 0;
    void* round_out = nullptr;  // where the current round's kernel publishes (result_dev or the exchange area)
    // small device staging area for points / challenges
    void* stage_dev = nullptr;
    size_t stage_bytes = 0;
    // communicator of sharded sumchecks (dpb_comm_init); nranks == 1 without one
    void* nccl_comm = nullptr;
    int rank = 0, nranks = 1;
    void* gather_dev = nullptr;   // send area (first half) and all-gather result (second half is unused slack)
    void* gather_host = nullptr;  // pinned copy of the all-gather result
    size_t gather_bytes = 0;
    // Single-node exchange of the per-round partial sums: a POSIX shared-memory segment that every rank maps and
    // registers with CUDA, so each rank's round kernel publishes straight into memory all hosts poll
    // (api_comm.cu).  Off (nullptr) when the ranks are not on one host or the set-up failed: NCCL all-gather then.
    void* xch_host = nullptr;
    void* xch_dev = nullptr;
    size_t xch_bytes = 0;
    unsigned int xseq = 0;     // exchanges made so far; every rank counts the same
    unsigned int done_value = 0;  // what the next launch writes into its completion flag
    // resident last-rounds kernel (generic_round.cuh): its mailbox in mapped pinned memory, the stream it
    // runs on (so that it never blocks other work of this context) and the sumcheck that owns it right now
    void* tail_box_host = nullptr;
    void* tail_box_dev = nullptr;
    cudaStream_t tail_stream = nullptr;
    cudaEvent_t tail_ev[2] = {nullptr, nullptr};
    const void* tail_owner = nullptr;
    // ring of pinned staging slots for small host-to-device copies that must not block (upload_small)
    static constexpr int kStageSlots = 8;
    static constexpr size_t kStageSlotBytes = 64 * 1024;
    void* up_host = nullptr;
    cudaEvent_t up_ev[kStageSlots] = {};
    bool up_used[kStageSlots] = {};
    int up_next = 0;
    // Device memory of the context (device_alloc / device_free, api_core.cu).  Requests below 2 GiB are cut out of
    // arenas of 8 GiB that the library takes from the stream-ordered pool and keeps (first fit by address, freed
    // ranges merged with their neighbours); larger requests get a block of their own, and the last of those (up to
    // 16 blocks, 96 GiB) are kept for a request of the same size.  Why: a proof asks for the same few hundred sizes layer after layer,
    // and the stream-ordered allocator was measured to take milliseconds per block of 128 MB..1 GiB in that pattern
    // (1.6 s of a 3.3 s GPT-2 walk), differently from run to run.  Every allocation of a context is used on its one
    // stream, so handing a freed range to the next request is as safe as the pool's own stream-ordered reuse.
    struct Arena {
        char* base = nullptr;  // nullptr: released
        size_t bytes = 0, used = 0;
        std::map<size_t, size_t> free_ranges;  // offset -> length
    };
    struct Live {
        int32_t arena;  // index into arenas, or -1: a block of its own
        size_t bytes;
    };
    struct Block {
        void* p;
        size_t bytes;
    };
    std::mutex block_mu;
    std::vector<Arena> arenas;
    std::unordered_map<void*, Live> block_live;
    std::vector<Block> big_free;  // kept blocks of 2 GiB and more, oldest first
    // side streams of dpb_pcs_batch_commit (the commitments of a batch run next to each other), made on first use
    static constexpr int kMsmStreams = 4;
    cudaStream_t msm_stream[kMsmStreams] = {};
    cudaEvent_t msm_ev[kMsmStreams + 1] = {};
    void* msm_host = nullptr;  // pinned: the window sums of the commitments in flight
    // the block of device memory the last sumcheck used, kept for the next one (dpb_sumcheck_begin)
    void* slab_cache = nullptr;
    size_t slab_cache_bytes = 0;
    bool slab_cache_busy = false;
    bool tail_enabled = true;
    uint64_t sumcheck_launches = 0;  // kernels launched by the sumcheck entry points
    unsigned long long tail_wait_ns = 1ull * 1000 * 1000 * 1000;
    // optional per-kernel timing log (dpb_profile_enable)
    bool profile = false;
    cudaEvent_t prof_ev[2] = {nullptr, nullptr};
    std::vector<dpb_profile_entry> prof_log;
};

struct dpb_mle {
    dpb_ctx* ctx = nullptr;
    int dtype = 0;
    uint64_t len = 0;
    void* ptr = nullptr;
    bool owns = false;
    bool zero_pad = false;  // in a sumcheck over more variables: zero above its length (else: constant in the early rounds)
    // Set on the tables dpb_eq_table / dpb_eq_tables return: the point (challenge elements, native bytes) the table
    // is the eq table of.  A sumcheck whose terms all carry such a table runs its large rounds in split-eq form.
    std::vector<uint8_t> eq_point;
};

namespace dpb {

inline uint32_t grid_for(const dpb_ctx* ctx, uint64_t work_items, uint32_t per_sm = 8) {
    uint64_t b = (work_items + kThreads - 1) / kThreads;
    const uint64_t cap = (uint64_t)ctx->sm_count * per_sm;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    if (b > ctx->max_blocks) b = ctx->max_blocks;
    return (uint32_t)b;
}

template <class F>
inline ReduceScratch<F> reduce_scratch(const dpb_ctx* ctx) {
    ReduceScratch<F> rs;
    rs.partials = (typename F::E*)ctx->partials;
    rs.counter = ctx->counter;
    rs.chunk_out = ctx->chunk_out_dev;
    rs.done_value = ctx->done_value;
    return rs;
}

int device_alloc(dpb_ctx* ctx, size_t bytes, void** out);
void device_free(dpb_ctx* ctx, void* p);
// Queues a copy of a (small) host buffer to device memory on the context's stream and returns at once: the
// bytes are taken now, into pinned staging slots, so the caller may free or reuse `src` immediately.
int upload_small(dpb_ctx* ctx, void* dst, const void* src, size_t bytes);
int new_mle(dpb_ctx* ctx, int dtype, uint64_t len, dpb_mle** out);
// copies `n` challenge elements from host memory to the staging area and returns the device pointer
int stage_to_device(dpb_ctx* ctx, const void* host, size_t bytes, size_t offset, void** dev);

// Every rank contributes `bytes` of host data; out receives nranks * bytes in rank order (api_comm.cu).  With one
// rank: a copy.  Bounded wait; DPB_EINVAL when nranks * bytes exceeds the context's exchange buffer.
int comm_allgather_host(dpb_ctx* ctx, const void* in, size_t bytes, void* out);

// What the batched logup prover knows about a layer sumcheck it is about to run (host/logup.hpp): the instances in the
// order of the sumcheck's tables, and the layer's constants.  sumcheck_hint_logup hands it to a sumcheck right after
// dpb_sumcheck_begin; when the sumcheck runs in split-eq form with that single eq table, its large rounds then use
// the layer's own formula (sc_round_logup) instead of the term list.  The hint must describe the polynomial the term
// list describes; a hint the sumcheck cannot use is ignored.
struct LogupHintInst {
    int kind;        // 0 inner layer (4 tables), 1 lookup input layer (2 * ncol tables), 2 table input layer (2 + 2 * ncol)
    uint32_t first;  // index of its first table
    uint32_t ncol;
    alignas(16) uint8_t alpha[32], constant[32], sep[32];  // challenge elements: alpha_j, and for input layers c and s
};
void sumcheck_hint_logup(dpb_sc* sc, const LogupHintInst* inst, uint32_t n_inst, const void* lambda, uint32_t eq_table);

}  // namespace dpb
