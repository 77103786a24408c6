// C ABI: context, table handles, layout conversion, eq tables and partial
// evaluation (fix_high / fix_low / evaluate).
#include <algorithm>
#include <atomic>
#include <mutex>

#include "common.cuh"
#include "fix_kernels.cuh"
#include "poly_kernels.cuh"

namespace dpb {

std::string& last_error_slot() {
    static thread_local std::string s;
    return s;
}

static std::atomic<bool> g_trace{false};
static std::mutex g_trace_mu;
static std::vector<std::pair<std::string, std::pair<double, uint64_t>>> g_trace_log;
bool trace_on() { return g_trace.load(std::memory_order_relaxed); }
void trace_add(const char* phase, double seconds) {
    std::lock_guard<std::mutex> lock(g_trace_mu);
    for (auto& e : g_trace_log)
        if (e.first == phase) {
            e.second.first += seconds;
            e.second.second++;
            return;
        }
    g_trace_log.push_back({phase, {seconds, 1}});
}

int fail(int code, const char* fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    last_error_slot() = buf;
    return code;
}

constexpr size_t kArenaBytes = (size_t)8 << 30;   // what the library takes from the pool at a time
constexpr size_t kBigBlock = (size_t)2 << 30;     // requests of this size and more get a block of their own
constexpr size_t kBigKeepCount = 16;              // freed big blocks kept for a request of the same size
constexpr size_t kBigKeepBytes = (size_t)96 << 30;
constexpr size_t kAllocAlign = 256;

// DPB_ARENA=0: every request goes to the stream-ordered allocator itself (to compare the two)
static bool arena_enabled() {
    static const bool v = [] {
        const char* e = getenv("DPB_ARENA");
        return !(e && e[0] == '0');
    }();
    return v;
}

// gives unused memory back to the pool: arenas nothing lives in, and the kept big blocks
static void arena_release_unused(dpb_ctx* ctx) {
    for (auto& a : ctx->arenas) {
        if (a.base && a.used == 0) {
            cudaFreeAsync(a.base, ctx->stream);
            a.base = nullptr;
            a.bytes = 0;
            a.free_ranges.clear();
        }
    }
    for (const auto& b : ctx->big_free) cudaFreeAsync(b.p, ctx->stream);
    ctx->big_free.clear();
}

static cudaError_t pool_alloc(dpb_ctx* ctx, size_t bytes, void** out) {
    cudaError_t e = cudaMallocAsync(out, bytes, ctx->stream);
    if (e == cudaErrorMemoryAllocation) {
        // what the library keeps may be what stands in the way: give it back and ask again
        cudaGetLastError();
        arena_release_unused(ctx);
        e = cudaMallocAsync(out, bytes, ctx->stream);
    }
    if (e != cudaSuccess) cudaGetLastError();
    return e;
}

int device_alloc(dpb_ctx* ctx, size_t bytes, void** out) {
    if (bytes == 0) bytes = 16;
    bytes = (bytes + kAllocAlign - 1) & ~(kAllocAlign - 1);
    std::lock_guard<std::mutex> lock(ctx->block_mu);
    if (!arena_enabled()) {
        const cudaError_t e = pool_alloc(ctx, bytes, out);
        if (e != cudaSuccess)
            return fail(e == cudaErrorMemoryAllocation ? DPB_ENOMEM : DPB_ECUDA, "device allocation of %zu bytes: %s", bytes,
                        cudaGetErrorString(e));
        return DPB_OK;
    }
    if (bytes >= kBigBlock) {
        for (size_t i = ctx->big_free.size(); i-- > 0;) {  // newest first
            if (ctx->big_free[i].bytes != bytes) continue;
            *out = ctx->big_free[i].p;
            ctx->big_free.erase(ctx->big_free.begin() + i);
            ctx->block_live[*out] = {-1, bytes};
            return DPB_OK;
        }
        const cudaError_t e = pool_alloc(ctx, bytes, out);
        if (e != cudaSuccess)
            return fail(e == cudaErrorMemoryAllocation ? DPB_ENOMEM : DPB_ECUDA, "device allocation of %zu bytes: %s", bytes,
                        cudaGetErrorString(e));
        ctx->block_live[*out] = {-1, bytes};
        return DPB_OK;
    }
    // first fit by address over the arenas
    for (int pass = 0; pass < 2; pass++) {
        for (size_t ai = 0; ai < ctx->arenas.size(); ai++) {
            auto& a = ctx->arenas[ai];
            if (!a.base || a.bytes - a.used < bytes) continue;
            for (auto it = a.free_ranges.begin(); it != a.free_ranges.end(); ++it) {
                if (it->second < bytes) continue;
                const size_t off = it->first, len = it->second;
                a.free_ranges.erase(it);
                if (len > bytes) a.free_ranges[off + bytes] = len - bytes;
                a.used += bytes;
                *out = a.base + off;
                ctx->block_live[*out] = {(int32_t)ai, bytes};
                return DPB_OK;
            }
        }
        if (pass == 1) break;
        // a new arena: 8 GiB, less when the device cannot give that much (never less than the request)
        size_t want = kArenaBytes;
        void* base = nullptr;
        cudaError_t e = cudaErrorMemoryAllocation;
        while (want >= bytes) {
            e = cudaMallocAsync(&base, want, ctx->stream);
            if (e == cudaSuccess) break;
            cudaGetLastError();
            if (e != cudaErrorMemoryAllocation) break;
            if (want == bytes) break;
            want = std::max(bytes, want / 2);
        }
        if (e != cudaSuccess) {
            arena_release_unused(ctx);
            want = std::max(bytes, (size_t)256 << 20);
            e = cudaMallocAsync(&base, want, ctx->stream);
            if (e != cudaSuccess) {
                cudaGetLastError();
                return fail(e == cudaErrorMemoryAllocation ? DPB_ENOMEM : DPB_ECUDA, "device allocation of %zu bytes: %s", bytes,
                            cudaGetErrorString(e));
            }
        }
        dpb_ctx::Arena* slot = nullptr;
        for (auto& a : ctx->arenas)
            if (!a.base) {
                slot = &a;
                break;
            }
        if (!slot) {
            ctx->arenas.emplace_back();
            slot = &ctx->arenas.back();
        }
        slot->base = (char*)base;
        slot->bytes = want;
        slot->used = 0;
        slot->free_ranges.clear();
        slot->free_ranges[0] = want;
    }
    return fail(DPB_ENOMEM, "device allocation of %zu bytes: no arena could hold it", bytes);
}

void device_free(dpb_ctx* ctx, void* p) {
    if (!p) return;
    std::lock_guard<std::mutex> lock(ctx->block_mu);
    auto it = ctx->block_live.find(p);
    if (it == ctx->block_live.end()) {
        cudaFreeAsync(p, ctx->stream);  // not from the arenas (DPB_ARENA=0)
        return;
    }
    const dpb_ctx::Live live = it->second;
    ctx->block_live.erase(it);
    if (live.arena < 0) {
        ctx->big_free.push_back({p, live.bytes});
        size_t total = 0;
        for (const auto& b : ctx->big_free) total += b.bytes;
        while (ctx->big_free.size() > kBigKeepCount || total > kBigKeepBytes) {
            cudaFreeAsync(ctx->big_free.front().p, ctx->stream);
            total -= ctx->big_free.front().bytes;
            ctx->big_free.erase(ctx->big_free.begin());
        }
        return;
    }
    auto& a = ctx->arenas[live.arena];
    size_t off = (size_t)((char*)p - a.base), len = live.bytes;
    a.used -= len;
    // merge with the free range after and the one before
    auto next = a.free_ranges.lower_bound(off);
    if (next != a.free_ranges.end() && next->first == off + len) {
        len += next->second;
        next = a.free_ranges.erase(next);
    }
    if (next != a.free_ranges.begin()) {
        auto prev = std::prev(next);
        if (prev->first + prev->second == off) {
            off = prev->first;
            len += prev->second;
            a.free_ranges.erase(prev);
        }
    }
    a.free_ranges[off] = len;
}

int upload_small(dpb_ctx* ctx, void* dst, const void* src, size_t bytes) {
    size_t done = 0;
    while (done < bytes) {
        const int slot = ctx->up_next;
        ctx->up_next = (slot + 1) % dpb_ctx::kStageSlots;
        // a slot is reused only after the copy that last read it has run (long ago, as a rule)
        if (ctx->up_used[slot]) DPB_CUDA(cudaEventSynchronize(ctx->up_ev[slot]));
        const size_t n = std::min(bytes - done, dpb_ctx::kStageSlotBytes);
        char* stage = (char*)ctx->up_host + (size_t)slot * dpb_ctx::kStageSlotBytes;
        memcpy(stage, (const char*)src + done, n);
        DPB_CUDA(cudaMemcpyAsync((char*)dst + done, stage, n, cudaMemcpyHostToDevice, ctx->stream));
        DPB_CUDA(cudaEventRecord(ctx->up_ev[slot], ctx->stream));
        ctx->up_used[slot] = true;
        done += n;
    }
    return DPB_OK;
}

int new_mle(dpb_ctx* ctx, int dtype, uint64_t len, dpb_mle** out) {
    dpb_mle* m = new (std::nothrow) dpb_mle();
    if (!m) return fail(DPB_ENOMEM, "host allocation failed");
    m->ctx = ctx;
    m->dtype = dtype;
    m->len = len;
    m->owns = true;
    int rc = device_alloc(ctx, len * dtype_size(dtype), &m->ptr);
    if (rc != DPB_OK) {
        delete m;
        return rc;
    }
    *out = m;
    return DPB_OK;
}

int stage_to_device(dpb_ctx* ctx, const void* host, size_t bytes, size_t offset, void** dev) {
    if (offset + bytes > ctx->stage_bytes)
        return fail(DPB_EINVAL, "staging area too small (%zu + %zu > %zu)", offset, bytes,
                    ctx->stage_bytes);
    *dev = (char*)ctx->stage_dev + offset;
    return upload_small(ctx, *dev, host, bytes);
}

// eq(x, pt) table over m variables into freshly allocated device memory.
template <class F>
static int eq_table_dev(dpb_ctx* ctx, const typename F::E* pt_dev, uint32_t m,
                        typename F::E** out) {
    typedef typename F::E E;
    const uint64_t n = 1ull << m;
    E* res = nullptr;
    DPB_TRY(device_alloc(ctx, n * sizeof(E), (void**)&res));
    constexpr uint32_t kDirect = 10;
    if (m <= kDirect) {
        eq_direct<F><<<grid_for(ctx, n), kThreads, 0, ctx->stream>>>(pt_dev, m, res);
    } else {
        E* lo = nullptr;
        E* hi = nullptr;
        DPB_TRY(device_alloc(ctx, sizeof(E) << kDirect, (void**)&lo));
        eq_direct<F><<<grid_for(ctx, 1ull << kDirect), kThreads, 0, ctx->stream>>>(pt_dev, kDirect, lo);
        int rc = eq_table_dev<F>(ctx, pt_dev + kDirect, m - kDirect, &hi);
        if (rc != DPB_OK) {
            device_free(ctx, lo);
            device_free(ctx, res);
            return rc;
        }
        eq_combine<F><<<grid_for(ctx, n), kThreads, 0, ctx->stream>>>(lo, kDirect, hi, n, res);
        device_free(ctx, lo);
        device_free(ctx, hi);
    }
    DPB_CUDA(cudaGetLastError());
    *out = res;
    return DPB_OK;
}

template <class F>
static int eq_table_impl(dpb_ctx* ctx, const void* point, uint32_t m, dpb_mle** out) {
    typedef typename F::E E;
    void* pt_dev = nullptr;
    if (m > 0) DPB_TRY(stage_to_device(ctx, point, m * sizeof(E), 0, &pt_dev));
    E* res = nullptr;
    DPB_TRY(eq_table_dev<F>(ctx, (const E*)pt_dev, m, &res));
    dpb_mle* h = new (std::nothrow) dpb_mle();
    if (!h) return fail(DPB_ENOMEM, "host allocation failed");
    h->ctx = ctx;
    h->dtype = F::kChalDtype;
    h->len = 1ull << m;
    h->ptr = res;
    h->owns = true;
    if (m) h->eq_point.assign((const uint8_t*)point, (const uint8_t*)point + m * sizeof(E));
    *out = h;
    return DPB_OK;
}

// Binds k variables from the top (high = true) or the bottom, at most 5 per
// pass so every pass keeps the whole device busy.
template <class F>
static int fix_vars_impl(dpb_ctx* ctx, const void* in, int dtype_in, uint64_t len,
                         const void* point_host, uint32_t k, bool high, void** out_ptr) {
    typedef typename F::E E;
    void* pt_dev = nullptr;
    DPB_TRY(stage_to_device(ctx, point_host, k * sizeof(E), 0, &pt_dev));
    const E* pt = (const E*)pt_dev;
    const void* cur = in;
    int cur_dtype = dtype_in;
    uint64_t cur_len = len;
    void* owned = nullptr;  // intermediate we must free
    uint32_t done = 0;
    E* w = nullptr;
    DPB_TRY(device_alloc(ctx, sizeof(E) * 32, (void**)&w));
    while (done < k) {
        const uint32_t g = (k - done) < 5 ? (k - done) : 5;
        // high: bind the top g of the variables still free, i.e. point[k-done-g .. k-done)
        // low : bind the bottom g, i.e. point[done .. done+g)
        const E* sub = high ? pt + (k - done - g) : pt + done;
        eq_direct<F><<<1, 32, 0, ctx->stream>>>(sub, g, w);
        const uint64_t n_out = cur_len >> g;
        E* nxt = nullptr;
        int rc = device_alloc(ctx, n_out * sizeof(E), (void**)&nxt);
        if (rc != DPB_OK) {
            device_free(ctx, owned);
            device_free(ctx, w);
            return rc;
        }
        if (high)
            fix_high_sum<F><<<grid_for(ctx, n_out), kThreads, 0, ctx->stream>>>(cur, cur_dtype, w, g, n_out, nxt);
        else
            fix_low_sum<F><<<grid_for(ctx, n_out), kThreads, 0, ctx->stream>>>(cur, cur_dtype, w, g, n_out, nxt);
        device_free(ctx, owned);
        owned = nxt;
        cur = nxt;
        cur_dtype = F::kChalDtype;
        cur_len = n_out;
        done += g;
    }
    device_free(ctx, w);
    DPB_CUDA(cudaGetLastError());
    *out_ptr = owned;
    return DPB_OK;
}

static int fix_common(dpb_ctx* ctx, const dpb_mle* mle, const void* point, uint32_t k, bool high,
                      dpb_mle** out) {
    if (!ctx || !mle || !out || (!point && k)) return fail(DPB_EINVAL, "null argument");
    const uint32_t n = log2u(mle->len);
    if (k == 0 || k > n) return fail(DPB_EINVAL, "cannot bind %u of %u variables", k, n);
    if (k * dtype_size(chal_dtype(mle->dtype)) > ctx->stage_bytes)
        return fail(DPB_EINVAL, "point too long");
    void* res = nullptr;
    int rc = is_gl(mle->dtype)
                 ? fix_vars_impl<GlFam>(ctx, mle->ptr, mle->dtype, mle->len, point, k, high, &res)
                 : fix_vars_impl<FrFam>(ctx, mle->ptr, mle->dtype, mle->len, point, k, high, &res);
    if (rc != DPB_OK) return rc;
    dpb_mle* h = new (std::nothrow) dpb_mle();
    if (!h) return fail(DPB_ENOMEM, "host allocation failed");
    h->ctx = ctx;
    h->dtype = chal_dtype(mle->dtype);
    h->len = mle->len >> k;
    h->ptr = res;
    h->owns = true;
    *out = h;
    return DPB_OK;
}

}  // namespace dpb

using namespace dpb;

template <class F>
int eq_tables_impl(dpb_ctx* ctx, const void* points, const uint32_t* num_vars, uint32_t n, dpb_mle** out_owner,
                          dpb_mle** out_tables) {
    typedef typename F::E E;
    std::vector<EqBatchDesc> desc(n);
    std::vector<uint64_t> part_prefix(n + 1), out_prefix(n + 1);
    uint64_t pt = 0, parts = 0, outs = 0;
    for (uint32_t t = 0; t < n; t++) {
        const uint32_t m = num_vars[t], h = (m + 1) / 2;
        if (m > 34) return fail(DPB_EINVAL, "eq table %u over %u variables is too large", t, m);
        desc[t].m = m;
        desc[t].pt_off = (uint32_t)pt;
        desc[t].part_off = parts;
        desc[t].out_off = outs;
        part_prefix[t] = parts;
        out_prefix[t] = outs;
        pt += m;
        parts += (1ull << h) + (1ull << (m - h));
        outs += 1ull << m;
    }
    part_prefix[n] = parts;
    out_prefix[n] = outs;
    if (pt > 0xFFFFFFFFull) return fail(DPB_EINVAL, "too many coordinates");
    // one scratch block: [descriptors | part prefix | table prefix | points | parts]
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off = (off + bytes + 31) & ~(size_t)31;
        return o;
    };
    const size_t o_desc = take(n * sizeof(EqBatchDesc)), o_pp = take((n + 1) * 8), o_op = take((n + 1) * 8),
                 o_pts = take((size_t)pt * sizeof(E)), meta = off, o_parts = take(parts * sizeof(E));
    void* scratch = nullptr;
    DPB_TRY(device_alloc(ctx, off, &scratch));
    std::vector<uint8_t> blob(meta, 0);
    memcpy(blob.data() + o_desc, desc.data(), n * sizeof(EqBatchDesc));
    memcpy(blob.data() + o_pp, part_prefix.data(), (n + 1) * 8);
    memcpy(blob.data() + o_op, out_prefix.data(), (n + 1) * 8);
    if (pt) memcpy(blob.data() + o_pts, points, (size_t)pt * sizeof(E));
    int rc = upload_small(ctx, scratch, blob.data(), meta);
    dpb_mle* owner = nullptr;
    if (rc == DPB_OK) rc = new_mle(ctx, F::kChalDtype, outs, &owner);
    if (rc != DPB_OK) {
        device_free(ctx, scratch);
        return rc;
    }
    char* sb = (char*)scratch;
    eq_batch_parts<F><<<grid_for(ctx, parts), kThreads, 0, ctx->stream>>>(
        (const EqBatchDesc*)(sb + o_desc), (const uint64_t*)(sb + o_pp), n, (const E*)(sb + o_pts), (E*)(sb + o_parts));
    eq_batch_combine<F><<<grid_for(ctx, outs), kThreads, 0, ctx->stream>>>(
        (const EqBatchDesc*)(sb + o_desc), (const uint64_t*)(sb + o_op), n, (const E*)(sb + o_parts), (E*)owner->ptr);
    cudaError_t e = cudaGetLastError();
    device_free(ctx, scratch);
    if (e != cudaSuccess) {
        dpb_mle_free(owner);
        return fail(DPB_ECUDA, "eq tables: %s", cudaGetErrorString(e));
    }
    for (uint32_t t = 0; t < n; t++) {
        rc = dpb_mle_view(owner, out_prefix[t], 1ull << num_vars[t], &out_tables[t]);
        if (rc == DPB_OK && num_vars[t])
            out_tables[t]->eq_point.assign((const uint8_t*)points + (size_t)desc[t].pt_off * sizeof(E),
                                           (const uint8_t*)points + (size_t)(desc[t].pt_off + num_vars[t]) * sizeof(E));
        if (rc != DPB_OK) {
            for (uint32_t q = 0; q < t; q++) dpb_mle_free(out_tables[q]);
            dpb_mle_free(owner);
            return rc;
        }
    }
    *out_owner = owner;
    return DPB_OK;
}

extern "C" {

const char* dpb_last_error(void) { return last_error_slot().c_str(); }

int dpb_init(int device, dpb_ctx** out) {
    if (!out) return fail(DPB_EINVAL, "null argument");
    int n_dev = 0;
    cudaError_t e = cudaGetDeviceCount(&n_dev);
    if (e != cudaSuccess || n_dev == 0)
        return fail(DPB_ECUDA, "no CUDA device available (%s); this library has no CPU path",
                    e == cudaSuccess ? "device count is 0" : cudaGetErrorString(e));
    if (device < 0 || device >= n_dev) return fail(DPB_EINVAL, "device %d out of range", device);
    DPB_CUDA(cudaSetDevice(device));
    dpb_ctx* ctx = new (std::nothrow) dpb_ctx();
    if (!ctx) return fail(DPB_ENOMEM, "host allocation failed");
    ctx->device = device;
    cudaDeviceProp prop;
    DPB_CUDA(cudaGetDeviceProperties(&prop, device));
    ctx->sm_count = prop.multiProcessorCount;
    DPB_CUDA(cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking));
    // keep freed blocks in the stream-ordered pool instead of returning them to the driver
    cudaMemPool_t pool;
    DPB_CUDA(cudaDeviceGetDefaultMemPool(&pool, device));
    uint64_t thresh = UINT64_MAX;
    DPB_CUDA(cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &thresh));
    // The resident last-rounds kernel needs the host to answer while it runs.  When launches are known to block the
    // launching thread (CUDA_LAUNCH_BLOCKING, or a tool injected into the process that serialises kernels) it is
    // not started at all; otherwise the first one still finds out by itself (its bounded wait for the host's first
    // sign of life) and the context falls back then.
    {
        const char* blocking = getenv("CUDA_LAUNCH_BLOCKING");
        const char* injected = getenv("CUDA_INJECTION64_PATH");
        const char* assume_async = getenv("DPB_ASSUME_ASYNC_LAUNCHES");  // skips this check (the kernel's own stays)
        if (!(assume_async && assume_async[0] == '1') &&
            ((blocking && blocking[0] && strcmp(blocking, "0") != 0) || (injected && injected[0])))
            ctx->tail_enabled = false;
    }
    ctx->max_blocks = (uint32_t)ctx->sm_count * 8;
    DPB_CUDA(cudaMalloc(&ctx->partials, (size_t)ctx->max_blocks * kMaxAcc * sizeof(Fr)));
    DPB_CUDA(cudaMalloc((void**)&ctx->counter, 256));
    DPB_CUDA(cudaMemset(ctx->counter, 0, 256));
    ctx->result_bytes = 64 * 1024;
    DPB_CUDA(cudaHostAlloc(&ctx->result_host, ctx->result_bytes, cudaHostAllocMapped));
    DPB_CUDA(cudaHostGetDevicePointer(&ctx->result_dev, ctx->result_host, 0));
    memset(ctx->result_host, 0, ctx->result_bytes);
    ctx->stage_bytes = 64 * 1024;
    DPB_CUDA(cudaMalloc(&ctx->stage_dev, ctx->stage_bytes));
    DPB_CUDA(cudaEventCreate(&ctx->prof_ev[0]));
    DPB_CUDA(cudaEventCreate(&ctx->prof_ev[1]));
    DPB_CUDA(cudaHostAlloc(&ctx->up_host, dpb_ctx::kStageSlots * dpb_ctx::kStageSlotBytes, cudaHostAllocDefault));
    for (int i = 0; i < dpb_ctx::kStageSlots; i++)
        DPB_CUDA(cudaEventCreateWithFlags(&ctx->up_ev[i], cudaEventDisableTiming));
    DPB_CUDA(cudaHostAlloc(&ctx->tail_box_host, 8192, cudaHostAllocMapped));
    DPB_CUDA(cudaHostGetDevicePointer(&ctx->tail_box_dev, ctx->tail_box_host, 0));
    memset(ctx->tail_box_host, 0, 8192);
    DPB_CUDA(cudaStreamCreateWithFlags(&ctx->tail_stream, cudaStreamNonBlocking));
    DPB_CUDA(cudaEventCreateWithFlags(&ctx->tail_ev[0], cudaEventDisableTiming));
    DPB_CUDA(cudaEventCreateWithFlags(&ctx->tail_ev[1], cudaEventDisableTiming));
    *out = ctx;
    return DPB_OK;
}

void dpb_shutdown(dpb_ctx* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->slab_cache) device_free(ctx, ctx->slab_cache);
    {
        // tables the caller never freed die with the context
        std::lock_guard<std::mutex> lock(ctx->block_mu);
        for (auto& a : ctx->arenas)
            if (a.base) cudaFreeAsync(a.base, ctx->stream);
        ctx->arenas.clear();
        for (const auto& kv : ctx->block_live)
            if (kv.second.arena < 0) cudaFreeAsync(kv.first, ctx->stream);
        ctx->block_live.clear();
        for (const auto& b : ctx->big_free) cudaFreeAsync(b.p, ctx->stream);
        ctx->big_free.clear();
    }
    cudaStreamSynchronize(ctx->stream);
    cudaStreamSynchronize(ctx->tail_stream);
    for (int i = 0; i < dpb_ctx::kMsmStreams; i++)
        if (ctx->msm_stream[i]) {
            cudaStreamSynchronize(ctx->msm_stream[i]);
            cudaStreamDestroy(ctx->msm_stream[i]);
        }
    for (int i = 0; i <= dpb_ctx::kMsmStreams; i++)
        if (ctx->msm_ev[i]) cudaEventDestroy(ctx->msm_ev[i]);
    if (ctx->msm_host) cudaFreeHost(ctx->msm_host);
    cudaStreamDestroy(ctx->tail_stream);
    cudaEventDestroy(ctx->tail_ev[0]);
    cudaEventDestroy(ctx->tail_ev[1]);
    cudaFreeHost(ctx->tail_box_host);
    cudaFreeHost(ctx->up_host);
    for (int i = 0; i < dpb_ctx::kStageSlots; i++) cudaEventDestroy(ctx->up_ev[i]);
    cudaFree(ctx->partials);
    cudaFree(ctx->counter);
    cudaFree(ctx->stage_dev);
    cudaFreeHost(ctx->result_host);
    cudaEventDestroy(ctx->prof_ev[0]);
    cudaEventDestroy(ctx->prof_ev[1]);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
}

int dpb_trim(dpb_ctx* ctx) {
    if (!ctx) return fail(DPB_EINVAL, "null context");
    DPB_CUDA(cudaSetDevice(ctx->device));
    if (ctx->slab_cache && !ctx->slab_cache_busy) {
        device_free(ctx, ctx->slab_cache);
        ctx->slab_cache = nullptr;
        ctx->slab_cache_bytes = 0;
    }
    {
        std::lock_guard<std::mutex> lock(ctx->block_mu);
        arena_release_unused(ctx);
    }
    DPB_CUDA(cudaStreamSynchronize(ctx->stream));
    cudaMemPool_t pool;
    DPB_CUDA(cudaDeviceGetDefaultMemPool(&pool, ctx->device));
    DPB_CUDA(cudaMemPoolTrimTo(pool, 0));
    return DPB_OK;
}

int dpb_sync(dpb_ctx* ctx) {
    if (!ctx) return fail(DPB_EINVAL, "null context");
    DPB_CUDA(cudaStreamSynchronize(ctx->stream));
    return DPB_OK;
}

void* dpb_stream(dpb_ctx* ctx) { return ctx ? (void*)ctx->stream : nullptr; }

uint64_t dpb_sumcheck_launches(const dpb_ctx* ctx) { return ctx ? ctx->sumcheck_launches : 0; }

int dpb_resident_rounds(dpb_ctx* ctx, int enable, uint32_t wait_ms) {
    if (!ctx) return fail(DPB_EINVAL, "null context");
    ctx->tail_enabled = enable != 0;
    if (wait_ms) ctx->tail_wait_ns = (unsigned long long)wait_ms * 1000000ull;
    return DPB_OK;
}

int dpb_profile_enable(dpb_ctx* ctx, int on) {
    if (!ctx) return fail(DPB_EINVAL, "null context");
    if (on) ctx->prof_log.clear();
    ctx->profile = on != 0;
    return DPB_OK;
}

int dpb_trace_enable(int on) {
    std::lock_guard<std::mutex> lock(g_trace_mu);
    if (on) g_trace_log.clear();
    g_trace.store(on != 0);
    return DPB_OK;
}

int dpb_trace_read(char* out, size_t cap, size_t* needed) {
    if (!needed) return fail(DPB_EINVAL, "null argument");
    std::string text;
    {
        std::lock_guard<std::mutex> lock(g_trace_mu);
        char line[160];
        for (const auto& e : g_trace_log) {
            snprintf(line, sizeof line, "%s\t%.6f\t%llu\n", e.first.c_str(), e.second.first * 1e3,
                     (unsigned long long)e.second.second);
            text += line;
        }
    }
    *needed = text.size() + 1;
    if (out && cap >= text.size() + 1) memcpy(out, text.c_str(), text.size() + 1);
    return DPB_OK;
}

int dpb_profile_read(dpb_ctx* ctx, dpb_profile_entry* out, uint32_t cap, uint32_t* n) {
    if (!ctx || !n || (!out && cap)) return fail(DPB_EINVAL, "null argument");
    *n = (uint32_t)ctx->prof_log.size();
    for (uint32_t i = 0; i < *n && i < cap; i++) out[i] = ctx->prof_log[i];
    return DPB_OK;
}

int dpb_mle_alloc(dpb_ctx* ctx, int dtype, uint64_t len, dpb_mle** out) {
    if (!ctx || !out) return fail(DPB_EINVAL, "null argument");
    if (!valid_dtype(dtype)) return fail(DPB_EINVAL, "unknown dtype %d", dtype);
    if (!is_pow2(len)) return fail(DPB_EINVAL, "length %llu is not a power of two", (unsigned long long)len);
    return new_mle(ctx, dtype, len, out);
}

int dpb_mle_from_host(dpb_ctx* ctx, int dtype, const void* evals, uint64_t len, int form,
                      dpb_mle** out) {
    if (!ctx || !out || !evals) return fail(DPB_EINVAL, "null argument");
    if (!valid_dtype(dtype)) return fail(DPB_EINVAL, "unknown dtype %d", dtype);
    if (!is_pow2(len)) return fail(DPB_EINVAL, "length %llu is not a power of two", (unsigned long long)len);
    if (form == DPB_FORM_CANONICAL && dtype != DPB_FR)
        return fail(DPB_EINVAL, "canonical form applies to DPB_FR tables only");
    if (form == DPB_FORM_I64 && dtype == DPB_GL_EXT)
        return fail(DPB_EINVAL, "i64 input yields base-field or Fr tables");
    if (form < DPB_FORM_NATIVE || form > DPB_FORM_I64) return fail(DPB_EINVAL, "unknown form %d", form);
    if (is_int_dtype(dtype) && form != DPB_FORM_NATIVE)
        return fail(DPB_EINVAL, "integer tables take their integers as they are (DPB_FORM_NATIVE)");
    dpb_mle* m = nullptr;
    DPB_TRY(new_mle(ctx, dtype, len, &m));
    int rc = DPB_OK;
    if (form == DPB_FORM_NATIVE) {
        cudaError_t e = cudaMemcpyAsync(m->ptr, evals, len * dtype_size(dtype), cudaMemcpyHostToDevice, ctx->stream);
        if (e != cudaSuccess) rc = fail(DPB_ECUDA, "upload: %s", cudaGetErrorString(e));
    } else if (form == DPB_FORM_CANONICAL) {
        cudaError_t e = cudaMemcpyAsync(m->ptr, evals, len * 32, cudaMemcpyHostToDevice, ctx->stream);
        if (e != cudaSuccess) rc = fail(DPB_ECUDA, "upload: %s", cudaGetErrorString(e));
        else fr_canonical_to_mont<<<grid_for(ctx, len), kThreads, 0, ctx->stream>>>((const Fr*)m->ptr, (Fr*)m->ptr, len);
    } else {
        void* tmp = nullptr;
        rc = device_alloc(ctx, len * 8, &tmp);
        if (rc == DPB_OK) {
            cudaError_t e = cudaMemcpyAsync(tmp, evals, len * 8, cudaMemcpyHostToDevice, ctx->stream);
            if (e != cudaSuccess) rc = fail(DPB_ECUDA, "upload: %s", cudaGetErrorString(e));
            else if (dtype == DPB_FR)
                fr_from_i64_kernel<<<grid_for(ctx, len), kThreads, 0, ctx->stream>>>((const int64_t*)tmp, (Fr*)m->ptr, len);
            else
                gl_from_i64_kernel<<<grid_for(ctx, len), kThreads, 0, ctx->stream>>>((const int64_t*)tmp, (uint64_t*)m->ptr, len);
            device_free(ctx, tmp);
        }
    }
    if (rc == DPB_OK) {
        // the host buffer may be pageable and reused by the caller right away
        cudaError_t e = cudaStreamSynchronize(ctx->stream);
        if (e == cudaSuccess) e = cudaGetLastError();
        if (e != cudaSuccess) rc = fail(DPB_ECUDA, "upload: %s", cudaGetErrorString(e));
    }
    if (rc != DPB_OK) {
        dpb_mle_free(m);
        return rc;
    }
    *out = m;
    return DPB_OK;
}

int dpb_mle_from_device(dpb_ctx* ctx, int dtype, void* dev_ptr, uint64_t len, dpb_mle** out) {
    if (!ctx || !out || !dev_ptr) return fail(DPB_EINVAL, "null argument");
    if (!valid_dtype(dtype)) return fail(DPB_EINVAL, "unknown dtype %d", dtype);
    if (!is_pow2(len)) return fail(DPB_EINVAL, "length %llu is not a power of two", (unsigned long long)len);
    if (((uintptr_t)dev_ptr & 15) != 0) return fail(DPB_EINVAL, "device pointer must be 16-byte aligned");
    dpb_mle* m = new (std::nothrow) dpb_mle();
    if (!m) return fail(DPB_ENOMEM, "host allocation failed");
    m->ctx = ctx;
    m->dtype = dtype;
    m->len = len;
    m->ptr = dev_ptr;
    m->owns = false;
    *out = m;
    return DPB_OK;
}

int dpb_mle_view(const dpb_mle* mle, uint64_t offset, uint64_t len, dpb_mle** out) {
    if (!mle || !out) return fail(DPB_EINVAL, "null argument");
    if (!is_pow2(len) || offset + len > mle->len)
        return fail(DPB_EINVAL, "view [%llu, +%llu) outside a table of %llu", (unsigned long long)offset,
                    (unsigned long long)len, (unsigned long long)mle->len);
    const size_t byte_off = offset * dtype_size(mle->dtype);
    if (byte_off & 15) return fail(DPB_EINVAL, "view must start on a 16-byte boundary");
    dpb_mle* m = new (std::nothrow) dpb_mle();
    if (!m) return fail(DPB_ENOMEM, "host allocation failed");
    m->ctx = mle->ctx;
    m->dtype = mle->dtype;
    m->len = len;
    m->ptr = (char*)mle->ptr + byte_off;
    m->owns = false;
    *out = m;
    return DPB_OK;
}

int dpb_mle_zero_padded(const dpb_mle* mle, dpb_mle** out) {
    if (!mle || !out) return fail(DPB_EINVAL, "null argument");
    dpb_mle* m = new (std::nothrow) dpb_mle();
    if (!m) return fail(DPB_ENOMEM, "host allocation failed");
    *m = *mle;
    m->owns = false;
    m->zero_pad = true;
    *out = m;
    return DPB_OK;
}

int dpb_linear_combination(dpb_ctx* ctx, dpb_mle* const* mles, const void* coeffs, uint32_t n, dpb_mle** out) {
    if (!ctx || !mles || !coeffs || !out) return fail(DPB_EINVAL, "null argument");
    if (n < 1) return fail(DPB_EINVAL, "no tables");
    const bool gl = mles[0] && is_gl(mles[0]->dtype);
    uint64_t max_len = 0;
    std::vector<LinCombSrc> src(n);
    for (uint32_t j = 0; j < n; j++) {
        const dpb_mle* m = mles[j];
        if (!m || m->ctx != ctx || !valid_dtype(m->dtype) || is_gl(m->dtype) != gl)
            return fail(DPB_EINVAL, "table %u is null, foreign or of another field", j);
        src[j].ptr = m->ptr;
        src[j].len = m->len;
        src[j].dtype = m->dtype;
        src[j].pad = 0;
        if (m->len > max_len) max_len = m->len;
    }
    const size_t es = gl ? 16 : 32;
    void *d_src = nullptr, *d_coef = nullptr;
    DPB_TRY(device_alloc(ctx, n * sizeof(LinCombSrc), &d_src));
    int rc = device_alloc(ctx, n * es, &d_coef);
    if (rc == DPB_OK) rc = upload_small(ctx, d_src, src.data(), n * sizeof(LinCombSrc));
    if (rc == DPB_OK) rc = upload_small(ctx, d_coef, coeffs, n * es);
    dpb_mle* res = nullptr;
    if (rc == DPB_OK) rc = new_mle(ctx, gl ? DPB_GL_EXT : DPB_FR, max_len, &res);
    if (rc == DPB_OK) {
        if (gl)
            linear_combination_kernel<GlFam><<<grid_for(ctx, max_len), kThreads, 0, ctx->stream>>>(
                (const LinCombSrc*)d_src, (const Gl2*)d_coef, n, max_len, (Gl2*)res->ptr);
        else
            linear_combination_kernel<FrFam><<<grid_for(ctx, max_len), kThreads, 0, ctx->stream>>>(
                (const LinCombSrc*)d_src, (const Fr*)d_coef, n, max_len, (Fr*)res->ptr);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) rc = fail(DPB_ECUDA, "linear combination: %s", cudaGetErrorString(e));
    }
    device_free(ctx, d_src);
    device_free(ctx, d_coef);
    if (rc != DPB_OK) {
        if (res) dpb_mle_free(res);
        return rc;
    }
    *out = res;
    return DPB_OK;
}

int dpb_rope_permuted_eq(dpb_ctx* ctx, const dpb_mle* eq, int layout, uint64_t row_size, dpb_mle** out) {
    if (!ctx || !eq || !out) return fail(DPB_EINVAL, "null argument");
    if (eq->ctx != ctx) return fail(DPB_EINVAL, "table of another context");
    if (eq->dtype != DPB_FR && eq->dtype != DPB_GL_EXT) return fail(DPB_EINVAL, "an eq table holds challenge elements");
    if (layout != 0 && layout != 1) return fail(DPB_EINVAL, "layout is 0 (adjacent pairs) or 1 (rotate half)");
    if (eq->len < 2 || (eq->len & 1)) return fail(DPB_EINVAL, "table length must be even");
    if (layout == 1 && (row_size < 2 || (row_size & 1) || eq->len % row_size))
        return fail(DPB_EINVAL, "rotate half: the row size must be even and divide the table length");
    dpb_mle* res = nullptr;
    DPB_TRY(new_mle(ctx, eq->dtype, eq->len, &res));
    if (eq->dtype == DPB_FR)
        rope_permuted_eq_kernel<FrFam><<<grid_for(ctx, eq->len), kThreads, 0, ctx->stream>>>(
            (const Fr*)eq->ptr, eq->len, layout, row_size, (Fr*)res->ptr);
    else
        rope_permuted_eq_kernel<GlFam><<<grid_for(ctx, eq->len), kThreads, 0, ctx->stream>>>(
            (const Gl2*)eq->ptr, eq->len, layout, row_size, (Gl2*)res->ptr);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        dpb_mle_free(res);
        return fail(DPB_ECUDA, "permuted eq: %s", cudaGetErrorString(e));
    }
    *out = res;
    return DPB_OK;
}

int dpb_mle_free(dpb_mle* mle) {
    if (!mle) return DPB_OK;
    if (mle->owns) device_free(mle->ctx, mle->ptr);
    delete mle;
    return DPB_OK;
}

int dpb_mle_to_host(const dpb_mle* mle, void* out, uint64_t len, int form) {
    if (!mle || !out) return fail(DPB_EINVAL, "null argument");
    if (len > mle->len) return fail(DPB_EINVAL, "asked for %llu of %llu entries", (unsigned long long)len,
                                    (unsigned long long)mle->len);
    dpb_ctx* ctx = mle->ctx;
    if (form == DPB_FORM_NATIVE) {
        DPB_CUDA(cudaMemcpyAsync(out, mle->ptr, len * dtype_size(mle->dtype), cudaMemcpyDeviceToHost, ctx->stream));
    } else if (form == DPB_FORM_CANONICAL && mle->dtype == DPB_FR) {
        void* tmp = nullptr;
        DPB_TRY(device_alloc(ctx, len * 32, &tmp));
        fr_mont_to_canonical<<<grid_for(ctx, len), kThreads, 0, ctx->stream>>>((const Fr*)mle->ptr, (Fr*)tmp, len);
        cudaError_t e = cudaMemcpyAsync(out, tmp, len * 32, cudaMemcpyDeviceToHost, ctx->stream);
        device_free(ctx, tmp);
        if (e != cudaSuccess) return fail(DPB_ECUDA, "download: %s", cudaGetErrorString(e));
    } else {
        return fail(DPB_EINVAL, "form %d not available for dtype %d", form, mle->dtype);
    }
    DPB_CUDA(cudaStreamSynchronize(ctx->stream));
    DPB_CUDA(cudaGetLastError());
    return DPB_OK;
}

uint64_t dpb_mle_len(const dpb_mle* mle) { return mle ? mle->len : 0; }
int dpb_mle_dtype(const dpb_mle* mle) { return mle ? mle->dtype : DPB_EINVAL; }
void* dpb_mle_device_ptr(const dpb_mle* mle) { return mle ? mle->ptr : nullptr; }

int dpb_eq_table(dpb_ctx* ctx, int family_dtype, const void* point, uint32_t m, dpb_mle** out) {
    if (!ctx || !out || (!point && m)) return fail(DPB_EINVAL, "null argument");
    if (!valid_dtype(family_dtype)) return fail(DPB_EINVAL, "unknown dtype %d", family_dtype);
    if (m > 34) return fail(DPB_EINVAL, "eq table over %u variables is too large", m);
    return is_gl(family_dtype) ? eq_table_impl<GlFam>(ctx, point, m, out)
                               : eq_table_impl<FrFam>(ctx, point, m, out);
}

int dpb_eq_tables(dpb_ctx* ctx, int family_dtype, const void* points, const uint32_t* num_vars, uint32_t n,
                  dpb_mle** out_owner, dpb_mle** out_tables) {
    if (!ctx || !num_vars || !out_owner || !out_tables) return fail(DPB_EINVAL, "null argument");
    if (n == 0) return fail(DPB_EINVAL, "no tables");
    if (!valid_dtype(family_dtype)) return fail(DPB_EINVAL, "unknown dtype %d", family_dtype);
    bool any = false;
    for (uint32_t t = 0; t < n; t++) any = any || num_vars[t] > 0;
    if (any && !points) return fail(DPB_EINVAL, "null argument");
    return is_gl(family_dtype) ? eq_tables_impl<GlFam>(ctx, points, num_vars, n, out_owner, out_tables)
                               : eq_tables_impl<FrFam>(ctx, points, num_vars, n, out_owner, out_tables);
}

int dpb_fix_high(dpb_ctx* ctx, const dpb_mle* mle, const void* point, uint32_t k, dpb_mle** out) {
    return fix_common(ctx, mle, point, k, true, out);
}

int dpb_fix_low(dpb_ctx* ctx, const dpb_mle* mle, const void* point, uint32_t k, dpb_mle** out) {
    return fix_common(ctx, mle, point, k, false, out);
}

int dpb_mle_evaluate(dpb_ctx* ctx, const dpb_mle* mle, const void* point, uint32_t n, void* out) {
    if (!ctx || !mle || !out) return fail(DPB_EINVAL, "null argument");
    if ((1ull << n) != mle->len)
        return fail(DPB_EINVAL, "point of %u coordinates for a table of %llu entries", n,
                    (unsigned long long)mle->len);
    if (n == 0) {
        // a constant: widen the single entry
        if (is_int_dtype(mle->dtype)) {
            int64_t x = 0;
            int32_t x32 = 0;
            const bool narrow = dtype_size(mle->dtype) == 4;
            DPB_CUDA(cudaMemcpyAsync(narrow ? (void*)&x32 : (void*)&x, mle->ptr, narrow ? 4 : 8, cudaMemcpyDeviceToHost,
                                     ctx->stream));
            DPB_CUDA(cudaStreamSynchronize(ctx->stream));
            if (narrow) x = x32;
            if (is_gl(mle->dtype)) {
                const uint64_t mag = x < 0 ? (uint64_t)0 - (uint64_t)x : (uint64_t)x;
                const Gl2 v = gl2_make(x < 0 ? (GL_P - mag % GL_P) % GL_P : mag % GL_P, 0);
                memcpy(out, &v, sizeof v);
            } else {
                const Fr v = fr_from_i64(x);
                memcpy(out, &v, sizeof v);
            }
            return DPB_OK;
        }
        if (mle->dtype == DPB_GL_BASE) {
            uint64_t v[2] = {0, 0};
            DPB_CUDA(cudaMemcpyAsync(v, mle->ptr, 8, cudaMemcpyDeviceToHost, ctx->stream));
            DPB_CUDA(cudaStreamSynchronize(ctx->stream));
            memcpy(out, v, 16);
            return DPB_OK;
        }
        DPB_CUDA(cudaMemcpyAsync(out, mle->ptr, dtype_size(mle->dtype), cudaMemcpyDeviceToHost, ctx->stream));
        DPB_CUDA(cudaStreamSynchronize(ctx->stream));
        return DPB_OK;
    }
    dpb_mle* res = nullptr;
    DPB_TRY(fix_common(ctx, mle, point, n, false, &res));
    int rc = dpb_mle_to_host(res, out, 1, DPB_FORM_NATIVE);
    dpb_mle_free(res);
    return rc;
}

int dpb_mle_evaluate_many(dpb_ctx* ctx, dpb_mle* const* mles, uint32_t n, const void* point, uint32_t num_vars,
                          void* out) {
    if (!ctx || !mles || !out || (!point && num_vars)) return fail(DPB_EINVAL, "null argument");
    if (n == 0) return DPB_OK;
    if (num_vars > 40) return fail(DPB_EINVAL, "a point of %u coordinates", num_vars);
    const bool gl = mles[0] && is_gl(mles[0]->dtype);
    const size_t es = gl ? 16 : 32;
    // per number of variables m: the eq table of the first m coordinates and prod_{j >= m} (1 - point[j])
    std::vector<dpb_mle*> eq(num_vars + 1, nullptr);
    auto free_eq = [&]() {
        for (auto* m : eq) dpb_mle_free(m);
    };
    std::vector<EvalManySrc> src(n);
    std::vector<uint8_t> scale((size_t)n * es);
    for (uint32_t t = 0; t < n; t++) {
        const dpb_mle* m = mles[t];
        if (!m || m->ctx != ctx || !valid_dtype(m->dtype) || is_gl(m->dtype) != gl || m->len == 0 || (m->len & (m->len - 1)) ||
            m->len > (1ull << num_vars)) {
            free_eq();
            return fail(DPB_EINVAL, "table %u is null, foreign, of another field, not a power of two or longer than 2^%u", t, num_vars);
        }
        uint32_t mv = 0;
        while ((1ull << mv) < m->len) mv++;
        if (!eq[mv]) {
            const int rc = dpb_eq_table(ctx, gl ? DPB_GL_EXT : DPB_FR, point, mv, &eq[mv]);
            if (rc != DPB_OK) {
                free_eq();
                return rc;
            }
        }
        src[t].ptr = m->ptr;
        src[t].eq = eq[mv]->ptr;
        src[t].len = m->len;
        src[t].dtype = m->dtype;
        src[t].pad = 0;
        if (gl) {
            Gl2 sc = GlFam::one();
            for (uint32_t j = mv; j < num_vars; j++) sc = GlFam::mul(sc, GlFam::sub(GlFam::one(), ((const Gl2*)point)[j]));
            memcpy(scale.data() + (size_t)t * es, &sc, es);
        } else {
            Fr sc = FrFam::one();
            for (uint32_t j = mv; j < num_vars; j++) sc = FrFam::mul(sc, FrFam::sub(FrFam::one(), ((const Fr*)point)[j]));
            memcpy(scale.data() + (size_t)t * es, &sc, es);
        }
    }
    uint64_t longest = 0;
    for (const auto& t : src) longest = std::max(longest, t.len);
    // enough blocks to fill the GPU a few times over, at most one slice per 256 entries of the longest table
    uint32_t slices = (uint32_t)std::max<uint64_t>(1, std::min<uint64_t>((longest + kThreads - 1) / kThreads,
                                                                         ((uint64_t)ctx->sm_count * 8 + n - 1) / n));
    void *d_src = nullptr, *d_scale = nullptr, *d_partial = nullptr, *d_out = nullptr;
    int rc = device_alloc(ctx, (size_t)n * sizeof(EvalManySrc), &d_src);
    if (rc == DPB_OK) rc = device_alloc(ctx, (size_t)n * es, &d_scale);
    if (rc == DPB_OK) rc = device_alloc(ctx, (size_t)n * slices * es, &d_partial);
    if (rc == DPB_OK) rc = device_alloc(ctx, (size_t)n * es, &d_out);
    if (rc == DPB_OK) rc = upload_small(ctx, d_src, src.data(), (size_t)n * sizeof(EvalManySrc));
    if (rc == DPB_OK) rc = upload_small(ctx, d_scale, scale.data(), (size_t)n * es);
    if (rc == DPB_OK) {
        // the grid's second dimension holds at most 65535 blocks
        for (uint32_t first = 0; first < n; first += 65535) {
            const uint32_t cnt = std::min<uint32_t>(65535, n - first);
            const dim3 grid(slices, cnt);
            if (gl)
                evaluate_many_kernel<GlFam><<<grid, kThreads, 0, ctx->stream>>>((const EvalManySrc*)d_src + first, slices,
                                                                                 (Gl2*)d_partial + (size_t)first * slices);
            else
                evaluate_many_kernel<FrFam><<<grid, kThreads, 0, ctx->stream>>>((const EvalManySrc*)d_src + first, slices,
                                                                                 (Fr*)d_partial + (size_t)first * slices);
        }
        const uint32_t blocks = (n + kThreads - 1) / kThreads;
        if (gl)
            evaluate_many_finish<GlFam><<<blocks, kThreads, 0, ctx->stream>>>((const Gl2*)d_partial, slices, (const Gl2*)d_scale, n,
                                                                                (Gl2*)d_out);
        else
            evaluate_many_finish<FrFam><<<blocks, kThreads, 0, ctx->stream>>>((const Fr*)d_partial, slices, (const Fr*)d_scale, n,
                                                                                (Fr*)d_out);
        cudaError_t e = cudaGetLastError();
        if (e == cudaSuccess) e = cudaMemcpyAsync(out, d_out, (size_t)n * es, cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) rc = fail(DPB_ECUDA, "evaluate many: %s", cudaGetErrorString(e));
    }
    device_free(ctx, d_src);
    device_free(ctx, d_scale);
    device_free(ctx, d_partial);
    device_free(ctx, d_out);
    free_eq();
    return rc;
}

}  // extern "C"
