// C ABI: logup-GKR fraction tree of one instance, every level resident on the
// device (the batched prover walks the levels top-down and needs all of them,
// zkml/src/lookup/logup_gkr/prover.rs:144-147).
#include "common.cuh"
#include "logup_kernels.cuh"

using namespace dpb;

struct dpb_logup {
    dpb_ctx* ctx = nullptr;
    bool gl = false;
    uint32_t m = 0;        // columns have 2^m entries
    void* slab = nullptr;  // all levels, numerators then denominators per level
    std::vector<void*> num, den;  // level l (1-based) at index l-1, 2^(m-l) entries each
};

namespace dpb {

constexpr uint64_t kSmallLevel = 1024;  // levels of at most this many fractions are finished by one block

template <class F>
static int build_tree(dpb_logup* lu, int kind, dpb_mle* const* columns, uint32_t n_cols,
                      const dpb_mle* mult, const void* constant_chal, const void* sep_chal) {
    typedef typename F::E E;
    dpb_ctx* ctx = lu->ctx;
    const uint32_t m = lu->m;
    const uint32_t levels = m - 1;
    // level l has 2 * 2^(m-l) entries; total < 2 * 2^m
    size_t total = 0;
    for (uint32_t l = 1; l <= levels; l++) total += 2ull << (m - l);
    DPB_TRY(device_alloc(ctx, total * sizeof(E), &lu->slab));
    {
        E* p = (E*)lu->slab;
        for (uint32_t l = 1; l <= levels; l++) {
            lu->num.push_back(p);
            p += 1ull << (m - l);
            lu->den.push_back(p);
            p += 1ull << (m - l);
        }
    }
    LogupCols<F> c;
    memset(&c, 0, sizeof c);
    c.n_cols = n_cols;
    memcpy(&c.constant, constant_chal, sizeof(E));
    E sep;
    memcpy(&sep, sep_chal, sizeof(E));
    E pw = F::one();
    for (uint32_t j = 0; j < n_cols; j++) {
        c.col[j] = columns[j]->ptr;
        c.dtype[j] = columns[j]->dtype;
        c.sep_pow[j] = pw;
        pw = F::mul(pw, sep);
    }
    uint64_t half = 1ull << (m - 1);
    if (kind == DPB_LOGUP_LOOKUP)
        logup_initial_lookup<F><<<grid_for(ctx, half), kThreads, 0, ctx->stream>>>(c, half, (E*)lu->num[0], (E*)lu->den[0]);
    else
        logup_initial_table<F><<<grid_for(ctx, half), kThreads, 0, ctx->stream>>>(c, mult->ptr, mult->dtype, half,
                                                                                   (E*)lu->num[0], (E*)lu->den[0]);
    for (uint32_t l = 2; l <= levels; l++) {
        half = 1ull << (m - l);
        if (half <= kSmallLevel) {
            // levels l..levels in one launch (they lie one behind the other in the slab)
            logup_small_levels<F><<<1, kThreads, 0, ctx->stream>>>((const E*)lu->num[l - 2], (const E*)lu->den[l - 2], half,
                                                                   (E*)lu->num[l - 1]);
            break;
        }
        logup_next_level<F><<<grid_for(ctx, half), kThreads, 0, ctx->stream>>>(
            (const E*)lu->num[l - 2], (const E*)lu->den[l - 2], half, (E*)lu->num[l - 1], (E*)lu->den[l - 1]);
    }
    DPB_CUDA(cudaGetLastError());
    return DPB_OK;
}

}  // namespace dpb

extern "C" {

int dpb_logup_build(dpb_ctx* ctx, int kind, dpb_mle* const* columns, uint32_t n_cols,
                    const dpb_mle* mult, const void* constant_chal, const void* sep_chal,
                    dpb_logup** out) {
    if (!ctx || !columns || !constant_chal || !sep_chal || !out) return fail(DPB_EINVAL, "null argument");
    if (kind != DPB_LOGUP_LOOKUP && kind != DPB_LOGUP_TABLE) return fail(DPB_EINVAL, "unknown kind %d", kind);
    if (n_cols < 1 || n_cols > (uint32_t)kMaxLogupCols)
        return fail(DPB_EINVAL, "No column evals were provided or too many (%u, max %d)", n_cols, kMaxLogupCols);
    if ((kind == DPB_LOGUP_TABLE) != (mult != nullptr))
        return fail(DPB_EINVAL, "multiplicities are required for tables and only for tables");
    for (uint32_t j = 0; j < n_cols; j++)
        if (!columns[j] || columns[j]->ctx != ctx) return fail(DPB_EINVAL, "column %u is null or foreign", j);
    const uint64_t len = columns[0]->len;
    const bool gl = is_gl(columns[0]->dtype);
    for (uint32_t j = 1; j < n_cols; j++) {
        if (columns[j]->len != len) return fail(DPB_EINVAL, "All sets of evaluations should be the same length");
        if (is_gl(columns[j]->dtype) != gl) return fail(DPB_EINVAL, "columns mix fields");
    }
    if (mult && (mult->len != len || is_gl(mult->dtype) != gl))
        return fail(DPB_EINVAL, "Multiplicities length was not equal to column evaluations length, multiplicities: %llu, columns: %llu",
                    (unsigned long long)mult->len, (unsigned long long)len);
    if (len < 4) return fail(DPB_EINVAL, "columns need at least 4 entries, got %llu", (unsigned long long)len);
    dpb_logup* lu = new (std::nothrow) dpb_logup();
    if (!lu) return fail(DPB_ENOMEM, "host allocation failed");
    lu->ctx = ctx;
    lu->gl = gl;
    lu->m = log2u(len);
    int rc = gl ? build_tree<GlFam>(lu, kind, columns, n_cols, mult, constant_chal, sep_chal)
                : build_tree<FrFam>(lu, kind, columns, n_cols, mult, constant_chal, sep_chal);
    if (rc != DPB_OK) {
        dpb_logup_free(lu);
        return rc;
    }
    *out = lu;
    return DPB_OK;
}

uint32_t dpb_logup_num_levels(const dpb_logup* lu) { return lu ? lu->m - 1 : 0; }

int dpb_logup_level(const dpb_logup* lu, uint32_t level, dpb_mle* out_views[4]) {
    if (!lu || !out_views) return fail(DPB_EINVAL, "null argument");
    if (level < 1 || level > lu->m - 1) return fail(DPB_EINVAL, "level %u outside 1..%u", level, lu->m - 1);
    const uint64_t half = 1ull << (lu->m - level - 1);
    const size_t es = lu->gl ? 16 : 32;
    const int dt = lu->gl ? DPB_GL_EXT : DPB_FR;
    char* base[2] = {(char*)lu->num[level - 1], (char*)lu->den[level - 1]};
    for (int a = 0; a < 2; a++) {
        for (int h = 0; h < 2; h++) {
            dpb_mle* v = new (std::nothrow) dpb_mle();
            if (!v) return fail(DPB_ENOMEM, "host allocation failed");
            v->ctx = lu->ctx;
            v->dtype = dt;
            v->len = half;
            v->ptr = base[a] + (size_t)h * half * es;
            v->owns = false;
            out_views[a * 2 + h] = v;
        }
    }
    return DPB_OK;
}

int dpb_logup_outputs(const dpb_logup* lu, void* out4) {
    if (!lu || !out4) return fail(DPB_EINVAL, "null argument");
    const size_t es = lu->gl ? 16 : 32;
    const uint32_t top = lu->m - 1;
    dpb_ctx* ctx = lu->ctx;
    DPB_CUDA(cudaMemcpyAsync(out4, lu->num[top - 1], 2 * es, cudaMemcpyDeviceToHost, ctx->stream));
    DPB_CUDA(cudaMemcpyAsync((char*)out4 + 2 * es, lu->den[top - 1], 2 * es, cudaMemcpyDeviceToHost, ctx->stream));
    DPB_CUDA(cudaStreamSynchronize(ctx->stream));
    return DPB_OK;
}

int dpb_logup_outputs_batch(const dpb_logup* const* lus, uint32_t n, void* out) {
    if (!lus || !out || n == 0) return fail(DPB_EINVAL, "null argument");
    for (uint32_t i = 0; i < n; i++)
        if (!lus[i] || lus[i]->ctx != lus[0]->ctx || lus[i]->gl != lus[0]->gl)
            return fail(DPB_EINVAL, "tree %u is null, of another context or of another field", i);
    dpb_ctx* ctx = lus[0]->ctx;
    const size_t es = lus[0]->gl ? 16 : 32;
    // gathered on the device, then one copy to the host and one wait, instead of one of each per tree
    void* gathered = nullptr;
    DPB_TRY(device_alloc(ctx, (size_t)n * 4 * es, &gathered));
    cudaError_t e = cudaSuccess;
    for (uint32_t i = 0; i < n && e == cudaSuccess; i++) {
        const uint32_t top = lus[i]->m - 1;
        char* dst = (char*)gathered + (size_t)i * 4 * es;
        e = cudaMemcpyAsync(dst, lus[i]->num[top - 1], 2 * es, cudaMemcpyDeviceToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(dst + 2 * es, lus[i]->den[top - 1], 2 * es, cudaMemcpyDeviceToDevice, ctx->stream);
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(out, gathered, (size_t)n * 4 * es, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    device_free(ctx, gathered);
    if (e != cudaSuccess) return fail(DPB_ECUDA, "logup outputs: %s", cudaGetErrorString(e));
    return DPB_OK;
}

void dpb_logup_free(dpb_logup* lu) {
    if (!lu) return;
    device_free(lu->ctx, lu->slab);
    delete lu;
}

}  // extern "C"
