// C ABI: lookup witness generation (LookupOp::generate_witness, zkml/src/lookup/operation/mod.rs:103-160;
// ChunkingInfo, zkml/src/lookup/operation/decomposer.rs:182-383; table multiplicities,
// zkml/src/lookup/context.rs:313-371).
#include "common.cuh"
#include "lookup_kernels.cuh"

struct dpb_lookup_counts {
    dpb_ctx* ctx = nullptr;
    uint32_t bits = 0;
    unsigned long long* dev = nullptr;
};

namespace dpb {

constexpr uint32_t kCheckTableBits = 16;  // SHIFT_CHECK_TABLE_BIT_SIZE, ZERO_CHECK_TABLE_BIT_SIZE (table/mod.rs:20-23)

static int64_t table_min_input(uint32_t bits, int sign) {
    // Table::min_input_value (zkml/src/lookup/table/mod.rs:135-142)
    if (sign == DPB_SIGN_POSITIVE) return 0;
    if (sign == DPB_SIGN_MIXED) return -(1ll << (bits - 1));
    return -(1ll << bits) + 1;
}

template <class F>
static int witness_impl(dpb_ctx* ctx, const dpb_chunking_info& ci, int64_t fpm, int64_t padding_value, const int64_t* tensor,
                        int tensor_on_device, const uint64_t* shape, uint32_t rank, const int64_t* table_out,
                        int outputs_on_device, uint32_t num_value_columns, dpb_lookup_counts* const counts[4],
                        dpb_mle** out_owner, dpb_mle** out_in, uint32_t in_cap, uint32_t* n_in, dpb_mle** out_out,
                        uint32_t out_cap, uint32_t* n_out) {
    typedef typename SmallToField<F>::T T;
    const uint64_t rows = rank == 1 ? 1 : shape[rank - 2], cols = shape[rank - 1];
    uint64_t n_slices = 1;
    for (uint32_t a = 0; a + 2 < rank; a++) n_slices *= shape[a];
    const uint32_t prow_bits = log2u(rows), pcol_bits = log2u(cols);
    const uint32_t p_bits = prow_bits + pcol_bits;
    const uint64_t P = 1ull << p_bits;
    const uint32_t value_in = num_value_columns != 1 ? 1 : 0;
    const uint32_t n_in_per = ci.n_shifted_chunks + value_in * ci.n_value_chunks + ci.n_zeroing_chunks;
    const uint32_t n_out_per = ci.n_value_chunks + ci.n_zeroing_chunks;
    const uint64_t total_in = n_slices * n_in_per, total_out = n_slices * n_out_per;
    *n_in = (uint32_t)total_in;
    *n_out = (uint32_t)total_out;
    if (total_in > in_cap || total_out > out_cap)
        return fail(DPB_EINVAL, "room for %u + %u columns, %llu + %llu needed", in_cap, out_cap, (unsigned long long)total_in,
                    (unsigned long long)total_out);
    if ((total_in + total_out) * P > (1ull << 36)) return fail(DPB_EINVAL, "witness of more than 2^36 entries");

    std::vector<void*> to_free;
    auto cleanup = [&](int code) {
        for (void* p : to_free) device_free(ctx, p);
        return code;
    };
    const uint64_t numel = n_slices * rows * cols;
    const int64_t* t_dev = tensor;
    if (!tensor_on_device) {
        void* p = nullptr;
        int rc = device_alloc(ctx, numel * 8, &p);
        if (rc != DPB_OK) return rc;
        to_free.push_back(p);
        cudaError_t e = cudaMemcpyAsync(p, tensor, numel * 8, cudaMemcpyHostToDevice, ctx->stream);
        if (e != cudaSuccess) return cleanup(fail(DPB_ECUDA, "tensor upload: %s", cudaGetErrorString(e)));
        t_dev = (const int64_t*)p;
    }
    const int64_t* out_dev = table_out;
    if (table_out && !outputs_on_device) {
        void* p = nullptr;
        const size_t bytes = (size_t)8 << ci.value_chunk_bits;
        int rc = device_alloc(ctx, bytes, &p);
        if (rc != DPB_OK) return cleanup(rc);
        to_free.push_back(p);
        cudaError_t e = cudaMemcpyAsync(p, table_out, bytes, cudaMemcpyHostToDevice, ctx->stream);
        if (e != cudaSuccess) return cleanup(fail(DPB_ECUDA, "table upload: %s", cudaGetErrorString(e)));
        out_dev = (const int64_t*)p;
    }
    void* d_err = nullptr;
    int rc = device_alloc(ctx, sizeof(int), &d_err);
    if (rc != DPB_OK) return cleanup(rc);
    to_free.push_back(d_err);
    cudaMemsetAsync(d_err, 0, sizeof(int), ctx->stream);

    dpb_mle* owner = new (std::nothrow) dpb_mle();
    if (!owner) return cleanup(fail(DPB_ENOMEM, "host allocation failed"));
    owner->ctx = ctx;
    owner->dtype = SmallToField<F>::kDtype;
    owner->len = (total_in + total_out) * P;
    owner->owns = true;
    rc = device_alloc(ctx, owner->len * sizeof(T), &owner->ptr);
    if (rc != DPB_OK) {
        delete owner;
        return cleanup(rc);
    }
    LookupWitnessArgs a;
    memset(&a, 0, sizeof a);
    a.tensor = t_dev;
    a.rows = rows;
    a.cols = cols;
    a.pcol_bits = pcol_bits;
    a.p_bits = p_bits;
    a.n_slices = n_slices;
    a.fpm = fpm;
    a.rc = 1ll << (ci.right_shift - 1);
    a.pad_rescaled = padding_value * fpm + a.rc;
    a.ci = ci;
    a.table_out = out_dev;
    a.table_min = table_min_input(ci.value_chunk_bits, ci.table_sign);
    for (int h = 0; h < 4; h++) a.counts[h] = counts[h] ? counts[h]->dev : nullptr;
    a.n_in_per = n_in_per;
    a.n_out_per = n_out_per;
    a.value_in_column = value_in;
    a.error = (int*)d_err;
    T* in_cols = (T*)owner->ptr;
    T* out_cols = in_cols + total_in * P;
    a.direct_rows = counts[1] && ci.value_chunk_bits <= kLookupDirectBits ? 1u << ci.value_chunk_bits : 0;
    const size_t smem = lookup_witness_smem<F>(a.direct_rows);
    cudaError_t e = cudaFuncSetAttribute(lookup_witness_kernel<F>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    // few, large blocks: each adds its block-local counters to device memory once
    const uint64_t work = n_slices << p_bits;
    uint64_t blocks = (work + 511) / 512;
    const uint64_t cap = (uint64_t)ctx->sm_count * 2;
    if (blocks > cap) blocks = cap;
    if (e == cudaSuccess) {
        lookup_witness_kernel<F><<<(uint32_t)blocks, 512, smem, ctx->stream>>>(a, in_cols, out_cols);
        e = cudaGetLastError();
    }
    int err_host = 0;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&err_host, d_err, sizeof(int), cudaMemcpyDeviceToHost, ctx->stream);
    // the error word is needed before returning, and a host tensor is only read during the call
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cleanup(DPB_OK);
    if (e != cudaSuccess) {
        dpb_mle_free(owner);
        return fail(DPB_ECUDA, "lookup witness: %s", cudaGetErrorString(e));
    }
    if (err_host) {
        dpb_mle_free(owner);
        return fail(DPB_EINVAL, "Input value out of range for SignedZeroCheckTable, min: -32768, max: 32767");
    }
    for (uint64_t c = 0; c < total_in + total_out; c++) {
        dpb_mle* v = new (std::nothrow) dpb_mle();
        if (!v) return fail(DPB_ENOMEM, "host allocation failed");
        v->ctx = ctx;
        v->dtype = owner->dtype;
        v->len = P;
        v->ptr = (char*)owner->ptr + c * P * sizeof(T);
        v->owns = false;
        (c < total_in ? out_in[c] : out_out[c - total_in]) = v;
    }
    *out_owner = owner;
    return DPB_OK;
}

}  // namespace dpb

using namespace dpb;

extern "C" int dpb_chunking_info_new(uint32_t right_shift, uint32_t table_bits, int table_sign, uint32_t max_bit_size,
                                     uint32_t n_value_chunks, dpb_chunking_info* out) {
    if (!out) return fail(DPB_EINVAL, "null argument");
    if (right_shift == 0) return fail(DPB_EINVAL, "Right shift must be greater than zero to decompose value, got 0");
    if (table_sign < DPB_SIGN_POSITIVE || table_sign > DPB_SIGN_MIXED) return fail(DPB_EINVAL, "unknown table sign %d", table_sign);
    if (table_bits < 1 || table_bits > 30) return fail(DPB_EINVAL, "table bit size %u outside 1..30", table_bits);
    if (n_value_chunks < 1 || n_value_chunks > (uint32_t)kLookupMaxChunks)
        return fail(DPB_EINVAL, "%u value chunks (1..%d)", n_value_chunks, kLookupMaxChunks);
    if (max_bit_size < 1 || max_bit_size > 62) return fail(DPB_EINVAL, "max bit size %u outside 1..62", max_bit_size);
    const uint32_t value_bits = table_bits * n_value_chunks;
    if (right_shift + value_bits > 62) return fail(DPB_EINVAL, "shift %u + value bits %u exceed 62", right_shift, value_bits);
    dpb_chunking_info ci;
    memset(&ci, 0, sizeof ci);
    ci.right_shift = right_shift;
    ci.value_chunk_bits = table_bits;
    ci.n_value_chunks = n_value_chunks;
    ci.table_sign = table_sign;
    ci.n_shifted_chunks = (right_shift + kCheckTableBits - 1) / kCheckTableBits;
    const uint32_t above = max_bit_size > right_shift + value_bits ? max_bit_size - (right_shift + value_bits) : 0;
    ci.n_zeroing_chunks = (above + kCheckTableBits - 1) / kCheckTableBits;
    if (ci.n_shifted_chunks > (uint32_t)kLookupMaxChunks || ci.n_zeroing_chunks > (uint32_t)kLookupMaxChunks)
        return fail(DPB_EINVAL, "more than %d chunks of a kind", kLookupMaxChunks);
    ci.shifted_chunk_multiplier = right_shift % kCheckTableBits ? 1ll << (kCheckTableBits - right_shift % kCheckTableBits) : 1;
    if (table_sign == DPB_SIGN_MIXED) {
        ci.value_chunk_offset = 1ll << (table_bits - 1);
        const int64_t combined = 1ll << (value_bits - 1);
        const int64_t first = std::max(1ll << (max_bit_size - 1), (long long)(combined << right_shift));
        ci.offset = first + (ci.n_zeroing_chunks > 0 ? (combined << right_shift) : 0);
        if (ci.n_zeroing_chunks > 0)
            ci.top_zeroing_chunk_offset = ci.offset >> (right_shift + value_bits + (ci.n_zeroing_chunks - 1) * kCheckTableBits);
    }
    *out = ci;
    return DPB_OK;
}

extern "C" int dpb_lookup_counts_new(dpb_ctx* ctx, uint32_t table_bits, dpb_lookup_counts** out) {
    if (!ctx || !out) return fail(DPB_EINVAL, "null argument");
    if (table_bits < 1 || table_bits > 30) return fail(DPB_EINVAL, "table bit size %u outside 1..30", table_bits);
    dpb_lookup_counts* c = new (std::nothrow) dpb_lookup_counts();
    if (!c) return fail(DPB_ENOMEM, "host allocation failed");
    c->ctx = ctx;
    c->bits = table_bits;
    void* p = nullptr;
    int rc = device_alloc(ctx, (size_t)8 << table_bits, &p);
    if (rc != DPB_OK) {
        delete c;
        return rc;
    }
    c->dev = (unsigned long long*)p;
    cudaError_t e = cudaMemsetAsync(p, 0, (size_t)8 << table_bits, ctx->stream);
    if (e != cudaSuccess) {
        device_free(ctx, p);
        delete c;
        return fail(DPB_ECUDA, "clearing counters: %s", cudaGetErrorString(e));
    }
    *out = c;
    return DPB_OK;
}

extern "C" int dpb_lookup_counts_to_host(const dpb_lookup_counts* c, uint64_t* out, uint64_t len) {
    if (!c || !out) return fail(DPB_EINVAL, "null argument");
    if (len != (1ull << c->bits)) return fail(DPB_EINVAL, "length %llu, table has %llu rows", (unsigned long long)len, 1ull << c->bits);
    cudaError_t e = cudaMemcpyAsync(out, c->dev, len * 8, cudaMemcpyDeviceToHost, c->ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(c->ctx->stream);
    if (e != cudaSuccess) return fail(DPB_ECUDA, "reading counters: %s", cudaGetErrorString(e));
    return DPB_OK;
}

extern "C" void dpb_lookup_counts_free(dpb_lookup_counts* c) {
    if (!c) return;
    if (c->dev) device_free(c->ctx, c->dev);
    delete c;
}

namespace dpb {

// counters[rows[i]] += 1 for i < n; equal rows of a warp are merged into one atomic
__global__ void __launch_bounds__(kThreads)
    lookup_count_rows_kernel(const int64_t* rows, uint64_t n, uint64_t n_rows, unsigned long long* counters,
                             unsigned int* bad) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    // whole warps iterate together so that the match below sees every lane of the warp
    const uint64_t n_up = (n + 31) & ~(uint64_t)31;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_up; i += stride) {
        const bool live = i < n;
        const int64_t r = live ? rows[i] : -1;
        const bool ok = live && r >= 0 && (uint64_t)r < n_rows;
        if (live && !ok) atomicAdd(bad, 1u);
        const unsigned long long key = ok ? (unsigned long long)r : ~0ull;
        const unsigned peers = __match_any_sync(0xffffffffu, key);
        if (ok && (unsigned)(__ffs(peers) - 1) == (threadIdx.x & 31u))
            atomicAdd(&counters[r], (unsigned long long)__popc(peers));
    }
}

}  // namespace dpb

extern "C" int dpb_lookup_counts_add_rows(dpb_ctx* ctx, dpb_lookup_counts* c, const int64_t* rows, int rows_on_device,
                                          uint64_t n) {
    if (!ctx || !c || (!rows && n)) return fail(DPB_EINVAL, "null argument");
    if (c->ctx != ctx) return fail(DPB_EINVAL, "the counters belong to another context");
    if (n == 0) return DPB_OK;
    const int64_t* dev = rows;
    void* tmp = nullptr;
    if (!rows_on_device) {
        DPB_TRY(device_alloc(ctx, n * sizeof(int64_t), &tmp));
        cudaError_t e = cudaMemcpyAsync(tmp, rows, n * sizeof(int64_t), cudaMemcpyHostToDevice, ctx->stream);
        if (e != cudaSuccess) {
            device_free(ctx, tmp);
            return fail(DPB_ECUDA, "copying rows: %s", cudaGetErrorString(e));
        }
        dev = (const int64_t*)tmp;
    }
    unsigned int* bad = nullptr;
    int rc = device_alloc(ctx, sizeof(unsigned int), (void**)&bad);
    if (rc != DPB_OK) {
        device_free(ctx, tmp);
        return rc;
    }
    unsigned int h_bad = 0;
    cudaError_t e = cudaMemsetAsync(bad, 0, sizeof(unsigned int), ctx->stream);
    if (e == cudaSuccess) {
        lookup_count_rows_kernel<<<grid_for(ctx, n), kThreads, 0, ctx->stream>>>(dev, n, 1ull << c->bits, c->dev, bad);
        e = cudaGetLastError();
    }
    if (e == cudaSuccess) e = cudaMemcpyAsync(&h_bad, bad, sizeof(unsigned int), cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    device_free(ctx, bad);
    device_free(ctx, tmp);
    if (e != cudaSuccess) return fail(DPB_ECUDA, "counting rows: %s", cudaGetErrorString(e));
    if (h_bad) return fail(DPB_EINVAL, "%u rows lie outside the table's 2^%u rows (they were not counted)", h_bad, c->bits);
    return DPB_OK;
}

extern "C" int dpb_lookup_multiplicities(dpb_ctx* ctx, const dpb_lookup_counts* c, int family_dtype, dpb_mle** out) {
    if (!ctx || !c || !out) return fail(DPB_EINVAL, "null argument");
    if (!valid_dtype(family_dtype)) return fail(DPB_EINVAL, "unknown dtype %d", family_dtype);
    const uint64_t n = 1ull << c->bits;
    dpb_mle* m = nullptr;
    int rc = new_mle(ctx, is_gl(family_dtype) ? DPB_GL_BASE : DPB_FR, n, &m);
    if (rc != DPB_OK) return rc;
    if (is_gl(family_dtype))
        lookup_multiplicities_kernel<GlFam><<<grid_for(ctx, n), kThreads, 0, ctx->stream>>>(c->dev, n, (uint64_t*)m->ptr);
    else
        lookup_multiplicities_kernel<FrFam><<<grid_for(ctx, n), kThreads, 0, ctx->stream>>>(c->dev, n, (Fr*)m->ptr);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        dpb_mle_free(m);
        return fail(DPB_ECUDA, "multiplicities: %s", cudaGetErrorString(e));
    }
    *out = m;
    return DPB_OK;
}

extern "C" int dpb_lookup_witness(dpb_ctx* ctx, int family_dtype, const dpb_chunking_info* info, int64_t fixed_point_multiplier,
                                  int64_t padding_value, const int64_t* tensor, int tensor_on_device, const uint64_t* shape,
                                  uint32_t rank, const int64_t* value_table_outputs, int outputs_on_device,
                                  uint32_t num_value_columns, dpb_lookup_counts* shift_counts,
                                  dpb_lookup_counts* value_counts, dpb_lookup_counts* zero_counts,
                                  dpb_lookup_counts* signed_zero_counts, dpb_mle** out_owner, dpb_mle** out_input_columns,
                                  uint32_t in_cap, uint32_t* n_in, dpb_mle** out_output_columns, uint32_t out_cap,
                                  uint32_t* n_out) {
    if (!ctx || !info || !tensor || !shape || !out_owner || !out_input_columns || !n_in || !out_output_columns || !n_out)
        return fail(DPB_EINVAL, "null argument");
    if (!valid_dtype(family_dtype)) return fail(DPB_EINVAL, "unknown dtype %d", family_dtype);
    if (rank < 1 || rank > 8) return fail(DPB_EINVAL, "Input tensor must have rank at least 1 (and at most 8), got %u", rank);
    for (uint32_t a = 0; a < rank; a++)
        if (shape[a] == 0) return fail(DPB_EINVAL, "axis %u is empty", a);
    const dpb_chunking_info& ci = *info;
    if (ci.right_shift == 0 || ci.right_shift > 62 || ci.value_chunk_bits < 1 || ci.value_chunk_bits > 30 || ci.n_value_chunks < 1 ||
        ci.n_value_chunks > (uint32_t)kLookupMaxChunks || ci.n_shifted_chunks > (uint32_t)kLookupMaxChunks ||
        ci.n_zeroing_chunks > (uint32_t)kLookupMaxChunks || ci.table_sign < DPB_SIGN_POSITIVE || ci.table_sign > DPB_SIGN_MIXED)
        return fail(DPB_EINVAL, "chunking info out of range");
    if (num_value_columns != 1 && num_value_columns != 2) return fail(DPB_EINVAL, "tables have one or two columns, got %u", num_value_columns);
    if (num_value_columns == 2 && !value_table_outputs) return fail(DPB_EINVAL, "a two-column table needs its output column");
    // Multiple value chunks are only supported for requantisation tables (decomposer.rs:199-204), which have one column
    if (ci.n_value_chunks > 1 && num_value_columns != 1)
        return fail(DPB_EINVAL, "Multiple value chunks are currently only supported for Requantisation tables");
    dpb_lookup_counts* counts[4] = {shift_counts, value_counts, zero_counts, signed_zero_counts};
    const uint32_t want_bits[4] = {kCheckTableBits, ci.value_chunk_bits, kCheckTableBits, kCheckTableBits};
    for (int h = 0; h < 4; h++)
        if (counts[h] && (counts[h]->bits != want_bits[h] || counts[h]->ctx != ctx))
            return fail(DPB_EINVAL, "counter %d has 2^%u rows, its table 2^%u (or another context)", h, counts[h]->bits, want_bits[h]);
    if (is_int_dtype(family_dtype)) {  // integer columns: the chunks as they are, eight bytes each
        return is_gl(family_dtype)
                   ? witness_impl<IntColumns<GlFam>>(ctx, ci, fixed_point_multiplier, padding_value, tensor, tensor_on_device,
                                                     shape, rank, value_table_outputs, outputs_on_device, num_value_columns,
                                                     counts, out_owner, out_input_columns, in_cap, n_in, out_output_columns,
                                                     out_cap, n_out)
                   : witness_impl<IntColumns<FrFam>>(ctx, ci, fixed_point_multiplier, padding_value, tensor, tensor_on_device,
                                                     shape, rank, value_table_outputs, outputs_on_device, num_value_columns,
                                                     counts, out_owner, out_input_columns, in_cap, n_in, out_output_columns,
                                                     out_cap, n_out);
    }
    return is_gl(family_dtype)
               ? witness_impl<GlFam>(ctx, ci, fixed_point_multiplier, padding_value, tensor, tensor_on_device, shape, rank,
                                     value_table_outputs, outputs_on_device, num_value_columns, counts, out_owner,
                                     out_input_columns, in_cap, n_in, out_output_columns, out_cap, n_out)
               : witness_impl<FrFam>(ctx, ci, fixed_point_multiplier, padding_value, tensor, tensor_on_device, shape, rank,
                                     value_table_outputs, outputs_on_device, num_value_columns, counts, out_owner,
                                     out_input_columns, in_cap, n_in, out_output_columns, out_cap, n_out);
}
