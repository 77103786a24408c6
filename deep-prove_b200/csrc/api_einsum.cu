// C ABI: einsum axis fixing (AxesMapping::fix_axes ->
// FixedAxesMapping::mles_from_tensor, zkml/src/layers/einsum/axis.rs:478-500,
// 1142-1234).
#include "common.cuh"
#include "einsum_kernels.cuh"

namespace dpb {

template <class F>
static int einsum_impl(dpb_ctx* ctx, const int64_t* tensor, int tensor_on_device, const uint64_t* shape,
                       const uint8_t* kind, const void* const* points, const uint32_t* point_len, uint32_t rank,
                       dpb_mle** out_owner, dpb_mle** out_mles, uint32_t out_cap, uint32_t* n_out) {
    typedef typename F::E E;
    // strides of the unpadded row-major tensor
    uint64_t stride[kMaxEinsumRank];
    uint64_t numel = 1;
    for (int a = (int)rank - 1; a >= 0; a--) {
        stride[a] = numel;
        numel *= shape[a];
    }
    EinsumKept kept;
    memset(&kept, 0, sizeof kept);
    uint64_t outer_dims[kMaxEinsumRank], outer_stride[kMaxEinsumRank];
    uint32_t n_outer = 0;
    uint64_t S = 1, C = 1, O = 1;
    for (uint32_t a = 0; a < rank; a++) {
        if (kind[a] == DPB_AXIS_OUTER) {
            if (!points[a] && shape[a] > 1) return fail(DPB_EINVAL, "outer axis %u has no point", a);
            if ((1ull << point_len[a]) < shape[a])
                return fail(DPB_EINVAL, "axis %u of size %llu needs more than %u variables", a, (unsigned long long)shape[a], point_len[a]);
            outer_dims[n_outer] = shape[a];
            outer_stride[n_outer] = stride[a];
            n_outer++;
            O *= shape[a];
        } else if (kind[a] == DPB_AXIS_STACKED || kind[a] == DPB_AXIS_CONTRACTED) {
            kept.dim[kept.n_kept] = shape[a];
            kept.stride[kept.n_kept] = stride[a];
            kept.n_kept++;
            (kind[a] == DPB_AXIS_STACKED ? S : C) *= shape[a];
        } else {
            return fail(DPB_EINVAL, "axis %u has unknown kind %u", a, kind[a]);
        }
    }
    if (O > (1ull << 24)) return fail(DPB_EINVAL, "outer axes span %llu entries (max 2^24)", (unsigned long long)O);
    if (out_cap < S) {
        *n_out = (uint32_t)S;
        return fail(DPB_EINVAL, "room for %u tables, %llu needed", out_cap, (unsigned long long)S);
    }
    const uint32_t c_vars = log2u(C);
    const uint64_t c_pad = 1ull << c_vars;

    // device copies: tensor, per-axis eq weights, flat weights, outer offsets
    const int64_t* t_dev = tensor;
    void* t_owned = nullptr;
    std::vector<void*> to_free;
    auto cleanup = [&](int code) {
        for (void* p : to_free) device_free(ctx, p);
        return code;
    };
    if (!tensor_on_device) {
        int rc = device_alloc(ctx, numel * 8, &t_owned);
        if (rc != DPB_OK) return rc;
        to_free.push_back(t_owned);
        cudaError_t e = cudaMemcpyAsync(t_owned, tensor, numel * 8, cudaMemcpyHostToDevice, ctx->stream);
        if (e != cudaSuccess) return cleanup(fail(DPB_ECUDA, "tensor upload: %s", cudaGetErrorString(e)));
        t_dev = (const int64_t*)t_owned;
    }
    std::vector<dpb_mle*> eqs;
    auto free_eqs = [&]() {
        for (auto* m : eqs) dpb_mle_free(m);
    };
    std::vector<const E*> w_ptrs;
    for (uint32_t a = 0; a < rank; a++) {
        if (kind[a] != DPB_AXIS_OUTER) continue;
        dpb_mle* eq = nullptr;
        int rc = dpb_eq_table(ctx, F::kChalDtype, points[a], point_len[a], &eq);
        if (rc != DPB_OK) {
            free_eqs();
            return cleanup(rc);
        }
        eqs.push_back(eq);
        w_ptrs.push_back((const E*)eq->ptr);
    }
    std::vector<uint64_t> off(O);
    for (uint64_t o = 0; o < O; o++) {
        uint64_t rem = o, acc = 0;
        for (int a = (int)n_outer - 1; a >= 0; a--) {
            acc += (rem % outer_dims[a]) * outer_stride[a];
            rem /= outer_dims[a];
        }
        off[o] = acc;
    }
    void *d_off = nullptr, *d_w = nullptr, *d_wptr = nullptr, *d_dims = nullptr;
    int rc = device_alloc(ctx, O * 8, &d_off);
    if (rc == DPB_OK) { to_free.push_back(d_off); rc = device_alloc(ctx, O * sizeof(E), &d_w); }
    if (rc == DPB_OK) { to_free.push_back(d_w); rc = device_alloc(ctx, (n_outer + 1) * sizeof(void*), &d_wptr); }
    if (rc == DPB_OK) { to_free.push_back(d_wptr); rc = device_alloc(ctx, (n_outer + 1) * 8, &d_dims); }
    if (rc == DPB_OK) to_free.push_back(d_dims);
    if (rc != DPB_OK) {
        free_eqs();
        return cleanup(rc);
    }
    rc = upload_small(ctx, d_off, off.data(), O * 8);
    if (rc == DPB_OK && n_outer) {
        rc = upload_small(ctx, d_wptr, w_ptrs.data(), n_outer * sizeof(void*));
        if (rc == DPB_OK) rc = upload_small(ctx, d_dims, outer_dims, n_outer * 8);
    }
    if (rc != DPB_OK) {
        free_eqs();
        return cleanup(rc);
    }
    einsum_outer_weights<F><<<grid_for(ctx, O), kThreads, 0, ctx->stream>>>((const E* const*)d_wptr, (const uint64_t*)d_dims,
                                                                              n_outer, O, (E*)d_w);
    // output slab: S tables of c_pad entries, pad zeroed
    dpb_mle* owner = new (std::nothrow) dpb_mle();
    if (!owner) {
        free_eqs();
        return cleanup(fail(DPB_ENOMEM, "host allocation failed"));
    }
    owner->ctx = ctx;
    owner->dtype = F::kChalDtype;
    owner->len = S * c_pad;
    owner->owns = true;
    rc = device_alloc(ctx, S * c_pad * sizeof(E), &owner->ptr);
    if (rc != DPB_OK) {
        delete owner;
        free_eqs();
        return cleanup(rc);
    }
    if (c_pad != C) cudaMemsetAsync(owner->ptr, 0, S * c_pad * sizeof(E), ctx->stream);
    const uint64_t n_outputs = S * C;
    const bool innermost_is_outer = rank > 0 && kind[rank - 1] == DPB_AXIS_OUTER;
    if (innermost_is_outer)
        einsum_contract_warp<F><<<grid_for(ctx, n_outputs * 32), kThreads, 0, ctx->stream>>>(
            t_dev, kept, (const uint64_t*)d_off, (const E*)d_w, O, n_outputs, C, c_pad, (E*)owner->ptr);
    else
        einsum_contract_thread<F><<<grid_for(ctx, n_outputs), kThreads, 0, ctx->stream>>>(
            t_dev, kept, (const uint64_t*)d_off, (const E*)d_w, O, n_outputs, C, c_pad, (E*)owner->ptr);
    cudaError_t e = cudaGetLastError();
    // a host tensor is only read during the call: wait for its copy (device tensors need no wait)
    if (e == cudaSuccess && !tensor_on_device) e = cudaStreamSynchronize(ctx->stream);
    free_eqs();
    cleanup(DPB_OK);
    if (e != cudaSuccess) {
        dpb_mle_free(owner);
        return fail(DPB_ECUDA, "einsum: %s", cudaGetErrorString(e));
    }
    for (uint64_t s = 0; s < S; s++) {
        dpb_mle* v = new (std::nothrow) dpb_mle();
        if (!v) return fail(DPB_ENOMEM, "host allocation failed");
        v->ctx = ctx;
        v->dtype = F::kChalDtype;
        v->len = c_pad;
        v->ptr = (char*)owner->ptr + s * c_pad * sizeof(E);
        v->owns = false;
        out_mles[s] = v;
    }
    *out_owner = owner;
    *n_out = (uint32_t)S;
    return DPB_OK;
}

}  // namespace dpb

using namespace dpb;

extern "C" int dpb_einsum_fix_axes(dpb_ctx* ctx, int family_dtype, const int64_t* tensor, int tensor_on_device,
                                   const uint64_t* shape, const uint8_t* axis_kind, const void* const* axis_points,
                                   const uint32_t* axis_point_len, uint32_t rank, dpb_mle** out_owner,
                                   dpb_mle** out_mles, uint32_t out_cap, uint32_t* n_out) {
    if (!ctx || !tensor || !shape || !axis_kind || !axis_points || !axis_point_len || !out_owner || !out_mles || !n_out)
        return fail(DPB_EINVAL, "null argument");
    if (!valid_dtype(family_dtype)) return fail(DPB_EINVAL, "unknown dtype %d", family_dtype);
    if (rank < 1 || rank > (uint32_t)kMaxEinsumRank) return fail(DPB_EINVAL, "rank %u outside 1..%d", rank, kMaxEinsumRank);
    for (uint32_t a = 0; a < rank; a++)
        if (shape[a] == 0) return fail(DPB_EINVAL, "axis %u is empty", a);
    return is_gl(family_dtype)
               ? einsum_impl<GlFam>(ctx, tensor, tensor_on_device, shape, axis_kind, axis_points, axis_point_len, rank,
                                    out_owner, out_mles, out_cap, n_out)
               : einsum_impl<FrFam>(ctx, tensor, tensor_on_device, shape, axis_kind, axis_points, axis_point_len, rank,
                                    out_owner, out_mles, out_cap, n_out);
}
