// Multilinear-table kernels outside the sumcheck loop: layout conversion, eq
// tables, partial evaluation of the top / bottom variables.
#pragma once
#include "family.cuh"

namespace dpb {

// ---- layout conversion ---------------------------------------------------
// in and out may be the same array
__global__ void fr_canonical_to_mont(const Fr* in, Fr* out, uint64_t n) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        FrFam::store(out, i, fr_to_mont(FrFam::load(in, DPB_FR, i)));
}
__global__ void fr_mont_to_canonical(const Fr* in, Fr* out, uint64_t n) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        FrFam::store(out, i, fr_from_mont(FrFam::load(in, DPB_FR, i)));
}
__global__ void fr_from_i64_kernel(const int64_t* __restrict__ in, Fr* __restrict__ out,
                                   uint64_t n) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        FrFam::store(out, i, fr_from_i64(in[i]));
}
__global__ void gl_from_i64_kernel(const int64_t* __restrict__ in, uint64_t* __restrict__ out,
                                   uint64_t n) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const int64_t x = in[i];
        // |x| < 2^63 < p, so the magnitude is already canonical
        out[i] = x < 0 ? GL_P - ((uint64_t)0 - (uint64_t)x) : (uint64_t)x;
    }
}

// ---- eq tables -------------------------------------------------------------
// out[i] = prod_j (bit_j(i) ? pt[j] : 1 - pt[j]),  i < 2^m, directly (m small).
template <class F>
__global__ void eq_direct(const typename F::E* __restrict__ pt, uint32_t m,
                          typename F::E* __restrict__ out) {
    typedef typename F::E E;
    const uint64_t n = 1ull << m;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        E acc = F::one();
        for (uint32_t j = 0; j < m; j++) {
            const E r = pt[j];
            acc = F::mul(acc, ((i >> j) & 1) ? r : F::sub(F::one(), r));
        }
        F::store(out, i, acc);
    }
}
// out[i] = hi[i >> lo_bits] * lo[i & (2^lo_bits - 1)]
template <class F>
__global__ void eq_combine(const typename F::E* __restrict__ lo, uint32_t lo_bits,
                           const typename F::E* __restrict__ hi, uint64_t n,
                           typename F::E* __restrict__ out) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t mask = (1ull << lo_bits) - 1;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        F::store(out, i,
                 F::mul(F::load(hi, F::kChalDtype, i >> lo_bits), F::load(lo, F::kChalDtype, i & mask)));
}

// ---- many eq tables at once -----------------------------------------------------
// Table t has m_t variables and its point at pts[pt_off[t] ..].  Its table is
// the outer product of a "low" part over the first h_t = ceil(m_t / 2) variables
// and a "high" part over the rest, each computed directly (at most m_t / 2 + 1
// multiplies per entry of tables of about sqrt(2^m_t) entries), then one
// multiply per output entry.  Work items of all tables are laid end to end;
// `prefix` holds the first item of every table (n + 1 entries) and a thread
// finds its table by binary search.
struct EqBatchDesc {
    uint32_t m;        // variables
    uint32_t pt_off;   // first coordinate in the points array
    uint64_t part_off; // low part at parts[part_off], high part right after it
    uint64_t out_off;  // table at out[out_off]
};

__device__ __forceinline__ uint32_t find_segment(const uint64_t* __restrict__ prefix, uint32_t n, uint64_t item) {
    uint32_t lo = 0, hi = n;
    while (hi - lo > 1) {
        const uint32_t mid = (lo + hi) >> 1;
        if (prefix[mid] <= item) lo = mid;
        else hi = mid;
    }
    return lo;
}

template <class F>
__global__ void __launch_bounds__(kThreads)
    eq_batch_parts(const EqBatchDesc* __restrict__ desc, const uint64_t* __restrict__ prefix, uint32_t n,
                   const typename F::E* __restrict__ pts, typename F::E* __restrict__ parts) {
    typedef typename F::E E;
    const uint64_t total = prefix[n];
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t w = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += stride) {
        const uint32_t t = find_segment(prefix, n, w);
        const EqBatchDesc d = desc[t];
        const uint32_t h = (d.m + 1) / 2;
        uint64_t i = w - prefix[t];
        uint32_t first = 0, bits = h;  // low part: coordinates [0, h)
        if (i >= (1ull << h)) {        // high part: coordinates [h, m)
            i -= 1ull << h;
            first = h;
            bits = d.m - h;
        }
        E acc = F::one();
        for (uint32_t j = 0; j < bits; j++) {
            const E r = pts[d.pt_off + first + j];
            acc = F::mul(acc, ((i >> j) & 1) ? r : F::sub(F::one(), r));
        }
        F::store(parts, d.part_off + (w - prefix[t]), acc);
    }
}

template <class F>
__global__ void __launch_bounds__(kThreads)
    eq_batch_combine(const EqBatchDesc* __restrict__ desc, const uint64_t* __restrict__ prefix, uint32_t n,
                     const typename F::E* __restrict__ parts, typename F::E* __restrict__ out) {
    const uint64_t total = prefix[n];
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t w = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; w < total; w += stride) {
        const uint32_t t = find_segment(prefix, n, w);
        const EqBatchDesc d = desc[t];
        const uint32_t h = (d.m + 1) / 2;
        const uint64_t i = w - prefix[t];
        const uint64_t lo = i & ((1ull << h) - 1), hi = i >> h;
        F::store(out, d.out_off + i,
                 F::mul(F::load(parts, F::kChalDtype, d.part_off + lo),
                        F::load(parts, F::kChalDtype, d.part_off + (1ull << h) + hi)));
    }
}

// Many tables evaluated at one point: table t (2^m_t entries, any layout of its family) against the eq table of the
// point's first m_t coordinates: partial[t * slices + s] = sum over slice s of table_t[x] * eq_{m_t}[x].
struct EvalManySrc {
    const void* ptr;
    const void* eq;  // eq table over this table's variables (challenge elements)
    uint64_t len;
    int32_t dtype;
    int32_t pad;
};
template <class F>
__global__ void __launch_bounds__(kThreads)
    evaluate_many_kernel(const EvalManySrc* __restrict__ src, uint32_t slices, typename F::E* __restrict__ partial) {
    typedef typename F::E E;
    const EvalManySrc t = src[blockIdx.y];
    E acc[1] = {F::zero()};
    const uint64_t stride = (uint64_t)slices * blockDim.x;
    for (uint64_t x = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; x < t.len; x += stride)
        acc[0] = F::add(acc[0], F::mul(F::load(t.ptr, t.dtype, x), ((const E*)t.eq)[x]));
    block_sum<F, 1>(acc);
    if (threadIdx.x == 0) partial[(size_t)blockIdx.y * slices + blockIdx.x] = acc[0];
}
// out[t] = scale[t] * sum_s partial[t * slices + s]
template <class F>
__global__ void __launch_bounds__(kThreads)
    evaluate_many_finish(const typename F::E* __restrict__ partial, uint32_t slices, const typename F::E* __restrict__ scale,
                         uint32_t n, typename F::E* __restrict__ out) {
    typedef typename F::E E;
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n) return;
    E acc = F::zero();
    for (uint32_t s = 0; s < slices; s++) acc = F::add(acc, partial[(size_t)t * slices + s]);
    out[t] = F::mul(acc, scale[t]);
}

// One source table of a linear combination.
struct LinCombSrc {
    const void* ptr;
    uint64_t len;
    int32_t dtype;
    int32_t pad;
};

// The eq table of a rotary layer with its entries moved and negated the way the rotation pairs them
// (RopeLayout::permuted_eq_poly, zkml/src/layers/transformer/positional/rope.rs:238-258).
// layout 0 (adjacent pairs): out[i] = eq[i + 1] for even i, -eq[i - 1] for odd i.
// layout 1 (rotate half, rows of `row` entries): out[i] = eq[i + row/2] in a row's first half, -eq[i - row/2] in its second.
template <class F>
__global__ void __launch_bounds__(kThreads)
    rope_permuted_eq_kernel(const typename F::E* __restrict__ eq, uint64_t len, int layout, uint64_t row,
                            typename F::E* __restrict__ out) {
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += stride) {
        bool first;
        uint64_t src;
        if (layout == 0) {
            first = (i & 1) == 0;
            src = i ^ 1;
        } else {
            const uint64_t half = row >> 1, c = i % row;
            first = c < half;
            src = first ? i + half : i - half;
        }
        const typename F::E v = eq[src];
        out[i] = first ? v : F::neg(v);
    }
}

// out[i] = sum_j coeff[j] * table_j[i], tables shorter than the output read as zero beyond their length.
// Consecutive threads read consecutive entries of each table in turn.
template <class F>
__global__ void __launch_bounds__(kThreads)
    linear_combination_kernel(const LinCombSrc* __restrict__ src, const typename F::E* __restrict__ coeff, uint32_t n,
                              uint64_t len, typename F::E* __restrict__ out) {
    typedef typename F::E E;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < len; i += stride) {
        E acc = F::zero();
        for (uint32_t j = 0; j < n; j++) {
            const LinCombSrc s = src[j];
            if (i < s.len) acc = F::add(acc, F::mul(coeff[j], F::load(s.ptr, s.dtype, i)));
        }
        F::store(out, i, acc);
    }
}

}  // namespace dpb
