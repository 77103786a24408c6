// Einsum axis fixing: contract the OUTER axes of an integer tensor against
// per-axis eq weights, keep the stacked and contracted axes
// (FixedAxesMapping::mles_from_tensor, zkml/src/layers/einsum/axis.rs:1142-1234).
//
//   out[q] = sum_o W[o] * T[kept_off(q) + outer_off[o]],   W[o] = prod_a w_a[o_a]
//
// The tensor stays in its native form (signed 64-bit quantised values, 8 bytes
// per entry instead of a 32-byte field element).  A term of the sum is
// (integer) * (field element): the products are added up as plain integers
// (16 wide multiply-adds per term for BN254, 4 for Goldilocks, no reduction) and
// reduced once per output; a negative entry adds its magnitude times the
// negated weight.
#pragma once
#include "family.cuh"
#include "gl_words.cuh"

namespace dpb {

constexpr int kMaxEinsumRank = 8;

struct EinsumKept {
    uint32_t n_kept;
    uint64_t dim[kMaxEinsumRank];     // kept axes, outermost first
    uint64_t stride[kMaxEinsumRank];  // their strides in the tensor (entries)
};

template <class F>
struct EinsumAcc;
template <>
struct EinsumAcc<FrFam> {
    FrIntAcc a;
    __device__ __forceinline__ void zero() { a = fr_intacc_zero(); }
    __device__ __forceinline__ void mac(const Fr& w, int64_t x) { fr_intacc_mac(a, w, x); }
    __device__ __forceinline__ Fr finish() const { return fr_intacc_finish(a); }
};
template <>
struct EinsumAcc<GlFam> {
    glw::A8 s0, s1;
    __device__ __forceinline__ void zero() { s0 = s1 = glw::acc_zero(); }
    __device__ __forceinline__ void mac(const Gl2& w, int64_t x) {
        const uint64_t mag = x < 0 ? (uint64_t)0 - (uint64_t)x : (uint64_t)x;
        const uint64_t c0 = x < 0 ? gl_neg(w.c0) : w.c0, c1 = x < 0 ? gl_neg(w.c1) : w.c1;
        const glw::W m = glw::make_w((uint32_t)mag, (uint32_t)(mag >> 32));
        glw::acc_mac(s0, m, glw::make_w((uint32_t)c0, (uint32_t)(c0 >> 32)));
        glw::acc_mac(s1, m, glw::make_w((uint32_t)c1, (uint32_t)(c1 >> 32)));
    }
    __device__ __forceinline__ Gl2 finish() const {
        return gl2_make(glw::to_u64(glw::canon(glw::acc_reduce(s0))), glw::to_u64(glw::canon(glw::acc_reduce(s1))));
    }
};

// W[o] = prod over outer axes of w_a[coordinate of o on axis a]; o is the flat
// row-major index over the outer axes.
template <class F>
__global__ void einsum_outer_weights(const typename F::E* const* __restrict__ w, const uint64_t* __restrict__ dims,
                                     uint32_t n_outer, uint64_t n, typename F::E* __restrict__ out) {
    typedef typename F::E E;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t o = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; o < n; o += stride) {
        uint64_t rem = o;
        E acc = F::one();
        for (int a = (int)n_outer - 1; a >= 0; a--) {
            const uint64_t c = rem % dims[a];
            rem /= dims[a];
            acc = F::mul(acc, w[a][c]);
        }
        F::store(out, o, acc);
    }
}

__device__ __forceinline__ uint64_t einsum_kept_offset(const EinsumKept& k, uint64_t q) {
    uint64_t off = 0;
    for (int a = (int)k.n_kept - 1; a >= 0; a--) {
        off += (q % k.dim[a]) * k.stride[a];
        q /= k.dim[a];
    }
    return off;
}

// One thread per output entry: right when the innermost tensor axis is kept
// (neighbouring outputs are neighbouring tensor entries).
// Output entry q = s * C + c lands at out[s * c_pad + c]; the pad is zeroed by the caller.
template <class F>
__global__ void einsum_contract_thread(const int64_t* __restrict__ t, EinsumKept kept, const uint64_t* __restrict__ outer_off,
                                       const typename F::E* __restrict__ w, uint64_t n_outer, uint64_t n_out,
                                       uint64_t c_size, uint64_t c_pad, typename F::E* __restrict__ out) {
    typedef typename F::E E;
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t q = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; q < n_out; q += stride) {
        const uint64_t base = einsum_kept_offset(kept, q);
        EinsumAcc<F> acc;
        acc.zero();
        for (uint64_t o = 0; o < n_outer; o++) acc.mac(F::load(w, F::kChalDtype, o), t[base + outer_off[o]]);
        F::store(out, (q / c_size) * c_pad + (q % c_size), acc.finish());
    }
}

// One warp per output entry, lanes striding over the outer index: right when
// the innermost tensor axis is an outer axis.
template <class F>
__global__ void einsum_contract_warp(const int64_t* __restrict__ t, EinsumKept kept, const uint64_t* __restrict__ outer_off,
                                     const typename F::E* __restrict__ w, uint64_t n_outer, uint64_t n_out,
                                     uint64_t c_size, uint64_t c_pad, typename F::E* __restrict__ out) {
    typedef typename F::E E;
    const uint32_t lane = threadIdx.x & 31;
    const uint64_t warp = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint64_t n_warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    for (uint64_t q = warp; q < n_out; q += n_warps) {
        const uint64_t base = einsum_kept_offset(kept, q);
        EinsumAcc<F> part;
        part.zero();
        for (uint64_t o = lane; o < n_outer; o += 32) part.mac(F::load(w, F::kChalDtype, o), t[base + outer_off[o]]);
        E acc = part.finish();
        for (int off = 16; off > 0; off >>= 1) acc = F::add(acc, F::shfl_down(acc, off));
        if (lane == 0) F::store(out, (q / c_size) * c_pad + (q % c_size), acc);
    }
}

}  // namespace dpb
