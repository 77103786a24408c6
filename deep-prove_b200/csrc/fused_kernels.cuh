// The product shape of a sumcheck: a single term  f_1 * f_2 * ... * f_K
// (coefficient one) over K tables that all have every variable of the
// sumcheck and share one storage layout.  This is the f*g*h microbenchmark
// shape and the v1*v2*eq shape of the Hadamard prover
// (zkml/src/layers/hadamard.rs:106-115).
//
// This header holds the shape detection the sumcheck entry points use and the
// plain first-round kernel (one thread per pair, evaluations at 0..=K) that the
// allocation-free entry point launches; the rounds of an ordinary sumcheck of
// this shape run the sampled kernels of fused_v2.cuh / fused_v4.cuh.
#pragma once
#include <functional>
#include <type_traits>

#include "common.cuh"

namespace dpb {

constexpr int kFusedNone = 0;
constexpr int kFusedProduct = 1;  // single product of K = k full-size tables, coefficient one

// ---- input adaptors --------------------------------------------------------
// Goldilocks tables that still hold base-field entries are multiplied in the
// base field (one 64-bit multiply instead of three).
template <class F, bool BASE>
struct FusedIn;

template <>
struct FusedIn<GlFam, true> {
    typedef uint64_t T;
    __device__ __forceinline__ static void load2(const void* p, uint64_t q, T (&a)[2]) {
        const ulonglong2 u = ((const ulonglong2*)p)[q];
        a[0] = u.x; a[1] = u.y;
    }
    __device__ __forceinline__ static T add(T a, T b) { return gl_add(a, b); }
    __device__ __forceinline__ static T sub(T a, T b) { return gl_sub(a, b); }
    __device__ __forceinline__ static T mul(T a, T b) { return gl_mul(a, b); }
    __device__ __forceinline__ static T zero() { return 0; }
    __device__ __forceinline__ static Gl2 widen(T a) { return gl2_from_base(a); }
};

template <class F>
struct FusedIn<F, false> {
    typedef typename F::E T;
    __device__ __forceinline__ static void load2(const void* p, uint64_t q, T (&a)[2]) {
        a[0] = F::load(p, F::kChalDtype, 2 * q);
        a[1] = F::load(p, F::kChalDtype, 2 * q + 1);
    }
    __device__ __forceinline__ static T add(const T& a, const T& b) { return F::add(a, b); }
    __device__ __forceinline__ static T sub(const T& a, const T& b) { return F::sub(a, b); }
    __device__ __forceinline__ static T mul(const T& a, const T& b) { return F::mul(a, b); }
    __device__ __forceinline__ static T zero() { return F::zero(); }
    __device__ __forceinline__ static T widen(const T& a) { return a; }
};

template <int K>
struct FusedPtrs {
    const void* in[K];
    void* out[K];
};

// Round 0: acc[x] = sum_p prod_j (f_j[2p] + x (f_j[2p+1] - f_j[2p])),  x = 0..K.
template <class F, int K, bool BASE>
__global__ void __launch_bounds__(kThreads)
    fused_product_eval0(FusedPtrs<K> ptrs, uint64_t n_pairs, ReduceScratch<F> rs,
                        typename F::E* out) {
    typedef FusedIn<F, BASE> In;
    typedef typename In::T T;
    typedef typename F::E E;
    T acc[K + 1];
#pragma unroll
    for (int x = 0; x <= K; x++) acc[x] = In::zero();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n_pairs; p += stride) {
        T val[K], delta[K];
#pragma unroll
        for (int j = 0; j < K; j++) {
            T a[2];
            In::load2(ptrs.in[j], p, a);
            val[j] = a[0];
            delta[j] = In::sub(a[1], a[0]);
        }
#pragma unroll
        for (int x = 0; x <= K; x++) {
            T prod = val[0];
#pragma unroll
            for (int j = 1; j < K; j++) prod = In::mul(prod, val[j]);
            acc[x] = In::add(acc[x], prod);
            if (x < K) {
#pragma unroll
                for (int j = 0; j < K; j++) val[j] = In::add(val[j], delta[j]);
            }
        }
    }
    E wide[K + 1];
#pragma unroll
    for (int x = 0; x <= K; x++) wide[x] = In::widen(acc[x]);
    grid_sum_publish<F, K + 1>(wide, rs, out);
}

// ---- host side ---------------------------------------------------------------
// Returns kFusedProduct when the term list is one coefficient-one product of
// all k (2..4) tables, each used once, all full-size and in one layout.
inline int detect_fused_shape(const MleDesc*, size_t k, uint32_t num_vars, const dpb_term* terms,
                              uint32_t n_terms, bool gl, const std::function<uint32_t(uint32_t)>& nv,
                              const std::function<int(uint32_t)>& dtype) {
    if (n_terms != 1 || k < 2 || k > 4 || terms[0].n_factors != k || num_vars < 2) return kFusedNone;
    bool seen[4] = {false, false, false, false};
    for (uint32_t j = 0; j < k; j++) {
        const uint32_t id = terms[0].idx[j];
        if (id >= k || seen[id]) return kFusedNone;
        seen[id] = true;
        if (nv(j) != num_vars || dtype(j) != dtype(0)) return kFusedNone;
    }
    // integer tables: only 32-bit integers of the BN254 family have fused rounds (products of up to three)
    if (dtype(0) == DPB_GL_I64 || dtype(0) == DPB_GL_I32 || dtype(0) == DPB_FR_I64) return kFusedNone;
    if (dtype(0) == DPB_FR_I32 && k > 3) return kFusedNone;
    if (gl) {
        Gl2 c;
        memcpy(&c, terms[0].coeff, sizeof c);
        if (!GlFam::is_one(c)) return kFusedNone;
    } else {
        Fr c;
        memcpy(&c, terms[0].coeff, sizeof c);
        if (!FrFam::is_one(c)) return kFusedNone;
    }
    return kFusedProduct;
}
}  // namespace dpb
