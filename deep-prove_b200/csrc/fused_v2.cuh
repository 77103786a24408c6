// Fused product-sumcheck rounds, second generation.
//
// Same data movement as fused_kernels.cuh (round 0 reads the tables once;
// every later round reads the previous tables once, writes the half-size
// tables and evaluates from registers) but far fewer instructions per pair:
//
//  * The round polynomial P of degree K is sampled at 0, (1), "infinity" (its
//    leading coefficient), -1 and, for K = 4, 2.  At 0, 1 and infinity the
//    factor values are the table entries and their differences themselves, so
//    no per-point increments are needed.  P(1) is only computed in round 0;
//    later rounds the host derives it from the previous round
//    (P_i(0) + P_i(1) = P_{i-1}(r_{i-1})).  The host turns these samples into the
//    evaluations at 0..=K; field arithmetic is exact, so the result is the same
//    bit pattern the plain evaluation gives.
//  * Goldilocks products are accumulated as unreduced 128-bit integers in
//    160-bit accumulators and reduced once per thread (gl_fast.cuh).
//
// Output slots of every kernel (K+1 challenge elements):
//   [0] P(0)   [1] P(1) (round 0 only, else zero)   [2] prod_j (f_j(0) - f_j(1)) = (-1)^K P(inf)
//   [3] P(-1) (K >= 3)   [4] P(2) (K = 4)
#pragma once
#include "common.cuh"
#include "gl_fast.cuh"

namespace dpb {

// ---- per-layout arithmetic --------------------------------------------------
// T: value held in registers; C: the challenge; Acc: accumulator of products.
struct OpsGlBase {
    typedef GlFam F;
    typedef uint64_t T;
    typedef glf::Acc160 Acc;
    static constexpr int kLoadWords = 1;
    __device__ __forceinline__ static T sub_c(T a, T c) { return glf::sub_c(a, c); }
    __device__ __forceinline__ static T add_c(T a, T c) { return glf::add_c(a, c); }
    __device__ __forceinline__ static T mul(T a, T b) { return glf::mul(a, b); }
    __device__ __forceinline__ static Acc acc_zero() { return glf::acc_zero(); }
    __device__ __forceinline__ static void mac(Acc& acc, T a, T b) { glf::acc_mac(acc, a, b); }
    __device__ __forceinline__ static Gl2 finish(const Acc& acc) {
        return gl2_make(glf::canon(glf::acc_reduce(acc)), 0);
    }
    __device__ __forceinline__ static void load2(const void* p, uint64_t q, T (&a)[2]) {
        const ulonglong2 u = ((const ulonglong2*)p)[q];
        a[0] = u.x;
        a[1] = u.y;
    }
};

struct OpsGlExt {
    typedef GlFam F;
    typedef glf::L2 T;
    struct Acc {
        glf::Acc160 s00, s11, s01;
    };
    __device__ __forceinline__ static T sub_c(const T& a, const T& c) {
        T r;
        r.c0 = glf::sub_c(a.c0, c.c0);
        r.c1 = glf::sub_c(a.c1, c.c1);
        return r;
    }
    __device__ __forceinline__ static T add_c(const T& a, const T& c) {
        T r;
        r.c0 = glf::add_c(a.c0, c.c0);
        r.c1 = glf::add_c(a.c1, c.c1);
        return r;
    }
    __device__ __forceinline__ static T mul(const T& a, const T& b) { return glf::mul2(a, b); }
    __device__ __forceinline__ static Acc acc_zero() {
        Acc a;
        a.s00 = a.s11 = a.s01 = glf::acc_zero();
        return a;
    }
    __device__ __forceinline__ static void mac(Acc& acc, const T& a, const T& b) {
        glf::acc_mac(acc.s00, a.c0, b.c0);
        glf::acc_mac(acc.s11, a.c1, b.c1);
        glf::acc_mac(acc.s01, a.c0, b.c1);
        glf::acc_mac(acc.s01, a.c1, b.c0);
    }
    __device__ __forceinline__ static Gl2 finish(const Acc& acc) {
        const uint64_t s11 = glf::canon(glf::acc_reduce(acc.s11));
        const uint64_t c0 = gl_add(glf::canon(glf::acc_reduce(acc.s00)), gl_mul_small(s11, (uint32_t)GL_NONRES));
        return gl2_make(c0, glf::canon(glf::acc_reduce(acc.s01)));
    }
    __device__ __forceinline__ static T load1(const void* p, uint64_t i) {
        const ulonglong2 u = ((const ulonglong2*)p)[i];
        T r;
        r.c0 = u.x;
        r.c1 = u.y;
        return r;
    }
    __device__ __forceinline__ static void load2(const void* p, uint64_t q, T (&a)[2]) {
        a[0] = load1(p, 2 * q);
        a[1] = load1(p, 2 * q + 1);
    }
};

// Extension arithmetic with two accumulators per sample: the non-residue is
// folded into the left operand of the lazy product (one small multiply per
// product) instead of keeping a third 160-bit sum alive.
struct OpsGlExt2 : OpsGlExt {
    struct Acc {
        glf::Acc160 s0, s1;
    };
    __device__ __forceinline__ static Acc acc_zero() {
        Acc a;
        a.s0 = a.s1 = glf::acc_zero();
        return a;
    }
    __device__ __forceinline__ static void mac(Acc& acc, const T& a, const T& b) {
        glf::acc_mac(acc.s0, a.c0, b.c0);
        glf::acc_mac(acc.s0, glf::mul7(a.c1), b.c1);
        glf::acc_mac(acc.s1, a.c0, b.c1);
        glf::acc_mac(acc.s1, a.c1, b.c0);
    }
    __device__ __forceinline__ static Gl2 finish(const Acc& acc) {
        return gl2_make(glf::canon(glf::acc_reduce(acc.s0)), glf::canon(glf::acc_reduce(acc.s1)));
    }
};

struct OpsFr {
    typedef FrFam F;
    typedef Fr T;
    typedef Fr Acc;
    __device__ __forceinline__ static T sub_c(const T& a, const T& c) { return fr_sub(a, c); }
    __device__ __forceinline__ static T add_c(const T& a, const T& c) { return fr_add(a, c); }
    __device__ __forceinline__ static T mul(const T& a, const T& b) { return fr_mul(a, b); }
    __device__ __forceinline__ static Acc acc_zero() { return fr_zero(); }
    __device__ __forceinline__ static void mac(Acc& acc, const T& a, const T& b) { acc = fr_add(acc, fr_mul(a, b)); }
    __device__ __forceinline__ static Fr finish(const Acc& acc) { return acc; }
    __device__ __forceinline__ static void load2(const void* p, uint64_t q, T (&a)[2]) {
        a[0] = FrFam::load(p, DPB_FR, 2 * q);
        a[1] = FrFam::load(p, DPB_FR, 2 * q + 1);
    }
};

// acc[slot] += prod_j v[j]
template <class Ops, int K>
__device__ __forceinline__ void mac_product(typename Ops::Acc& acc, const typename Ops::T (&v)[K]) {
    if (K == 2) {
        Ops::mac(acc, v[0], v[1]);
    } else {
        typename Ops::T t = Ops::mul(v[0], v[1]);
#pragma unroll
        for (int j = 2; j < K - 1; j++) t = Ops::mul(t, v[j]);
        Ops::mac(acc, t, v[K - 1]);
    }
}

// Adds one pair's contribution to every sample.  f0[j], f1[j] are canonical.
template <class Ops, int K, bool WITH_P1>
__device__ __forceinline__ void sample_pair(typename Ops::Acc (&acc)[K + 1], const typename Ops::T (&f0)[K],
                                            const typename Ops::T (&f1)[K]) {
    typedef typename Ops::T T;
    mac_product<Ops, K>(acc[0], f0);
    if (WITH_P1) mac_product<Ops, K>(acc[1], f1);
    T e[K];
#pragma unroll
    for (int j = 0; j < K; j++) e[j] = Ops::sub_c(f0[j], f1[j]);  // f(0) - f(1)
    mac_product<Ops, K>(acc[2], e);
    if (K >= 3) {
        T m[K];
#pragma unroll
        for (int j = 0; j < K; j++) m[j] = Ops::add_c(e[j], f0[j]);  // f(-1) = 2 f(0) - f(1)
        mac_product<Ops, K>(acc[3], m);
    }
    if (K >= 4) {
        T g[K];
#pragma unroll
        for (int j = 0; j < K; j++) g[j] = Ops::add_c(Ops::sub_c(f1[j], f0[j]), f1[j]);  // f(2) = 2 f(1) - f(0)
        mac_product<Ops, K>(acc[K], g);
    }
}

// The same sampling, fed one table at a time: keeps only the running products
// of the K-1 tables seen so far (fewer live registers than holding every
// table's pair).  Call absorb<J>() for J = 0..K-1 in order.
template <class Ops, int K, bool WITH_P1>
struct Sampler {
    typedef typename Ops::T T;
    T p0, p1, pinf, pm1, p2;
    template <int J>
    __device__ __forceinline__ void absorb(typename Ops::Acc (&acc)[K + 1], const T& f0, const T& f1) {
        const T e = Ops::sub_c(f0, f1);
        T m = e, g = e;
        if (K >= 3) m = Ops::add_c(e, f0);
        if (K >= 4) g = Ops::add_c(Ops::sub_c(f1, f0), f1);
        if (J == 0) {
            p0 = f0;
            p1 = f1;
            pinf = e;
            pm1 = m;
            p2 = g;
        } else if (J < K - 1) {
            p0 = Ops::mul(p0, f0);
            if (WITH_P1) p1 = Ops::mul(p1, f1);
            pinf = Ops::mul(pinf, e);
            if (K >= 3) pm1 = Ops::mul(pm1, m);
            if (K >= 4) p2 = Ops::mul(p2, g);
        } else {
            Ops::mac(acc[0], p0, f0);
            if (WITH_P1) Ops::mac(acc[1], p1, f1);
            Ops::mac(acc[2], pinf, e);
            if (K >= 3) Ops::mac(acc[3], pm1, m);
            if (K >= 4) Ops::mac(acc[K], p2, g);
        }
    }
};

template <int K>
struct V2Ptrs {
    const void* in[K];
    void* out[K];
};

template <class Ops, int K>
__device__ __forceinline__ void publish(typename Ops::Acc (&acc)[K + 1], ReduceScratch<typename Ops::F> rs,
                                        typename Ops::F::E* out) {
    typename Ops::F::E wide[K + 1];
#pragma unroll
    for (int x = 0; x <= K; x++) wide[x] = Ops::finish(acc[x]);
    grid_sum_publish<typename Ops::F, K + 1>(wide, rs, out);
}

// Round 0: samples only.
template <class Ops, int K, int MINB = 1>
__global__ void __launch_bounds__(kThreads, MINB)
    v2_eval0(V2Ptrs<K> ptrs, uint64_t n_pairs, ReduceScratch<typename Ops::F> rs, typename Ops::F::E* out) {
    typedef typename Ops::T T;
    typename Ops::Acc acc[K + 1];
#pragma unroll
    for (int x = 0; x <= K; x++) acc[x] = Ops::acc_zero();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n_pairs; p += stride) {
        T f0[K], f1[K];
#pragma unroll
        for (int j = 0; j < K; j++) {
            T a[2];
            Ops::load2(ptrs.in[j], p, a);
            f0[j] = a[0];
            f1[j] = a[1];
        }
        sample_pair<Ops, K, true>(acc, f0, f1);
    }
    publish<Ops, K>(acc, rs, out);
}

// ---- folds -------------------------------------------------------------------
// What a fold needs to know about the challenge r = (r0, r1): r0, r1 and 7*r1.
struct GlChal {
    uint64_t r0, r1, r1x7;
};

// Rounds >= 1 over Goldilocks.  BASE_IN: the input tables hold base elements
// (round 1); otherwise extension elements.  One thread per output pair.
template <int K, bool BASE_IN, int MINB>
__global__ void __launch_bounds__(kThreads, MINB)
    v2_fold_eval_gl(V2Ptrs<K> ptrs, GlChal r, uint64_t n_pairs, ReduceScratch<GlFam> rs, Gl2* out) {
    typedef OpsGlExt Ops;
    typedef glf::L2 T;
    Ops::Acc acc[K + 1];
#pragma unroll
    for (int x = 0; x <= K; x++) acc[x] = Ops::acc_zero();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n_pairs; p += stride) {
        T f[2][K];
#pragma unroll
        for (int j = 0; j < K; j++) {
            if (BASE_IN) {
                const ulonglong2* s = (const ulonglong2*)ptrs.in[j] + 2 * p;
                const ulonglong2 u = s[0], v = s[1];
                const uint64_t a[4] = {u.x, u.y, v.x, v.y};
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const uint64_t d = glf::sub_c(a[2 * h + 1], a[2 * h]);
                    f[h][j].c0 = glf::canon(glf::add_c(glf::mul(r.r0, d), a[2 * h]));
                    f[h][j].c1 = glf::canon(glf::mul(r.r1, d));
                }
            } else {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const T a0 = Ops::load1(ptrs.in[j], 4 * p + 2 * h);
                    const T a1 = Ops::load1(ptrs.in[j], 4 * p + 2 * h + 1);
                    const T d = Ops::sub_c(a1, a0);
                    glf::Acc160 s0 = glf::acc_zero(), s1 = glf::acc_zero();
                    glf::acc_mac(s0, d.c0, r.r0);
                    glf::acc_mac(s0, d.c1, r.r1x7);
                    glf::acc_mac(s1, d.c0, r.r1);
                    glf::acc_mac(s1, d.c1, r.r0);
                    f[h][j].c0 = glf::canon(glf::add_c(glf::acc_reduce(s0), a0.c0));
                    f[h][j].c1 = glf::canon(glf::add_c(glf::acc_reduce(s1), a0.c1));
                }
            }
            ulonglong2* o = (ulonglong2*)ptrs.out[j] + 2 * p;
            o[0] = make_ulonglong2(f[0][j].c0, f[0][j].c1);
            o[1] = make_ulonglong2(f[1][j].c0, f[1][j].c1);
        }
        sample_pair<Ops, K, false>(acc, f[0], f[1]);
    }
    publish<Ops, K>(acc, rs, out);
}

// Rounds >= 1 over BN254.
template <int K, int MINB = 1>
__global__ void __launch_bounds__(kThreads, MINB)
    v2_fold_eval_fr(V2Ptrs<K> ptrs, frw::FixedMul rk, uint64_t n_pairs, ReduceScratch<FrFam> rs, Fr* out) {
    typedef OpsFr Ops;
    Fr acc[K + 1];
#pragma unroll
    for (int x = 0; x <= K; x++) acc[x] = fr_zero();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n_pairs; p += stride) {
        Fr f[2][K];
#pragma unroll
        for (int j = 0; j < K; j++) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const Fr a0 = FrFam::load(ptrs.in[j], DPB_FR, 4 * p + 2 * h);
                const Fr a1 = FrFam::load(ptrs.in[j], DPB_FR, 4 * p + 2 * h + 1);
                f[h][j] = fr_add(a0, fr_mul_fixed(rk, fr_sub(a1, a0)));  // the challenge is fixed for the launch
                FrFam::store(ptrs.out[j], 2 * p + h, f[h][j]);
            }
        }
        sample_pair<Ops, K, false>(acc, f[0], f[1]);
    }
    publish<Ops, K>(acc, rs, out);
}

// ---- host: samples -> evaluations at 0..=K -----------------------------------
// raw[] as laid out above; claim = P(0) + P(1) when P(1) was not sampled.
// Also returns the coefficients (low to high) so the next round's claim can be
// evaluated.
template <class F>
inline void samples_to_evals(int K, const typename F::E* raw, bool have_p1, const typename F::E& claim,
                             typename F::E* evals, typename F::E* coeffs) {
    typedef typename F::E E;
    const E p0 = raw[0];
    const E p1 = have_p1 ? raw[1] : F::sub(claim, p0);
    const E lead = (K & 1) ? F::neg(raw[2]) : raw[2];
    const E two = F::from_u64(2);
    static const E inv2 = F::inv(F::from_u64(2)), inv6 = F::inv(F::from_u64(6));  // inversions are slow: once per process
    E c[5];
    for (int i = 0; i < 5; i++) c[i] = F::zero();
    c[0] = p0;
    c[K] = lead;
    if (K == 2) {
        c[1] = F::sub(F::sub(p1, p0), lead);
    } else if (K == 3) {
        // p(1) + p(-1) = 2 (c0 + c2);  p(1) = c0 + c1 + c2 + c3
        const E pm1 = raw[3];
        c[2] = F::sub(F::mul(F::add(p1, pm1), inv2), p0);
        c[1] = F::sub(F::sub(F::sub(p1, p0), c[2]), lead);
    } else {  // K == 4
        const E pm1 = raw[3], p2 = raw[4];
        c[2] = F::sub(F::sub(F::mul(F::add(p1, pm1), inv2), p0), lead);
        const E s = F::mul(F::sub(p1, pm1), inv2);  // c1 + c3
        // p(2) = c0 + 2 c1 + 4 c2 + 8 c3 + 16 c4  ->  6 c3 = p(2) - c0 - 4 c2 - 16 c4 - 2 s
        E t = F::sub(p2, p0);
        t = F::sub(t, F::mul(F::from_u64(4), c[2]));
        t = F::sub(t, F::mul(F::from_u64(16), lead));
        t = F::sub(t, F::mul(two, s));
        c[3] = F::mul(t, inv6);
        c[1] = F::sub(s, c[3]);
    }
    for (int x = 0; x <= K; x++) {
        const E X = F::from_u64((uint64_t)x);
        E v = c[K];
        for (int i = K - 1; i >= 0; i--) v = F::add(F::mul(v, X), c[i]);
        evals[x] = v;
    }
    evals[0] = p0;
    evals[1] = p1;
    for (int i = 0; i <= K; i++) coeffs[i] = c[i];
}

template <class F>
inline typename F::E eval_coeffs(int K, const typename F::E* c, const typename F::E& x) {
    typename F::E v = c[K];
    for (int i = K - 1; i >= 0; i--) v = F::add(F::mul(v, x), c[i]);
    return v;
}

}  // namespace dpb
