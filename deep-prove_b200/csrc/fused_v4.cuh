// Goldilocks fused rounds on the word-level arithmetic of gl_words.cuh.
// Same staging (cp.async ring per thread), sampling (0, 1, inf, -1, 2) and
// table-at-a-time streaming as fused_v3.cuh; only the arithmetic differs.
#pragma once
#include "fused_v3.cuh"
#include "gl_words.cuh"

namespace dpb {

struct OpsWBase {
    typedef GlFam F;
    typedef glw::W T;
    typedef glw::A8 Acc;
    __device__ __forceinline__ static T sub_c(const T& a, const T& c) { return glw::sub_c(a, c); }
    __device__ __forceinline__ static T add_c(const T& a, const T& c) { return glw::add_c(a, c); }
    __device__ __forceinline__ static T mul(const T& a, const T& b) { return glw::mul(a, b); }
    __device__ __forceinline__ static Acc acc_zero() { return glw::acc_zero(); }
    __device__ __forceinline__ static void mac(Acc& acc, const T& a, const T& b) { glw::acc_mac(acc, a, b); }
    __device__ __forceinline__ static Gl2 finish(const Acc& acc) {
        return gl2_make(glw::to_u64(glw::canon(glw::acc_reduce(acc))), 0);
    }
};

struct OpsWExt {
    typedef GlFam F;
    typedef glw::W2 T;
    struct Acc {
        glw::A8 s0, s1;
    };
    __device__ __forceinline__ static T sub_c(const T& a, const T& c) { return glw::sub_c(a, c); }
    __device__ __forceinline__ static T add_c(const T& a, const T& c) { return glw::add_c(a, c); }
    __device__ __forceinline__ static T mul(const T& a, const T& b) { return glw::mul(a, b); }
    __device__ __forceinline__ static Acc acc_zero() {
        Acc a;
        a.s0 = a.s1 = glw::acc_zero();
        return a;
    }
    __device__ __forceinline__ static void mac(Acc& acc, const T& a, const T& b) {
        glw::acc_mac(acc.s0, a.c0, b.c0);
        glw::acc_mac(acc.s0, glw::mul7(a.c1), b.c1);
        glw::acc_mac(acc.s1, a.c0, b.c1);
        glw::acc_mac(acc.s1, a.c1, b.c0);
    }
    __device__ __forceinline__ static Gl2 finish(const Acc& acc) {
        return gl2_make(glw::to_u64(glw::canon(glw::acc_reduce(acc.s0))), glw::to_u64(glw::canon(glw::acc_reduce(acc.s1))));
    }
};

__device__ __forceinline__ glw::W2 as_w2(const uint4& v) {
    glw::W2 r;
    r.c0 = glw::make_w(v.x, v.y);
    r.c1 = glw::make_w(v.z, v.w);
    return r;
}

// Round 0, staged.
template <int K, bool BASE, int STAGES, int MINB>
__global__ void __launch_bounds__(kStageThreads, MINB)
    v4_eval0_gl(V2Ptrs<K> ptrs, uint64_t n_pairs, ReduceScratch<GlFam> rs, Gl2* out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int CH = BASE ? 1 : 2;
    Stager<K, CH, STAGES> st;
    st.base = (uint4*)smem_raw;
    typedef typename std::conditional<BASE, OpsWBase, OpsWExt>::type Ops;
    typename Ops::Acc acc[K + 1];
#pragma unroll
    for (int x = 0; x <= K; x++) acc[x] = Ops::acc_zero();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t p0 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) st.issue(s, ptrs.in, p0 + s * stride, p0 + s * stride < n_pairs);
    int cur = 0;
    for (uint64_t p = p0; p < n_pairs; p += stride) {
        const uint64_t pn = p + (uint64_t)(STAGES - 1) * stride;
        int nxt = cur + STAGES - 1;
        if (nxt >= STAGES) nxt -= STAGES;
        st.issue(nxt, ptrs.in, pn, pn < n_pairs);
        cp_async_wait<STAGES - 1>();
        Sampler<Ops, K, true> smp;
        auto one_table = [&](auto jc) {
            constexpr int j = decltype(jc)::value;
            if constexpr (BASE) {
                const uint4 v = st.get(cur, j, 0);
                smp.template absorb<j>(acc, glw::make_w(v.x, v.y), glw::make_w(v.z, v.w));
            } else {
                smp.template absorb<j>(acc, as_w2(st.get(cur, j, 0)), as_w2(st.get(cur, j, 1)));
            }
        };
        one_table(std::integral_constant<int, 0>());
        one_table(std::integral_constant<int, 1>());
        if constexpr (K >= 3) one_table(std::integral_constant<int, 2>());
        if constexpr (K >= 4) one_table(std::integral_constant<int, 3>());
        if (++cur == STAGES) cur = 0;
    }
    cp_async_wait<0>();
    publish<Ops, K>(acc, rs, out);
}

// Rounds >= 1, staged: fold, store and sample one table at a time.
template <int K, bool BASE_IN, int STAGES, int MINB>
__global__ void __launch_bounds__(kStageThreads, MINB)
    v4_fold_eval_gl(V2Ptrs<K> ptrs, glw::Chal r, uint64_t n_pairs, ReduceScratch<GlFam> rs, Gl2* out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int CH = BASE_IN ? 2 : 4;
    Stager<K, CH, STAGES> st;
    st.base = (uint4*)smem_raw;
    typedef OpsWExt Ops;
    typedef glw::W2 T;
    Ops::Acc acc[K + 1];
#pragma unroll
    for (int x = 0; x <= K; x++) acc[x] = Ops::acc_zero();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    const uint64_t p0 = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) st.issue(s, ptrs.in, p0 + s * stride, p0 + s * stride < n_pairs);
    int cur = 0;
    for (uint64_t p = p0; p < n_pairs; p += stride) {
        const uint64_t pn = p + (uint64_t)(STAGES - 1) * stride;
        int nxt = cur + STAGES - 1;
        if (nxt >= STAGES) nxt -= STAGES;
        st.issue(nxt, ptrs.in, pn, pn < n_pairs);
        cp_async_wait<STAGES - 1>();
        Sampler<Ops, K, false> smp;
        auto one_table = [&](auto jc) {
            constexpr int j = decltype(jc)::value;
            T f0, f1;
            if constexpr (BASE_IN) {
                const uint4 u = st.get(cur, j, 0), v = st.get(cur, j, 1);
                f0 = glw::fold_base(glw::make_w(u.x, u.y), glw::make_w(u.z, u.w), r);
                f1 = glw::fold_base(glw::make_w(v.x, v.y), glw::make_w(v.z, v.w), r);
            } else {
                f0 = glw::fold_ext(as_w2(st.get(cur, j, 0)), as_w2(st.get(cur, j, 1)), r);
                f1 = glw::fold_ext(as_w2(st.get(cur, j, 2)), as_w2(st.get(cur, j, 3)), r);
            }
            uint4* o = (uint4*)ptrs.out[j] + 2 * p;
            o[0] = make_uint4(f0.c0.lo, f0.c0.hi, f0.c1.lo, f0.c1.hi);
            o[1] = make_uint4(f1.c0.lo, f1.c0.hi, f1.c1.lo, f1.c1.hi);
            smp.template absorb<j>(acc, f0, f1);
        };
        one_table(std::integral_constant<int, 0>());
        one_table(std::integral_constant<int, 1>());
        if constexpr (K >= 3) one_table(std::integral_constant<int, 2>());
        if constexpr (K >= 4) one_table(std::integral_constant<int, 3>());
        if (++cur == STAGES) cur = 0;
    }
    cp_async_wait<0>();
    publish<Ops, K>(acc, rs, out);
}

}  // namespace dpb
