// Goldilocks fused rounds with asynchronous staging of the inputs.
//
// The arithmetic is that of fused_v2.cuh.  What changes is how table entries
// reach the registers: every thread streams the 16-byte chunks of its NEXT
// items from global to shared memory with cp.async while it works on the
// current item, so the integer pipes do not idle on HBM latency and the data in
// flight costs no registers.  Each thread only ever reads back the chunks it
// copied itself (chunk c of thread t lives at [c][t], stride 16 B across the
// warp: conflict-free 128-bit shared loads), so no block-wide barrier is
// needed: cp.async.wait_group orders a thread's own copies.
#pragma once
#include <type_traits>

#include "fused_v2.cuh"

namespace dpb {

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    const uint32_t s = (uint32_t)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

constexpr int kStageThreads = 256;

// Per-thread staging ring: STAGES slots of K tables x CH chunks of 16 bytes.
template <int K, int CH, int STAGES>
struct Stager {
    uint4* base;  // this block's shared memory
    __device__ __forceinline__ uint4* slot(int s, int j, int c) const {
        return base + (((size_t)s * K + j) * CH + c) * kStageThreads + threadIdx.x;
    }
    // item `p` of every table: CH consecutive chunks starting at chunk p * CH
    __device__ __forceinline__ void issue(int s, const void* const (&in)[K], uint64_t p, bool valid) const {
        if (valid) {
#pragma unroll
            for (int j = 0; j < K; j++) {
                const uint4* g = (const uint4*)in[j] + p * CH;
#pragma unroll
                for (int c = 0; c < CH; c++) cp_async16(slot(s, j, c), g + c);
            }
        }
        cp_async_commit();  // an empty group keeps the group count uniform
    }
    __device__ __forceinline__ uint4 get(int s, int j, int c) const { return *slot(s, j, c); }
    static constexpr size_t bytes() { return (size_t)STAGES * K * CH * kStageThreads * sizeof(uint4); }
};

__device__ __forceinline__ void fold_base4(const uint64_t (&a)[4], const GlChal& r, glf::L2 (&f)[2]) {
#pragma unroll
    for (int h = 0; h < 2; h++) {
        const uint64_t d = glf::sub_c(a[2 * h + 1], a[2 * h]);
        f[h].c0 = glf::canon(glf::add_c(glf::mul(r.r0, d), a[2 * h]));
        f[h].c1 = glf::canon(glf::mul(r.r1, d));
    }
}
__device__ __forceinline__ glf::L2 fold_ext2(const glf::L2& a0, const glf::L2& a1, const GlChal& r) {
    const glf::L2 d = OpsGlExt::sub_c(a1, a0);
    glf::Acc160 s0 = glf::acc_zero(), s1 = glf::acc_zero();
    glf::acc_mac(s0, d.c0, r.r0);
    glf::acc_mac(s0, d.c1, r.r1x7);
    glf::acc_mac(s1, d.c0, r.r1);
    glf::acc_mac(s1, d.c1, r.r0);
    glf::L2 f;
    f.c0 = glf::canon(glf::add_c(glf::acc_reduce(s0), a0.c0));
    f.c1 = glf::canon(glf::add_c(glf::acc_reduce(s1), a0.c1));
    return f;
}
__device__ __forceinline__ glf::L2 as_l2(const uint4& v) {
    glf::L2 r;
    r.c0 = (uint64_t)v.x | ((uint64_t)v.y << 32);
    r.c1 = (uint64_t)v.z | ((uint64_t)v.w << 32);
    return r;
}

// Round 0 over Goldilocks, staged.  BASE: base-field tables.
template <int K, bool BASE, int STAGES>
__global__ void __launch_bounds__(kStageThreads)
    v3_eval0_gl(V2Ptrs<K> ptrs, uint64_t n_pairs, ReduceScratch<GlFam> rs, Gl2* out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int CH = BASE ? 1 : 2;
    Stager<K, CH, STAGES> st;
    st.base = (uint4*)smem_raw;
    typedef typename std::conditional<BASE, OpsGlBase, OpsGlExt>::type Ops;
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
        typename Ops::T f0[K], f1[K];
#pragma unroll
        for (int j = 0; j < K; j++) {
            if constexpr (BASE) {
                const uint4 v = st.get(cur, j, 0);
                f0[j] = (uint64_t)v.x | ((uint64_t)v.y << 32);
                f1[j] = (uint64_t)v.z | ((uint64_t)v.w << 32);
            } else {
                f0[j] = as_l2(st.get(cur, j, 0));
                f1[j] = as_l2(st.get(cur, j, 1));
            }
        }
        sample_pair<Ops, K, true>(acc, f0, f1);
        if (++cur == STAGES) cur = 0;
    }
    cp_async_wait<0>();
    publish<Ops, K>(acc, rs, out);
}

// Rounds >= 1 over Goldilocks, staged.  Tables are folded, stored and fed to
// the sampler one at a time.
template <int K, bool BASE_IN, int STAGES, int MINB>
__global__ void __launch_bounds__(kStageThreads, MINB)
    v3_fold_eval_gl(V2Ptrs<K> ptrs, GlChal r, uint64_t n_pairs, ReduceScratch<GlFam> rs, Gl2* out) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    constexpr int CH = BASE_IN ? 2 : 4;
    Stager<K, CH, STAGES> st;
    st.base = (uint4*)smem_raw;
    typedef OpsGlExt2 Ops;
    typedef glf::L2 T;
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
            T f[2];
            if constexpr (BASE_IN) {
                const uint4 u = st.get(cur, j, 0), v = st.get(cur, j, 1);
                const uint64_t a[4] = {(uint64_t)u.x | ((uint64_t)u.y << 32), (uint64_t)u.z | ((uint64_t)u.w << 32),
                                       (uint64_t)v.x | ((uint64_t)v.y << 32), (uint64_t)v.z | ((uint64_t)v.w << 32)};
                fold_base4(a, r, f);
            } else {
                f[0] = fold_ext2(as_l2(st.get(cur, j, 0)), as_l2(st.get(cur, j, 1)), r);
                f[1] = fold_ext2(as_l2(st.get(cur, j, 2)), as_l2(st.get(cur, j, 3)), r);
            }
            ulonglong2* o = (ulonglong2*)ptrs.out[j] + 2 * p;
            o[0] = make_ulonglong2(f[0].c0, f[0].c1);
            o[1] = make_ulonglong2(f[1].c0, f[1].c1);
            smp.template absorb<j>(acc, f[0], f[1]);
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
