// Product-sumcheck rounds over 32-bit integer tables (DPB_FR_I32), BN254 family.
//
// The tensors and lookup columns the reference proves about are small signed
// integers that only become field elements at the prover's door
// (Tensor::to_field, zkml/src/layers/einsum/prove.rs:66-91).  Over BN254 every
// field product costs 128 wide multiply-adds, and the first two rounds of a
// sumcheck carry about two thirds of its products; with the integers kept as
// they are, those rounds need almost none:
//
//  * round 0: the samples P(0), P(1), prod (f(0) - f(1)) and P(-1) of a product
//    of K <= 3 tables are products of integers below 2^34 in magnitude, i.e.
//    102-bit integers.  A thread adds them up exactly in 128-bit registers and
//    converts each sum to a field element once, at the end.  The round reads
//    4 bytes per entry and is bound by HBM, not by the multiplier.
//  * round 1: the fold  a0 + r (a1 - a0)  of two integers by the challenge is
//    |a0| * (+-R) + |a1 - a0| * (+-r R)  as integers mod p, two rows of eight
//    words times one word each: 16 wide multiply-adds and the two-word
//    reduction of frw::mul_fixed instead of a full product.  The samples are
//    then taken from the folded field elements as in every later round.
//
// Sums of exact integers reduced mod p equal the sums of the reduced terms, so
// the round messages are bit-identical to those over the converted tables.
#pragma once
#include "fused_v2.cuh"

namespace dpb {

// |x| < 2^127 as a field element (Montgomery form)
__device__ __forceinline__ Fr fr_from_i128(__int128 x) {
    const bool neg = x < 0;
    const unsigned __int128 mag = neg ? (unsigned __int128)0 - (unsigned __int128)x : (unsigned __int128)x;
    Fr a;
    a.l[0] = (uint64_t)mag;
    a.l[1] = (uint64_t)(mag >> 64);
    a.l[2] = a.l[3] = 0;
    a = fr_to_mont(a);
    return neg ? fr_neg(a) : a;
}

// Round 0: samples of the product of K int32 tables, in the slots of fused_v2.cuh.
template <int K>
__global__ void __launch_bounds__(kThreads)
    v2_eval0_fr_i32(V2Ptrs<K> ptrs, uint64_t n_pairs, ReduceScratch<FrFam> rs, Fr* out) {
    static_assert(K == 2 || K == 3, "products of two or three integer tables");
    __int128 acc[4] = {0, 0, 0, 0};
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n_pairs; p += stride) {
        __int128 p0 = 1, p1 = 1, pinf = 1, pm1 = 1;
#pragma unroll
        for (int j = 0; j < K; j++) {
            const int2 v = ((const int2*)ptrs.in[j])[p];
            const int64_t f0 = v.x, f1 = v.y, e = f0 - f1, m = e + f0;  // f(0), f(1), f(0) - f(1), f(-1)
            p0 *= f0;
            p1 *= f1;
            pinf *= e;
            pm1 *= m;
        }
        acc[0] += p0;
        acc[1] += p1;
        acc[2] += pinf;
        if (K >= 3) acc[3] += pm1;
    }
    Fr wide[K + 1];
#pragma unroll
    for (int x = 0; x <= K; x++) wide[x] = fr_from_i128(acc[x]);
    grid_sum_publish<FrFam, K + 1>(wide, rs, out);
}

// What the integer fold needs of the challenge: the rows  +-R * 2^64  and  +-(r R) * 2^64  mod p (the factor 2^64
// pays for the two reduction words), words little-endian.
struct IntFoldKey {
    uint32_t one_pos[8], one_neg[8], r_pos[8], r_neg[8];
};

// a0 + r (a1 - a0) for integers a0, a1 of 32 bits
__device__ __forceinline__ Fr fold_i32(const IntFoldKey& k, int32_t a0, int32_t a1) {
    const int64_t d = (int64_t)a1 - (int64_t)a0;  // below 2^32 in magnitude
    const uint32_t ma = a0 < 0 ? (uint32_t)0 - (uint32_t)a0 : (uint32_t)a0;
    const uint32_t md = d < 0 ? (uint32_t)(-d) : (uint32_t)d;
    return frw::to_fr(frw::lin2_rows(ma, a0 < 0 ? k.one_neg : k.one_pos, md, d < 0 ? k.r_neg : k.r_pos));
}

// Round 1 over int32 tables: fold by the challenge (integers in, field elements out), then the usual samples.
template <int K, int MINB = 1>
__global__ void __launch_bounds__(kThreads, MINB)
    v2_fold_eval_fr_i32(V2Ptrs<K> ptrs, IntFoldKey key, uint64_t n_pairs, ReduceScratch<FrFam> rs, Fr* out) {
    typedef OpsFr Ops;
    __shared__ IntFoldKey k;
    if (threadIdx.x < 32) ((uint32_t*)&k)[threadIdx.x] = ((const uint32_t*)&key)[threadIdx.x];
    __syncthreads();
    Fr acc[K + 1];
#pragma unroll
    for (int x = 0; x <= K; x++) acc[x] = fr_zero();
    const uint64_t stride = (uint64_t)gridDim.x * blockDim.x;
    for (uint64_t p = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; p < n_pairs; p += stride) {
        Fr f[2][K];
#pragma unroll
        for (int j = 0; j < K; j++) {
            const int4 a = ((const int4*)ptrs.in[j])[p];  // entries 4p .. 4p+3
            f[0][j] = fold_i32(k, a.x, a.y);
            f[1][j] = fold_i32(k, a.z, a.w);
            FrFam::store(ptrs.out[j], 2 * p, f[0][j]);
            FrFam::store(ptrs.out[j], 2 * p + 1, f[1][j]);
        }
        sample_pair<Ops, K, false>(acc, f[0], f[1]);
    }
    publish<Ops, K>(acc, rs, out);
}

// Host: the four rows for the challenge r (Montgomery form).  c * 2^64 as an integer mod p is the Montgomery
// product of c * R (= c times R^2, reduced) with the plain integer 2^64.
inline void int_fold_key(const Fr& r, IntFoldKey& out) {
    Fr two64;
    two64.l[0] = 0;
    two64.l[1] = 1;
    two64.l[2] = two64.l[3] = 0;
    auto row = [&](const Fr& c, uint32_t* w) {
        const Fr v = fr_mul(fr_mul(c, fr_rr()), two64);
        for (int i = 0; i < 4; i++) {
            w[2 * i] = (uint32_t)v.l[i];
            w[2 * i + 1] = (uint32_t)(v.l[i] >> 32);
        }
    };
    row(fr_one(), out.one_pos);
    row(fr_neg(fr_one()), out.one_neg);
    row(r, out.r_pos);
    row(fr_neg(r), out.r_neg);
}

}  // namespace dpb
