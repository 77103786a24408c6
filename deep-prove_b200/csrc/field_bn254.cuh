// BN254 scalar field Fr (the field the reference prover is instantiated on,
// zkml/src/lookup/logup_gkr/mod.rs:22 `type F = ark_bn254::Fr`), host and device.
//
// Storage form: four 64-bit little-endian limbs holding a*R mod r with
// R = 2^256 (Montgomery form), the in-memory form of arkworks' 4-limb
// Montgomery backend. Canonical form (plain integer < r, 32 bytes LE) is what
// ark_serialize writes; conversions are provided.
//
// r = 21888242871839275222246405745257275088548364400416034343698204186575808495617
#pragma once
#include <cstdint>

#include "field_gl.cuh"  // DPB_HD, mul64wide

namespace dpb {

struct alignas(16) Fr {
    uint64_t l[4];
};

// Constants as macros so both host and device code inline them as immediates.
#define DPB_FR_P0 0x43e1f593f0000001ULL
#define DPB_FR_P1 0x2833e84879b97091ULL
#define DPB_FR_P2 0xb85045b68181585dULL
#define DPB_FR_P3 0x30644e72e131a029ULL
#define DPB_FR_INV 0xc2e1f593efffffffULL  // -r^{-1} mod 2^64
// R mod r (Montgomery form of 1)
#define DPB_FR_R0 0xac96341c4ffffffbULL
#define DPB_FR_R1 0x36fc76959f60cd29ULL
#define DPB_FR_R2_ 0x666ea36f7879462eULL
#define DPB_FR_R3 0x0e0a77c19a07df2fULL
// R^2 mod r
#define DPB_FR_RR0 0x1bb8e645ae216da7ULL
#define DPB_FR_RR1 0x53fe3ab1e35c59e3ULL
#define DPB_FR_RR2 0x8c49833d53bb8085ULL
#define DPB_FR_RR3 0x0216d0b17f4e44a5ULL

}  // namespace dpb
#if defined(__CUDACC__)
#include "fr_words.cuh"
#endif
namespace dpb {

DPB_HD Fr fr_zero() {
    Fr r;
    r.l[0] = r.l[1] = r.l[2] = r.l[3] = 0;
    return r;
}
DPB_HD Fr fr_one() {
    Fr r;
    r.l[0] = DPB_FR_R0;
    r.l[1] = DPB_FR_R1;
    r.l[2] = DPB_FR_R2_;
    r.l[3] = DPB_FR_R3;
    return r;
}
DPB_HD Fr fr_rr() {
    Fr r;
    r.l[0] = DPB_FR_RR0;
    r.l[1] = DPB_FR_RR1;
    r.l[2] = DPB_FR_RR2;
    r.l[3] = DPB_FR_RR3;
    return r;
}
DPB_HD bool fr_eq(const Fr& a, const Fr& b) {
    return a.l[0] == b.l[0] && a.l[1] == b.l[1] && a.l[2] == b.l[2] && a.l[3] == b.l[3];
}
DPB_HD bool fr_is_zero(const Fr& a) { return (a.l[0] | a.l[1] | a.l[2] | a.l[3]) == 0; }

// a + b + carry_in -> sum, carry_out
DPB_HD uint64_t adc(uint64_t a, uint64_t b, uint64_t& carry) {
    uint64_t s = a + b;
    uint64_t c1 = s < a;
    uint64_t t = s + carry;
    uint64_t c2 = t < s;
    carry = c1 + c2;
    return t;
}
// a - b - borrow_in -> diff, borrow_out
DPB_HD uint64_t sbb(uint64_t a, uint64_t b, uint64_t& borrow) {
    uint64_t d = a - b;
    uint64_t b1 = a < b;
    uint64_t t = d - borrow;
    uint64_t b2 = d < borrow;
    borrow = b1 + b2;
    return t;
}
// acc + x*y + carry -> low 64 bits; carry <- high 64 bits
DPB_HD uint64_t mac(uint64_t acc, uint64_t x, uint64_t y, uint64_t& carry) {
    uint64_t lo, hi;
    mul64wide(x, y, lo, hi);
    uint64_t s = lo + acc;
    hi += (s < lo);
    uint64_t t = s + carry;
    hi += (t < s);
    carry = hi;
    return t;
}

// Conditionally subtract r so the result is < r (input < 2r).
DPB_HD Fr fr_reduce_once(const Fr& a) {
    uint64_t bw = 0;
    Fr d;
    d.l[0] = sbb(a.l[0], DPB_FR_P0, bw);
    d.l[1] = sbb(a.l[1], DPB_FR_P1, bw);
    d.l[2] = sbb(a.l[2], DPB_FR_P2, bw);
    d.l[3] = sbb(a.l[3], DPB_FR_P3, bw);
    return bw ? a : d;
}

DPB_HD Fr fr_add_portable(const Fr& a, const Fr& b) {
    uint64_t c = 0;
    Fr s;
    s.l[0] = adc(a.l[0], b.l[0], c);
    s.l[1] = adc(a.l[1], b.l[1], c);
    s.l[2] = adc(a.l[2], b.l[2], c);
    s.l[3] = adc(a.l[3], b.l[3], c);  // r < 2^254: no carry out
    return fr_reduce_once(s);
}

DPB_HD Fr fr_sub_portable(const Fr& a, const Fr& b) {
    uint64_t bw = 0;
    Fr d;
    d.l[0] = sbb(a.l[0], b.l[0], bw);
    d.l[1] = sbb(a.l[1], b.l[1], bw);
    d.l[2] = sbb(a.l[2], b.l[2], bw);
    d.l[3] = sbb(a.l[3], b.l[3], bw);
    if (bw) {
        uint64_t c = 0;
        d.l[0] = adc(d.l[0], DPB_FR_P0, c);
        d.l[1] = adc(d.l[1], DPB_FR_P1, c);
        d.l[2] = adc(d.l[2], DPB_FR_P2, c);
        d.l[3] = adc(d.l[3], DPB_FR_P3, c);
    }
    return d;
}

// Device code uses the 32-bit word routines of fr_words.cuh; host code the
// portable 64-bit limb ones above.  Same values either way.
DPB_HD Fr fr_add(const Fr& a, const Fr& b) {
#if defined(__CUDA_ARCH__)
    return frw::to_fr(frw::add(frw::from_fr(a), frw::from_fr(b)));
#else
    return fr_add_portable(a, b);
#endif
}
DPB_HD Fr fr_sub(const Fr& a, const Fr& b) {
#if defined(__CUDA_ARCH__)
    return frw::to_fr(frw::sub(frw::from_fr(a), frw::from_fr(b)));
#else
    return fr_sub_portable(a, b);
#endif
}

DPB_HD Fr fr_neg(const Fr& a) { return fr_is_zero(a) ? a : fr_sub(fr_zero(), a); }

// Montgomery product a*b/R mod r (coarsely integrated operand scanning; the
// top limb of r leaves two spare bits so the running sum fits five limbs).
DPB_HD Fr fr_mul_portable(const Fr& a, const Fr& b) {
    const uint64_t p[4] = {DPB_FR_P0, DPB_FR_P1, DPB_FR_P2, DPB_FR_P3};
    uint64_t t0 = 0, t1 = 0, t2 = 0, t3 = 0, t4 = 0;
#if defined(__CUDA_ARCH__)
#pragma unroll
#endif
    for (int i = 0; i < 4; i++) {
        uint64_t c = 0;
        uint64_t bi = b.l[i];
        t0 = mac(t0, a.l[0], bi, c);
        t1 = mac(t1, a.l[1], bi, c);
        t2 = mac(t2, a.l[2], bi, c);
        t3 = mac(t3, a.l[3], bi, c);
        t4 += c;
        uint64_t m = t0 * DPB_FR_INV;
        c = 0;
        (void)mac(t0, m, p[0], c);
        t0 = mac(t1, m, p[1], c);
        t1 = mac(t2, m, p[2], c);
        t2 = mac(t3, m, p[3], c);
        t3 = t4 + c;
        t4 = 0;
    }
    Fr r;
    r.l[0] = t0;
    r.l[1] = t1;
    r.l[2] = t2;
    r.l[3] = t3;
    return fr_reduce_once(r);
}

DPB_HD Fr fr_mul(const Fr& a, const Fr& b) {
#if defined(__CUDA_ARCH__)
    return frw::to_fr(frw::mul(frw::from_fr(a), frw::from_fr(b)));
#else
    return fr_mul_portable(a, b);
#endif
}

#if defined(__CUDACC__)
// a * c for the multiplicand c whose constants `k` were made by fr_fixed_table (device only)
__device__ __forceinline__ Fr fr_mul_fixed(const frw::FixedMul& k, const Fr& a) {
    return frw::to_fr(frw::mul_fixed(frw::from_fr(a), k));
}
// Sum of integer * field-element products, lazily: see frw::IntAcc.  `w` in Montgomery form; the result is the
// Montgomery form of sum x_o * w_o.  A negative x adds |x| * (r - w).
struct FrIntAcc {
    frw::IntAcc a;
};
__device__ __forceinline__ FrIntAcc fr_intacc_zero() {
    FrIntAcc r;
    r.a = frw::intacc_zero();
    return r;
}
__device__ __forceinline__ void fr_intacc_mac(FrIntAcc& acc, const Fr& w, int64_t x) {
    const uint64_t mag = x < 0 ? (uint64_t)0 - (uint64_t)x : (uint64_t)x;
    frw::intacc_mac(acc.a, frw::from_fr(x < 0 ? fr_neg(w) : w), mag);
}
__device__ __forceinline__ Fr fr_intacc_finish(const FrIntAcc& acc) {
    // S = lo + 2^256 hi: lo * R / R = lo mod r, hi * R^2 / R = hi * 2^256 mod r (inputs below 2^256 are fine: the
    // other factor is below r, so the Montgomery product stays below 2 r before its last subtraction)
    frw::F8 lo, hi;
    frw::intacc_split(acc.a, lo, hi);
    const Fr a = frw::to_fr(frw::mul(lo, frw::from_fr(fr_one())));
    const Fr b = frw::to_fr(frw::mul(hi, frw::from_fr(fr_rr())));
    return fr_add(a, b);
}

// Integer -> Montgomery form without a full product: |x| = lo + 2^32 hi, and x R = lo * (+-R) + hi * (+-2^32 R)
// mod r; the rows below hold those four constants times 2^64 (what frw::lin2_rows divides out again).
static __device__ __constant__ const uint32_t kIntRowOnePos[8] = {0x7c5fb586u, 0xb4c6edf9u, 0xbfeb93beu, 0x708c8d50u,
                                                                  0x04f7e0efu, 0x9ffd1de4u, 0x9a392866u, 0x215b02acu};
static __device__ __constant__ const uint32_t kIntRowOneNeg[8] = {0x73a04a7bu, 0x8f1b079au, 0xb9cddcd2u, 0xb7a75af7u,
                                                                  0x7c89776du, 0x185327d2u, 0x46f877c3u, 0x0f094bc6u};
static __device__ __constant__ const uint32_t kIntRowHiPos[8] = {0xaf8b5a7au, 0x54c81065u, 0x97aa45f6u, 0x2b82a1efu,
                                                                 0x330a5a6du, 0xbe492693u, 0x8229aff4u, 0x1847e486u};
static __device__ __constant__ const uint32_t kIntRowHiNeg[8] = {0x4074a587u, 0xef19e52eu, 0xe20f2a9au, 0xfcb14658u,
                                                                 0x4e76fdefu, 0xfa071f23u, 0x5f07f034u, 0x181c69ecu};
__device__ __forceinline__ Fr fr_from_int_rows(int64_t x) {
    const uint64_t mag = x < 0 ? (uint64_t)0 - (uint64_t)x : (uint64_t)x;
    const bool neg = x < 0;
    return frw::to_fr(frw::lin2_rows((uint32_t)mag, neg ? kIntRowOneNeg : kIntRowOnePos, (uint32_t)(mag >> 32),
                                     neg ? kIntRowHiNeg : kIntRowHiPos));
}

// 2^(32 i + 64) mod r as a plain integer, i = 0..7
DPB_HD Fr fr_fixed_power(int i) {
    Fr x;
    x.l[0] = x.l[1] = x.l[2] = x.l[3] = 0;
    const int e = 32 * i + 64;
    if (e < 254) {
        x.l[e / 64] = 1ull << (e % 64);
    } else if (e == 256) {
        x = fr_one();  // 2^256 mod r
    } else {  // 2^288 mod r
        x.l[0] = 0x93e7886515b8b9daULL;
        x.l[1] = 0x16df2426b05ea154ULL;
        x.l[2] = 0x1271b743302ab839ULL;
        x.l[3] = 0x06bc037eec6c226eULL;
    }
    return x;
}
// Constants of frw::mul_fixed for the multiplicand c (Montgomery form): row i is
// c * 2^(32 i + 64) / 2^256 mod r (a Montgomery product of c with the plain power).
DPB_HD void fr_fixed_row(const Fr& c, int i, uint32_t* row) {
    const Fr ci = fr_mul(c, fr_fixed_power(i));
    for (int w = 0; w < 4; w++) {
        row[2 * w] = (uint32_t)ci.l[w];
        row[2 * w + 1] = (uint32_t)(ci.l[w] >> 32);
    }
}
inline void fr_fixed_table(const Fr& c, frw::FixedMul& out) {
    for (int i = 0; i < 8; i++) fr_fixed_row(c, i, out.c[i]);
}
#endif

DPB_HD Fr fr_sqr(const Fr& a) { return fr_mul(a, a); }
DPB_HD Fr fr_double(const Fr& a) { return fr_add(a, a); }

// canonical integer (< r) -> Montgomery form
DPB_HD Fr fr_to_mont(const Fr& a) { return fr_mul(a, fr_rr()); }
// Montgomery form -> canonical integer
DPB_HD Fr fr_from_mont(const Fr& a) {
    Fr one;
    one.l[0] = 1;
    one.l[1] = one.l[2] = one.l[3] = 0;
    return fr_mul(a, one);
}
// Signed 64-bit integer -> field element; negative x maps to r - |x|, the
// rule of the reference's Element -> field conversion
// (zkml/src/quantization/mod.rs:220-267).
DPB_HD Fr fr_from_i64(int64_t x) {
    Fr a;
    uint64_t mag = x < 0 ? (uint64_t)0 - (uint64_t)x : (uint64_t)x;
    a.l[0] = mag;
    a.l[1] = a.l[2] = a.l[3] = 0;
    a = fr_to_mont(a);
    return x < 0 ? fr_neg(a) : a;
}
DPB_HD Fr fr_from_u64(uint64_t x) {
    Fr a;
    a.l[0] = x;
    a.l[1] = a.l[2] = a.l[3] = 0;
    return fr_to_mont(a);
}

inline Fr fr_pow(Fr a, const uint64_t e[4]) {
    Fr r = fr_one();
    for (int i = 255; i >= 0; i--) {
        r = fr_mul(r, r);
        if ((e[i / 64] >> (i % 64)) & 1) r = fr_mul(r, a);
    }
    return r;
}
// Host-side inverse (Montgomery form in and out) by the binary extended Euclidean algorithm: about 500 shift /
// subtract steps on four words instead of the 380 Montgomery products of a^(r-2): every sumcheck that runs in
// split-eq form inverts once when it begins.  inv(0) = 0, as with the power.
inline Fr fr_inv(const Fr& a) {
    typedef unsigned __int128 u128;
    struct U {
        uint64_t w[4];
    };
    const U P = {{DPB_FR_P0, DPB_FR_P1, DPB_FR_P2, DPB_FR_P3}};
    auto is_zero = [](const U& x) { return (x.w[0] | x.w[1] | x.w[2] | x.w[3]) == 0; };
    auto is_one = [](const U& x) { return x.w[0] == 1 && (x.w[1] | x.w[2] | x.w[3]) == 0; };
    auto geq = [](const U& x, const U& y) {
        for (int i = 3; i >= 0; i--)
            if (x.w[i] != y.w[i]) return x.w[i] > y.w[i];
        return true;
    };
    auto add = [](U& x, const U& y) {
        u128 c = 0;
        for (int i = 0; i < 4; i++) {
            c += (u128)x.w[i] + y.w[i];
            x.w[i] = (uint64_t)c;
            c >>= 64;
        }
    };
    auto sub = [](U& x, const U& y) {
        uint64_t b = 0;
        for (int i = 0; i < 4; i++) {
            const u128 d = (u128)x.w[i] - y.w[i] - b;
            x.w[i] = (uint64_t)d;
            b = (uint64_t)(d >> 64) & 1;
        }
    };
    auto shr1 = [](U& x) {
        for (int i = 0; i < 3; i++) x.w[i] = (x.w[i] >> 1) | (x.w[i + 1] << 63);
        x.w[3] >>= 1;
    };
    auto halve = [&](U& x) {  // x / 2 mod r for x < r (r < 2^254: x + r does not overflow)
        if (x.w[0] & 1) add(x, P);
        shr1(x);
    };
    auto sub_mod = [&](U& x, const U& y) {  // x - y mod r for x, y < r
        if (!geq(x, y)) add(x, P);
        sub(x, y);
    };
    U u = {{a.l[0], a.l[1], a.l[2], a.l[3]}}, v = P, x1 = {{1, 0, 0, 0}}, x2 = {{0, 0, 0, 0}};
    if (is_zero(u)) return a;
    while (!is_one(u) && !is_one(v)) {
        while (!(u.w[0] & 1)) {
            shr1(u);
            halve(x1);
        }
        while (!(v.w[0] & 1)) {
            shr1(v);
            halve(x2);
        }
        if (geq(u, v)) {
            sub(u, v);
            sub_mod(x1, x2);
        } else {
            sub(v, u);
            sub_mod(x2, x1);
        }
    }
    const U& y = is_one(u) ? x1 : x2;  // (a R)^-1 as a plain integer
    Fr r;
    r.l[0] = y.w[0];
    r.l[1] = y.w[1];
    r.l[2] = y.w[2];
    r.l[3] = y.w[3];
    // Montgomery products by R^2 lift it: (a R)^-1 -> a^-1 -> a^-1 R
    return fr_mul(fr_mul(r, fr_rr()), fr_rr());
}

}  // namespace dpb
