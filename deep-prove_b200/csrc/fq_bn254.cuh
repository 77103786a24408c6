// BN254 base field Fq (the coordinate field of G1), 4 x 64-bit limbs in Montgomery form.
// Host and device share the code: the curve arithmetic of the MSM runs on the device, the last few additions and
// the conversion to affine coordinates on the host.  q = 21888242871839275222246405745257275088696311157297823662689037894645226208583.
#pragma once
#include <cstdint>

#include "field_bn254.cuh"  // DPB_HD

namespace dpb {

struct alignas(16) Fq {
    uint64_t l[4];
};

#define DPB_FQ_Q0 0x3c208c16d87cfd47ULL
#define DPB_FQ_Q1 0x97816a916871ca8dULL
#define DPB_FQ_Q2 0xb85045b68181585dULL
#define DPB_FQ_Q3 0x30644e72e131a029ULL
#define DPB_FQ_INV 0x87d20782e4866389ULL  // -q^{-1} mod 2^64

}  // namespace dpb
#if defined(__CUDACC__)
#include "fq_words.cuh"
namespace dpb {
__device__ __forceinline__ frw::F8 fq_words(const Fq& a) {
    frw::F8 r;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        r.w[2 * i] = (uint32_t)a.l[i];
        r.w[2 * i + 1] = (uint32_t)(a.l[i] >> 32);
    }
    return r;
}
__device__ __forceinline__ Fq fq_from_words(const frw::F8& a) {
    Fq r;
#pragma unroll
    for (int i = 0; i < 4; i++) r.l[i] = (uint64_t)a.w[2 * i] | ((uint64_t)a.w[2 * i + 1] << 32);
    return r;
}
}  // namespace dpb
#endif
namespace dpb {

// (hi, lo) = a * b + c + d; never overflows 128 bits
DPB_HD void fq_mac(uint64_t a, uint64_t b, uint64_t c, uint64_t d, uint64_t& lo, uint64_t& hi) {
#if defined(__CUDA_ARCH__)
    const uint64_t pl = a * b, ph = __umul64hi(a, b);
    uint64_t s = pl + c;
    uint64_t carry = s < pl;
    const uint64_t t = s + d;
    carry += t < s;
    lo = t;
    hi = ph + carry;
#else
    const unsigned __int128 t = (unsigned __int128)a * b + c + d;
    lo = (uint64_t)t;
    hi = (uint64_t)(t >> 64);
#endif
}

DPB_HD Fq fq_zero() {
    Fq r;
    r.l[0] = r.l[1] = r.l[2] = r.l[3] = 0;
    return r;
}
DPB_HD Fq fq_one() {  // R mod q
    Fq r;
    r.l[0] = 0xd35d438dc58f0d9dULL;
    r.l[1] = 0x0a78eb28f5c70b3dULL;
    r.l[2] = 0x666ea36f7879462cULL;
    r.l[3] = 0x0e0a77c19a07df2fULL;
    return r;
}
DPB_HD Fq fq_rr() {  // R^2 mod q
    Fq r;
    r.l[0] = 0xf32cfc5b538afa89ULL;
    r.l[1] = 0xb5e71911d44501fbULL;
    r.l[2] = 0x47ab1eff0a417ff6ULL;
    r.l[3] = 0x06d89f71cab8351fULL;
    return r;
}
DPB_HD Fq fq_three() {  // 3 R mod q: the curve's b
    Fq r;
    r.l[0] = 0x7a17caa950ad28d7ULL;
    r.l[1] = 0x1f6ac17ae15521b9ULL;
    r.l[2] = 0x334bea4e696bd284ULL;
    r.l[3] = 0x2a1f6744ce179d8eULL;
    return r;
}
DPB_HD bool fq_is_zero(const Fq& a) { return (a.l[0] | a.l[1] | a.l[2] | a.l[3]) == 0; }
DPB_HD bool fq_eq(const Fq& a, const Fq& b) {
    return a.l[0] == b.l[0] && a.l[1] == b.l[1] && a.l[2] == b.l[2] && a.l[3] == b.l[3];
}
DPB_HD bool fq_geq_q(const Fq& a) {
    const uint64_t q[4] = {DPB_FQ_Q0, DPB_FQ_Q1, DPB_FQ_Q2, DPB_FQ_Q3};
    for (int i = 3; i >= 0; i--) {
        if (a.l[i] > q[i]) return true;
        if (a.l[i] < q[i]) return false;
    }
    return true;
}
DPB_HD Fq fq_sub_q(const Fq& a) {
    const uint64_t q[4] = {DPB_FQ_Q0, DPB_FQ_Q1, DPB_FQ_Q2, DPB_FQ_Q3};
    Fq r;
    uint64_t borrow = 0;
    for (int i = 0; i < 4; i++) {
        const uint64_t t = a.l[i] - q[i];
        const uint64_t b1 = a.l[i] < q[i];
        r.l[i] = t - borrow;
        borrow = b1 | (t < borrow);
    }
    return r;
}
DPB_HD Fq fq_add(const Fq& a, const Fq& b) {
#if defined(__CUDA_ARCH__)
    return fq_from_words(fqw::add(fq_words(a), fq_words(b)));
#endif
    Fq r;
    uint64_t carry = 0;
    for (int i = 0; i < 4; i++) {
        const uint64_t s = a.l[i] + b.l[i];
        const uint64_t c1 = s < a.l[i];
        r.l[i] = s + carry;
        carry = c1 | (r.l[i] < s);
    }
    return fq_geq_q(r) ? fq_sub_q(r) : r;  // a + b < 2q < 2^255: no carry out
}
DPB_HD Fq fq_sub(const Fq& a, const Fq& b) {
#if defined(__CUDA_ARCH__)
    return fq_from_words(fqw::sub(fq_words(a), fq_words(b)));
#endif
    const uint64_t q[4] = {DPB_FQ_Q0, DPB_FQ_Q1, DPB_FQ_Q2, DPB_FQ_Q3};
    Fq r;
    uint64_t borrow = 0;
    for (int i = 0; i < 4; i++) {
        const uint64_t t = a.l[i] - b.l[i];
        const uint64_t b1 = a.l[i] < b.l[i];
        r.l[i] = t - borrow;
        borrow = b1 | (t < borrow);
    }
    if (borrow) {
        uint64_t carry = 0;
        for (int i = 0; i < 4; i++) {
            const uint64_t s = r.l[i] + q[i];
            const uint64_t c1 = s < r.l[i];
            r.l[i] = s + carry;
            carry = c1 | (r.l[i] < s);
        }
    }
    return r;
}
DPB_HD Fq fq_neg(const Fq& a) { return fq_is_zero(a) ? a : fq_sub(fq_zero(), a); }
DPB_HD Fq fq_dbl(const Fq& a) { return fq_add(a, a); }

// Montgomery product a b / 2^256 mod q (coarsely integrated operand scanning on 64-bit limbs)
DPB_HD Fq fq_mul(const Fq& a, const Fq& b) {
#if defined(__CUDA_ARCH__)
    return fq_from_words(fqw::mul(fq_words(a), fq_words(b)));  // the word-level product of fq_words.cuh
#endif
    const uint64_t q[4] = {DPB_FQ_Q0, DPB_FQ_Q1, DPB_FQ_Q2, DPB_FQ_Q3};
    uint64_t t[6] = {0, 0, 0, 0, 0, 0};
    for (int i = 0; i < 4; i++) {
        uint64_t carry = 0;
        for (int j = 0; j < 4; j++) fq_mac(a.l[j], b.l[i], t[j], carry, t[j], carry);
        uint64_t s = t[4] + carry;
        t[5] = s < carry;
        t[4] = s;
        const uint64_t m = t[0] * DPB_FQ_INV;
        uint64_t lo;
        fq_mac(m, q[0], t[0], 0, lo, carry);
        for (int j = 1; j < 4; j++) fq_mac(m, q[j], t[j], carry, t[j - 1], carry);
        s = t[4] + carry;
        t[3] = s;
        t[4] = t[5] + (s < carry);
    }
    Fq r;
    r.l[0] = t[0];
    r.l[1] = t[1];
    r.l[2] = t[2];
    r.l[3] = t[3];
    return (t[4] || fq_geq_q(r)) ? fq_sub_q(r) : r;
}
DPB_HD Fq fq_sqr(const Fq& a) { return fq_mul(a, a); }
DPB_HD Fq fq_to_mont(const Fq& a) { return fq_mul(a, fq_rr()); }
DPB_HD Fq fq_from_mont(const Fq& a) {
    Fq one;
    one.l[0] = 1;
    one.l[1] = one.l[2] = one.l[3] = 0;
    return fq_mul(a, one);
}
// a^(q - 2): the inverse (once per MSM on the host, for the affine result; once per point when synthetic bases
// are made on the device)
DPB_HD Fq fq_inv(const Fq& a) {
    const uint64_t e[4] = {DPB_FQ_Q0 - 2, DPB_FQ_Q1, DPB_FQ_Q2, DPB_FQ_Q3};
    Fq r = fq_one();
    for (int i = 255; i >= 0; i--) {
        r = fq_sqr(r);
        if ((e[i / 64] >> (i % 64)) & 1) r = fq_mul(r, a);
    }
    return r;
}

}  // namespace dpb
