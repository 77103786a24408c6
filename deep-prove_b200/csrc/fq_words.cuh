// Device-side BN254 Fq arithmetic on 32-bit words: the Montgomery product of fr_words.cuh (coarsely integrated
// operand scanning, every 32x32 product a wide multiply-add onto an aligned word pair with the carries riding the
// multiply chains) for the base-field modulus q.  The curve additions of the multi-scalar multiplication are made of
// these products; the portable 64-bit-limb routines of fq_bn254.cuh stay for the host.
#pragma once
#include <cstdint>

#include "field_bn254.cuh"  // frw::F8 and the chain helpers

namespace dpb {
namespace fqw {

using frw::F8;

// modulus q, words little-endian, and -q^{-1} mod 2^32
#define DPB_FQW_Q0 0xd87cfd47u
#define DPB_FQW_Q1 0x3c208c16u
#define DPB_FQW_Q2 0x6871ca8du
#define DPB_FQW_Q3 0x97816a91u
#define DPB_FQW_Q4 0x8181585du
#define DPB_FQW_Q5 0xb85045b6u
#define DPB_FQW_Q6 0xe131a029u
#define DPB_FQW_Q7 0x30644e72u
#define DPB_FQW_INV 0xe4866389u

// the odd words of q times y onto four aligned pairs, with a carry in of (lead != 0)
__device__ __forceinline__ void chain_q_odd_lead(uint32_t* c, uint32_t& top, uint32_t y, uint32_t lead) {
    asm("{ .reg .u32 t;\n\t"
        "add.cc.u32 t, %10, 0xffffffff;\n\t"
        "madc.lo.cc.u32 %0, %11, %9, %0; madc.hi.cc.u32 %1, %11, %9, %1;\n\t"
        "madc.lo.cc.u32 %2, %12, %9, %2; madc.hi.cc.u32 %3, %12, %9, %3;\n\t"
        "madc.lo.cc.u32 %4, %13, %9, %4; madc.hi.cc.u32 %5, %13, %9, %5;\n\t"
        "madc.lo.cc.u32 %6, %14, %9, %6; madc.hi.cc.u32 %7, %14, %9, %7;\n\t"
        "addc.u32 %8, %8, 0; }"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]), "+r"(c[4]), "+r"(c[5]), "+r"(c[6]), "+r"(c[7]), "+r"(top)
        : "r"(y), "r"(lead), "r"(DPB_FQW_Q1), "r"(DPB_FQW_Q3), "r"(DPB_FQW_Q5), "r"(DPB_FQW_Q7));
}

// one word of b (see frw::mont_step: the same schedule with q's words)
template <int I>
__device__ __forceinline__ void mont_step(uint32_t* P, uint32_t* Q, const uint32_t* a, uint32_t bi) {
    frw::chain_mul(P + I, P[I + 8], a[0], a[2], a[4], a[6], bi);
    frw::chain_mul(Q + I + 1, Q[I + 9], a[1], a[3], a[5], a[7], bi);
    const uint32_t w = I ? P[I] + Q[I] : P[I];
    const uint32_t m = w * DPB_FQW_INV;
    frw::chain_mul(P + I, P[I + 8], DPB_FQW_Q0, DPB_FQW_Q2, DPB_FQW_Q4, DPB_FQW_Q6, m);
    if (I) chain_q_odd_lead(Q + I + 1, Q[I + 9], m, Q[I]);
    else frw::chain_mul(Q + I + 1, Q[I + 9], DPB_FQW_Q1, DPB_FQW_Q3, DPB_FQW_Q5, DPB_FQW_Q7, m);
}

// a < 2q -> a mod q
__device__ __forceinline__ F8 reduce_once(const F8& a) {
    F8 d;
    asm("{ .reg .u32 m, q0,q1,q2,q3,q4,q5,q6,q7;\n\t"
        "sub.cc.u32 %0, %8, 0xd87cfd47; subc.cc.u32 %1, %9, 0x3c208c16; subc.cc.u32 %2, %10, 0x6871ca8d;\n\t"
        "subc.cc.u32 %3, %11, 0x97816a91; subc.cc.u32 %4, %12, 0x8181585d; subc.cc.u32 %5, %13, 0xb85045b6;\n\t"
        "subc.cc.u32 %6, %14, 0xe131a029; subc.cc.u32 %7, %15, 0x30644e72; subc.u32 m, 0, 0;\n\t"
        "and.b32 q0, m, 0xd87cfd47; and.b32 q1, m, 0x3c208c16; and.b32 q2, m, 0x6871ca8d; and.b32 q3, m, 0x97816a91;\n\t"
        "and.b32 q4, m, 0x8181585d; and.b32 q5, m, 0xb85045b6; and.b32 q6, m, 0xe131a029; and.b32 q7, m, 0x30644e72;\n\t"
        "add.cc.u32 %0, %0, q0; addc.cc.u32 %1, %1, q1; addc.cc.u32 %2, %2, q2; addc.cc.u32 %3, %3, q3;\n\t"
        "addc.cc.u32 %4, %4, q4; addc.cc.u32 %5, %5, q5; addc.cc.u32 %6, %6, q6; addc.u32 %7, %7, q7; }"
        : "=&r"(d.w[0]), "=&r"(d.w[1]), "=&r"(d.w[2]), "=&r"(d.w[3]), "=&r"(d.w[4]), "=&r"(d.w[5]), "=&r"(d.w[6]),
          "=&r"(d.w[7])
        : "r"(a.w[0]), "r"(a.w[1]), "r"(a.w[2]), "r"(a.w[3]), "r"(a.w[4]), "r"(a.w[5]), "r"(a.w[6]), "r"(a.w[7]));
    return d;
}

// Montgomery product a * b / 2^256 mod q
__device__ __forceinline__ F8 mul(const F8& a, const F8& b) {
    uint32_t E[18], O[18];
#pragma unroll
    for (int i = 0; i < 18; i++) E[i] = O[i] = 0;
    mont_step<0>(E, O, a.w, b.w[0]);
    mont_step<1>(O, E, a.w, b.w[1]);
    mont_step<2>(E, O, a.w, b.w[2]);
    mont_step<3>(O, E, a.w, b.w[3]);
    mont_step<4>(E, O, a.w, b.w[4]);
    mont_step<5>(O, E, a.w, b.w[5]);
    mont_step<6>(E, O, a.w, b.w[6]);
    mont_step<7>(O, E, a.w, b.w[7]);
    F8 s;
    asm("add.cc.u32 %0, %8, %16; addc.cc.u32 %1, %9, %17; addc.cc.u32 %2, %10, %18; addc.cc.u32 %3, %11, %19;\n\t"
        "addc.cc.u32 %4, %12, %20; addc.cc.u32 %5, %13, %21; addc.cc.u32 %6, %14, %22; addc.u32 %7, %15, %23;"
        : "=&r"(s.w[0]), "=&r"(s.w[1]), "=&r"(s.w[2]), "=&r"(s.w[3]), "=&r"(s.w[4]), "=&r"(s.w[5]), "=&r"(s.w[6]),
          "=&r"(s.w[7])
        : "r"(E[8]), "r"(E[9]), "r"(E[10]), "r"(E[11]), "r"(E[12]), "r"(E[13]), "r"(E[14]), "r"(E[15]), "r"(O[8]),
          "r"(O[9]), "r"(O[10]), "r"(O[11]), "r"(O[12]), "r"(O[13]), "r"(O[14]), "r"(O[15]));
    return fqw::reduce_once(s);
}

__device__ __forceinline__ F8 add(const F8& a, const F8& b) {
    F8 s;
    asm("add.cc.u32 %0, %8, %16; addc.cc.u32 %1, %9, %17; addc.cc.u32 %2, %10, %18; addc.cc.u32 %3, %11, %19;\n\t"
        "addc.cc.u32 %4, %12, %20; addc.cc.u32 %5, %13, %21; addc.cc.u32 %6, %14, %22; addc.u32 %7, %15, %23;"
        : "=&r"(s.w[0]), "=&r"(s.w[1]), "=&r"(s.w[2]), "=&r"(s.w[3]), "=&r"(s.w[4]), "=&r"(s.w[5]), "=&r"(s.w[6]),
          "=&r"(s.w[7])
        : "r"(a.w[0]), "r"(a.w[1]), "r"(a.w[2]), "r"(a.w[3]), "r"(a.w[4]), "r"(a.w[5]), "r"(a.w[6]), "r"(a.w[7]),
          "r"(b.w[0]), "r"(b.w[1]), "r"(b.w[2]), "r"(b.w[3]), "r"(b.w[4]), "r"(b.w[5]), "r"(b.w[6]), "r"(b.w[7]));
    return fqw::reduce_once(s);  // a + b < 2q < 2^255
}

__device__ __forceinline__ F8 sub(const F8& a, const F8& b) {
    F8 d;
    asm("{ .reg .u32 m, q0,q1,q2,q3,q4,q5,q6,q7;\n\t"
        "sub.cc.u32 %0, %8, %16; subc.cc.u32 %1, %9, %17; subc.cc.u32 %2, %10, %18; subc.cc.u32 %3, %11, %19;\n\t"
        "subc.cc.u32 %4, %12, %20; subc.cc.u32 %5, %13, %21; subc.cc.u32 %6, %14, %22; subc.cc.u32 %7, %15, %23;\n\t"
        "subc.u32 m, 0, 0;\n\t"
        "and.b32 q0, m, 0xd87cfd47; and.b32 q1, m, 0x3c208c16; and.b32 q2, m, 0x6871ca8d; and.b32 q3, m, 0x97816a91;\n\t"
        "and.b32 q4, m, 0x8181585d; and.b32 q5, m, 0xb85045b6; and.b32 q6, m, 0xe131a029; and.b32 q7, m, 0x30644e72;\n\t"
        "add.cc.u32 %0, %0, q0; addc.cc.u32 %1, %1, q1; addc.cc.u32 %2, %2, q2; addc.cc.u32 %3, %3, q3;\n\t"
        "addc.cc.u32 %4, %4, q4; addc.cc.u32 %5, %5, q5; addc.cc.u32 %6, %6, q6; addc.u32 %7, %7, q7; }"
        : "=&r"(d.w[0]), "=&r"(d.w[1]), "=&r"(d.w[2]), "=&r"(d.w[3]), "=&r"(d.w[4]), "=&r"(d.w[5]), "=&r"(d.w[6]),
          "=&r"(d.w[7])
        : "r"(a.w[0]), "r"(a.w[1]), "r"(a.w[2]), "r"(a.w[3]), "r"(a.w[4]), "r"(a.w[5]), "r"(a.w[6]), "r"(a.w[7]),
          "r"(b.w[0]), "r"(b.w[1]), "r"(b.w[2]), "r"(b.w[3]), "r"(b.w[4]), "r"(b.w[5]), "r"(b.w[6]), "r"(b.w[7]));
    return d;
}

}  // namespace fqw
}  // namespace dpb
