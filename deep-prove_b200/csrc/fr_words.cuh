// Device-side BN254 Fr arithmetic on 32-bit words.
//
// The portable routines of field_bn254.cuh multiply 64-bit limbs; on the GPU
// each 64x64 product expands into a long sequence of 32-bit multiply-adds and
// register shuffles.  Here a field element is eight 32-bit words and the
// Montgomery product is coarsely integrated operand scanning over words: per
// word of b, eight 32x32 products accumulate into the running sum, then eight
// more for the reduction step.  Every product is a wide multiply-add that adds
// its 64-bit result to an aligned word pair with carry in and out, so the 128
// multiplies carry almost all of the additions; measured on sm_100a a wide
// multiply-add costs about four issue cycles and a carry-chained add about one,
// which makes the multiply count the floor.
//
// The word layout is the little-endian split of the four 64-bit limbs, so a
// conversion is a register reinterpretation.
#pragma once
// Included by field_bn254.cuh (after the definition of Fr) and by nothing else.
#include <cstdint>

namespace dpb {
namespace frw {

struct F8 {
    uint32_t w[8];
};

__device__ __forceinline__ F8 from_fr(const Fr& a) {
    F8 r;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        r.w[2 * i] = (uint32_t)a.l[i];
        r.w[2 * i + 1] = (uint32_t)(a.l[i] >> 32);
    }
    return r;
}
__device__ __forceinline__ Fr to_fr(const F8& a) {
    Fr r;
#pragma unroll
    for (int i = 0; i < 4; i++) r.l[i] = (uint64_t)a.w[2 * i] | ((uint64_t)a.w[2 * i + 1] << 32);
    return r;
}

// modulus r, words little-endian
#define DPB_FRW_P0 0xf0000001u
#define DPB_FRW_P1 0x43e1f593u
#define DPB_FRW_P2 0x79b97091u
#define DPB_FRW_P3 0x2833e848u
#define DPB_FRW_P4 0x8181585du
#define DPB_FRW_P5 0xb85045b6u
#define DPB_FRW_P6 0xe131a029u
#define DPB_FRW_P7 0x30644e72u
#define DPB_FRW_INV 0xefffffffu  // -r^{-1} mod 2^32

// Four wide multiply-adds on one carry chain: the four aligned word pairs
// (c0,c1) .. (c6,c7) += (x0, x1, x2, x3) * y, the carry out goes into top.  Each
// mad.lo.cc / madc.hi.cc pair with the same operands is one 32x32+64 multiply-add
// with carry in and out on the device, so a chain is four multiply instructions
// and one add.  With LEAD the chain starts with a carry in of (lead != 0).
#define DPB_FRW_CHAIN_BODY(FIRST, X0, X1, X2, X3)                                      \
    FIRST ".lo.cc.u32 %0, " X0 ", %9, %0; madc.hi.cc.u32 %1, " X0 ", %9, %1;\n\t"      \
    "madc.lo.cc.u32 %2, " X1 ", %9, %2; madc.hi.cc.u32 %3, " X1 ", %9, %3;\n\t"        \
    "madc.lo.cc.u32 %4, " X2 ", %9, %4; madc.hi.cc.u32 %5, " X2 ", %9, %5;\n\t"        \
    "madc.lo.cc.u32 %6, " X3 ", %9, %6; madc.hi.cc.u32 %7, " X3 ", %9, %7;\n\t"        \
    "addc.u32 %8, %8, 0;"
#define DPB_FRW_CHAIN_OUT(c, top)                                                                           \
    "+r"((c)[0]), "+r"((c)[1]), "+r"((c)[2]), "+r"((c)[3]), "+r"((c)[4]), "+r"((c)[5]), "+r"((c)[6]), \
        "+r"((c)[7]), "+r"(top)

// c points at the first word of the first pair; x are four words of a
__device__ __forceinline__ void chain_mul(uint32_t* c, uint32_t& top, uint32_t x0, uint32_t x1, uint32_t x2,
                                          uint32_t x3, uint32_t y) {
    asm(DPB_FRW_CHAIN_BODY("mad", "%10", "%11", "%12", "%13")
        : DPB_FRW_CHAIN_OUT(c, top)
        : "r"(y), "r"(x0), "r"(x1), "r"(x2), "r"(x3));
}
// the same with the even words of the modulus
__device__ __forceinline__ void chain_mod_even(uint32_t* c, uint32_t& top, uint32_t y) {
    asm(DPB_FRW_CHAIN_BODY("mad", "0xf0000001", "0x79b97091", "0x8181585d", "0xe131a029")
        : DPB_FRW_CHAIN_OUT(c, top)
        : "r"(y));
}
// the odd words of the modulus; LEAD: carry in of (lead != 0)
template <bool LEAD>
__device__ __forceinline__ void chain_mod_odd(uint32_t* c, uint32_t& top, uint32_t y, uint32_t lead) {
    if (LEAD) {
        asm("{ .reg .u32 t;\n\t"
            "add.cc.u32 t, %10, 0xffffffff;\n\t" DPB_FRW_CHAIN_BODY("madc", "0x43e1f593", "0x2833e848", "0xb85045b6",
                                                                   "0x30644e72") " }"
            : DPB_FRW_CHAIN_OUT(c, top)
            : "r"(y), "r"(lead));
    } else {
        asm(DPB_FRW_CHAIN_BODY("mad", "0x43e1f593", "0x2833e848", "0xb85045b6", "0x30644e72")
            : DPB_FRW_CHAIN_OUT(c, top)
            : "r"(y));
    }
}

// One word of b: the running sum is held as two arrays indexed by absolute word
// position.  P holds 64-bit pairs that start at positions of the parity of I, Q
// pairs that start at the other parity; the true sum is P + Q.  Products of the
// even words of a with b_I start at position I (in P), those of the odd words at
// I + 1 (in Q), so every multiply-add lands on an aligned pair.  The reduction
// word m clears position I of the sum: P[I] becomes -Q[I] mod 2^32, and the carry
// that P[I] + Q[I] sends to position I + 1 is exactly (Q[I] != 0); it enters the
// odd-word chain of the modulus.  Position I is never looked at again.
template <int I>
__device__ __forceinline__ void mont_step(uint32_t* P, uint32_t* Q, const uint32_t* a, uint32_t bi) {
    chain_mul(P + I, P[I + 8], a[0], a[2], a[4], a[6], bi);
    chain_mul(Q + I + 1, Q[I + 9], a[1], a[3], a[5], a[7], bi);
    const uint32_t w = I ? P[I] + Q[I] : P[I];
    const uint32_t m = w * DPB_FRW_INV;
    chain_mod_even(P + I, P[I + 8], m);
    if (I) chain_mod_odd<true>(Q + I + 1, Q[I + 9], m, Q[I]);
    else chain_mod_odd<false>(Q + I + 1, Q[I + 9], m, 0);
}

// a < 2r -> a mod r: subtract r; on a borrow add it back through a mask
__device__ __forceinline__ F8 reduce_once(const F8& a) {
    F8 d;
    asm("{ .reg .u32 m, q0,q1,q2,q3,q4,q5,q6,q7;\n\t"
        "sub.cc.u32 %0, %8, 0xf0000001; subc.cc.u32 %1, %9, 0x43e1f593; subc.cc.u32 %2, %10, 0x79b97091;\n\t"
        "subc.cc.u32 %3, %11, 0x2833e848; subc.cc.u32 %4, %12, 0x8181585d; subc.cc.u32 %5, %13, 0xb85045b6;\n\t"
        "subc.cc.u32 %6, %14, 0xe131a029; subc.cc.u32 %7, %15, 0x30644e72; subc.u32 m, 0, 0;\n\t"
        "and.b32 q0, m, 0xf0000001; and.b32 q1, m, 0x43e1f593; and.b32 q2, m, 0x79b97091; and.b32 q3, m, 0x2833e848;\n\t"
        "and.b32 q4, m, 0x8181585d; and.b32 q5, m, 0xb85045b6; and.b32 q6, m, 0xe131a029; and.b32 q7, m, 0x30644e72;\n\t"
        "add.cc.u32 %0, %0, q0; addc.cc.u32 %1, %1, q1; addc.cc.u32 %2, %2, q2; addc.cc.u32 %3, %3, q3;\n\t"
        "addc.cc.u32 %4, %4, q4; addc.cc.u32 %5, %5, q5; addc.cc.u32 %6, %6, q6; addc.u32 %7, %7, q7; }"
        : "=&r"(d.w[0]), "=&r"(d.w[1]), "=&r"(d.w[2]), "=&r"(d.w[3]), "=&r"(d.w[4]), "=&r"(d.w[5]), "=&r"(d.w[6]),
          "=&r"(d.w[7])
        : "r"(a.w[0]), "r"(a.w[1]), "r"(a.w[2]), "r"(a.w[3]), "r"(a.w[4]), "r"(a.w[5]), "r"(a.w[6]), "r"(a.w[7]));
    return d;
}

// Montgomery product a * b / 2^256 mod r
__device__ __forceinline__ F8 mul(const F8& a, const F8& b) {
    uint32_t E[18], O[18];  // pairs at even / odd positions; only a window of ten words is live at a time
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
    // positions 0..7 of the sum are clear; positions 8..15 hold a value below 2r
    F8 s;
    asm("add.cc.u32 %0, %8, %16; addc.cc.u32 %1, %9, %17; addc.cc.u32 %2, %10, %18; addc.cc.u32 %3, %11, %19;\n\t"
        "addc.cc.u32 %4, %12, %20; addc.cc.u32 %5, %13, %21; addc.cc.u32 %6, %14, %22; addc.u32 %7, %15, %23;"
        : "=&r"(s.w[0]), "=&r"(s.w[1]), "=&r"(s.w[2]), "=&r"(s.w[3]), "=&r"(s.w[4]), "=&r"(s.w[5]), "=&r"(s.w[6]),
          "=&r"(s.w[7])
        : "r"(E[8]), "r"(E[9]), "r"(E[10]), "r"(E[11]), "r"(E[12]), "r"(E[13]), "r"(E[14]), "r"(E[15]), "r"(O[8]),
          "r"(O[9]), "r"(O[10]), "r"(O[11]), "r"(O[12]), "r"(O[13]), "r"(O[14]), "r"(O[15]));
    return reduce_once(s);
}

// Product by a multiplicand that is fixed for a whole launch (the challenge of a fold).
// With a = sum_i a_i 2^(32 i), a * c / 2^256 = sum_i a_i * C_i for the eight constants
// C_i = c * 2^(32 i) / 2^256 mod r, which the host computes once per round.  The sum of
// the eight rows needs no interleaved reduction: 64 multiply-adds, all landing on the
// same aligned pairs, give a 289-bit value; two reduction words bring it below 2r (the
// host folds their factor 2^-64 into the constants).  80 wide multiply-adds instead
// of 128.
struct FixedMul {
    uint32_t c[8][8];  // C_i * 2^64 mod r, words little-endian
};
__device__ __forceinline__ F8 mul_fixed(const F8& a, const FixedMul& k) {
    uint32_t E[12], O[12];  // pairs at even / odd positions
#pragma unroll
    for (int i = 0; i < 12; i++) E[i] = O[i] = 0;
#pragma unroll
    for (int i = 0; i < 8; i++) {
        chain_mul(E, E[8], k.c[i][0], k.c[i][2], k.c[i][4], k.c[i][6], a.w[i]);
        chain_mul(O + 1, O[9], k.c[i][1], k.c[i][3], k.c[i][5], k.c[i][7], a.w[i]);
    }
    // reduction word for position 0 (only E holds it), then for position 1 (O's pair and E's left-over word)
    const uint32_t m0 = E[0] * DPB_FRW_INV;
    chain_mod_even(E, E[8], m0);
    chain_mod_odd<false>(O + 1, O[9], m0, 0);
    const uint32_t m1 = (O[1] + E[1]) * DPB_FRW_INV;
    chain_mod_even(O + 1, O[9], m1);
    chain_mod_odd<true>(E + 2, E[10], m1, E[1]);
    F8 s;
    asm("add.cc.u32 %0, %8, %16; addc.cc.u32 %1, %9, %17; addc.cc.u32 %2, %10, %18; addc.cc.u32 %3, %11, %19;\n\t"
        "addc.cc.u32 %4, %12, %20; addc.cc.u32 %5, %13, %21; addc.cc.u32 %6, %14, %22; addc.u32 %7, %15, %23;"
        : "=&r"(s.w[0]), "=&r"(s.w[1]), "=&r"(s.w[2]), "=&r"(s.w[3]), "=&r"(s.w[4]), "=&r"(s.w[5]), "=&r"(s.w[6]),
          "=&r"(s.w[7])
        : "r"(E[2]), "r"(E[3]), "r"(E[4]), "r"(E[5]), "r"(E[6]), "r"(E[7]), "r"(E[8]), "r"(E[9]), "r"(O[2]),
          "r"(O[3]), "r"(O[4]), "r"(O[5]), "r"(O[6]), "r"(O[7]), "r"(O[8]), "r"(O[9]));
    return reduce_once(s);
}

// Two small integers times two rows, the reduction of mul_fixed: what turns an integer, or the fold of two
// integers by a challenge, into a field element for a fraction of a product's cost.
// (ma * row_a + md * row_d) / 2^64 mod p, ma and md below 2^32
__device__ __forceinline__ F8 lin2_rows(uint32_t ma, const uint32_t* ra, uint32_t md, const uint32_t* rd) {
    uint32_t E[12], O[12];  // pairs at even / odd positions, as in mul_fixed
#pragma unroll
    for (int i = 0; i < 12; i++) E[i] = O[i] = 0;
    chain_mul(E, E[8], ra[0], ra[2], ra[4], ra[6], ma);
    chain_mul(O + 1, O[9], ra[1], ra[3], ra[5], ra[7], ma);
    chain_mul(E, E[8], rd[0], rd[2], rd[4], rd[6], md);
    chain_mul(O + 1, O[9], rd[1], rd[3], rd[5], rd[7], md);
    const uint32_t m0 = E[0] * DPB_FRW_INV;
    chain_mod_even(E, E[8], m0);
    chain_mod_odd<false>(O + 1, O[9], m0, 0);
    const uint32_t m1 = (O[1] + E[1]) * DPB_FRW_INV;
    chain_mod_even(O + 1, O[9], m1);
    chain_mod_odd<true>(E + 2, E[10], m1, E[1]);
    F8 s;
    asm("add.cc.u32 %0, %8, %16; addc.cc.u32 %1, %9, %17; addc.cc.u32 %2, %10, %18; addc.cc.u32 %3, %11, %19;\n\t"
        "addc.cc.u32 %4, %12, %20; addc.cc.u32 %5, %13, %21; addc.cc.u32 %6, %14, %22; addc.u32 %7, %15, %23;"
        : "=&r"(s.w[0]), "=&r"(s.w[1]), "=&r"(s.w[2]), "=&r"(s.w[3]), "=&r"(s.w[4]), "=&r"(s.w[5]), "=&r"(s.w[6]),
          "=&r"(s.w[7])
        : "r"(E[2]), "r"(E[3]), "r"(E[4]), "r"(E[5]), "r"(E[6]), "r"(E[7]), "r"(E[8]), "r"(E[9]), "r"(O[2]),
          "r"(O[3]), "r"(O[4]), "r"(O[5]), "r"(O[6]), "r"(O[7]), "r"(O[8]), "r"(O[9]));
    return reduce_once(s);
}

// Sum of (64-bit integer) * (field element) products kept as one unreduced integer: what the contraction of an
// integer tensor against eq weights is made of.  A term is 16 wide multiply-adds and no reduction; the sum of up to
// 2^24 terms stays below 2^352 and is reduced once (two Montgomery products).  Layout as in mul: E holds word pairs
// at even positions, O at odd positions, value = E + O; words 0..11.
struct IntAcc {
    uint32_t E[12], O[12];
};
__device__ __forceinline__ IntAcc intacc_zero() {
    IntAcc a;
#pragma unroll
    for (int i = 0; i < 12; i++) a.E[i] = a.O[i] = 0;
    return a;
}
// four pairs starting at c += (x0..x3) * y, the carry runs on through three more words
__device__ __forceinline__ void chain_mul_long(uint32_t* c, uint32_t x0, uint32_t x1, uint32_t x2, uint32_t x3, uint32_t y) {
    asm("mad.lo.cc.u32 %0, %12, %11, %0; madc.hi.cc.u32 %1, %12, %11, %1;\n\t"
        "madc.lo.cc.u32 %2, %13, %11, %2; madc.hi.cc.u32 %3, %13, %11, %3;\n\t"
        "madc.lo.cc.u32 %4, %14, %11, %4; madc.hi.cc.u32 %5, %14, %11, %5;\n\t"
        "madc.lo.cc.u32 %6, %15, %11, %6; madc.hi.cc.u32 %7, %15, %11, %7;\n\t"
        "addc.cc.u32 %8, %8, 0; addc.cc.u32 %9, %9, 0; addc.u32 %10, %10, 0;"
        : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3]), "+r"(c[4]), "+r"(c[5]), "+r"(c[6]), "+r"(c[7]), "+r"(c[8]),
          "+r"(c[9]), "+r"(c[10])
        : "r"(y), "r"(x0), "r"(x1), "r"(x2), "r"(x3));
}
// acc += mag * w, mag a 64-bit magnitude, w any 256-bit value
__device__ __forceinline__ void intacc_mac(IntAcc& a, const F8& w, uint64_t mag) {
    const uint32_t m0 = (uint32_t)mag, m1 = (uint32_t)(mag >> 32);
    chain_mul_long(a.E, w.w[0], w.w[2], w.w[4], w.w[6], m0);      // positions (0,1) .. (6,7)
    chain_mul_long(a.O + 1, w.w[1], w.w[3], w.w[5], w.w[7], m0);  // positions (1,2) .. (7,8)
    if (m1) {  // quantised values seldom need the upper word
        chain_mul_long(a.O + 1, w.w[0], w.w[2], w.w[4], w.w[6], m1);  // one word up: (1,2) .. (7,8)
        // two words up: (2,3) .. (8,9); the carry has one word of room left (the sum stays below 2^352)
        asm("mad.lo.cc.u32 %0, %10, %9, %0; madc.hi.cc.u32 %1, %10, %9, %1;\n\t"
            "madc.lo.cc.u32 %2, %11, %9, %2; madc.hi.cc.u32 %3, %11, %9, %3;\n\t"
            "madc.lo.cc.u32 %4, %12, %9, %4; madc.hi.cc.u32 %5, %12, %9, %5;\n\t"
            "madc.lo.cc.u32 %6, %13, %9, %6; madc.hi.cc.u32 %7, %13, %9, %7;\n\t"
            "addc.cc.u32 %8, %8, 0;"
            : "+r"(a.E[2]), "+r"(a.E[3]), "+r"(a.E[4]), "+r"(a.E[5]), "+r"(a.E[6]), "+r"(a.E[7]), "+r"(a.E[8]),
              "+r"(a.E[9]), "+r"(a.E[10])
            : "r"(m1), "r"(w.w[1]), "r"(w.w[3]), "r"(w.w[5]), "r"(w.w[7]));
    }
}
// the sum as words 0..10 (E + O), low 8 words and the words above them
__device__ __forceinline__ void intacc_split(const IntAcc& a, F8& lo, F8& hi) {
    uint32_t s[12];
    asm("add.cc.u32 %0, %12, %24; addc.cc.u32 %1, %13, %25; addc.cc.u32 %2, %14, %26; addc.cc.u32 %3, %15, %27;\n\t"
        "addc.cc.u32 %4, %16, %28; addc.cc.u32 %5, %17, %29; addc.cc.u32 %6, %18, %30; addc.cc.u32 %7, %19, %31;\n\t"
        "addc.cc.u32 %8, %20, %32; addc.cc.u32 %9, %21, %33; addc.cc.u32 %10, %22, %34; addc.u32 %11, %23, %35;"
        : "=&r"(s[0]), "=&r"(s[1]), "=&r"(s[2]), "=&r"(s[3]), "=&r"(s[4]), "=&r"(s[5]), "=&r"(s[6]), "=&r"(s[7]),
          "=&r"(s[8]), "=&r"(s[9]), "=&r"(s[10]), "=&r"(s[11])
        : "r"(a.E[0]), "r"(a.E[1]), "r"(a.E[2]), "r"(a.E[3]), "r"(a.E[4]), "r"(a.E[5]), "r"(a.E[6]), "r"(a.E[7]),
          "r"(a.E[8]), "r"(a.E[9]), "r"(a.E[10]), "r"(a.E[11]), "r"(a.O[0]), "r"(a.O[1]), "r"(a.O[2]), "r"(a.O[3]),
          "r"(a.O[4]), "r"(a.O[5]), "r"(a.O[6]), "r"(a.O[7]), "r"(a.O[8]), "r"(a.O[9]), "r"(a.O[10]), "r"(a.O[11]));
#pragma unroll
    for (int i = 0; i < 8; i++) lo.w[i] = s[i];
#pragma unroll
    for (int i = 0; i < 4; i++) hi.w[i] = s[8 + i];
#pragma unroll
    for (int i = 4; i < 8; i++) hi.w[i] = 0;
}

__device__ __forceinline__ F8 add(const F8& a, const F8& b) {
    F8 s;
    asm("add.cc.u32 %0, %8, %16; addc.cc.u32 %1, %9, %17; addc.cc.u32 %2, %10, %18; addc.cc.u32 %3, %11, %19;\n\t"
        "addc.cc.u32 %4, %12, %20; addc.cc.u32 %5, %13, %21; addc.cc.u32 %6, %14, %22; addc.u32 %7, %15, %23;"
        : "=&r"(s.w[0]), "=&r"(s.w[1]), "=&r"(s.w[2]), "=&r"(s.w[3]), "=&r"(s.w[4]), "=&r"(s.w[5]), "=&r"(s.w[6]),
          "=&r"(s.w[7])
        : "r"(a.w[0]), "r"(a.w[1]), "r"(a.w[2]), "r"(a.w[3]), "r"(a.w[4]), "r"(a.w[5]), "r"(a.w[6]), "r"(a.w[7]),
          "r"(b.w[0]), "r"(b.w[1]), "r"(b.w[2]), "r"(b.w[3]), "r"(b.w[4]), "r"(b.w[5]), "r"(b.w[6]), "r"(b.w[7]));
    return reduce_once(s);  // a + b < 2r < 2^255: no carry out of the top word
}

// a - b mod r: on a borrow add r back through a mask
__device__ __forceinline__ F8 sub(const F8& a, const F8& b) {
    F8 d;
    asm("{ .reg .u32 m, q0,q1,q2,q3,q4,q5,q6,q7;\n\t"
        "sub.cc.u32 %0, %8, %16; subc.cc.u32 %1, %9, %17; subc.cc.u32 %2, %10, %18; subc.cc.u32 %3, %11, %19;\n\t"
        "subc.cc.u32 %4, %12, %20; subc.cc.u32 %5, %13, %21; subc.cc.u32 %6, %14, %22; subc.cc.u32 %7, %15, %23;\n\t"
        "subc.u32 m, 0, 0;\n\t"
        "and.b32 q0, m, 0xf0000001; and.b32 q1, m, 0x43e1f593; and.b32 q2, m, 0x79b97091; and.b32 q3, m, 0x2833e848;\n\t"
        "and.b32 q4, m, 0x8181585d; and.b32 q5, m, 0xb85045b6; and.b32 q6, m, 0xe131a029; and.b32 q7, m, 0x30644e72;\n\t"
        "add.cc.u32 %0, %0, q0; addc.cc.u32 %1, %1, q1; addc.cc.u32 %2, %2, q2; addc.cc.u32 %3, %3, q3;\n\t"
        "addc.cc.u32 %4, %4, q4; addc.cc.u32 %5, %5, q5; addc.cc.u32 %6, %6, q6; addc.u32 %7, %7, q7; }"
        : "=&r"(d.w[0]), "=&r"(d.w[1]), "=&r"(d.w[2]), "=&r"(d.w[3]), "=&r"(d.w[4]), "=&r"(d.w[5]), "=&r"(d.w[6]),
          "=&r"(d.w[7])
        : "r"(a.w[0]), "r"(a.w[1]), "r"(a.w[2]), "r"(a.w[3]), "r"(a.w[4]), "r"(a.w[5]), "r"(a.w[6]), "r"(a.w[7]),
          "r"(b.w[0]), "r"(b.w[1]), "r"(b.w[2]), "r"(b.w[3]), "r"(b.w[4]), "r"(b.w[5]), "r"(b.w[6]), "r"(b.w[7]));
    return d;
}

}  // namespace frw
}  // namespace dpb
