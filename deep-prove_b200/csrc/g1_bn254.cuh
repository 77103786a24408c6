// BN254 G1 (y^2 = x^3 + 3 over Fq): affine and Jacobian points, the additions the bucket method needs.
// The point at infinity is Z = 0 in Jacobian coordinates and (0, 0) in affine ones ((0, 0) is not on the curve).
#pragma once
#include "fq_bn254.cuh"

namespace dpb {

struct G1Affine {
    Fq x, y;  // Montgomery form
};
struct G1Jac {
    Fq X, Y, Z;
};

DPB_HD G1Jac g1_infinity() {
    G1Jac p;
    p.X = fq_one();
    p.Y = fq_one();
    p.Z = fq_zero();
    return p;
}
DPB_HD bool g1_is_infinity(const G1Jac& p) { return fq_is_zero(p.Z); }
DPB_HD bool g1_affine_is_infinity(const G1Affine& p) { return fq_is_zero(p.x) && fq_is_zero(p.y); }
DPB_HD G1Jac g1_from_affine(const G1Affine& p) {
    if (g1_affine_is_infinity(p)) return g1_infinity();
    G1Jac r;
    r.X = p.x;
    r.Y = p.y;
    r.Z = fq_one();
    return r;
}
DPB_HD G1Affine g1_affine_neg(const G1Affine& p) {
    G1Affine r;
    r.x = p.x;
    r.y = fq_neg(p.y);
    return r;
}

// 2 P for a = 0 (dbl-2009-l: 2 products, 5 squarings)
DPB_HD G1Jac g1_double(const G1Jac& p) {
    if (g1_is_infinity(p)) return p;
    const Fq A = fq_sqr(p.X), B = fq_sqr(p.Y), C = fq_sqr(B);
    Fq D = fq_sub(fq_sub(fq_sqr(fq_add(p.X, B)), A), C);
    D = fq_dbl(D);
    const Fq E = fq_add(fq_dbl(A), A), F = fq_sqr(E);
    G1Jac r;
    r.X = fq_sub(F, fq_dbl(D));
    Fq C8 = fq_dbl(fq_dbl(fq_dbl(C)));
    r.Y = fq_sub(fq_mul(E, fq_sub(D, r.X)), C8);
    r.Z = fq_dbl(fq_mul(p.Y, p.Z));
    return r;
}

// P + Q, Q affine (madd-2007-bl: 7 products, 4 squarings); every special case handled
DPB_HD G1Jac g1_add_mixed(const G1Jac& p, const G1Affine& q) {
    if (g1_affine_is_infinity(q)) return p;
    if (g1_is_infinity(p)) return g1_from_affine(q);
    const Fq Z1Z1 = fq_sqr(p.Z);
    const Fq U2 = fq_mul(q.x, Z1Z1);
    const Fq S2 = fq_mul(fq_mul(q.y, p.Z), Z1Z1);
    const Fq H = fq_sub(U2, p.X);
    const Fq rr = fq_dbl(fq_sub(S2, p.Y));
    if (fq_is_zero(H)) {
        if (fq_is_zero(rr)) return g1_double(p);  // the same point
        return g1_infinity();                     // opposite points
    }
    const Fq HH = fq_sqr(H);
    const Fq I = fq_dbl(fq_dbl(HH));
    const Fq J = fq_mul(H, I);
    const Fq V = fq_mul(p.X, I);
    G1Jac r;
    r.X = fq_sub(fq_sub(fq_sqr(rr), J), fq_dbl(V));
    r.Y = fq_sub(fq_mul(rr, fq_sub(V, r.X)), fq_dbl(fq_mul(p.Y, J)));
    r.Z = fq_sub(fq_sub(fq_sqr(fq_add(p.Z, H)), Z1Z1), HH);
    return r;
}

// P + Q, both Jacobian (add-2007-bl: 11 products, 5 squarings)
DPB_HD G1Jac g1_add(const G1Jac& p, const G1Jac& q) {
    if (g1_is_infinity(p)) return q;
    if (g1_is_infinity(q)) return p;
    const Fq Z1Z1 = fq_sqr(p.Z), Z2Z2 = fq_sqr(q.Z);
    const Fq U1 = fq_mul(p.X, Z2Z2), U2 = fq_mul(q.X, Z1Z1);
    const Fq S1 = fq_mul(fq_mul(p.Y, q.Z), Z2Z2), S2 = fq_mul(fq_mul(q.Y, p.Z), Z1Z1);
    const Fq H = fq_sub(U2, U1);
    const Fq rr = fq_dbl(fq_sub(S2, S1));
    if (fq_is_zero(H)) {
        if (fq_is_zero(rr)) return g1_double(p);
        return g1_infinity();
    }
    const Fq I = fq_sqr(fq_dbl(H));
    const Fq J = fq_mul(H, I);
    const Fq V = fq_mul(U1, I);
    G1Jac r;
    r.X = fq_sub(fq_sub(fq_sqr(rr), J), fq_dbl(V));
    r.Y = fq_sub(fq_mul(rr, fq_sub(V, r.X)), fq_dbl(fq_mul(S1, J)));
    r.Z = fq_mul(fq_sub(fq_sub(fq_sqr(fq_add(p.Z, q.Z)), Z1Z1), Z2Z2), H);
    return r;
}

// k P for a small k, double-and-add from the top bit
DPB_HD G1Jac g1_mul_small(const G1Jac& p, uint32_t k) {
    G1Jac r = g1_infinity();
    int top = 31;
    while (top >= 0 && !((k >> top) & 1)) top--;
    for (int b = top; b >= 0; b--) {
        r = g1_double(r);
        if ((k >> b) & 1) r = g1_add(r, p);
    }
    return r;
}

// affine coordinates (one inversion)
DPB_HD G1Affine g1_to_affine(const G1Jac& p) {
    G1Affine r;
    if (g1_is_infinity(p)) {
        r.x = r.y = fq_zero();
        return r;
    }
    const Fq zi = fq_inv(p.Z), zi2 = fq_sqr(zi);
    r.x = fq_mul(p.X, zi2);
    r.y = fq_mul(p.Y, fq_mul(zi2, zi));
    return r;
}

DPB_HD bool g1_affine_on_curve(const G1Affine& p) {
    if (g1_affine_is_infinity(p)) return true;
    return fq_eq(fq_sqr(p.y), fq_add(fq_mul(fq_sqr(p.x), p.x), fq_three()));
}

}  // namespace dpb
