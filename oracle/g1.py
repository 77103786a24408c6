"""CPU restatement of the commit step's group arithmetic: BN254 G1 (y^2 = x^3 + 3 over Fq) with Python integers,
a naive multi-scalar multiplication, and a seeded synthetic set of G1 points standing in for a structured
reference string.

TEST INFRASTRUCTURE ONLY.  The reference's commitment scheme (HyperKZG in dp-crypto's arkyper module, rev 22e8e93)
is not part of the reference tree; its commit is, by the scheme's published definition, sum_i evals[i] * G_i
(the call site is CommittedPolynomial::batch_commit, zkml/src/poly_commit/context.rs:56-90).  Pinned by the curve's
public constants: the generator (1, 2) and its double (the EIP-196 test vector), the group order r, and the group
laws (tests/test_oracle_g1.py).  Points are (x, y) pairs, the point at infinity is None here and (0, 0) at the
library's boundary."""
import numpy as np

Q = 21888242871839275222246405745257275088696311157297823662689037894645226208583
R_ORDER = 21888242871839275222246405745257275088548364400416034343698204186575808495617
GENERATOR = (1, 2)


def on_curve(p):
    return p is None or (p[1] * p[1] - p[0] * p[0] * p[0] - 3) % Q == 0


def neg(p):
    return None if p is None else (p[0], (-p[1]) % Q)


def add(p, q):
    if p is None:
        return q
    if q is None:
        return p
    x1, y1 = p
    x2, y2 = q
    if x1 == x2:
        if (y1 + y2) % Q == 0:
            return None
        lam = 3 * x1 * x1 * pow(2 * y1, -1, Q) % Q
    else:
        lam = (y2 - y1) * pow(x2 - x1, -1, Q) % Q
    x3 = (lam * lam - x1 - x2) % Q
    return (x3, (lam * (x1 - x3) - y1) % Q)


def mul(k, p):
    k %= R_ORDER
    acc = None
    while k:
        if k & 1:
            acc = add(acc, p)
        p = add(p, p)
        k >>= 1
    return acc


def msm(scalars, points):
    """sum_i scalars[i] * points[i], term by term (scalars are integers mod r; negative ones allowed)."""
    acc = None
    for s, p in zip(scalars, points):
        acc = add(acc, mul(int(s) % R_ORDER, p))
    return acc


def synthetic_bases(n, seed=0):
    """n seeded G1 points: multiples of the generator by a running product of seeded factors.  They stand in for
    an SRS's powers (tau^i G): the MSM treats the points as opaque, and the group law is what is checked."""
    rng = np.random.default_rng(seed)
    out = []
    p = mul(int(rng.integers(2, 2**62)), GENERATOR)
    for _ in range(n):
        out.append(p)
        p = add(add(p, p), mul(int(rng.integers(1, 2**16)), GENERATOR))  # cheap, never repeats in practice
    return out


def boundary(p):
    return (0, 0) if p is None else p
