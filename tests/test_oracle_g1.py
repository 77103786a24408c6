"""Pins of the G1 oracle (oracle/g1.py): the curve's public constants and the group laws."""
import numpy as np

from oracle import g1


def test_generator_double_and_order():
    assert g1.on_curve(g1.GENERATOR)
    # the double of (1, 2), the well-known test vector of the curve's addition precompile
    assert g1.add(g1.GENERATOR, g1.GENERATOR) == (
        1368015179489954701390400359078579693043519447331113978918064868415326638035,
        9918110051302171585080402603319702774565515993150576347155970296011118125764)
    assert g1.mul(g1.R_ORDER, g1.GENERATOR) is None and g1.mul(g1.R_ORDER - 1, g1.GENERATOR) == g1.neg(g1.GENERATOR)


def test_group_laws_and_msm_linearity():
    rng = np.random.default_rng(1)
    pts = g1.synthetic_bases(6, seed=2)
    assert all(g1.on_curve(p) for p in pts) and len(set(pts)) == 6
    a, b, c = pts[:3]
    assert g1.add(g1.add(a, b), c) == g1.add(a, g1.add(b, c)) and g1.add(a, b) == g1.add(b, a)
    assert g1.add(a, g1.neg(a)) is None and g1.add(a, None) == a
    k1, k2 = int(rng.integers(1, 2**62)), int(rng.integers(1, 2**62))
    assert g1.mul(k1 + k2, a) == g1.add(g1.mul(k1, a), g1.mul(k2, a))
    s = [int(x) for x in rng.integers(-2**31, 2**31, size=6)]
    t = [int(x) for x in rng.integers(0, 2**62, size=6)]
    lhs = g1.msm([x + y for x, y in zip(s, t)], pts)
    assert lhs == g1.add(g1.msm(s, pts), g1.msm(t, pts))
