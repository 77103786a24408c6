"""Multi-scalar multiplication over BN254 G1 (dpb_msm_g1, dpb_pcs_batch_commit: the commit of the polynomial
commitment scheme, zkml/src/poly_commit/context.rs:56-90) against the Python restatement of the group law
(oracle/g1.py).  Group arithmetic is exact, so results are compared as integers.  Small sizes against the naive
sum; the window sizes that large inputs select through sparse scalars and repeated points; the full chunk size 2^20
through linearity."""
import importlib

import numpy as np
import pytest

from oracle import g1
from oracle import oracle as orc

pytestmark = pytest.mark.gpu

F = orc.FrField


@pytest.fixture(scope="module")
def pcs(dpb):
    return importlib.import_module("deep_prove_b200.pcs")


@pytest.fixture(scope="module")
def points():
    return g1.synthetic_bases(1024, seed=5)


def fr_table(vals):
    return F.table_from_ints([int(v) % g1.R_ORDER for v in vals])


@pytest.mark.parametrize("n", [1, 2, 16, 256])
def test_msm_full_width_scalars(dpb, ctx, pcs, points, n):
    rng = np.random.default_rng(6000 + n)
    scalars = [F.random_scalar(rng) for _ in range(n)]
    if n >= 16:
        scalars[0], scalars[1], scalars[2] = 0, g1.R_ORDER - 1, 1
    bases = pcs.G1Bases(ctx, points[:n])
    got = pcs.msm(ctx, bases, ctx.upload(fr_table(scalars), dpb.FR))
    assert got == g1.boundary(g1.msm(scalars, points[:n]))
    bases.free()


def test_msm_special_cases(dpb, ctx, pcs, points):
    """The same point twice in one bucket (a doubling), a point and its negative in one bucket (infinity), all
    scalars zero, and the empty sum."""
    p = points[3]
    pts = [p, p, g1.neg(p), points[4]]
    bases = pcs.G1Bases(ctx, pts)
    for scalars in ([5, 5, 0, 0], [7, 0, 7, 0], [7, 7, 7, 9], [0, 0, 0, 0], [g1.R_ORDER - 2, 2, 0, 1]):
        got = pcs.msm(ctx, bases, ctx.upload(fr_table(scalars), dpb.FR))
        assert got == g1.boundary(g1.msm(scalars, pts))
    bases.free()
    with pytest.raises(dpb.DpbError) as e:
        pcs.G1Bases(ctx, [(1, 3)])  # not on the curve
    assert e.value.code == dpb.EINVAL
    with pytest.raises(dpb.DpbError) as e:
        pcs.G1Bases(ctx, [(g1.Q + 1, 2)])  # coordinate not reduced
    assert e.value.code == dpb.EINVAL


@pytest.mark.parametrize("dtype_name", ["FR_I32", "FR_I64"])
def test_msm_integer_tables(dpb, ctx, pcs, points, dtype_name):
    """Quantised tensors and lookup columns commit as integers: negative entries add the negated point."""
    dt = getattr(dpb, dtype_name)
    rng = np.random.default_rng(6100)
    n = 1024
    lim = 2**31 if dtype_name == "FR_I32" else 2**63
    x = rng.integers(-lim, lim, size=n, dtype=np.int64)
    x[:4] = [0, -1, lim - 1, -lim]
    x[8::3] >>= 18
    bases = pcs.G1Bases(ctx, points)
    got = pcs.msm(ctx, bases, ctx.upload_ints(x, dt))
    assert got == g1.boundary(g1.msm([int(v) for v in x], points))
    # the same integers as field elements give the same commitment
    assert pcs.msm(ctx, bases, ctx.upload(F.table_from_i64(x), dpb.FR)) == got
    bases.free()


@pytest.mark.parametrize("log2_n", [14, 18])
def test_msm_large_window_sizes(dpb, ctx, pcs, points, log2_n):
    """2^14 and 2^18 scalars select windows of 13 and 16 bits.  The points are the 1024 distinct ones repeated, the
    scalars are zero except at 300 places, so the naive sum stays affordable."""
    rng = np.random.default_rng(6200 + log2_n)
    n = 1 << log2_n
    reps = n // len(points)
    arr = np.tile(pcs.points_to_array(points), (reps, 1))
    bases = pcs.G1Bases(ctx, arr)
    where = rng.choice(n, size=300, replace=False)
    vals = [F.random_scalar(rng) for _ in range(300)]
    table = np.zeros((n, 4), dtype=np.uint64)
    table[where] = F.table_from_ints(vals)
    got = pcs.msm(ctx, bases, ctx.upload(table, dpb.FR))
    assert got == g1.boundary(g1.msm(vals, [points[i % len(points)] for i in where]))
    bases.free()


def test_commit_is_linear_at_the_full_chunk_size(dpb, ctx, pcs, points):
    """2^20 evaluations (the largest chunk the reference commits to): commit(s) + commit(t) = commit(s + t) and
    commit(3 s) = 3 commit(s), for dense 32-bit integer tables, and batch_commit returns the single commits."""
    rng = np.random.default_rng(6300)
    n = 1 << 20
    arr = np.tile(pcs.points_to_array(points), (n // len(points), 1))
    bases = pcs.G1Bases(ctx, arr)
    s = rng.integers(-2**30, 2**30, size=n, dtype=np.int64)
    t = rng.integers(-2**30, 2**30, size=n, dtype=np.int64)
    ms, mt, mst = ctx.upload_ints(s, dpb.FR_I32), ctx.upload_ints(t, dpb.FR_I32), ctx.upload_ints(s + t, dpb.FR_I64)
    cs, ct, cst = pcs.batch_commit(ctx, bases, [ms, mt, mst])
    point = lambda c: None if c == (0, 0) else c
    assert g1.on_curve(point(cs)) and g1.add(point(cs), point(ct)) == point(cst)
    assert pcs.msm(ctx, bases, ms) == cs
    assert point(pcs.msm(ctx, bases, ctx.upload_ints(3 * s, dpb.FR_I64))) == g1.mul(3, point(cs))
    # and with full-width field scalars: commit(f) + commit(-f) = 0, commit(f) + commit(s) = commit(f + s)
    f = F.random_table_fast(rng, n)
    cf = pcs.msm(ctx, bases, ctx.upload(f, dpb.FR))
    lc = dpb.linear_combination(ctx, [ctx.upload(f, dpb.FR), ms], orc.scalars_to_array(F, [F.one, F.one]))
    assert g1.add(point(cf), point(cs)) == point(pcs.msm(ctx, bases, lc))
    neg = dpb.linear_combination(ctx, [ctx.upload(f, dpb.FR)], orc.scalars_to_array(F, [F.neg(F.one)]))
    assert g1.add(point(cf), point(pcs.msm(ctx, bases, neg))) is None
    bases.free()


@pytest.mark.parametrize("values", ["few", "int16"])
def test_msm_crowded_buckets(dpb, ctx, pcs, values):
    """Columns of few distinct values (signs, zero checks) and 16-bit chunks put tens of thousands of points into a
    handful of buckets: those are summed in chunks of 2048 points by many blocks.  The bases are the consecutive
    multiples of the generator, so sum_i s_i (i + 1) G is ONE scalar multiplication on the CPU side."""
    rng = np.random.default_rng(6400)
    n = 1 << 17
    if values == "few":
        x = rng.choice(np.array([0, 1, -1, 2, 255], dtype=np.int64), size=n)
    else:
        x = rng.integers(0, 1 << 16, size=n, dtype=np.int64)  # 13-bit window: the second window has 7 huge buckets
    bases = pcs.G1Bases.synthetic(ctx, n)
    k = int(sum(int(v) * (i + 1) for i, v in enumerate(x)) % g1.R_ORDER)
    want = g1.boundary(g1.mul(k, g1.GENERATOR))
    for dt in (dpb.FR_I32, dpb.FR_I64):
        assert pcs.msm(ctx, bases, ctx.upload_ints(x, dt)) == want
    assert pcs.msm(ctx, bases, ctx.upload(F.table_from_i64(x), dpb.FR)) == want
    bases.free()


def test_batch_commit_many_polynomials(dpb, ctx, pcs):
    """More polynomials than are in flight together (16), of mixed sizes and layouts: batch_commit returns what one
    commitment at a time returns, and what one scalar multiplication gives on the CPU side."""
    rng = np.random.default_rng(6500)
    bases = pcs.G1Bases.synthetic(ctx, 1 << 12)
    polys, want = [], []
    for i in range(40):
        n = 1 << int(rng.integers(0, 13))
        x = rng.integers(-(1 << 20), 1 << 20, size=n, dtype=np.int64)
        if i % 3 == 0:
            polys.append(ctx.upload(F.table_from_i64(x), dpb.FR))
        else:
            polys.append(ctx.upload_ints(x, dpb.FR_I32 if i % 3 == 1 else dpb.FR_I64))
        k = int(sum(int(v) * (j + 1) for j, v in enumerate(x)) % g1.R_ORDER)
        want.append(g1.boundary(g1.mul(k, g1.GENERATOR)) if k else (0, 0))
    got = pcs.batch_commit(ctx, bases, polys)
    assert list(got) == want
    assert [pcs.msm(ctx, bases, p) for p in polys[:5]] == want[:5]
    bases.free()
