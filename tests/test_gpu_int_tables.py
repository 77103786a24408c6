"""Integer tables (DPB_GL_I64 / GL_I32 / FR_I64 / FR_I32): the quantised tensors and lookup columns stay integers on
the device and stand for the field elements they map to (negative x -> p - |x|, zkml/src/quantization/mod.rs:220-267).
Everything computed from them must be bit-identical to what the oracle computes from the converted tables: the
product sumcheck (BN254 32-bit tables run their first round in integer arithmetic and their first fold through two
precomputed rows; every other layout converts at load), generic term lists that mix integer and field tables, folds,
evaluation, the linear combination and the logup fraction tree."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import family_dtype, gpu_sumcheck_prove, upload

pytestmark = pytest.mark.gpu

FIELDS = [orc.FrField, orc.GlField]


def int_dtypes(dpb, F):
    return (dpb.FR_I32, dpb.FR_I64) if F is orc.FrField else (dpb.GL_I32, dpb.GL_I64)


def draw(rng, dpb, dtype, n):
    if dtype in (dpb.FR_I32, dpb.GL_I32):
        x = rng.integers(-2**31, 2**31, size=n, dtype=np.int64)
        x[:4] = [-2**31, 2**31 - 1, 0, -1][: min(4, n)]
    else:
        x = rng.integers(-2**63, 2**63 - 1, size=n, dtype=np.int64, endpoint=True)
        x[:4] = [-2**63, 2**63 - 1, 0, -1][: min(4, n)]
    if n > 8:
        x[8::5] >>= 20  # small magnitudes too (16-bit lookup chunks, 12-bit weights)
    return x


@pytest.mark.parametrize("F", FIELDS)
def test_round_trip_fold_evaluate(dpb, ctx, F):
    rng = np.random.default_rng(8100)
    for dt in int_dtypes(dpb, F):
        n = 11
        x = draw(rng, dpb, dt, 1 << n)
        m = ctx.upload_ints(x, dt)
        assert m.dtype == dt and np.array_equal(m.to_host(), x.astype(dpb.INT_DTYPES[dt]))
        t = F.table_from_i64(x)
        pt = [F.random_scalar(rng) for _ in range(n)]
        pa = orc.scalars_to_array(F, pt)
        assert orc.array_to_scalars(F, ctx.evaluate(m, pa))[0] == orc.evaluate(F, t, pt)
        for k in (1, 4, 7):
            assert (ctx.fix_high(m, pa[:k]).to_host() == orc.fix_high_variables(F, t, pt[:k])).all()
            assert (ctx.fix_low(m, pa[:k]).to_host() == orc.fix_low_variables(F, t, pt[:k])).all()
        one = ctx.upload_ints(x[:1], dt)  # a one-entry table: its value, widened on the host
        want_one = F.from_int(int(x[0]))
        assert orc.array_to_scalars(F, ctx.evaluate(one, np.zeros((0, F.elem_words), np.uint64)))[0] == want_one
        c = [F.random_scalar(rng), F.random_scalar(rng)]
        other = F.random_table_fast(rng, 1 << n)
        lc = dpb.linear_combination(ctx, [m, upload(dpb, ctx, F, other)], orc.scalars_to_array(F, c))
        assert (lc.to_host() == orc.linear_combination(F, [t, other], c)).all()


@pytest.mark.parametrize("n", [2, 3, 4, 5, 8, 13, 16, 20, 21])
@pytest.mark.parametrize("k", [2, 3])
def test_product_sumcheck_over_int32_tables_bn254(dpb, ctx, n, k):
    """The integer rounds of the BN254 family: every round message, the point and the final evaluations equal the
    oracle's over the converted tables, from two variables up to the sizes where grids wrap around."""
    F = orc.FrField
    rng = np.random.default_rng(8200 + 10 * n + k)
    xs = [draw(rng, dpb, dpb.FR_I32, 1 << n) for _ in range(k)]
    terms = {tuple(range(k)): F.one}
    want = orc.sumcheck_prove(F, n, [F.table_from_i64(x) for x in xs], terms, orc.Transcript(F))
    mles = [ctx.upload_ints(x, dpb.FR_I32) for x in xs]
    got = gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F))
    assert got == want
    for m, x in zip(mles, xs):
        assert np.array_equal(m.to_host(), x.astype(np.int32))  # borrowed, not modified
        m.free()


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("n", [6, 14])
def test_product_sumcheck_other_int_layouts(dpb, ctx, F, n):
    """64-bit integers of both families, 32-bit integers over Goldilocks and a product of four 32-bit tables over
    BN254: converted at load by the general rounds."""
    rng = np.random.default_rng(8300 + n)
    cases = [(dt, 3) for dt in int_dtypes(dpb, F)] + [(int_dtypes(dpb, F)[0], 4)]
    for dt, k in cases:
        xs = [draw(rng, dpb, dt, 1 << n) for _ in range(k)]
        terms = {tuple(range(k)): F.one}
        want = orc.sumcheck_prove(F, n, [F.table_from_i64(x) for x in xs], terms, orc.Transcript(F))
        mles = [ctx.upload_ints(x, dt) for x in xs]
        assert gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F)) == want


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("n", [5, 12, 17])
def test_mixed_integer_and_field_tables(dpb, ctx, F, n):
    """A term list over integer tables of both widths, field tables, a smaller table and an eq table: the shape of
    a linking sumcheck whose witness columns stayed integers."""
    rng = np.random.default_rng(8400 + n)
    d32, d64 = int_dtypes(dpb, F)
    x0, x1, x2 = draw(rng, dpb, d32, 1 << n), draw(rng, dpb, d64, 1 << n), draw(rng, dpb, d32, 1 << (n - 2))
    f3 = F.random_table_fast(rng, 1 << n)
    pt = [F.random_scalar(rng) for _ in range(n)]
    c = [F.random_scalar(rng) for _ in range(3)]
    terms = {(4, 0, 1): c[0], (4, 0, 0, 3): c[1], (4, 2): F.one, (1, 3): c[2], (0,): F.one}
    tabs = [F.table_from_i64(x0), F.table_from_i64(x1), F.table_from_i64(x2), f3, orc.eq_evals(F, pt)]
    want = orc.sumcheck_prove(F, n, tabs, terms, orc.Transcript(F))
    mles = [ctx.upload_ints(x0, d32), ctx.upload_ints(x1, d64), ctx.upload_ints(x2, d32), upload(dpb, ctx, F, f3),
            ctx.eq_table(family_dtype(dpb, F), orc.scalars_to_array(F, pt))]
    assert gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F)) == want


@pytest.mark.parametrize("F", FIELDS)
def test_logup_tree_over_integer_columns(dpb, ctx, F):
    """Lookup columns are 16-bit chunks: the fraction tree built from 32-bit integer columns equals the oracle's
    tree over the converted columns, level by level."""
    rng = np.random.default_rng(8500)
    m = 12
    d32 = int_dtypes(dpb, F)[0]
    cols = [rng.integers(-2**15, 2**15, size=1 << m, dtype=np.int64) for _ in range(2)]
    cst, sep = F.random_scalar(rng), F.random_scalar(rng)
    want = orc.LogUpCircuit(F, 0, [F.table_from_i64(c) for c in cols], None, cst, sep)
    lu = ctx.logup(0, [ctx.upload_ints(c, d32) for c in cols], orc.scalars_to_array(F, [cst]),
                   orc.scalars_to_array(F, [sep]))
    for l in range(1, m):
        num, den = want.levels[l]
        half = num.shape[0] // 2
        got = [v.to_host() for v in lu.level(l)]
        assert (got[0] == num[:half]).all() and (got[1] == num[half:]).all()
        assert (got[2] == den[:half]).all() and (got[3] == den[half:]).all()
    assert orc.array_to_scalars(F, lu.outputs()) == want.outputs()


def test_integer_tables_argument_errors(dpb, ctx):
    x = np.arange(16, dtype=np.int64)
    with pytest.raises(dpb.DpbError) as e:
        import ctypes
        h = ctypes.c_void_p()
        dpb.check(dpb.lib.dpb_mle_from_host(ctx.h, dpb.FR_I64, x.ctypes.data, 16, dpb.FORM_I64, ctypes.byref(h)))
    assert e.value.code == dpb.EINVAL
    a, b = ctx.upload_ints(x, dpb.FR_I64), ctx.upload_ints(x, dpb.GL_I64)
    F = orc.FrField
    with pytest.raises(dpb.DpbError) as e:  # integer tables carry their family: no mixing
        ctx.sumcheck(4, [a, b], dpb.make_terms([(F.one, [0, 1])], F.to_native))
    assert e.value.code == dpb.EINVAL
