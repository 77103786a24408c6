"""GPU parity tests of the C-ABI primitives against the CPU oracle and the
committed fixtures.  Everything here is exact field arithmetic, so the bar is
bit-for-bit equality of every round message, folded table and tree level."""
import json
import os

import numpy as np
import pytest

from oracle import oracle as orc
from tests.golden import make_golden
from tests.helpers import family_dtype, gpu_sumcheck_prove, terms_array, upload

pytestmark = pytest.mark.gpu

FIELDS = [orc.FrField, orc.GlField]
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def golden(F):
    with open(os.path.join(GOLDEN, f"oracle_{F.name}.json")) as f:
        return json.load(f)


def hx(F, vals):
    return orc.serialize_scalars(F, vals).hex()


# ------------------------------------------------------------------ tables
def test_upload_forms(dpb, ctx):
    F = orc.FrField
    rng = np.random.default_rng(1)
    vals = [F.random_scalar(rng) for _ in range(64)]
    canon = np.frombuffer(b"".join(v.to_bytes(32, "little") for v in vals), dtype=np.uint64).reshape(-1, 4).copy()
    m = ctx.upload(canon, dpb.FR, dpb.FORM_CANONICAL)
    assert (m.to_host() == F.table_from_ints(vals)).all()
    assert (m.to_host(dpb.FORM_CANONICAL) == canon).all()
    xs = rng.integers(-2**62, 2**62, size=128, dtype=np.int64)
    xs[:4] = [0, -1, 1, -2**63 + 1]
    assert (ctx.upload_i64(xs, dpb.FR).to_host() == F.table_from_i64(xs)).all()
    assert (ctx.upload_i64(xs, dpb.GL_BASE).to_host() == orc.GlField.table_from_i64(xs)).all()


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("m", [0, 1, 5, 10, 11, 14])
def test_eq_table(dpb, ctx, F, m):
    rng = np.random.default_rng(10 + m)
    pt = [F.random_scalar(rng) for _ in range(m)]
    got = ctx.eq_table(family_dtype(dpb, F), orc.scalars_to_array(F, pt) if m else np.zeros((0, F.elem_words), np.uint64))
    assert (got.to_host() == orc.eq_evals(F, pt)).all()


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("n,k", [(7, 3), (12, 1), (12, 5), (12, 7), (12, 12), (17, 11)])
def test_fix_high_low(dpb, ctx, F, n, k):
    rng = np.random.default_rng(100 + n + k)
    t = F.random_table_fast(rng, 1 << n)
    pt = [F.random_scalar(rng) for _ in range(k)]
    m = upload(dpb, ctx, F, t)
    pa = orc.scalars_to_array(F, pt)
    assert (ctx.fix_high(m, pa).to_host() == orc.fix_high_variables(F, t, pt)).all()
    assert (ctx.fix_low(m, pa).to_host() == orc.fix_low_variables(F, t, pt)).all()


@pytest.mark.parametrize("F", FIELDS)
def test_fix_golden_and_evaluate(dpb, ctx, F):
    g = make_golden.golden_inputs(F, "fix")
    want = golden(F)
    m = upload(dpb, ctx, F, g["table"])
    pa = orc.scalars_to_array(F, g["point"])
    assert hx(F, orc.array_to_scalars(F, ctx.eq_table(family_dtype(dpb, F), pa[:4]).to_host())) == want["eq"]
    assert hx(F, orc.array_to_scalars(F, ctx.fix_high(m, pa[:3]).to_host())) == want["fix_high3"]
    assert hx(F, orc.array_to_scalars(F, ctx.fix_low(m, pa[:3]).to_host())) == want["fix_low3"]
    assert hx(F, orc.array_to_scalars(F, ctx.evaluate(m, pa))) == want["evaluate"]


@pytest.mark.parametrize("F", FIELDS)
def test_evaluate_little_endian(dpb, ctx, F):
    """zkml/src/lib.rs:357-369"""
    rng = np.random.default_rng(5)
    n = 9
    t = F.random_table(rng, 1 << n)
    m = upload(dpb, ctx, F, t)
    vals = F.table_to_ints(t)
    for idx in [0, 1, 77, 511]:
        pt = orc.scalars_to_array(F, [F.from_int((idx >> j) & 1) for j in range(n)])
        assert orc.array_to_scalars(F, ctx.evaluate(m, pt))[0] == vals[idx]


# ----------------------------------------------------------------- sumcheck
def product_case(F, rng, n, k, ext):
    if F is orc.GlField and ext:
        return [F.random_ext_table(rng, 1 << n) for _ in range(k)]
    return [F.random_table_fast(rng, 1 << n) for _ in range(k)]


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("n", [1, 2, 3, 4, 5, 6, 9, 13, 16])
@pytest.mark.parametrize("k", [2, 3, 4])
def test_product_sumcheck(dpb, ctx, F, n, k):
    """Single product of k full-size tables (the fused kernels), all rounds
    and final evaluations against the oracle."""
    rng = np.random.default_rng(1000 + 10 * n + k)
    for ext in ([False, True] if F is orc.GlField else [False]):
        tabs = product_case(F, rng, n, k, ext)
        terms = {tuple(range(k)): F.one}
        want = orc.sumcheck_prove(F, n, tabs, terms, orc.Transcript(F))
        mles = [upload(dpb, ctx, F, t) for t in tabs]
        got = gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F))
        assert got == want
        # inputs are borrowed, not modified
        for m, t in zip(mles, tabs):
            assert (m.to_host() == t).all()
            m.free()


@pytest.mark.parametrize("F,n,k", [(orc.GlField, 20, 2), (orc.GlField, 20, 3), (orc.GlField, 20, 4),
                                   (orc.GlField, 21, 3), (orc.GlField, 22, 3), (orc.FrField, 20, 2),
                                   (orc.FrField, 20, 3), (orc.FrField, 20, 4)])
def test_product_sumcheck_large(dpb, ctx, F, n, k):
    """The sizes at which the launcher picks the staged kernels (a launch with at least two items per thread of a
    full grid, i.e. 2^20 entries and up on a 148-SM part): round 0 over base or extension tables, round 1 with base
    or extension input, later rounds staged until they become too small, then the unstaged kernels and the resident
    one.  Every round message, the point and the final evaluations against the oracle."""
    rng = np.random.default_rng(7000 + 10 * n + k)
    for ext in ([False, True] if F is orc.GlField else [False]):
        tabs = product_case(F, rng, n, k, ext)
        terms = {tuple(range(k)): F.one}
        want = orc.sumcheck_prove(F, n, tabs, terms, orc.Transcript(F))
        mles = [upload(dpb, ctx, F, t) for t in tabs]
        got = gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F))
        assert got[0] == want[0]
        assert got[1:] == want[1:]
        for m, t in zip(mles, tabs):
            assert (m.to_host() == t).all()
            m.free()


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("k", [1, 10, 22])
def test_fix_high_low_large(dpb, ctx, F, k):
    """2^22 entries: several passes of up to five variables, grids larger than one wave."""
    n = 22
    rng = np.random.default_rng(7100 + k)
    t = F.random_table_fast(rng, 1 << n)
    pt = [F.random_scalar(rng) for _ in range(k)]
    m = upload(dpb, ctx, F, t)
    pa = orc.scalars_to_array(F, pt)
    assert (ctx.fix_high(m, pa).to_host() == orc.fix_high_variables(F, t, pt)).all()
    assert (ctx.fix_low(m, pa).to_host() == orc.fix_low_variables(F, t, pt)).all()
    m.free()


@pytest.mark.parametrize("F", FIELDS)
def test_product_sumcheck_golden(dpb, ctx, F):
    g = make_golden.golden_inputs(F, "prod3")
    mles = [upload(dpb, ctx, F, t) for t in g["tables"]]
    proof, point, finals = gpu_sumcheck_prove(dpb, ctx, F, g["n"], mles, {(0, 1, 2): F.one}, orc.Transcript(F))
    want = golden(F)["prod3"]
    assert orc.serialize_sumcheck_proof(F, proof).hex() == want["proof"]
    assert hx(F, point) == want["point"] and hx(F, finals) == want["finals"]


@pytest.mark.parametrize("F", FIELDS)
def test_generic_sumcheck_golden(dpb, ctx, F):
    """Tables of different sizes, coefficients, a repeated factor and a bare
    table term: the generic evaluation and fold kernels."""
    g = make_golden.golden_inputs(F, "mixed")
    mles = [upload(dpb, ctx, F, t) for t in g["tables"]]
    terms = make_golden.mixed_terms(F, g["coeffs"])
    proof, point, finals = gpu_sumcheck_prove(dpb, ctx, F, g["n"], mles, terms, orc.Transcript(F))
    want = golden(F)["mixed"]
    assert orc.serialize_sumcheck_proof(F, proof).hex() == want["proof"]
    assert hx(F, point) == want["point"] and hx(F, finals) == want["finals"]


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("n", [3, 8, 14])
def test_generic_sumcheck_random(dpb, ctx, F, n):
    rng = np.random.default_rng(2000 + n)
    sizes = [n, n, n - 1, n - 2, n, 1]
    tabs = [F.random_table_fast(rng, 1 << s) for s in sizes]
    if F is orc.GlField:
        tabs[4] = F.random_ext_table(rng, 1 << n)
    c = [F.random_scalar(rng) for _ in range(4)]
    terms = {(0, 1): c[0], (0, 2, 3): c[1], (4, 4, 1, 3, 5): c[2], (2,): c[3], (1, 4): F.one}
    want = orc.sumcheck_prove(F, n, tabs, terms, orc.Transcript(F))
    mles = [upload(dpb, ctx, F, t) for t in tabs]
    got = gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F))
    assert got == want


@pytest.mark.parametrize("F", FIELDS)
def test_hadamard_shape(dpb, ctx, F):
    """zkml/src/layers/hadamard.rs:93-131 with i64 inputs and a device-built eq table."""
    g = make_golden.golden_inputs(F, "hadamard")
    v1, v2 = upload(dpb, ctx, F, g["v1"]), upload(dpb, ctx, F, g["v2"])
    beta = ctx.eq_table(family_dtype(dpb, F), orc.scalars_to_array(F, g["point"]))
    proof, point, finals = gpu_sumcheck_prove(dpb, ctx, F, g["n"], [v1, v2, beta], {(0, 1, 2): F.one},
                                              orc.Transcript(F))
    want = golden(F)["hadamard"]
    assert orc.serialize_sumcheck_proof(F, proof).hex() == want["proof"]
    assert hx(F, point) == want["point"] and hx(F, finals[:2]) == want["claims"]


def test_sumcheck_state_errors(dpb, ctx):
    F = orc.GlField
    rng = np.random.default_rng(3)
    tabs = [upload(dpb, ctx, F, F.random_table(rng, 8)) for _ in range(2)]
    sc = ctx.sumcheck(3, tabs, terms_array(dpb, F, {(0, 1): F.one}))
    r = orc.scalars_to_array(F, [F.random_scalar(rng)])
    with pytest.raises(dpb.DpbError) as e:
        sc.finish(r)
    assert e.value.code == dpb.ESTATE
    sc.round(None)
    with pytest.raises(dpb.DpbError) as e:
        sc.round(None)  # later rounds need the challenge
    assert e.value.code == dpb.ESTATE
    sc.round(r)
    sc.round(r)
    with pytest.raises(dpb.DpbError) as e:
        sc.round(r)
    assert e.value.code == dpb.ESTATE
    sc.finish(r)
    sc.free()
    with pytest.raises(dpb.DpbError) as e:
        ctx.sumcheck(2, tabs, terms_array(dpb, F, {(0, 1): F.one}))  # tables larger than the sumcheck
    assert e.value.code == dpb.EINVAL
    with pytest.raises(dpb.DpbError) as e:
        ctx.sumcheck(3, tabs, terms_array(dpb, F, {(0, 5): F.one}))  # unknown table id
    assert e.value.code == dpb.EINVAL
    fr_tab = upload(dpb, ctx, orc.FrField, orc.FrField.random_table(rng, 8))
    with pytest.raises(dpb.DpbError) as e:
        ctx.sumcheck(3, [tabs[0], fr_tab], terms_array(dpb, F, {(0, 1): F.one}))  # mixed fields
    assert e.value.code == dpb.EINVAL


# -------------------------------------------------------------------- logup
@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("kind,ncols,m", [(0, 1, 2), (0, 1, 10), (0, 2, 7), (1, 2, 6), (1, 1, 12), (0, 3, 15)])
def test_logup_tree_levels(dpb, ctx, F, kind, ncols, m):
    """Every level of the fraction tree and the circuit outputs
    (zkml/src/lookup/logup_gkr/circuit.rs:88-184, 512-516, 558-560)."""
    rng = np.random.default_rng(3000 + 10 * m + ncols + kind)
    cols = [F.random_table_fast(rng, 1 << m) for _ in range(ncols)]
    mult = F.table_from_ints([int(x) for x in rng.integers(0, 9, size=1 << m)]) if kind == 1 else None
    cst, sep = F.random_scalar(rng), F.random_scalar(rng)
    want = orc.LogUpCircuit(F, kind, cols, mult, cst, sep)
    d_cols = [upload(dpb, ctx, F, c) for c in cols]
    d_mult = upload(dpb, ctx, F, mult) if kind == 1 else None
    lu = ctx.logup(kind, d_cols, orc.scalars_to_array(F, [cst]), orc.scalars_to_array(F, [sep]), d_mult)
    assert lu.num_levels == m - 1
    for l in range(1, m):
        num, den = want.levels[l]
        half = num.shape[0] // 2
        views = lu.level(l)
        got = [v.to_host() for v in views]
        assert (got[0] == num[:half]).all() and (got[1] == num[half:]).all()
        assert (got[2] == den[:half]).all() and (got[3] == den[half:]).all()
        for v in views:
            v.free()
    assert orc.array_to_scalars(F, lu.outputs()) == want.outputs()
    lu.free()


@pytest.mark.parametrize("F", FIELDS)
def test_logup_output_identity(dpb, ctx, F):
    """zkml/src/lookup/logup_gkr/circuit.rs:603-624: constant 0, separator 1 ->
    output fraction = -sum 1/v, on a 2^10 column as in the reference test."""
    rng = np.random.default_rng(4)
    col = F.random_table(rng, 1 << 10)
    lu = ctx.logup(0, [upload(dpb, ctx, F, col)], orc.scalars_to_array(F, [F.zero]),
                   orc.scalars_to_array(F, [F.one]))
    out = orc.array_to_scalars(F, lu.outputs())
    want = F.zero
    for v in F.table_to_ints(col):
        want = F.sub(want, F.inv(v))
    num = F.add(F.mul(out[0], out[3]), F.mul(out[1], out[2]))
    assert F.mul(num, F.inv(F.mul(out[2], out[3]))) == want


def test_logup_argument_errors(dpb, ctx):
    F = orc.FrField
    rng = np.random.default_rng(6)
    a = upload(dpb, ctx, F, F.random_table(rng, 16))
    b = upload(dpb, ctx, F, F.random_table(rng, 8))
    one = orc.scalars_to_array(F, [F.one])
    with pytest.raises(dpb.DpbError) as e:
        ctx.logup(0, [a, b], one, one)  # unequal lengths (structs.rs:175-181)
    assert e.value.code == dpb.EINVAL
    with pytest.raises(dpb.DpbError) as e:
        ctx.logup(1, [a], one, one)  # a table needs multiplicities
    assert e.value.code == dpb.EINVAL
    with pytest.raises(dpb.DpbError) as e:
        ctx.logup(1, [a], one, one, b)  # multiplicities of the wrong length (structs.rs:221-226)
    assert e.value.code == dpb.EINVAL
