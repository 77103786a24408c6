"""Sumchecks whose terms are all led by an eq table (built with the library, so
the table knows its point) run their large rounds in split-eq form: the eq table
is read from its original instead of being bound, and one evaluation point less
is computed.  The messages must be the same field elements as the direct form's:
these cases are large enough to reach those rounds (more than 256 pairs) and are
checked against the oracle, with the resident last-rounds kernel on and off."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import family_dtype, gpu_sumcheck_prove, upload

pytestmark = pytest.mark.gpu

FIELDS = [orc.FrField, orc.GlField]


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("resident", [True, False])
def test_one_eq_group(dpb, ctx, F, resident):
    """eq * (c1 a b + c2 a c + d): one group, degree 3, 2^12 entries."""
    rng = np.random.default_rng(9000)
    n = 12
    point = [F.random_scalar(rng) for _ in range(n)]
    tabs = [F.random_table_fast(rng, 1 << n) for _ in range(4)]
    c = [F.random_scalar(rng) for _ in range(2)]
    terms = {(4, 0, 1): c[0], (4, 0, 2): c[1], (4, 3): F.one}
    want = orc.sumcheck_prove(F, n, tabs + [orc.eq_evals(F, point)], terms, orc.Transcript(F))
    mles = [upload(dpb, ctx, F, t) for t in tabs] + [ctx.eq_table(family_dtype(dpb, F), orc.scalars_to_array(F, point))]
    ctx.resident_rounds(resident)
    try:
        got = gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F))
    finally:
        ctx.resident_rounds(True)
    assert got == want


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("resident", [True, False])
def test_groups_of_different_sizes(dpb, ctx, F, resident):
    """The batched logup shape: a group over all 13 variables and a group over the last 11, whose eq table is the
    eq table of the point's suffix, so that the moving eq tables share their coordinate in every round."""
    rng = np.random.default_rng(9100)
    n, m = 13, 11
    point = [F.random_scalar(rng) for _ in range(n)]
    big = [F.random_table_fast(rng, 1 << n) for _ in range(4)]
    small = [F.random_table_fast(rng, 1 << m) for _ in range(4)]
    a, lam = F.random_scalar(rng), F.random_scalar(rng)
    # tables 0..3 big, 4..7 small, 8 = eq over n, 9 = eq over the last m coordinates
    terms = {(8, 0, 3): F.one, (8, 1, 2): F.one, (8, 2, 3): lam,
             (9, 4, 7): a, (9, 5, 6): a, (9, 6, 7): F.mul(a, lam)}
    tabs = big + small + [orc.eq_evals(F, point), orc.eq_evals(F, point[n - m:])]
    want = orc.sumcheck_prove(F, n, tabs, terms, orc.Transcript(F))
    fam = family_dtype(dpb, F)
    owner, eqs = dpb.eq_tables(ctx, fam, [orc.scalars_to_array(F, point), orc.scalars_to_array(F, point[n - m:])])
    mles = [upload(dpb, ctx, F, t) for t in big + small] + eqs
    ctx.resident_rounds(resident)
    try:
        got = gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F))
    finally:
        ctx.resident_rounds(True)
    assert got == want


@pytest.mark.parametrize("F", FIELDS)
def test_shapes_that_must_stay_direct(dpb, ctx, F):
    """Two eq tables over different points (same_poly's shape) and an eq table used inside a product do not
    factor; an uploaded copy of an eq table carries no point.  All must still give the oracle's proof."""
    rng = np.random.default_rng(9200)
    n = 11
    p1 = [F.random_scalar(rng) for _ in range(n)]
    p2 = [F.random_scalar(rng) for _ in range(n)]
    f, g = F.random_table_fast(rng, 1 << n), F.random_table_fast(rng, 1 << n)
    fam = family_dtype(dpb, F)
    cases = [
        ({(0, 2): F.random_scalar(rng), (0, 3): F.random_scalar(rng)}, [p1, p2]),   # different points
        ({(2, 0, 1): F.one, (0, 2, 2): F.random_scalar(rng)}, [p1]),               # eq squared inside a product
    ]
    for terms, pts in cases:
        eq_tabs = [orc.eq_evals(F, p) for p in pts]
        tabs = [f, g] + eq_tabs
        want = orc.sumcheck_prove(F, n, tabs, terms, orc.Transcript(F))
        mles = [upload(dpb, ctx, F, f), upload(dpb, ctx, F, g)] + \
               [ctx.eq_table(fam, orc.scalars_to_array(F, p)) for p in pts]
        assert gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F)) == want
        mles = [upload(dpb, ctx, F, t) for t in tabs]  # no table knows its point
        assert gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F)) == want


@pytest.mark.parametrize("F", FIELDS)
def test_logup_batch_large_enough_for_split_rounds(dpb, ctx, F):
    """Batched logup-GKR over 2^12 and 2^10 lookups: the top layers have more than 256 pairs."""
    from deep_prove_b200 import prover
    rng = np.random.default_rng(9300)
    fam = family_dtype(dpb, F)
    o_in, d_in = [], []
    for m in (12, 10):
        cols = [F.random_table_fast(rng, 1 << m) for _ in range(2)]
        cst, sep = F.random_scalar(rng), F.random_scalar(rng)
        o_in.append(orc.LogUpInput(F, 0, cols, cst, sep, columns_per_instance=1))
        d_in.append(prover.LogUpInput.new_lookup([upload(dpb, ctx, F, c) for c in cols], orc.scalars_to_array(F, [cst]),
                                                 orc.scalars_to_array(F, [sep]), 1))
    got = prover.new_batch_multiple_sizes_prove(ctx, d_in, prover.Blake3Transcript(fam))
    assert got == orc.serialize_logup_proof(F, orc.logup_batch_prove(F, o_in, orc.Transcript(F)))
