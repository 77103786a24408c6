"""Claim batching of the opening proof (zkml/src/poly_commit/prover.rs:113-131,
140-255): zero-padded tables in a sumcheck, the random linear combination,
and the whole entry point against the oracle, bit for bit.  Shapes follow the
reference's own test (zkml/src/poly_commit/mod.rs:224-398): a handful of
polynomials of different sizes, one or two claims each, with and without
chunking."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import family_dtype, gpu_sumcheck_prove, upload

pytestmark = pytest.mark.gpu

FIELDS = [orc.FrField, orc.GlField]


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("n", [3, 6, 11])
def test_zero_padded_sumcheck(dpb, ctx, F, n):
    """Tables of fewer variables entered as zero-padded views: every round message, the point and the final
    evaluations equal the oracle's run on the materialised (zeros appended) tables."""
    rng = np.random.default_rng(8000 + n)
    sizes = [n, n - 1, max(n - 3, 1), 1, n - 2, n]
    tabs = [F.random_table_fast(rng, 1 << s) for s in sizes]
    c = [F.random_scalar(rng) for _ in range(3)]
    terms = {(0, 1): c[0], (1, 2, 5): c[1], (3, 4): c[2], (4, 5): F.one, (2,): F.one}
    want = orc.sumcheck_prove(F, n, [orc.zero_pad_table(F, t, n) for t in tabs], terms, orc.Transcript(F))
    owned = [upload(dpb, ctx, F, t) for t in tabs]
    views = [m.zero_padded() for m in owned]
    got = gpu_sumcheck_prove(dpb, ctx, F, n, views, terms, orc.Transcript(F))
    assert got == want
    for m, t in zip(owned, tabs):
        assert (m.to_host() == t).all()  # inputs are borrowed, not modified
    for m in views + owned:
        m.free()


@pytest.mark.parametrize("F", FIELDS)
def test_zero_padded_and_suffix_tables_together(dpb, ctx, F):
    """A smaller table WITHOUT the flag is a function of the last variables; with it, of the first."""
    rng = np.random.default_rng(8100)
    n = 7
    full, small_a, small_b = (F.random_table_fast(rng, 1 << s) for s in (n, 4, 4))
    terms = {(0, 1): F.one, (0, 2): F.random_scalar(rng)}
    # oracle: table 1 zero-padded (materialised), table 2 left small (suffix semantics are the oracle's default)
    want = orc.sumcheck_prove(F, n, [full, orc.zero_pad_table(F, small_a, n), small_b], terms, orc.Transcript(F))
    m = [upload(dpb, ctx, F, t) for t in (full, small_a, small_b)]
    pa = m[1].zero_padded()
    got = gpu_sumcheck_prove(dpb, ctx, F, n, [m[0], pa, m[2]], terms, orc.Transcript(F))
    assert got == want


@pytest.mark.parametrize("F", FIELDS)
def test_linear_combination(dpb, ctx, F):
    rng = np.random.default_rng(8200)
    tabs = [F.random_table_fast(rng, 1 << s) for s in (9, 4, 9, 1, 7)]
    coeffs = [F.random_scalar(rng) for _ in tabs]
    mles = [upload(dpb, ctx, F, t) for t in tabs]
    got = dpb.linear_combination(ctx, mles, orc.scalars_to_array(F, coeffs))
    assert (got.to_host() == orc.linear_combination(F, tabs, coeffs)).all()
    assert got.len == 1 << 9


@pytest.mark.parametrize("F", FIELDS)
def test_eq_tables_batch(dpb, ctx, F):
    """Many eq tables in one call equal the oracle's, table by table (sizes 0 .. 13 variables, odd and even)."""
    rng = np.random.default_rng(8250)
    sizes = [5, 0, 1, 12, 3, 13, 2, 8, 8, 1, 7]
    pts = [[F.random_scalar(rng) for _ in range(m)] for m in sizes]
    arrs = [orc.scalars_to_array(F, p) if p else np.zeros((0, F.elem_words), np.uint64) for p in pts]
    owner, tabs = dpb.eq_tables(ctx, family_dtype(dpb, F), arrs)
    for t, p in zip(tabs, pts):
        assert (t.to_host() == orc.eq_evals(F, p)).all()
    for t in tabs:
        t.free()
    owner.free()


def make_polys(F, rng, shapes):
    """shapes: (num_vars, num_chunks, num_claims) per polynomial -> oracle-side CommittedPoly list"""
    polys = []
    for nv, nchunks, nclaims in shapes:
        full = F.random_table_fast(rng, 1 << nv)
        m = nv - (nchunks.bit_length() - 1)
        chunks = [full[i << m:(i + 1) << m] for i in range(nchunks)]
        claims = []
        for _ in range(nclaims):
            pt = [F.random_scalar(rng) for _ in range(nv)]
            claims.append((pt, orc.evaluate(F, full, pt)))
        polys.append(orc.CommittedPoly(chunks, claims))
    return polys


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("chunked", [False, True])
def test_claims_batching_prove(dpb, ctx, F, chunked):
    from deep_prove_b200 import prover
    rng = np.random.default_rng(8300 + int(chunked))
    # five "model" polynomials of 10..13 variables with one or two claims, then four "witness" polynomials with one
    shapes = [(10, 1, 1), (12, 1, 2), (11, 1, 1), (13, 1, 2), (10, 1, 1), (10, 1, 1), (12, 1, 1), (11, 1, 1), (13, 1, 1)]
    if chunked:  # chunks of at most 2^10 entries, as with CHUNK_SIZE_THRESHOLD = 10 in the reference's test
        shapes = [(nv, 1 << max(nv - 10, 0), c) for nv, _, c in shapes]
    polys = make_polys(F, rng, shapes)
    want = orc.claims_batching_prove(F, polys, orc.Transcript(F))
    assert orc.claims_batching_verify(F, want, polys, orc.Transcript(F))

    gpu_polys, owned = [], []
    for p in polys:
        chunks = [upload(dpb, ctx, F, c) for c in p.chunks]
        owned += chunks
        claims = [(orc.scalars_to_array(F, pt), orc.scalars_to_array(F, [ev])[0]) for pt, ev in p.claims]
        gpu_polys.append(prover.CommittedPoly(chunks, claims))
    tr = prover.Blake3Transcript(family_dtype(dpb, F))
    got = prover.claims_batching_prove(ctx, tr, gpu_polys)
    n = len(want["point"])
    assert [orc.array_to_scalars(F, got["sumcheck"][i]) for i in range(n)] == want["sumcheck"]
    assert orc.array_to_scalars(F, got["point"]) == want["point"]
    assert orc.array_to_scalars(F, got["sumcheck_evals"]) == want["sumcheck_evals"]
    assert orc.array_to_scalars(F, got["rlc_challenges"]) == want["rlc_challenges"]
    assert (got["rlc"].to_host() == want["rlc"]).all()
    # the transcript ends in the same state as the oracle's
    ot = orc.Transcript(F)
    orc.claims_batching_prove(F, polys, ot)
    assert orc.array_to_scalars(F, tr.challenge_scalar().reshape(1, -1)) == [ot.challenge_scalar()]
    tr.free()
    got["rlc"].free()
    for m in owned:
        m.free()


@pytest.mark.parametrize("F", FIELDS)
def test_claims_batching_golden(dpb, ctx, F):
    """The committed fixture (tests/golden/oracle_*.json, key "claims")."""
    import json
    import os
    from deep_prove_b200 import prover
    from tests.golden import make_golden
    with open(os.path.join(os.path.dirname(__file__), "golden", f"oracle_{F.name}.json")) as f:
        want = json.load(f)["claims"]
    hx = lambda arr: orc.serialize_scalars(F, orc.array_to_scalars(F, arr)).hex()
    gpu_polys = []
    for p in make_golden.golden_inputs(F, "claims"):
        chunks = [upload(dpb, ctx, F, c) for c in p.chunks]
        claims = [(orc.scalars_to_array(F, pt), orc.scalars_to_array(F, [ev])[0]) for pt, ev in p.claims]
        gpu_polys.append(prover.CommittedPoly(chunks, claims))
    tr = prover.Blake3Transcript(family_dtype(dpb, F))
    got = prover.claims_batching_prove(ctx, tr, gpu_polys)
    assert hx(got["sumcheck"].reshape(-1, got["sumcheck"].shape[-1])) == want["proof"]
    assert hx(got["point"]) == want["point"] and hx(got["sumcheck_evals"]) == want["evals"]
    assert hx(got["rlc_challenges"]) == want["rlc_challenges"] and hx(got["rlc"].to_host()) == want["rlc"]


def test_claims_batching_argument_errors(dpb, ctx):
    from deep_prove_b200 import prover
    F = orc.FrField
    rng = np.random.default_rng(8400)
    a, b = upload(dpb, ctx, F, F.random_table_fast(rng, 16)), upload(dpb, ctx, F, F.random_table_fast(rng, 8))
    pt = orc.scalars_to_array(F, [F.random_scalar(rng) for _ in range(5)])
    ev = orc.scalars_to_array(F, [F.one])[0]
    tr = prover.Blake3Transcript(dpb.FR)
    with pytest.raises(dpb.DpbError) as e:  # chunks of different lengths
        prover.claims_batching_prove(ctx, tr, [prover.CommittedPoly([a, b], [(pt, ev)])])
    assert e.value.code == dpb.EINVAL
    with pytest.raises(dpb.DpbError) as e:  # three chunks
        prover.claims_batching_prove(ctx, tr, [prover.CommittedPoly([a, a, a], [(pt, ev)])])
    assert e.value.code == dpb.EINVAL
    tr.free()


@pytest.mark.parametrize("F", FIELDS)
def test_evaluate_many_zero_padded(dpb, ctx, F):
    """dpb_mle_evaluate_many: tables of several sizes and layouts (field, base, integers) at one point, each as its
    zero-padded extension (the convention of dpb_mle_zero_padded), against the oracle."""
    rng = np.random.default_rng(91)
    n = 9
    point = [F.random_scalar(rng) for _ in range(n)]
    tabs, mles = [], []
    for m in (9, 9, 6, 3, 0):
        ints = rng.integers(-(1 << 40), 1 << 40, size=1 << m, dtype=np.int64)
        tabs.append(F.table_from_i64(ints))
        mles.append(ctx.upload_ints(ints, dpb.FR_I64 if F is orc.FrField else dpb.GL_I64))
        t = F.random_table_fast(rng, 1 << m) if F is orc.FrField else F.random_table(rng, 1 << m)
        tabs.append(t)
        mles.append(upload(dpb, ctx, F, t))
    got = orc.array_to_scalars(F, dpb.evaluate_many(ctx, mles, orc.scalars_to_array(F, point)))
    want = [orc.evaluate(F, orc.zero_pad_table(F, t, n), point) for t in tabs]
    assert got == want
