"""GPU parity of the whole-protocol entry points (include/dpb_prover.h): the
C++ transcript drives the GPU rounds and the resulting proofs must equal the
oracle's byte for byte.  The cases mirror the reference's own tests."""
import importlib
import json
import os

import numpy as np
import pytest

from oracle import oracle as orc
from tests.golden import make_golden
from tests.helpers import family_dtype, terms_array, upload

pytestmark = pytest.mark.gpu

FIELDS = [orc.FrField, orc.GlField]
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def prover(dpb):
    return importlib.import_module("deep_prove_b200.prover")


def golden(F):
    with open(os.path.join(GOLDEN, f"oracle_{F.name}.json")) as f:
        return json.load(f)


def flat(F, arr):
    return orc.array_to_scalars(F, np.asarray(arr).reshape(-1, F.elem_words))


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("n", [1, 6, 12, 18])
def test_prove_sumcheck_matches_oracle(dpb, ctx, prover, F, n):
    """IOPProverState::prove on f*g*h, the microbenchmark shape."""
    rng = np.random.default_rng(50 + n)
    tabs = [F.random_table_fast(rng, 1 << n) for _ in range(3)]
    terms = {(0, 1, 2): F.one}
    want_proof, want_point, want_finals = orc.sumcheck_prove(F, n, tabs, terms, orc.Transcript(F))
    t = prover.Blake3Transcript(family_dtype(dpb, F))
    st = prover.IOPProverState.prove(ctx, n, [upload(dpb, ctx, F, x) for x in tabs], terms_array(dpb, F, terms), t)
    assert flat(F, st.proof) == [e for r in want_proof for e in r]
    assert flat(F, st.collect_raw_challenges()) == want_point
    assert flat(F, st.get_mle_flatten_final_evaluations()) == want_finals
    o = orc.Transcript(F)
    orc.sumcheck_verify(F, orc.extract_sum(F, want_proof), want_proof, n, 3, o)
    assert t.state() == (o.state, o.round)


@pytest.mark.parametrize("F", FIELDS)
def test_hadamard_prove(dpb, ctx, prover, F):
    """zkml/src/layers/hadamard.rs:173-209 (test_hadamard_proving): i64 inputs,
    claim = MLE of the element-wise product at a random point."""
    rng = np.random.default_rng(60)
    n = 10
    a = rng.integers(-128, 128, size=1 << n, dtype=np.int64)
    b = rng.integers(-128, 128, size=1 << n, dtype=np.int64)
    r = [F.random_scalar(rng) for _ in range(n)]
    base = dpb.FR if F is orc.FrField else dpb.GL_BASE
    v1, v2 = ctx.upload_i64(a, base), ctx.upload_i64(b, base)
    t = prover.Blake3Transcript(family_dtype(dpb, F))
    evals, point, claims = prover.hadamard_prove(ctx, t, orc.scalars_to_array(F, r), v1, v2)
    want = orc.hadamard_prove(F, orc.Transcript(F), r, F.table_from_i64(a), F.table_from_i64(b))
    assert flat(F, evals) == [e for rr in want["sumcheck"] for e in rr]
    assert flat(F, point) == want["point"] and flat(F, claims) == want["individual_claim"]
    # the verifier's checks (hadamard.rs:133-163)
    out_eval = orc.evaluate(F, F.table_from_i64(a * b), r)
    assert orc.extract_sum(F, want["sumcheck"]) == out_eval
    pt, expected = orc.sumcheck_verify(F, out_eval, want["sumcheck"], n, 3, orc.Transcript(F))
    c = flat(F, claims)
    assert F.mul(orc.identity_eval(F, r, pt), F.mul(c[0], c[1])) == expected
    assert orc.evaluate(F, F.table_from_i64(a), pt) == c[0]


@pytest.mark.parametrize("F", FIELDS)
def test_hadamard_golden(dpb, ctx, prover, F):
    g = make_golden.golden_inputs(F, "hadamard")
    t = prover.Blake3Transcript(family_dtype(dpb, F))
    evals, point, claims = prover.hadamard_prove(ctx, t, orc.scalars_to_array(F, g["point"]),
                                                 upload(dpb, ctx, F, g["v1"]), upload(dpb, ctx, F, g["v2"]))
    want = golden(F)["hadamard"]
    assert orc.serialize_scalars(F, flat(F, evals)).hex() == want["proof"]
    assert orc.serialize_scalars(F, flat(F, point)).hex() == want["point"]
    assert orc.serialize_scalars(F, flat(F, claims)).hex() == want["claims"]


@pytest.mark.parametrize("F", FIELDS)
def test_same_poly_prove(dpb, ctx, prover, F):
    """zkml/src/iop/same_poly.rs:193-229 (test_same_poly_proof): 14 claims on a 2^10 table."""
    rng = np.random.default_rng(61)
    n, m = 10, 14
    poly = F.random_table(rng, 1 << n)
    pts = [[F.random_scalar(rng) for _ in range(n)] for _ in range(m)]
    claims = [(p, orc.evaluate(F, poly, p)) for p in pts]
    want = orc.same_poly_prove(F, orc.Transcript(F), poly, claims)
    t = prover.Blake3Transcript(family_dtype(dpb, F))
    evals, point, ev = prover.same_poly_prove(ctx, t, upload(dpb, ctx, F, poly),
                                              np.stack([orc.scalars_to_array(F, p) for p in pts]))
    assert flat(F, evals) == [e for rr in want["sumcheck"] for e in rr]
    assert flat(F, point) == want["point"] and flat(F, ev)[0] == want["eval"]
    assert orc.evaluate(F, poly, want["point"]) == want["eval"]


def lookup_inputs(dpb, ctx, prover, F, rng, sizes, ncols=2, cpi=1):
    o_in, d_in, instances, columns = [], [], [], []
    for m in sizes:
        cols = [F.random_table_fast(rng, 1 << m) for _ in range(ncols)]
        cst, sep = F.random_scalar(rng), F.random_scalar(rng)
        o_in.append(orc.LogUpInput(F, 0, cols, cst, sep, columns_per_instance=cpi))
        d_in.append(prover.LogUpInput.new_lookup([upload(dpb, ctx, F, c) for c in cols],
                                                 orc.scalars_to_array(F, [cst]), orc.scalars_to_array(F, [sep]), cpi))
        instances += [dict(constant=cst, sep=sep, num_columns=cpi, kind=0, num_vars=m - 1)] * (ncols // cpi)
        columns += cols
    return o_in, d_in, instances, columns


@pytest.mark.parametrize("F", FIELDS)
def test_logup_batch_prove_reference_shape(dpb, ctx, prover, F):
    """zkml/src/lookup/logup_gkr/mod.rs:24-79 (test_logup_batch_prove): sizes
    2^11..2^7, two single-column lookup instances each; the GPU proof equals
    the oracle's, verifies, and every output claim is the column's MLE value."""
    rng = np.random.default_rng(62)
    o_in, d_in, instances, columns = lookup_inputs(dpb, ctx, prover, F, rng, [11, 10, 9, 8, 7])
    want = orc.logup_batch_prove(F, o_in, orc.Transcript(F))
    got = prover.new_batch_multiple_sizes_prove(ctx, d_in, prover.Blake3Transcript(family_dtype(dpb, F)))
    assert got == orc.serialize_logup_proof(F, want)
    res = orc.logup_batch_verify(F, want, instances, orc.Transcript(F))
    for (pt, ev), col in zip(res["output_claims"], columns):
        assert orc.evaluate(F, col, pt) == ev


@pytest.mark.parametrize("F", FIELDS)
def test_logup_golden(dpb, ctx, prover, F):
    g = make_golden.golden_inputs(F, "logup_lookup")
    S = lambda v: orc.scalars_to_array(F, [v])
    ins = [prover.LogUpInput.new_lookup([upload(dpb, ctx, F, c) for c in i["columns"]], S(i["constant"]),
                                        S(i["sep"]), i["cpi"]) for i in g]
    got = prover.new_batch_multiple_sizes_prove(ctx, ins, prover.Blake3Transcript(family_dtype(dpb, F)))
    assert got.hex() == golden(F)["logup_lookup"]
    g = make_golden.golden_inputs(F, "logup_table")
    tb = prover.LogUpInput.new_table([upload(dpb, ctx, F, c) for c in g["columns"]], upload(dpb, ctx, F, g["mult"]),
                                     S(g["constant"]), S(g["sep"]))
    got = prover.new_batch_multiple_sizes_prove(ctx, [tb], prover.Blake3Transcript(family_dtype(dpb, F)))
    assert got.hex() == golden(F)["logup_table"]


@pytest.mark.parametrize("F", FIELDS)
def test_logup_two_column_lookups_and_table(dpb, ctx, prover, F):
    """Two-column (input, output) lookups against their table: both proofs
    equal the oracle's and the fractions cancel (zkml/src/iop/verifier.rs:543-584)."""
    rng = np.random.default_rng(63)
    tbits, lbits = 8, 13
    t_in = np.arange(1 << tbits, dtype=np.int64) - (1 << (tbits - 1))
    t_out = np.maximum(t_in, 0)  # a ReLU table
    idx = rng.integers(0, 1 << tbits, size=1 << lbits)
    mult = np.bincount(idx, minlength=1 << tbits).astype(np.int64)
    cst, sep = F.random_scalar(rng), F.random_scalar(rng)
    S = lambda v: orc.scalars_to_array(F, [v])
    base = dpb.FR if F is orc.FrField else dpb.GL_BASE
    T = F.table_from_i64
    o_l = orc.LogUpInput(F, 0, [T(t_in[idx]), T(t_out[idx])], cst, sep, columns_per_instance=2)
    o_t = orc.LogUpInput(F, 1, [T(t_in), T(t_out)], cst, sep, mult=T(mult))
    d_l = prover.LogUpInput.new_lookup([ctx.upload_i64(t_in[idx], base), ctx.upload_i64(t_out[idx], base)],
                                       S(cst), S(sep), 2)
    d_t = prover.LogUpInput.new_table([ctx.upload_i64(t_in, base), ctx.upload_i64(t_out, base)],
                                      ctx.upload_i64(mult, base), S(cst), S(sep))
    fam = family_dtype(dpb, F)
    w_l = orc.logup_batch_prove(F, [o_l], orc.Transcript(F))
    w_t = orc.logup_batch_prove(F, [o_t], orc.Transcript(F))
    assert prover.new_batch_multiple_sizes_prove(ctx, [d_l], prover.Blake3Transcript(fam)) == orc.serialize_logup_proof(F, w_l)
    assert prover.new_batch_multiple_sizes_prove(ctx, [d_t], prover.Blake3Transcript(fam)) == orc.serialize_logup_proof(F, w_t)
    r_l = orc.logup_batch_verify(F, w_l, [dict(constant=cst, sep=sep, num_columns=2, kind=0, num_vars=lbits - 1)], orc.Transcript(F))
    r_t = orc.logup_batch_verify(F, w_t, [dict(constant=cst, sep=sep, num_columns=2, kind=1, num_vars=tbits - 1)], orc.Transcript(F))
    n, d = F.zero, F.one
    for nn, dd in zip(r_l["numerators"] + r_t["numerators"], r_l["denominators"] + r_t["denominators"]):
        n, d = F.add(F.mul(n, dd), F.mul(d, nn)), F.mul(d, dd)
    assert n == F.zero and d != F.zero


def test_logup_errors(dpb, ctx, prover):
    """Error behaviour of new_batch_multiple_sizes_prove (prover.rs:95-140) and
    LogUpInput::new_* (structs.rs:158-231)."""
    F = orc.FrField
    rng = np.random.default_rng(64)
    S = lambda v: orc.scalars_to_array(F, [v])
    small = upload(dpb, ctx, F, F.random_table(rng, 16))
    big = upload(dpb, ctx, F, F.random_table(rng, 64))
    t = lambda: prover.Blake3Transcript(dpb.FR)
    with pytest.raises(dpb.DpbError, match="No inputs provided"):
        prover.new_batch_multiple_sizes_prove(ctx, [], t())
    up = [prover.LogUpInput.new_lookup([small], S(F.one), S(F.one), 1),
          prover.LogUpInput.new_lookup([big], S(F.one), S(F.one), 1)]
    with pytest.raises(dpb.DpbError, match="decreasing size order"):
        prover.new_batch_multiple_sizes_prove(ctx, up, t())
    mixed = [prover.LogUpInput.new_lookup([big], S(F.one), S(F.one), 1),
             prover.LogUpInput.new_table([small], small, S(F.one), S(F.one))]
    with pytest.raises(dpb.DpbError, match="Not all proof types matched"):
        prover.new_batch_multiple_sizes_prove(ctx, mixed, t())
    with pytest.raises(dpb.DpbError, match="same length"):
        prover.new_batch_multiple_sizes_prove(ctx, [prover.LogUpInput.new_lookup([big, small], S(F.one), S(F.one), 2)], t())
    with pytest.raises(dpb.DpbError, match="Multiplicities length"):
        prover.new_batch_multiple_sizes_prove(ctx, [prover.LogUpInput.new_table([big], small, S(F.one), S(F.one))], t())


def test_phase_timers(dpb, ctx, prover):
    """dpb_trace_enable / dpb_trace_read: the whole-protocol entry points report where their host time goes."""
    F = orc.FrField
    rng = np.random.default_rng(77)
    assert dpb.trace_read() == {} or isinstance(dpb.trace_read(), dict)
    dpb.trace(True)
    cols = [ctx.upload(F.random_table_fast(rng, 1 << 9), dpb.FR) for _ in range(2)]
    one = orc.scalars_to_array(F, [F.one])
    d_in = prover.LogUpInput.new_lookup(cols, one, one, 1)
    prover.new_batch_multiple_sizes_prove(ctx, [d_in], prover.Blake3Transcript(dpb.FR))
    got = dpb.trace_read()
    dpb.trace(False)
    for phase in ("logup.trees", "logup.outputs", "logup.layer_expressions", "logup.eq_tables", "sumcheck.begin",
                  "sumcheck.rounds", "sumcheck.finish"):
        assert phase in got and got[phase][0] >= 0 and got[phase][1] >= 1
    assert got["sumcheck.begin"][1] == 8  # one sumcheck per tree level of a 2^9 instance
