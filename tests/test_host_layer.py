"""Host-side prover code that needs no GPU: the C++ transcript and the
expression algebra of libdpb.so against the oracle's Python restatements."""
import json
import os

import numpy as np
import pytest

from oracle import oracle as orc

FIELDS = [orc.FrField, orc.GlField]
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


@pytest.fixture(scope="module")
def prover(dpb):
    import importlib
    return importlib.import_module("deep_prove_b200.prover")


def fam(dpb, F):
    return dpb.FR if F is orc.FrField else dpb.GL_EXT


@pytest.mark.parametrize("F", FIELDS)
def test_transcript_matches_oracle_and_fixture(dpb, prover, F):
    t = prover.Blake3Transcript(fam(dpb, F), b"m2vec")
    o = orc.Transcript(F, b"m2vec")
    vals = [F.from_int(7), F.neg(F.one)]
    t.append_scalars(orc.scalars_to_array(F, vals))
    o.append_scalars(vals)
    got = [t.append_and_sample(b"initial_alpha"), t.challenge_scalar(), t.challenge_scalar()]
    want = [o.append_and_sample(b"initial_alpha"), o.challenge_scalar(), o.challenge_scalar()]
    got = [orc.array_to_scalars(F, g)[0] for g in got]
    assert got == want
    with open(os.path.join(GOLDEN, f"oracle_{F.name}.json")) as f:
        assert orc.serialize_scalars(F, got).hex() == json.load(f)["transcript"]
    assert t.state() == (o.state, o.round)


@pytest.mark.parametrize("F", FIELDS)
def test_transcript_long_sequences(dpb, prover, F):
    """Multi-chunk BLAKE3 inputs (more than 1024 bytes per absorb) and clones."""
    rng = np.random.default_rng(1)
    t = prover.Blake3Transcript(fam(dpb, F), b"a longer label \x00 with a zero byte")
    o = orc.Transcript(F, b"a longer label \x00 with a zero byte")
    for n in [0, 1, 3, 40, 70, 200]:
        vals = [F.random_scalar(rng) for _ in range(n)]
        t.append_scalars(orc.scalars_to_array(F, vals) if n else np.zeros((0, F.elem_words), np.uint64))
        o.append_scalars(vals)
        assert orc.array_to_scalars(F, t.challenge_scalar())[0] == o.challenge_scalar()
    c = t.clone()
    assert c.state() == t.state()
    c.append_and_sample(b"x")
    assert c.state() != t.state()
    assert t.state() == (o.state, o.round)


class OracleX:
    def __init__(self, F): self.F = F
    def wit(self, i): return orc.Expr.wit(i)
    def const(self, c): return orc.Expr.const(c)
    def chal(self, i, p, s, o): return orc.Expr.chal(i, p, s, o)


class LibX:
    def __init__(self, F, prover): self.F, self.P = F, prover
    def wit(self, i): return self.P.Expression.WitIn(i)
    def const(self, c): return self.P.Expression.Constant(self.F.to_native(c))
    def chal(self, i, p, s, o): return self.P.Expression.Challenge(i, p, self.F.to_native(s), self.F.to_native(o))


def sample_expr(X, F, consts):
    """The logup generic-layer and initial-lookup expressions
    (zkml/src/lookup/logup_gkr/circuit.rs:279-284, 397-401) plus a few extras."""
    one, zero = F.one, F.zero
    alpha2 = X.chal(0, 2, one, zero)
    lam = X.chal(1, 1, one, zero)
    layer = alpha2 * (X.wit(0) * X.wit(3) + X.wit(1) * X.wit(2) + lam * X.wit(2) * X.wit(3))
    d_lo = X.const(consts[0]) + X.const(one) * X.wit(4) + X.const(consts[1]) * X.wit(5)
    d_hi = X.const(consts[0]) + X.const(one) * X.wit(6) + X.const(consts[1]) * X.wit(7)
    lookup = X.chal(0, 3, one, zero) * (-d_hi - d_lo + lam * d_lo * d_hi)
    extra = X.chal(1, 0, consts[2], consts[3]) * X.wit(0) * X.wit(0) - X.wit(1) + X.const(zero) * X.wit(2)
    return (layer + lookup) * X.wit(8) + extra


@pytest.mark.parametrize("F", FIELDS)
def test_expression_expansion_and_evaluation(dpb, prover, F):
    rng = np.random.default_rng(2)
    consts = [F.random_scalar(rng) for _ in range(4)]
    chal = [F.random_scalar(rng) for _ in range(2)]
    want = orc.expr_to_terms(F, sample_expr(OracleX(F), F, consts), chal)
    terms = sample_expr(LibX(F, prover), F, consts).to_terms(fam(dpb, F), orc.scalars_to_array(F, chal))
    got = {}
    for t in terms:
        key = tuple(t.idx[j] for j in range(t.n_factors))
        got[key] = F.from_native(bytes(t.coeff)[:F.elem_words * 8])
    assert got == want
    wit = [F.random_scalar(rng) for _ in range(9)]
    ev = sample_expr(LibX(F, prover), F, consts).evaluate(fam(dpb, F), orc.scalars_to_array(F, wit),
                                                           orc.scalars_to_array(F, chal))
    assert orc.array_to_scalars(F, ev)[0] == orc.eval_expr(F, sample_expr(OracleX(F), F, consts), wit, chal)


def test_malformed_expression_is_rejected(dpb, prover):
    bad = prover.Expression([(prover.Expression.ADD, 0, 0, b"", b"")])
    with pytest.raises(dpb.DpbError) as e:
        bad.to_terms(dpb.FR, np.zeros((0, 4), np.uint64))
    assert e.value.code == dpb.EINVAL


# ------------------------------------------------------- closed-form evaluations between layers
@pytest.mark.parametrize("F", FIELDS)
def test_lookup_padding_evaluation_matches_the_oracle(dpb, prover, F):
    """dpb_lookup_padding_evaluation against the oracle's restatement, which tests/test_oracle_pins.py pins with
    the reference's own test (zkml/src/lookup/operation/mod.rs:354-415); ranks 1..4, power-of-two and ragged
    dimensions, and the reference's error for a point of the wrong length."""
    rng = np.random.default_rng(5100)
    f = fam(dpb, F)
    for _ in range(40):
        rank = int(rng.integers(1, 5))
        shape = [int(rng.integers(1, 12)) for _ in range(rank)]
        n_vars = sum(max(d - 1, 0).bit_length() for d in shape)
        point = [F.random_scalar(rng) for _ in range(n_vars)]
        pad = F.random_scalar(rng)
        want = orc.compute_lookup_padding_evaluation(F, pad, shape, orc.split_point(shape, point))
        pt = orc.scalars_to_array(F, point) if n_vars else np.zeros((0, F.elem_words), np.uint64)
        got = prover.lookup_padding_evaluation(f, orc.scalars_to_array(F, [pad]), shape, pt)
        assert orc.array_to_scalars(F, got)[0] == want
    with pytest.raises(dpb.DpbError) as e:
        prover.lookup_padding_evaluation(f, orc.scalars_to_array(F, [F.one]), [3, 5], orc.scalars_to_array(F, [F.one] * 4))
    assert "does not match total variables" in str(e.value)


@pytest.mark.parametrize("F", FIELDS)
def test_bias_evaluation_matches_the_oracle(dpb, prover, F):
    """dpb_bias_evaluation for output C(ijl) with BIAS(il), BIAS(l), BIAS(li) and BIAS(ijl)
    (zkml/src/layers/einsum/axis.rs:583-720; the first is the shape of the reference's test at axis.rs:1529)."""
    rng = np.random.default_rng(5200)
    f = fam(dpb, F)
    for bias_axes in ("il", "l", "li", "ijl"):
        for _ in range(8):
            shape = [int(rng.integers(1, 10)), int(rng.integers(2, 10)), int(rng.integers(1, 10))]
            n_vars = sum(max(d - 1, 0).bit_length() for d in shape)
            point = [F.random_scalar(rng) for _ in range(n_vars)]
            bias_eval = F.random_scalar(rng)
            split = orc.split_point(shape, point)
            want, want_pt = orc.compute_bias_evaluation(F, "ijl", bias_axes, split, bias_eval, shape)
            present = [a in bias_axes for a in "ijl"]
            pos = [bias_axes.index(a) if a in bias_axes else 0 for a in "ijl"]
            pt = orc.scalars_to_array(F, point) if n_vars else np.zeros((0, F.elem_words), np.uint64)
            got, got_pt = prover.bias_evaluation(f, shape, present, pos, pt, orc.scalars_to_array(F, [bias_eval]))
            assert orc.array_to_scalars(F, got)[0] == want
            assert (orc.array_to_scalars(F, got_pt) if len(want_pt) else []) == want_pt


@pytest.mark.parametrize("F", FIELDS)
def test_scalar_inverse_matches_the_oracle(dpb, prover, F):
    """dpb_scalar_inverse (the host inverse the split-eq planning uses; BN254: binary extended Euclid) against the
    oracle's inverse, on random values and on the edges 1, -1, 2, 0."""
    rng = np.random.default_rng(17)
    fam = dpb.FR if F is orc.FrField else dpb.GL_EXT
    vals = [F.one, F.neg(F.one), F.from_int(2), F.from_int(-7)] + [F.random_scalar(rng) for _ in range(300)]
    for v in vals:
        got = orc.array_to_scalars(F, prover.scalar_inverse(fam, orc.scalars_to_array(F, [v])).reshape(1, -1))[0]
        assert got == F.inv(v)
        assert F.mul(got, v) == F.one
    zero = orc.array_to_scalars(F, prover.scalar_inverse(fam, orc.scalars_to_array(F, [F.zero])).reshape(1, -1))[0]
    assert zero == F.zero
