"""Pins the CPU oracle (CPU only, no GPU needed).

The reference holds no golden proof or transcript vector for this path and its
sumcheck core (dp-crypto) is absent, so the oracle is pinned three ways:
  1. its C field arithmetic and kernels against naive Python big-int
     definitions on small cases;
  2. the reference's own algebraic tests, replayed against the oracle
     (file:line in each test);
  3. committed fixtures of its outputs (tests/golden), so that a later change
     of the oracle cannot move the target silently.
"""
import itertools
import json
import os

import numpy as np
import pytest

from oracle import blake3_py
from oracle import oracle as orc

FIELDS = [orc.FrField, orc.GlField]
GOLDEN = os.path.join(os.path.dirname(__file__), "golden")


def rand_table(F, rng, n, ext=False):
    if F is orc.GlField and ext:
        return F.random_ext_table(rng, n)
    return F.random_table(rng, n)


def naive_mle_eval(F, vals, point):
    """sum_x f(x) prod_i (x_i ? r_i : 1 - r_i), x little-endian"""
    tot = F.zero
    for i, v in enumerate(vals):
        w = F.one
        for j, r in enumerate(point):
            w = F.mul(w, r if (i >> j) & 1 else F.sub(F.one, r))
        tot = F.add(tot, F.mul(v, w))
    return tot


@pytest.mark.parametrize("F", FIELDS)
def test_field_mul_matches_bigint(F):
    rng = np.random.default_rng(1)
    fn = orc.lib().orc_gl2_mul1 if F is orc.GlField else orc.lib().orc_fr_mul1
    edge = [F.zero, F.one, F.neg(F.one)]
    vals = edge + [F.random_scalar(rng) for _ in range(40)]
    for a, b in itertools.product(vals[:8], vals):
        A, B = orc.scalars_to_array(F, [a]), orc.scalars_to_array(F, [b])
        out = np.zeros_like(A)
        fn(orc._ptr(A), orc._ptr(B), orc._ptr(out))
        assert orc.array_to_scalars(F, out)[0] == F.mul(a, b)


def test_fr_conversions():
    F = orc.FrField
    rng = np.random.default_rng(2)
    xs = np.array([0, 1, -1, 2**62, -(2**62), 12345, -98765], dtype=np.int64)
    t = F.table_from_i64(xs)
    # Element -> field: negative x is r - |x| (zkml/src/quantization/mod.rs:220-267)
    assert F.table_to_ints(t) == [int(x) % orc.FR_MOD for x in xs]
    vals = [F.random_scalar(rng) for _ in range(5)]
    assert F.table_to_ints(F.table_from_ints(vals)) == vals
    canon = np.frombuffer(b"".join(v.to_bytes(32, "little") for v in vals), dtype=np.uint64).reshape(-1, 4).copy()
    mont = np.empty_like(canon)
    orc.lib().orc_fr_to_mont(orc._ptr(canon), orc._ptr(mont), 5)
    assert F.table_to_ints(mont) == vals
    back = np.empty_like(canon)
    orc.lib().orc_fr_from_mont(orc._ptr(mont), orc._ptr(back), 5)
    assert (back == canon).all()


def test_blake3_known_answers():
    # Known-answer values of the BLAKE3 specification's test-vector input
    # pattern (byte i = i mod 251) are in the committed fixture; the empty-input
    # digest is the published one.
    assert blake3_py.blake3(b"").hex() == "af1349b9f5f9a1a6a0404dea36dcc9499bcb25c9adc112b7cc9a93cae41f3262"
    with open(os.path.join(GOLDEN, "blake3_kat.json")) as f:
        kat = json.load(f)
    for n, hx in kat.items():
        data = bytes(i % 251 for i in range(int(n)))
        assert blake3_py.blake3(data).hex() == hx, n


def test_blake3_matches_module_when_present():
    blake3 = pytest.importorskip("blake3")
    rng = np.random.default_rng(3)
    for n in [0, 1, 64, 65, 1024, 1025, 2048, 4097, 7000]:
        d = rng.bytes(n)
        assert blake3_py.blake3(d) == blake3.blake3(d).digest()


@pytest.mark.parametrize("F", FIELDS)
def test_evaluate_is_little_endian(F):
    """zkml/src/lib.rs:357-369 (test_vector_mle): evaluating at the LE bits of
    an index returns that entry."""
    rng = np.random.default_rng(4)
    n = 4
    t = rand_table(F, rng, 1 << n)
    vals = F.table_to_ints(t)
    for idx in [0, 1, 5, 10, 15]:
        pt = [F.from_int((idx >> j) & 1) for j in range(n)]
        assert orc.evaluate(F, t, pt) == vals[idx]
    pt = [F.random_scalar(rng) for _ in range(n)]
    assert orc.evaluate(F, t, pt) == naive_mle_eval(F, vals, pt)


@pytest.mark.parametrize("F", FIELDS)
def test_eq_evals(F):
    rng = np.random.default_rng(5)
    for m in [0, 1, 3, 6]:
        pt = [F.random_scalar(rng) for _ in range(m)]
        eq = orc.array_to_scalars(F, orc.eq_evals(F, pt))
        for i in range(1 << m):
            bits = [F.from_int((i >> j) & 1) for j in range(m)]
            assert eq[i] == orc.identity_eval(F, bits, pt)


def _triangular_fix(F, point, fix_row):
    """Closed form of the reference's test helper fix_mle_rec
    (zkml/src/layers/transformer/attention_mask/prove.rs:14-44): the MLE of the
    lower-triangular 0/1 matrix [row >= col] with its row (fix_row) or column
    variables bound to `point`, as a table over the other index."""
    n = len(point)
    out = []
    two = F.from_int(2)
    for idx in range(1 << n):
        acc = F.one
        for b in range(n):
            bit = F.from_int((idx >> b) & 1)
            c = point[b]
            same = F.add(F.sub(F.sub(F.one, bit), c), F.mul(two, F.mul(bit, c)))
            if fix_row:
                acc = F.add(F.mul(acc, same), F.mul(F.sub(F.one, bit), c))
            else:
                acc = F.add(F.mul(acc, same), F.mul(F.sub(F.one, c), bit))
        out.append(acc)
    return out


@pytest.mark.parametrize("F", FIELDS)
def test_fix_high_low_on_triangular_matrices(F):
    """zkml/src/layers/transformer/attention_mask/prove.rs:392-451
    (test_fix_lower_mle): fix_high binds the row (most significant) variables of
    a row-major matrix, fix_low the column variables."""
    rng = np.random.default_rng(6)
    nv = 4
    size = 1 << nv
    lower = [1 if r >= c else 0 for r in range(size) for c in range(size)]
    upper = [1 if r <= c else 0 for r in range(size) for c in range(size)]
    lower_t = F.table_from_ints(lower)
    upper_t = F.table_from_ints(upper)
    if F is orc.FrField:
        lower_t, upper_t = F.table_from_ints(lower), F.table_from_ints(upper)
    row_pt = [F.random_scalar(rng) for _ in range(nv)]
    col_pt = [F.random_scalar(rng) for _ in range(nv)]
    s = lambda t: orc.array_to_scalars(F, t)
    assert s(orc.fix_high_variables(F, lower_t, row_pt)) == _triangular_fix(F, row_pt, True)
    assert s(orc.fix_low_variables(F, lower_t, col_pt)) == _triangular_fix(F, col_pt, False)
    assert s(orc.fix_high_variables(F, upper_t, row_pt)) == _triangular_fix(F, row_pt, False)
    assert s(orc.fix_low_variables(F, upper_t, col_pt)) == _triangular_fix(F, col_pt, True)


@pytest.mark.parametrize("F", FIELDS)
def test_tensor_mle_row_then_column(F):
    """zkml/src/tensor/mod.rs:1875-1897 (test_tensor_mle): binding the row bits
    with fix_high and evaluating at the column bits addresses one entry."""
    rng = np.random.default_rng(7)
    rows, cols = 4, 8
    t = rand_table(F, rng, rows * cols)
    vals = F.table_to_ints(t)
    r, c = 3, 5
    row_bits = [F.from_int((r >> j) & 1) for j in range(2)]
    col_bits = [F.from_int((c >> j) & 1) for j in range(3)]
    fixed = orc.fix_high_variables(F, t, row_bits)
    assert orc.evaluate(F, fixed, col_bits) == vals[r * cols + c]


@pytest.mark.parametrize("F", FIELDS)
def test_sumcheck_round_matches_naive(F):
    rng = np.random.default_rng(8)
    n = 4
    tabs = [rand_table(F, rng, 1 << n), rand_table(F, rng, 1 << n, ext=True), rand_table(F, rng, 1 << (n - 2))]
    vals = [F.table_to_ints(t) for t in tabs]
    c0, c1 = F.random_scalar(rng), F.random_scalar(rng)
    terms = {(0, 1): c0, (0, 1, 2): c1, (2,): F.one}
    d = 3
    got = orc.sumcheck_round(F, n, tabs, terms, d)
    # naive: table 2 has 2 variables and depends on the LAST two of the four
    want = []
    for x in range(d + 1):
        X = F.from_int(x)
        tot = F.zero
        for p in range(1 << (n - 1)):
            def at(j):
                if len(vals[j]) == 1 << n:
                    f0, f1 = vals[j][2 * p], vals[j][2 * p + 1]
                else:
                    f0 = f1 = vals[j][(2 * p) >> 2]
                return F.add(f0, F.mul(X, F.sub(f1, f0)))
            for m, c in terms.items():
                pr = c
                for j in m:
                    pr = F.mul(pr, at(j))
                tot = F.add(tot, pr)
        want.append(tot)
    assert got == want


@pytest.mark.parametrize("F", FIELDS)
def test_sumcheck_prove_verify_roundtrip(F):
    """The f*g*eq sumcheck of zkml/src/layers/hadamard.rs:173-209
    (test_hadamard_proving): prove, verify, and check the claims by evaluation."""
    rng = np.random.default_rng(9)
    n = 5
    v1, v2 = rand_table(F, rng, 1 << n), rand_table(F, rng, 1 << n)
    r = [F.random_scalar(rng) for _ in range(n)]
    prod = [F.mul(a, b) for a, b in zip(F.table_to_ints(v1), F.table_to_ints(v2))]
    claim = naive_mle_eval(F, prod, r)
    pr = orc.hadamard_prove(F, orc.Transcript(F), r, v1, v2)
    assert orc.extract_sum(F, pr["sumcheck"]) == claim
    point, expected = orc.sumcheck_verify(F, claim, pr["sumcheck"], n, 3, orc.Transcript(F))
    assert point == pr["point"]
    beta = orc.identity_eval(F, r, point)
    assert F.mul(beta, F.mul(*pr["individual_claim"])) == expected
    assert orc.evaluate(F, v1, point) == pr["individual_claim"][0]
    assert orc.evaluate(F, v2, point) == pr["individual_claim"][1]


@pytest.mark.parametrize("F", FIELDS)
def test_same_poly(F):
    """zkml/src/iop/same_poly.rs:193-229 (test_same_poly_proof), smaller."""
    rng = np.random.default_rng(10)
    n, m = 6, 5
    poly = rand_table(F, rng, 1 << n)
    claims = []
    for _ in range(m):
        pt = [F.random_scalar(rng) for _ in range(n)]
        claims.append((pt, orc.evaluate(F, poly, pt)))
    pr = orc.same_poly_prove(F, orc.Transcript(F), poly, claims)
    t = orc.Transcript(F)
    chal = t.read_challenges(m)
    y = F.zero
    for a, (_, yi) in zip(chal, claims):
        y = F.add(y, F.mul(a, yi))
    point, expected = orc.sumcheck_verify(F, y, pr["sumcheck"], n, 2, t)
    comb = F.zero
    for a, (pt, _) in zip(chal, claims):
        comb = F.add(comb, F.mul(a, orc.identity_eval(F, pt, point)))
    assert F.mul(pr["eval"], comb) == expected
    assert orc.evaluate(F, poly, point) == pr["eval"]


@pytest.mark.parametrize("F", FIELDS)
def test_logup_circuit_output_identity(F):
    """zkml/src/lookup/logup_gkr/circuit.rs:603-624 (test_circuit_construction):
    with constant 0 and separator 1 the tree output is -sum 1/v."""
    rng = np.random.default_rng(11)
    col = rand_table(F, rng, 1 << 6)
    c = orc.LogUpCircuit(F, 0, [col], None, F.zero, F.one)
    out = c.outputs()
    assert len(out) == 4
    want = F.zero
    for v in F.table_to_ints(col):
        want = F.sub(want, F.inv(v))
    num = F.add(F.mul(out[0], out[3]), F.mul(out[1], out[2]))
    den = F.mul(out[2], out[3])
    assert F.mul(num, F.inv(den)) == want


def _mixed_lookup_inputs(F, rng, sizes):
    inputs, instances, columns = [], [], []
    for n in sizes:
        cols = [rand_table(F, rng, 1 << n), rand_table(F, rng, 1 << n)]
        cst, sep = F.random_scalar(rng), F.random_scalar(rng)
        inputs.append(orc.LogUpInput(F, 0, cols, cst, sep, columns_per_instance=1))
        instances += [dict(constant=cst, sep=sep, num_columns=1, kind=0, num_vars=n - 1)] * 2
        columns += cols
    return inputs, instances, columns


@pytest.mark.parametrize("F", FIELDS)
def test_logup_batch_prove_verify(F):
    """zkml/src/lookup/logup_gkr/mod.rs:24-79 (test_logup_batch_prove), at sizes
    2^7..2^3: mixed-size lookup instances, prove, verify, and every output claim
    equals the column's MLE at the claim point."""
    rng = np.random.default_rng(12)
    inputs, instances, columns = _mixed_lookup_inputs(F, rng, [7, 6, 5, 4, 3])
    proof = orc.logup_batch_prove(F, inputs, orc.Transcript(F))
    res = orc.logup_batch_verify(F, proof, instances, orc.Transcript(F))
    assert len(res["output_claims"]) == len(columns)
    for (pt, ev), col in zip(res["output_claims"], columns):
        assert orc.evaluate(F, col, pt) == ev
    assert [c[1] for c in proof["output_claims"]] == [c[1] for c in res["output_claims"]]


@pytest.mark.parametrize("F", FIELDS)
def test_logup_table_and_lookup_fractions_cancel(F):
    """The global check of zkml/src/iop/verifier.rs:543-584: the lookups'
    fractions plus the table's fraction sum to zero when the multiplicities
    count the lookups."""
    rng = np.random.default_rng(13)
    tbits, lbits = 4, 6
    table_in = list(range(1 << tbits))
    table_out = [(3 * x + 1) % 17 for x in table_in]
    idx = rng.integers(0, 1 << tbits, size=1 << lbits)
    look_in = [table_in[i] for i in idx]
    look_out = [table_out[i] for i in idx]
    mult = [0] * (1 << tbits)
    for i in idx:
        mult[i] += 1
    cst, sep = F.random_scalar(rng), F.random_scalar(rng)
    T = lambda v: F.table_from_ints(v)
    lk = orc.LogUpInput(F, 0, [T(look_in), T(look_out)], cst, sep, columns_per_instance=2)
    tb = orc.LogUpInput(F, 1, [T(table_in), T(table_out)], cst, sep, mult=T(mult))
    p_l = orc.logup_batch_prove(F, [lk], orc.Transcript(F))
    p_t = orc.logup_batch_prove(F, [tb], orc.Transcript(F))
    r_l = orc.logup_batch_verify(F, p_l, [dict(constant=cst, sep=sep, num_columns=2, kind=0, num_vars=lbits - 1)],
                                 orc.Transcript(F))
    r_t = orc.logup_batch_verify(F, p_t, [dict(constant=cst, sep=sep, num_columns=2, kind=1, num_vars=tbits - 1)],
                                 orc.Transcript(F))
    n, d = F.zero, F.one
    for nn, dd in zip(r_l["numerators"] + r_t["numerators"], r_l["denominators"] + r_t["denominators"]):
        n, d = F.add(F.mul(n, dd), F.mul(d, nn)), F.mul(d, dd)
    assert n == F.zero and d != F.zero
    # table claims: multiplicity poly first, then the columns (structs.rs:395-420)
    pt, ev = r_t["output_claims"][0]
    assert orc.evaluate(F, T(mult), pt) == ev


@pytest.mark.parametrize("F", FIELDS)
def test_zero_padding_convention(F):
    """A zero-padded table is its polynomial over the FIRST variables times (1 - x_j) for every added variable:
    the formula the reference's verifier uses for the padded eq tables (zkml/src/poly_commit/verifier.rs:300-311)."""
    rng = np.random.default_rng(14)
    m, n = 3, 6
    eq_point = [F.random_scalar(rng) for _ in range(m)]
    point = [F.random_scalar(rng) for _ in range(n)]
    padded = orc.zero_pad_table(F, orc.eq_evals(F, eq_point), n)
    want = orc.identity_eval(F, point[:m], eq_point)
    for p in point[m:]:
        want = F.mul(want, F.sub(F.one, p))
    assert orc.evaluate(F, padded, point) == want


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("chunked", [False, True])
def test_claims_batching_prove_verify(F, chunked):
    """The reference's own test of this path (zkml/src/poly_commit/mod.rs:224-398) at reduced sizes: polynomials
    of different sizes, one or two claims each, unchunked and cut into chunks; the prover's output passes the
    restated verifier (verifier.rs:203-330), the linear combination opens to sum_j c_j * eval_j at the sumcheck
    point, and a changed evaluation is rejected."""
    rng = np.random.default_rng(15 + int(chunked))
    polys = []
    for nv, nclaims in ((6, 1), (8, 2), (5, 1), (7, 2), (6, 1)):
        nchunks = 1 << max(nv - 5, 0) if chunked else 1
        full = F.random_table_fast(rng, 1 << nv)
        mv = nv - (nchunks.bit_length() - 1)
        claims = []
        for _ in range(nclaims):
            pt = [F.random_scalar(rng) for _ in range(nv)]
            claims.append((pt, orc.evaluate(F, full, pt)))
        polys.append(orc.CommittedPoly([full[i << mv:(i + 1) << mv] for i in range(nchunks)], claims))
    proof = orc.claims_batching_prove(F, polys, orc.Transcript(F))
    assert orc.claims_batching_verify(F, proof, polys, orc.Transcript(F))
    # the chunk coefficients rebuild a claim from the chunks' evaluations (mod.rs:38-45)
    p = polys[1]
    pt, ev = p.claims[0]
    acc = F.zero
    for c, chunk in zip(p.batching_coefficients_for_chunks(F, pt), p.chunks):
        acc = F.add(acc, F.mul(c, orc.evaluate(F, chunk, p.eq_point_per_chunk(pt))))
    assert acc == ev
    # the combined polynomial at the sumcheck point
    point, n_rlc = proof["point"], (len(proof["rlc"]) - 1).bit_length()
    lhs = orc.evaluate(F, proof["rlc"], point[:n_rlc])
    rhs = F.zero
    for c, e in zip(proof["rlc_challenges"], proof["sumcheck_evals"]):
        rhs = F.add(rhs, F.mul(c, e))
    assert lhs == rhs
    bad = dict(proof)
    bad["sumcheck_evals"] = list(proof["sumcheck_evals"])
    bad["sumcheck_evals"][0] = F.add(bad["sumcheck_evals"][0], F.one)
    assert not orc.claims_batching_verify(F, bad, polys, orc.Transcript(F))


@pytest.mark.parametrize("F", FIELDS)
def test_golden_fixture(F):
    """The oracle's outputs on seeded inputs are frozen in tests/golden."""
    from tests.golden import make_golden
    with open(os.path.join(GOLDEN, f"oracle_{F.name}.json")) as f:
        want = json.load(f)
    assert make_golden.generate(F) == want


# ------------------------------------------------------- padding and broadcast evaluations
def _pad_pow2(a, value=0):
    shape = [1 << max(d - 1, 0).bit_length() for d in a.shape]
    out = np.full(shape, value, dtype=np.int64)
    out[tuple(slice(0, d) for d in a.shape)] = a
    return out


@pytest.mark.parametrize("F", FIELDS)
def test_padding_eval_function(F):
    """zkml/src/lookup/operation/mod.rs:354-415, the reference's own test of compute_lookup_padding_evaluation:
    zero sub-tensors over the last two dimensions padded with the padding value, repeated over the unpadded
    leading indices, zero elsewhere; the MLE's evaluation at a random point equals the closed form."""
    rng = np.random.default_rng(4100)
    padding_value = 1
    for _ in range(30):
        rank = int(rng.integers(1, 5))
        shape = [int(rng.integers(1, 10)) for _ in range(rank)]
        lead = shape[: max(rank - 2, 0)]
        sub = _pad_pow2(np.zeros(shape[max(rank - 2, 0):], dtype=np.int64), padding_value)
        inter = np.broadcast_to(sub, tuple(lead) + sub.shape).copy()
        tensor = _pad_pow2(inter, 0)
        n_vars = sum(max(d - 1, 0).bit_length() for d in tensor.shape)
        point = [F.random_scalar(rng) for _ in range(n_vars)]
        mle_eval = orc.evaluate(F, F.table_from_i64(tensor.reshape(-1)), point)
        dim_points = orc.split_point(list(tensor.shape), point)
        got = orc.compute_lookup_padding_evaluation(F, F.from_int(padding_value), shape, dim_points)
        assert got == mle_eval, (shape, rank)


@pytest.mark.parametrize("F", FIELDS)
def test_broadcasted_bias_eval(F):
    """zkml/src/layers/einsum/axis.rs:1529-1590 for "A(ijk)@B(ikl)->C(ijl)+BIAS(il)": the bias broadcast along j,
    padded, evaluated at a random point equals compute_bias_evaluation of the bias's own evaluation."""
    rng = np.random.default_rng(4200)
    for _ in range(20):
        i, j, l = int(rng.integers(1, 10)), int(rng.integers(2, 10)), int(rng.integers(1, 10))
        out_shape = [i, j, l]
        bias = rng.integers(-1000, 1000, size=(i, l), dtype=np.int64)
        broadcast = np.broadcast_to(bias[:, None, :], (i, j, l)).copy()
        padded_b, padded_bias = _pad_pow2(broadcast), _pad_pow2(bias)
        n_vars = sum(max(d - 1, 0).bit_length() for d in padded_b.shape)
        point = [F.random_scalar(rng) for _ in range(n_vars)]
        want = orc.evaluate(F, F.table_from_i64(padded_b.reshape(-1)), point)
        split = orc.split_point(out_shape, point)
        bias_point = orc.bias_evaluation_point("ijl", "il", split)
        bias_eval = orc.evaluate(F, F.table_from_i64(padded_bias.reshape(-1)), bias_point)
        got, pt = orc.compute_bias_evaluation(F, "ijl", "il", split, bias_eval, out_shape)
        assert got == want and pt == bias_point


def _padded_mle(F, t):
    """The tensor zero-padded to powers of two per axis, as a table (last axis lowest variables)."""
    dims = [1 << max(d - 1, 0).bit_length() for d in t.shape]
    p = np.zeros(dims, dtype=np.int64)
    p[tuple(slice(0, d) for d in t.shape)] = t
    return F.table_from_i64(p.reshape(-1))


def einsum_cases(F, rng):
    """(name, lhs, lhs_fixes, rhs, subscripts per output, output points) of the layer shapes the path uses."""
    C, O, S = orc.AXIS_CONTRACTED, orc.AXIS_OUTER, orc.AXIS_STACKED
    lg = lambda d: max(d - 1, 0).bit_length()
    pt = lambda d: [F.random_scalar(rng) for _ in range(lg(d))]
    cases = []
    # dense layer: x[m, k] w[k, n]
    x, w = rng.integers(-99, 99, (6, 10)), rng.integers(-99, 99, (10, 5))
    rp, cp = pt(6), pt(5)
    cases.append(("dense", x, [((O, C), [rp, None])], [(w, (C, O), [None, cp])], ["mk,kn->mn"], [cp + rp]))
    # attention scores: q[h, s, d] k[h, t, d], stacked heads
    q, k = rng.integers(-9, 9, (3, 5, 4)), rng.integers(-9, 9, (3, 6, 4))
    hp, sp, tp = pt(3), pt(5), pt(6)
    cases.append(("qk", q, [((S, O, C), [hp, sp, None])], [(k, (S, O, C), [hp, tp, None])], ["hsd,htd->hst"],
                  [tp + sp + hp]))
    # one left tensor, two right tensors (a fused projection): two outputs, the left claims are merged
    w2 = rng.integers(-99, 99, (10, 3))
    rp2, cp2 = pt(6), pt(3)
    cases.append(("two outputs", x, [((O, C), [rp, None]), ((O, C), [rp2, None])],
                  [(w, (C, O), [None, cp]), (w2, (C, O), [None, cp2])], ["mk,kn->mn", "mk,kn->mn"],
                  [cp + rp, cp2 + rp2]))
    return cases


@pytest.mark.parametrize("F", FIELDS)
def test_einsum_prove_claims(F):
    """einsum_prove (EinSum::prove_internal restated): the sumcheck's claimed sum is the gamma-combination of the
    outputs' MLEs at their claim points (what EinSum::verify checks first, zkml/src/layers/einsum/verify.rs), the
    sumcheck verifies, and every input claim it hands on is true of the padded input tensor."""
    rng = np.random.default_rng(21)
    for name, lhs, fixes, rhs, subs, out_points in einsum_cases(F, rng):
        T = orc.Transcript(F)
        got = orc.einsum_prove(F, T, lhs, fixes, rhs, lhs_padded=_padded_mle(F, lhs))
        gamma = got["batching_challenge"]
        want, g = F.zero, F.one
        for (t, _, _), sub, pt in zip(rhs, subs, out_points):
            out = np.einsum(sub, lhs, t)
            want = F.add(want, F.mul(g, orc.evaluate(F, _padded_mle(F, out), pt)))
            g = F.mul(g, gamma)
        assert orc.extract_sum(F, got["sumcheck"]) == want, name
        V = orc.Transcript(F)
        assert V.append_and_sample(b"batching_challenge") == gamma
        n = len(got["point"])
        point, expected = orc.sumcheck_verify(F, want, got["sumcheck"], n, 2, V)
        assert point == got["point"], name
        # the last round's value is the expression at the final evaluations (left tables first, then right)
        R, S = len(rhs), len(got["stacking_coeffs"][0])
        ev, acc, g = got["evaluations"], F.zero, F.one
        for i in range(R):
            inner = F.zero
            for j in range(S):
                inner = F.add(inner, F.mul(got["stacking_coeffs"][i][j], F.mul(ev[i * S + j], ev[R * S + i * S + j])))
            acc = F.add(acc, F.mul(g, inner))
            g = F.mul(g, gamma)
        assert acc == expected, name
        for (t, _, _), (pt, ev) in zip(rhs, got["rhs_claims"]):
            assert orc.evaluate(F, _padded_mle(F, t), pt) == ev, name
        pt, ev = got["lhs_claim"]
        assert orc.evaluate(F, _padded_mle(F, lhs), pt) == ev, name
        assert (got["aggregation"] is not None) == (len(rhs) > 1)
