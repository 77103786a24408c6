"""Pins the oracle's lookup witness generation (CPU only) with the reference's own checks of that code:

  * decomposing a value and recombining its chunks gives the value back, and the value chunks with the
    zeroing chunks give the right-shifted value (proptest_value_decomposer,
    zkml/src/lookup/operation/decomposer.rs:781-797);
  * the verifier's field formula over the chunk columns gives the value back (proptest_input_recombiner,
    decomposer.rs:799-819);
  * recombining the looked-up outputs gives what the operation itself computes: rescale, shift, table with
    clamping (combine_outputs, decomposer.rs:503-590, used by compare_output_and_witness,
    zkml/src/lookup/operation/mod.rs:448-479);
  * every looked-up row is a row of its table and the counts add up to the number of lookups, which is what the
    logup argument needs of the multiplicities (zkml/src/lookup/context.rs:313-371).
"""
import numpy as np
import pytest

from oracle import oracle as orc

SIGNS = [orc.SIGN_POSITIVE, orc.SIGN_NEGATIVE, orc.SIGN_MIXED]


def full_recombination(ci, shifted, value, zeroing):
    """test_full_recombination (decomposer.rs:664-723), integers."""
    n = len(value[0])
    out = []
    for i in range(n):
        val = 0
        for j, c in enumerate(value):
            v = int(c[i])
            v = v + ci.value_chunk_offset if ci.sign == orc.SIGN_MIXED else (v if ci.sign == orc.SIGN_POSITIVE else -v)
            val += v << (j * ci.value_chunk_size)
        low = 0
        for j, c in enumerate(shifted):
            if j != ci.n_shifted - 1 or ci.right_shift % 16 == 0:
                low += int(c[i]) << (j * 16)
            else:
                low += (int(c[i]) // ci.shifted_chunk_multiplier) << (j * 16)
        acc = low + (val << ci.right_shift)
        for j, c in enumerate(zeroing):
            sh = ci.value_chunk_size * ci.n_value + ci.right_shift + j * 16
            if j != ci.n_zeroing - 1 or not ci.is_signed:
                acc += int(c[i]) << sh
            else:
                acc += (int(c[i]) + ci.top_zeroing_chunk_offset) << sh
        out.append(acc - ci.offset if ci.sign == orc.SIGN_MIXED else (acc if ci.sign == orc.SIGN_POSITIVE else -acc))
    return out


def recombination_after_shift(ci, value, zeroing):
    """test_recombination_after_shift (decomposer.rs:613-661)."""
    n = len(value[0])
    out = []
    for i in range(n):
        val = 0
        for j, c in enumerate(value):
            v = int(c[i])
            v = v + ci.value_chunk_offset if ci.sign == orc.SIGN_MIXED else (v if ci.sign == orc.SIGN_POSITIVE else -v)
            val += v << (j * ci.value_chunk_size)
        for j, c in enumerate(zeroing):
            sh = ci.value_chunk_size * ci.n_value + j * 16
            if j != ci.n_zeroing - 1 or not ci.is_signed:
                val += int(c[i]) << sh
            else:
                val += (int(c[i]) + ci.top_zeroing_chunk_offset) << sh
        out.append(val - (ci.offset >> ci.right_shift) if ci.sign == orc.SIGN_MIXED
                   else (val if ci.sign == orc.SIGN_POSITIVE else -val))
    return out


def draw_case(rng):
    """decomposer_input (decomposer.rs:735-764): the reference's strategy for its property tests."""
    right_shift = int(rng.integers(10, 28))
    bits = int(rng.integers(8, 16))
    sign = SIGNS[int(rng.integers(0, 3))]
    max_bit_size = int(rng.integers(right_shift + bits + 16, 63))
    if sign == orc.SIGN_MIXED:
        lo, hi = -(1 << (max_bit_size - 1)), (1 << (max_bit_size - 1)) - 1
    elif sign == orc.SIGN_POSITIVE:
        lo, hi = 0, (1 << max_bit_size) - 1
    else:
        lo, hi = -(1 << max_bit_size) + 1, 0
    inputs = rng.integers(lo, hi, size=int(rng.integers(1, 20)), endpoint=True, dtype=np.int64)
    inputs[0] = lo if rng.integers(0, 2) else hi  # the range's ends, always
    return right_shift, bits, sign, max_bit_size, inputs


def test_value_decomposer_recombines():
    rng = np.random.default_rng(9100)
    for _ in range(400):
        right_shift, bits, sign, max_bit_size, inputs = draw_case(rng)
        ci = orc.ChunkingInfo(right_shift, bits, sign, max_bit_size)
        shifted, value, zeroing = ci.decompose_input(inputs)
        # The chunks hold `covered` bits of value + offset.  For a signed operation whose chunks cover exactly
        # max_bit_size bits, the offset pushes the top 2^(right_shift + bits - 1) values of the range one bit
        # past the chunks and the reference's decomposition drops that bit (its own property test draws such a
        # value with probability below 2^-16); the oracle follows the reference there, and this test says so.
        covered = right_shift + bits + 16 * ci.n_zeroing
        dropped = [((int(v) + ci.offset) >> covered) << covered if sign == orc.SIGN_MIXED else 0 for v in inputs]
        assert all(d == 0 for d in dropped) or covered == max_bit_size
        assert full_recombination(ci, shifted, value, zeroing) == [int(v) - d for v, d in zip(inputs, dropped)]
        want = [(int(v) - d) >> right_shift if sign != orc.SIGN_NEGATIVE else -((-int(v)) >> right_shift)
                for v, d in zip(inputs, dropped)]
        assert recombination_after_shift(ci, value, zeroing) == want
        # chunks are rows of their tables
        for c in shifted:
            assert c.min() >= 0 and c.max() < (1 << 16)
        lo, hi = orc.table_input_range(bits, sign)
        assert value[0].min() >= lo and value[0].max() <= hi
        ci.table_output(value, zeroing, None)  # raises if a zeroing chunk is outside its table


@pytest.mark.parametrize("F", [orc.FrField, orc.GlField])
def test_input_recombiner_in_the_field(F):
    rng = np.random.default_rng(9200)
    for _ in range(60):
        right_shift, bits, sign, max_bit_size, inputs = draw_case(rng)
        ci = orc.ChunkingInfo(right_shift, bits, sign, max_bit_size)
        shifted, value, zeroing = ci.decompose_input(inputs)
        covered = right_shift + bits + 16 * ci.n_zeroing
        for i, x in enumerate(inputs.tolist()):
            if sign == orc.SIGN_MIXED and (x + ci.offset) >> covered:
                continue  # the bit the reference drops, see test_value_decomposer_recombines
            got = ci.combine_input_claims(F, [F.from_int(int(c[i])) for c in shifted],
                                          [F.from_int(int(c[i])) for c in value],
                                          [F.from_int(int(c[i])) for c in zeroing])
            assert got == F.from_int(x)


def combine_outputs(ci, value_out, zero_out, out_min, out_max):
    """combine_outputs (decomposer.rs:503-590) for one value chunk."""
    res = []
    for i in range(len(value_out[0])):
        value = int(value_out[0][i])
        if ci.is_signed:
            prod = 1
            for z in zero_out[:max(ci.n_zeroing - 1, 0)]:
                prod *= int(z[i])
            if ci.n_zeroing:
                last = int(zero_out[-1][i])
                bit = 1 - last * last
                lower = prod
                prod *= bit
                clamp = (last * (last + 1) // 2 + (bit - lower * bit)) * out_max + (last * (last - 1) // 2) * out_min
            else:
                clamp = 0
            res.append(clamp + prod * value)
        else:
            prod = 1
            for z in zero_out:
                prod *= int(z[i])
            clamp = (out_max if ci.sign == orc.SIGN_POSITIVE else out_min) if ci.n_zeroing else 1
            res.append(clamp + prod * (value - clamp))
    return res


@pytest.mark.parametrize("kind", ["relu", "requantise"])
@pytest.mark.parametrize("shape", [(5,), (3, 7), (2, 3, 5), (2, 4, 8)])
def test_witness_outputs_equal_the_operation(kind, shape):
    """LookupOp::apply (zkml/src/lookup/operation/mod.rs:46-58): rescale, add the rounding constant, shift,
    look up with clamping; the witness' outputs recombine to the same values on the unpadded entries and to the
    operation of the padding value elsewhere."""
    rng = np.random.default_rng(9300 + len(shape))
    bits, right_shift, max_bit_size, fpm, padding = 10, 13, 44, 37, 0
    lo, hi = orc.table_input_range(bits, orc.SIGN_MIXED)
    ins = np.arange(lo, hi + 1, dtype=np.int64)
    if kind == "relu":  # TableType::ReLU: input.clamp(0, input_max), two columns (tabletype.rs:126)
        table_out, n_cols = np.clip(ins, 0, hi), 2
    else:               # TableType::Requantise: clamp(min, max), one column (tabletype.rs:127)
        table_out, n_cols = None, 1
    ci = orc.ChunkingInfo(right_shift, bits, orc.SIGN_MIXED, max_bit_size)
    big = (1 << (max_bit_size - 2)) // fpm
    t = rng.integers(-big, big, size=shape, dtype=np.int64)
    t.reshape(-1)[::3] = rng.integers(-(1 << 12), 1 << 12, size=t.reshape(-1)[::3].shape)  # some inside the table
    w = orc.LookupOpWitness(ci, fpm, padding, t, table_out, n_cols)
    rows, cols = (1, shape[0]) if len(shape) == 1 else shape[-2:]
    prow, pcol = 1 << (rows - 1).bit_length(), 1 << (cols - 1).bit_length()
    shifted_in = (t * fpm + ci.rounding_constant()) >> right_shift
    want_unpadded = np.clip(shifted_in, 0 if kind == "relu" else lo, hi)
    pad_out = int(np.clip((padding * fpm + ci.rounding_constant()) >> right_shift, 0 if kind == "relu" else lo, hi))
    out_min, out_max = (0, hi) if kind == "relu" else (lo, hi)
    for c, (chunk, (vo, zo)) in enumerate(zip(want_unpadded.reshape(-1, rows, cols), w.outputs)):
        got = np.array(combine_outputs(ci, vo, zo, out_min, out_max)).reshape(prow, pcol)
        assert (got[:rows, :cols] == chunk).all()
        mask = np.ones((prow, pcol), bool)
        mask[:rows, :cols] = False
        assert (got[mask] == pad_out).all()
    assert len(w.input_columns()) == len(w.inputs) * (ci.n_shifted + (n_cols - 1) + ci.n_zeroing)
    assert len(w.output_columns()) == len(w.inputs) * (1 + ci.n_zeroing)


@pytest.mark.parametrize("F", [orc.FrField, orc.GlField])
def test_counts_and_multiplicities(F):
    rng = np.random.default_rng(9400)
    bits, right_shift, max_bit_size = 8, 20, 50
    lo, hi = orc.table_input_range(bits, orc.SIGN_MIXED)
    ins = np.arange(lo, hi + 1, dtype=np.int64)
    table_out = np.clip(ins, 0, hi)
    ci = orc.ChunkingInfo(right_shift, bits, orc.SIGN_MIXED, max_bit_size)
    t = rng.integers(-(1 << 47), 1 << 47, size=(3, 6, 10), dtype=np.int64)
    t[:, ::2, :] >>= 20
    w = orc.LookupOpWitness(ci, 1, 0, t, table_out, 2)
    shift, value, zero, signed = w.get_counts()
    lookups = 3 * 8 * 16
    assert sum(shift.values()) == lookups * ci.n_shifted
    assert sum(value.values()) == lookups
    assert sum(zero.values()) == lookups * (ci.n_zeroing - 1)
    assert sum(signed.values()) == lookups
    tables = {
        "shift": (orc.merged_table_column(16, orc.SIGN_POSITIVE, None), shift),
        "value": (orc.merged_table_column(bits, orc.SIGN_MIXED, table_out), value),
        "zero": (orc.merged_table_column(16, orc.SIGN_POSITIVE, (np.arange(1 << 16) == 0).astype(np.int64)), zero),
        "signed": (orc.merged_table_column(16, orc.SIGN_MIXED, np.sign(np.arange(-(1 << 15), 1 << 15))), signed),
    }
    for name, (col, counts) in tables.items():
        rows = set(col.tolist())
        assert set(counts) <= rows, name  # every looked-up row is in the table
        m = orc.array_to_scalars(F, orc.table_multiplicities(F, col, counts))
        assert len(m) == len(col)
        total = F.zero
        for x in m:
            total = F.add(total, x)
        assert total == F.from_int(sum(counts.values()))
    # a table with a repeated row: its lookups are split evenly between the copies
    col = np.array([0, 1, 2, 2], dtype=np.int64)
    m = orc.array_to_scalars(F, orc.table_multiplicities(F, col, {2: 6, 0: 1}))
    assert m == [F.one, F.zero, F.from_int(3), F.from_int(3)]


# ------------------------------------------------------------- linking sumcheck
def padded_2d(a, fill):
    rows, cols = a.shape
    prow, pcol = 1 << max(rows - 1, 0).bit_length(), 1 << max(cols - 1, 0).bit_length()
    out = np.full((prow, pcol), fill, dtype=np.int64)
    out[:rows, :cols] = a
    return out


def linking_case(F, kind, rng, shape=(3, 5, 6)):
    """A lookup operation's witness over a rank-3 tensor with everything the linking sumcheck needs."""
    bits, right_shift, max_bit_size, fpm, padding = 8, 12, 40, 5, 0
    lo, hi = orc.table_input_range(bits, orc.SIGN_MIXED)
    if kind == "relu":
        table_out, n_cols, n_value = np.clip(np.arange(lo, hi + 1, dtype=np.int64), 0, hi), 2, 1
        out_min, out_max = 0, hi
    else:  # requantisation over two value chunks
        table_out, n_cols, n_value = None, 1, 2
        out_min, out_max = lo, hi
    ci = orc.ChunkingInfo(right_shift, bits, orc.SIGN_MIXED, max_bit_size, n_value)
    big = (1 << (max_bit_size - 2)) // fpm
    t = rng.integers(-big, big, size=shape, dtype=np.int64)
    t.reshape(-1)[::2] >>= 22
    w = orc.LookupOpWitness(ci, fpm, padding, t, table_out, n_cols)
    # what the operation computes (LookupOp::apply, zkml/src/lookup/operation/mod.rs:46-58)
    full_bits = bits * n_value
    cl_lo, cl_hi = (0, hi) if kind == "relu" else (-(1 << (full_bits - 1)), (1 << (full_bits - 1)) - 1)
    op = lambda x: np.clip((x * fpm + ci.rounding_constant()) >> right_shift, cl_lo, cl_hi)
    outputs = [padded_2d(op(s), int(op(np.int64(padding)))) for s in t]
    return ci, w, outputs, out_min, out_max


@pytest.mark.parametrize("F", [orc.FrField, orc.GlField])
@pytest.mark.parametrize("kind", ["relu", "requantise2"])
def test_linking_sumcheck_ties_outputs_and_lookups(F, kind):
    """What prove_linking_sumcheck's claimed sum must be (debug_linking_sumcheck's check,
    zkml/src/lookup/operation/inputs/proving.rs:74-84): sum_c b_c * (MLE of the operation's padded output slice c at
    the claim's point + sum_j s^j * MLE of witness (c, j) at the logup point); and the sumcheck verifies, its final
    evaluations being the witness tables at its point."""
    rng = np.random.default_rng(9950)
    shape = (3, 5, 6)
    ci, w, outputs, out_min, out_max = linking_case(F, kind, rng, shape)
    mles = [F.table_from_i64(c) for c in w.output_columns()]
    n2d = 3 + 3
    claim_point = [F.random_scalar(rng) for _ in range(n2d + 2)]
    logup_point = [F.random_scalar(rng) for _ in range(n2d)]
    res = orc.lookup_linking_prove(F, orc.Transcript(F), orc.VARIANT_STANDARD, ci, out_min, out_max, shape, mles,
                                   claim_point, logup_point)
    chal = res["challenges"]
    s, betas = chal[0], chal[1:]
    assert len(betas) == 3
    # the slices' coefficients are the eq evaluations of the leading dimension's coordinates
    lead = orc.array_to_scalars(F, orc.eq_evals(F, claim_point[n2d:]))
    assert betas == lead[:3]
    per = ci.n_value + ci.n_zeroing
    want = F.zero
    for c in range(3):
        out_eval = orc.evaluate(F, F.table_from_i64(outputs[c].reshape(-1)), claim_point[:n2d])
        lk = F.zero
        if ci.n_value == 1:
            powers = [1] + [2 + j for j in range(ci.n_zeroing)]
        else:
            powers = [1 + j for j in range(ci.n_value)] + [1 + ci.n_value + j for j in range(ci.n_zeroing)]
        for j, p in enumerate(powers):
            lk = F.add(lk, F.mul(F.pow(s, p), orc.evaluate(F, mles[c * per + j], logup_point)))
        want = F.add(want, F.mul(betas[c], F.add(out_eval, lk)))
    assert orc.extract_sum(F, res["sumcheck"]) == want
    # the whole padded output tensor at the claim's point is the first half of that sum
    full = np.zeros((4, 8, 8), dtype=np.int64)
    full[:3] = np.stack(outputs)
    total_out = orc.evaluate(F, F.table_from_i64(full.reshape(-1)), claim_point)
    part = F.zero
    for c in range(3):
        part = F.add(part, F.mul(betas[c], orc.evaluate(F, F.table_from_i64(outputs[c].reshape(-1)), claim_point[:n2d])))
    assert part == total_out
    # verifier side: rounds check out, final evaluations are the tables at the point
    degree = len(res["sumcheck"][0]) - 1
    tr = orc.Transcript(F)
    tr.append_and_sample(b"sum")
    v_point, expected = orc.sumcheck_verify(F, want, res["sumcheck"], n2d, degree, tr)
    point = res["point"]
    assert v_point == point
    assert [orc.evaluate(F, m, point) for m in mles] == res["evaluations"]
    expr = orc.lookup_linking_expression(F, orc.VARIANT_STANDARD, 3, ci, out_min, out_max)
    wit = res["evaluations"] + [orc.identity_eval(F, claim_point[:n2d], point), orc.identity_eval(F, logup_point, point)]
    assert orc.eval_expr(F, expr, wit, chal) == expected


def test_eq_point_and_batching_challenges_shapes():
    F = orc.FrField
    rng = np.random.default_rng(9960)
    for shape in [(5,), (3, 7), (2, 3, 5), (2, 3, 4, 8)]:
        total = sum(max(d - 1, 0).bit_length() for d in shape)
        pt = [F.random_scalar(rng) for _ in range(total)]
        eq_point, chal = orc.eq_point_and_batching_challenges(F, shape, pt)
        n2d = sum(max(d - 1, 0).bit_length() for d in shape[-2:])
        assert eq_point == pt[:n2d]
        slices = int(np.prod(shape[:-2])) if len(shape) > 2 else 1
        assert len(chal) == slices
        # coefficient of slice (i0, i1, ..) = prod_k eq(bits of i_k, that dimension's coordinates)
        if len(shape) == 4:
            d1 = orc.array_to_scalars(F, orc.eq_evals(F, pt[n2d:n2d + 2]))     # second dimension (3 -> 2 vars)
            d0 = orc.array_to_scalars(F, orc.eq_evals(F, pt[n2d + 2:]))        # first dimension (2 -> 1 var)
            assert chal == [F.mul(d0[i], d1[j]) for i in range(2) for j in range(3)]
    with pytest.raises(ValueError):
        orc.eq_point_and_batching_challenges(F, (3, 7), [F.one])


@pytest.mark.parametrize("F", [orc.FrField, orc.GlField])
def test_softmax_variant_adds_the_row_sums(F):
    """LookupVariant::Softmax (variant.rs:264-287, build_eq_polys variant/proving.rs:238-251): on top of the
    Standard sum, 2^k * nu * sum_x eq(x, (1/2,..,1/2, r_rows)) P_c(x), which is nu times the sum along the last
    dimension of the operation's output, taken at the logup point's row coordinates."""
    rng = np.random.default_rng(9990)
    shape = (3, 5, 6)
    ci, w, outputs, out_min, out_max = linking_case(F, "relu", rng, shape)
    mles = [F.table_from_i64(c) for c in w.output_columns()]
    n2d, col_vars = 6, 3
    claim_point = [F.random_scalar(rng) for _ in range(n2d + 2)]
    logup_point = [F.random_scalar(rng) for _ in range(n2d)]
    std = orc.lookup_linking_prove(F, orc.Transcript(F), orc.VARIANT_STANDARD, ci, out_min, out_max, shape, mles,
                                   claim_point, logup_point)
    soft = orc.lookup_linking_prove(F, orc.Transcript(F), orc.VARIANT_SOFTMAX, ci, out_min, out_max, shape, mles,
                                    claim_point, logup_point)
    assert soft["challenges"][:-1] == std["challenges"] and len(soft["challenges"]) == 1 + 3 + 1
    nu, betas = soft["challenges"][-1], soft["challenges"][1:4]
    extra = F.zero
    for c in range(3):
        row_sums = outputs[c].sum(axis=1)                       # padded rows, summed along the last dimension
        at_rows = orc.evaluate(F, F.table_from_i64(row_sums), logup_point[col_vars:])
        extra = F.add(extra, F.mul(betas[c], at_rows))
    want = F.add(orc.extract_sum(F, std["sumcheck"]), F.mul(nu, extra))
    assert orc.extract_sum(F, soft["sumcheck"]) == want
    tr = orc.Transcript(F)
    tr.append_and_sample(b"sum")
    tr.append_and_sample(b"normalisation")
    degree = len(soft["sumcheck"][0]) - 1
    point, expected = orc.sumcheck_verify(F, want, soft["sumcheck"], n2d, degree, tr)
    half = F.inv(F.from_int(2))
    expr = orc.lookup_linking_expression(F, orc.VARIANT_SOFTMAX, 3, ci, out_min, out_max, shape[-1])
    wit = soft["evaluations"] + [orc.identity_eval(F, claim_point[:n2d], point), orc.identity_eval(F, logup_point, point),
                                 orc.identity_eval(F, [half] * col_vars + logup_point[col_vars:], point)]
    assert orc.eval_expr(F, expr, wit, soft["challenges"]) == expected


@pytest.mark.parametrize("F", [orc.FrField, orc.GlField])
@pytest.mark.parametrize("normalised_sum,with_weight", [(False, False), (True, True)])
def test_normalisation_variant(F, normalised_sum, with_weight):
    """LookupVariant::Normalisation (variant.rs:288-346): the output part (times the weight table when there is
    one), nu times the sums of squares along the last dimension (and nu^2 times the sums, when the sum is
    normalised too) at the logup point's row coordinates, the lookup columns, and iota times the product of each
    chunk's input and scaling tables at the logup point."""
    rng = np.random.default_rng(9995)
    shape = (3, 5, 6)
    ci, w, outputs, out_min, out_max = linking_case(F, "relu", rng, shape)
    n2d, col_vars, P = 6, 3, 64
    small = lambda: F.table_from_i64(rng.integers(-50, 50, size=P, dtype=np.int64))
    inputs, scalings = [small() for _ in range(3)], [small() for _ in range(3)]
    w_int = rng.integers(-50, 50, size=P, dtype=np.int64)
    weight = F.table_from_i64(w_int) if with_weight else None
    mles = [F.table_from_i64(c) for c in w.output_columns()] + inputs + scalings
    claim_point = [F.random_scalar(rng) for _ in range(n2d + 2)]
    logup_point = [F.random_scalar(rng) for _ in range(n2d)]
    res = orc.lookup_linking_prove(F, orc.Transcript(F), orc.VARIANT_NORMALISATION, ci, out_min, out_max, shape, mles,
                                   claim_point, logup_point, normalised_sum=normalised_sum, weight=weight)
    chal = res["challenges"]
    assert len(chal) == 1 + 3 + 2
    s, betas, nu, iota = chal[0], chal[1:4], chal[4], chal[5]
    per = ci.n_value + ci.n_zeroing
    want = F.zero
    for c in range(3):
        out = outputs[c]
        if with_weight:
            lead = orc.evaluate(F, F.table_from_i64((out * w_int.reshape(out.shape)).reshape(-1)), claim_point[:n2d])
        else:
            lead = orc.evaluate(F, F.table_from_i64(out.reshape(-1)), claim_point[:n2d])
        rows = logup_point[col_vars:]
        part = F.add(lead, F.mul(nu, orc.evaluate(F, F.table_from_i64((out * out).sum(axis=1)), rows)))
        if normalised_sum:
            part = F.add(part, F.mul(F.mul(nu, nu), orc.evaluate(F, F.table_from_i64(out.sum(axis=1)), rows)))
        lk = F.zero
        for j, p in enumerate([1] + [2 + k for k in range(ci.n_zeroing)]):
            lk = F.add(lk, F.mul(F.pow(s, p), orc.evaluate(F, mles[c * per + j], logup_point)))
        prod_tab = [F.mul(a, b) for a, b in zip(orc.array_to_scalars(F, orc._widen(F, inputs[c])),
                                                orc.array_to_scalars(F, orc._widen(F, scalings[c])))]
        lk = F.add(lk, F.mul(iota, orc.evaluate(F, orc.scalars_to_array(F, prod_tab), logup_point)))
        want = F.add(want, F.mul(betas[c], F.add(part, lk)))
    assert orc.extract_sum(F, res["sumcheck"]) == want
    tr = orc.Transcript(F)
    for label in (b"sum", b"normalisation", b"input"):
        tr.append_and_sample(label)
    degree = len(res["sumcheck"][0]) - 1
    point, expected = orc.sumcheck_verify(F, want, res["sumcheck"], n2d, degree, tr)
    half = F.inv(F.from_int(2))
    expr = orc.lookup_linking_expression(F, orc.VARIANT_NORMALISATION, 3, ci, out_min, out_max, shape[-1],
                                         normalised_sum, with_weight)
    wit = res["evaluations"] + [orc.identity_eval(F, claim_point[:n2d], point), orc.identity_eval(F, logup_point, point),
                                orc.identity_eval(F, [half] * col_vars + logup_point[col_vars:], point)]
    if with_weight:
        assert res["weight_eval"] == orc.evaluate(F, weight, point)
        wit.append(res["weight_eval"])
    assert orc.eval_expr(F, expr, wit, chal) == expected
