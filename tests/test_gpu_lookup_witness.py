"""Lookup witness generation on the device (dpb_lookup_witness, dpb_lookup_counts_*, dpb_lookup_multiplicities)
against the oracle's restatement of LookupOp::generate_witness and the multiplicity computation: every chunk column
and every looked-up column bit for bit, the per-table counts, and that the columns and multiplicities satisfy the
logup argument they are made for."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import family_dtype

FIELDS = [orc.FrField, orc.GlField]


def test_chunking_info_matches_the_oracle(dpb):
    """Host-only: the numbers of ChunkingInfo::new over the reference's own test strategy and beyond."""
    rng = np.random.default_rng(9500)
    for _ in range(500):
        right_shift = int(rng.integers(1, 40))
        bits = int(rng.integers(2, 17))
        n_value = int(rng.integers(1, 3))
        sign = int(rng.integers(0, 3))
        if right_shift + bits * n_value > 60:
            continue
        max_bit_size = int(rng.integers(max(right_shift + bits * n_value - 3, 1), 63))
        want = orc.ChunkingInfo(right_shift, bits, sign, max_bit_size, n_value)
        if want.n_zeroing > 4 or want.n_shifted > 4:
            with pytest.raises(dpb.DpbError):
                dpb.ChunkingInfo.new(right_shift, bits, sign, max_bit_size, n_value)
            continue
        got = dpb.ChunkingInfo.new(right_shift, bits, sign, max_bit_size, n_value)
        assert (got.n_shifted_chunks, got.n_zeroing_chunks, got.offset, got.value_chunk_offset,
                got.shifted_chunk_multiplier, got.top_zeroing_chunk_offset) == \
               (want.n_shifted, want.n_zeroing, want.offset, want.value_chunk_offset,
                want.shifted_chunk_multiplier, want.top_zeroing_chunk_offset)
    with pytest.raises(dpb.DpbError) as e:
        dpb.ChunkingInfo.new(0, 8, 2, 40)
    assert "Right shift must be greater than zero" in str(e.value)


def value_table(kind, bits):
    """(sign, output column or None, columns): integer stand-ins for the reference's tables.  'exp' is a
    decreasing table over non-positive inputs with the shape of TableType::Exp (tabletype.rs:90-99); its values
    come from float32 arithmetic here and are data, not part of what is checked."""
    if kind == "relu":
        lo, hi = orc.table_input_range(bits, orc.SIGN_MIXED)
        return orc.SIGN_MIXED, np.clip(np.arange(lo, hi + 1, dtype=np.int64), 0, hi), 2
    if kind == "requantise":
        return orc.SIGN_MIXED, None, 1
    if kind == "exp":
        lo, hi = orc.table_input_range(bits, orc.SIGN_NEGATIVE)
        x = np.arange(lo, hi + 1, dtype=np.int64)
        out = np.rint(np.exp(x.astype(np.float32) / np.float32(1 << (bits - 3))) * np.float32(1 << 20)).astype(np.int64)
        out[0] = 0
        return orc.SIGN_NEGATIVE, out, 2
    if kind == "positive":
        return orc.SIGN_POSITIVE, (np.arange(1 << bits, dtype=np.int64) * 2654435761) % 1000003 - 500000, 2
    raise ValueError(kind)


def draw_tensor(rng, shape, sign, max_bit_size, fpm):
    big = (1 << (max_bit_size - 2)) // fpm
    if sign == orc.SIGN_MIXED:
        t = rng.integers(-big, big, size=shape, dtype=np.int64)
    elif sign == orc.SIGN_POSITIVE:
        t = rng.integers(0, big, size=shape, dtype=np.int64)
    else:
        t = -rng.integers(0, big, size=shape, dtype=np.int64)
    flat = t.reshape(-1)
    flat[::3] >>= int(rng.integers(10, 30))  # small magnitudes too
    flat[::7] = 0
    return t


def check_case(dpb, ctx, F, kind, bits, right_shift, max_bit_size, shape, fpm, padding, rng, n_value=1, device_tensor=False):
    sign, table_out, n_cols = value_table(kind, bits)
    want_ci = orc.ChunkingInfo(right_shift, bits, sign, max_bit_size, n_value)
    ci = dpb.ChunkingInfo.new(right_shift, bits, sign, max_bit_size, n_value)
    t = draw_tensor(rng, shape, sign, max_bit_size, fpm)
    want = orc.LookupOpWitness(want_ci, fpm, padding, t, table_out, n_cols)
    counts = [dpb.LookupCounts(ctx, b) for b in (16, bits, 16, 16)]
    fam = family_dtype(dpb, F)
    dev = ctx.upload_tensor_i64(t) if device_tensor else None
    owner, ins, outs = dpb.lookup_witness(ctx, fam, ci, fpm, padding, t, table_out, n_cols, counts, device_tensor=dev)
    try:
        want_in, want_out = want.input_columns(), want.output_columns()
        assert len(ins) == len(want_in) and len(outs) == len(want_out)
        for got, col in zip(ins + outs, want_in + want_out):
            assert got.len == col.size
            assert np.array_equal(got.to_host(), F.table_from_i64(col))
        # counts: dense rows on the device, merged keys in the oracle
        shift, value, zero, signed = want.get_counts()
        lo, _ = orc.table_input_range(bits, sign)
        got_counts = [c.to_host() for c in counts]
        sep = orc.COLUMN_SEPARATOR

        def dense(d, n, key_to_row):
            a = np.zeros(n, dtype=np.uint64)
            for k, c in d.items():
                a[key_to_row(k)] += c
            return a

        def input_of(key):  # merged key = input + 2^32 * output, |input| < 2^31
            return ((key + (1 << 31)) % sep) - (1 << 31)

        assert np.array_equal(got_counts[0], dense(shift, 1 << 16, lambda k: k))
        assert np.array_equal(got_counts[1], dense(value, 1 << bits, (lambda k: k - lo) if n_cols == 1 else (lambda k: input_of(k) - lo)))
        assert np.array_equal(got_counts[2], dense(zero, 1 << 16, input_of))
        assert np.array_equal(got_counts[3], dense(signed, 1 << 16, lambda k: input_of(k) + (1 << 15)))
        # multiplicities against the reference's computation over the merged table column
        m = counts[1].multiplicities(fam)
        col = orc.merged_table_column(bits, sign, table_out)
        assert F.table_to_ints(m.to_host()) == orc.array_to_scalars(F, orc.table_multiplicities(F, col, value))
        m.free()
    finally:
        for v in ins + outs:
            v.free()
        owner.free()
        for c in counts:
            c.free()
        if dev is not None:
            dev[0].free()
    return want


@pytest.mark.gpu
@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("kind,bits,right_shift,max_bit_size", [
    ("relu", 10, 13, 44), ("relu", 8, 16, 40), ("relu", 12, 27, 55), ("relu", 9, 12, 21), ("requantise", 10, 32, 60),
    ("exp", 11, 10, 40), ("exp", 8, 20, 28), ("positive", 9, 17, 50), ("positive", 16, 5, 21)])
def test_witness_columns_counts_multiplicities(dpb, ctx, F, kind, bits, right_shift, max_bit_size):
    rng = np.random.default_rng(9600 + bits + right_shift)
    for shape in [(5,), (3, 7), (2, 3, 5), (2, 2, 4, 8), (1, 1), (33, 65)]:
        check_case(dpb, ctx, F, kind, bits, right_shift, max_bit_size, shape, 37, 0 if kind != "exp" else -3, rng)


@pytest.mark.gpu
@pytest.mark.parametrize("F", FIELDS)
def test_integer_columns(dpb, ctx, F):
    """family_dtype = an integer layout: the columns are the chunks themselves (64-bit integers), equal to the
    oracle's integer columns, and the counters are the same as with field columns."""
    rng = np.random.default_rng(9650)
    for kind, bits, right_shift, max_bit_size, shape in [("relu", 10, 13, 44, (3, 7, 9)), ("exp", 8, 10, 34, (2, 12, 12)),
                                                         ("requantise", 10, 32, 60, (33, 65))]:
        sign, table_out, n_cols = value_table(kind, bits)
        t = draw_tensor(rng, shape, sign, max_bit_size, 5)
        want = orc.LookupOpWitness(orc.ChunkingInfo(right_shift, bits, sign, max_bit_size), 5, 0, t, table_out, n_cols)
        ci = dpb.ChunkingInfo.new(right_shift, bits, sign, max_bit_size)
        dt = dpb.FR_I64 if F is orc.FrField else dpb.GL_I64
        counts = [dpb.LookupCounts(ctx, b) for b in (16, bits, 16, 16)]
        counts_f = [dpb.LookupCounts(ctx, b) for b in (16, bits, 16, 16)]
        owner, ins, outs = dpb.lookup_witness(ctx, dt, ci, 5, 0, t, table_out, n_cols, counts)
        owner_f, ins_f, outs_f = dpb.lookup_witness(ctx, family_dtype(dpb, F), ci, 5, 0, t, table_out, n_cols, counts_f)
        for got, col in zip(ins + outs, want.input_columns() + want.output_columns()):
            assert got.dtype == dt and np.array_equal(got.to_host(), col)
        for a, b in zip(counts, counts_f):
            assert np.array_equal(a.to_host(), b.to_host())
        for h in ins + outs + ins_f + outs_f + [owner, owner_f] + counts + counts_f:
            h.free()


@pytest.mark.gpu
@pytest.mark.parametrize("F", FIELDS)
def test_two_value_chunks_and_device_tensor(dpb, ctx, F):
    rng = np.random.default_rng(9700)
    check_case(dpb, ctx, F, "requantise", 8, 12, 44, (3, 5, 9), 3, 0, rng, n_value=2)
    check_case(dpb, ctx, F, "relu", 10, 13, 44, (4, 17, 31), 5, 2, rng, device_tensor=True)


@pytest.mark.gpu
@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("side", [10, 11])
def test_large_tensor_with_constant_chunks(dpb, ctx, F, side):
    """2^20 and 2^22 entries whose zeroing chunks are all equal (the usual case: values far below the declared maximum),
    which is the case the block-local counters are for."""
    rng = np.random.default_rng(9800)
    bits, right_shift, max_bit_size = 12, 16, 60
    sign, table_out, n_cols = value_table("relu", bits)
    t = rng.integers(-(1 << 20), 1 << 20, size=(1 << side, 1 << side), dtype=np.int64)
    want_ci = orc.ChunkingInfo(right_shift, bits, sign, max_bit_size)
    want = orc.LookupOpWitness(want_ci, 1 << 5, 0, t, table_out, n_cols)
    ci = dpb.ChunkingInfo.new(right_shift, bits, sign, max_bit_size)
    counts = [dpb.LookupCounts(ctx, b) for b in (16, bits, 16, 16)]
    fam = family_dtype(dpb, F)
    for rep in range(2):  # counters add up over calls
        owner, ins, outs = dpb.lookup_witness(ctx, fam, ci, 1 << 5, 0, t, table_out, n_cols, counts)
        for got, col in zip(ins + outs, want.input_columns() + want.output_columns()):
            assert np.array_equal(got.to_host(), F.table_from_i64(col))
        for v in ins + outs:
            v.free()
        owner.free()
    shift, value, zero, signed = want.get_counts()
    got = [c.to_host() for c in counts]
    assert int(got[0].sum()) == 2 * sum(shift.values()) and int(got[1].sum()) == 2 * sum(value.values())
    assert int(got[2].sum()) == 2 * sum(zero.values()) and int(got[3].sum()) == 2 * sum(signed.values())
    for k, c in shift.items():
        assert got[0][k] == 2 * c
    assert len(zero) == 1 and len(signed) == 1  # one row each: every lookup of those tables hits it
    for c in counts:
        c.free()


@pytest.mark.gpu
def test_value_beyond_the_declared_size_is_an_error(dpb, ctx):
    """The reference fails with the signed zero-check table's range error (tabletype.rs:137-143) when an input is
    too large for max_bit_size; so does the call."""
    bits, right_shift, max_bit_size = 10, 13, 44
    sign, table_out, n_cols = value_table("relu", bits)
    ci = dpb.ChunkingInfo.new(right_shift, bits, sign, max_bit_size)
    t = np.array([[1, 2], [3, 3 << 53]], dtype=np.int64)
    with pytest.raises(ValueError):
        orc.LookupOpWitness(orc.ChunkingInfo(right_shift, bits, sign, max_bit_size), 1, 0, t, table_out, n_cols)
    with pytest.raises(dpb.DpbError) as e:
        dpb.lookup_witness(ctx, dpb.FR, ci, 1, 0, t, table_out, n_cols)
    assert e.value.code == dpb.EINVAL and "SignedZeroCheckTable" in str(e.value)
    with pytest.raises(dpb.DpbError):
        dpb.lookup_witness(ctx, dpb.FR, ci, 1, 0, t, None, 2)  # two columns need the output column


@pytest.mark.gpu
@pytest.mark.parametrize("F", FIELDS)
def test_witness_feeds_the_logup_argument(dpb, ctx, F):
    """The fractions of the lookups (value chunk in, value chunk out) and of the table with the device's
    multiplicities cancel: sum_lookups 1/(c + in + s*out) = sum_rows m/(c + in + s*out), which is the global check
    of zkml/src/iop/verifier.rs:543-584 on the trees' outputs."""
    rng = np.random.default_rng(9900)
    bits, right_shift, max_bit_size = 8, 12, 40
    sign, table_out, n_cols = value_table("relu", bits)
    ci = dpb.ChunkingInfo.new(right_shift, bits, sign, max_bit_size)
    t = draw_tensor(rng, (2, 16, 32), sign, max_bit_size, 7)
    counts = dpb.LookupCounts(ctx, bits)
    fam = family_dtype(dpb, F)
    owner, ins, outs = dpb.lookup_witness(ctx, fam, ci, 7, 0, t, table_out, n_cols, (None, counts, None, None))
    n_in_per, n_out_per = len(ins) // 2, len(outs) // 2
    cst, sep = F.random_scalar(rng), F.random_scalar(rng)
    c_arr, s_arr = orc.scalars_to_array(F, [cst]), orc.scalars_to_array(F, [sep])
    fracs = []
    for s in range(2):
        vin = ins[s * n_in_per + ci.n_shifted_chunks]
        vout = outs[s * n_out_per]
        lu = ctx.logup(0, [vin, vout], c_arr, s_arr)
        fracs.append(orc.array_to_scalars(F, lu.outputs()))
        lu.free()
    lo, hi = orc.table_input_range(bits, sign)
    tin = ctx.upload(F.table_from_i64(np.arange(lo, hi + 1, dtype=np.int64)), dpb.dtype_of_array(F.table_from_i64(np.arange(2)), F.name))
    tout = ctx.upload(F.table_from_i64(table_out), tin.dtype)
    mult = counts.multiplicities(fam)
    lu = ctx.logup(1, [tin, tout], c_arr, s_arr, mult)
    fracs.append(orc.array_to_scalars(F, lu.outputs()))
    lu.free()
    n, d = F.zero, F.one
    for n0, n1, d0, d1 in fracs:
        for nn, dd in ((n0, d0), (n1, d1)):
            n, d = F.add(F.mul(n, dd), F.mul(d, nn)), F.mul(d, dd)
    assert n == F.zero and d != F.zero
    for m in ins + outs + [tin, tout, mult]:
        m.free()
    owner.free()
    counts.free()


# ------------------------------------------------------------- linking sumcheck
@pytest.fixture(scope="module")
def prover(dpb):
    import importlib
    return importlib.import_module("deep_prove_b200.prover")


def flat(F, arr):
    return orc.array_to_scalars(F, np.asarray(arr).reshape(-1, F.elem_words))


@pytest.mark.gpu
@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("kind,bits,right_shift,max_bit_size,n_value,shape", [
    ("relu", 8, 12, 40, 1, (3, 5, 6)),          # two zeroing chunks, rank 3
    ("relu", 10, 13, 23, 1, (7, 9)),            # no zeroing chunk, rank 2
    ("relu", 9, 11, 30, 1, (2, 3, 17, 33)),     # one zeroing chunk, rank 4, 2^11 entries per slice
    ("requantise", 8, 12, 44, 2, (4, 16, 8)),   # two value chunks
    ("exp", 8, 10, 34, 1, (2, 12, 12)),         # a table over non-positive inputs
    ("positive", 9, 17, 26, 1, (11,)),          # no zeroing chunk, unsigned: the reference's 1 + value form
])
@pytest.mark.parametrize("variant", [0, 2])
def test_linking_sumcheck_on_the_device_witness(dpb, ctx, prover, F, kind, bits, right_shift, max_bit_size, n_value, shape,
                                                variant):
    """The witness columns come from dpb_lookup_witness and go straight into dpb_lookup_linking_prove; proof,
    point, evaluations, batching challenges and the transcript's state afterwards equal the oracle's."""
    rng = np.random.default_rng(9970 + bits + right_shift)
    sign, table_out, n_cols = value_table(kind, bits)
    fpm = 3
    t = draw_tensor(rng, shape, sign, max_bit_size, fpm)
    o_ci = orc.ChunkingInfo(right_shift, bits, sign, max_bit_size, n_value)
    want_w = orc.LookupOpWitness(o_ci, fpm, 0, t, table_out, n_cols)
    if table_out is None:
        out_min, out_max = orc.table_input_range(bits, sign)
    else:
        out_min, out_max = int(table_out[0]), int(table_out[-1])  # Table::min/max_output_value: the outputs at the ends
    o_mles = [F.table_from_i64(c) for c in want_w.output_columns()]
    dims = [1 << max(d - 1, 0).bit_length() for d in shape]
    total = sum(d.bit_length() - 1 for d in dims)
    n2d = sum(d.bit_length() - 1 for d in dims[-2:])
    claim_point = [F.random_scalar(rng) for _ in range(total)]
    logup_point = [F.random_scalar(rng) for _ in range(n2d)]
    o_tr = orc.Transcript(F)
    want = orc.lookup_linking_prove(F, o_tr, variant, o_ci, out_min, out_max, shape, o_mles, claim_point, logup_point)

    fam = family_dtype(dpb, F)
    ci = dpb.ChunkingInfo.new(right_shift, bits, sign, max_bit_size, n_value)
    owner, ins, outs = dpb.lookup_witness(ctx, fam, ci, fpm, 0, t, table_out, n_cols)
    tr = prover.Blake3Transcript(fam)
    got = prover.lookup_linking_prove(ctx, tr, variant, ci, out_min, out_max, shape, outs,
                                      orc.scalars_to_array(F, claim_point), orc.scalars_to_array(F, logup_point))
    assert flat(F, got["challenges"]) == want["challenges"]
    assert flat(F, got["sumcheck"]) == [e for r in want["sumcheck"] for e in r]
    assert flat(F, got["point"]) == want["point"]
    assert flat(F, got["evaluations"]) == want["evaluations"]
    assert tr.state() == (o_tr.state, o_tr.round)
    for m in ins + outs:
        m.free()
    owner.free()
    tr.free()


@pytest.mark.gpu
@pytest.mark.parametrize("F", FIELDS)
def test_linking_sumcheck_glu_and_errors(dpb, ctx, prover, F):
    rng = np.random.default_rng(9980)
    bits, right_shift, max_bit_size, shape = 8, 12, 40, (2, 6, 8)
    sign, table_out, n_cols = value_table("relu", bits)
    t = draw_tensor(rng, shape, sign, max_bit_size, 3)
    o_ci = orc.ChunkingInfo(right_shift, bits, sign, max_bit_size)
    w = orc.LookupOpWitness(o_ci, 3, 0, t, table_out, n_cols)
    glu = [F.random_table_fast(rng, 64) if F is orc.FrField else F.random_table(rng, 64) for _ in range(2)]
    o_mles = [F.table_from_i64(c) for c in w.output_columns()] + glu
    claim_point = [F.random_scalar(rng) for _ in range(7)]
    logup_point = [F.random_scalar(rng) for _ in range(6)]
    o_tr = orc.Transcript(F)
    want = orc.lookup_linking_prove(F, o_tr, orc.VARIANT_GLU, o_ci, 0, 127, shape, o_mles, claim_point, logup_point)
    fam = family_dtype(dpb, F)
    ci = dpb.ChunkingInfo.new(right_shift, bits, sign, max_bit_size)
    d_mles = [ctx.upload(np.ascontiguousarray(m), dpb.dtype_of_array(m, F.name)) for m in o_mles]
    tr = prover.Blake3Transcript(fam)
    got = prover.lookup_linking_prove(ctx, tr, prover.VARIANT_GLU, ci, 0, 127, shape, d_mles,
                                      orc.scalars_to_array(F, claim_point), orc.scalars_to_array(F, logup_point))
    assert flat(F, got["sumcheck"]) == [e for r in want["sumcheck"] for e in r]
    assert flat(F, got["evaluations"]) == want["evaluations"]
    assert tr.state() == (o_tr.state, o_tr.round)
    # a table too few, a claim point of the wrong length (the reference's error text)
    with pytest.raises(dpb.DpbError) as e:
        prover.lookup_linking_prove(ctx, tr, prover.VARIANT_GLU, ci, 0, 127, shape, d_mles[:-1],
                                    orc.scalars_to_array(F, claim_point), orc.scalars_to_array(F, logup_point))
    assert "witness tables" in str(e.value)
    with pytest.raises(dpb.DpbError) as e:
        prover.lookup_linking_prove(ctx, tr, prover.VARIANT_GLU, ci, 0, 127, shape, d_mles,
                                    orc.scalars_to_array(F, claim_point[:-1]), orc.scalars_to_array(F, logup_point))
    assert "does not match total variables" in str(e.value)
    for m in d_mles:
        m.free()
    tr.free()


@pytest.mark.gpu
@pytest.mark.parametrize("F", FIELDS)
def test_lookup_golden(dpb, ctx, prover, F):
    """The committed fixture (tests/golden, made by make_golden.py from the oracle): witness columns, counts,
    multiplicities and the linking proof of a seeded lookup operation."""
    import json
    import os
    from tests.golden import make_golden
    with open(os.path.join(os.path.dirname(__file__), "golden", f"oracle_{F.name}.json")) as f:
        want = json.load(f)["lookup"]
    g = make_golden.golden_inputs(F, "lookup")
    fam = family_dtype(dpb, F)
    ci = dpb.ChunkingInfo.new(g["right_shift"], g["bits"], orc.SIGN_MIXED, g["max_bit_size"])
    counts = [dpb.LookupCounts(ctx, b) for b in (16, g["bits"], 16, 16)]
    owner, ins, outs = dpb.lookup_witness(ctx, fam, ci, g["fpm"], g["padding"], g["tensor"], g["table_out"], 2, counts)
    for got, col in zip(ins + outs, want["columns"]):
        assert np.array_equal(got.to_host(), F.table_from_i64(np.array(col, dtype=np.int64)))
    assert len(ins) + len(outs) == len(want["columns"])
    lo, _ = orc.table_input_range(g["bits"], orc.SIGN_MIXED)
    sep = orc.COLUMN_SEPARATOR
    input_of = lambda key: ((key + (1 << 31)) % sep) - (1 << 31)
    rows = [lambda k: k, lambda k: input_of(k) - lo, input_of, lambda k: input_of(k) + (1 << 15)]
    for c, pairs, row in zip(counts, want["counts"], rows):
        dense = np.zeros(1 << c.bits, dtype=np.uint64)
        for key, n in pairs:
            dense[row(key)] += n
        assert np.array_equal(c.to_host(), dense)
    m = counts[1].multiplicities(fam)
    assert orc.serialize_scalars(F, F.table_to_ints(m.to_host())).hex() == want["multiplicities"]
    tr = prover.Blake3Transcript(fam)
    got = prover.lookup_linking_prove(ctx, tr, prover.VARIANT_STANDARD, ci, g["out_min"], g["out_max"], g["tensor"].shape,
                                      outs, orc.scalars_to_array(F, g["claim_point"]),
                                      orc.scalars_to_array(F, g["logup_point"]))
    hx = lambda a: orc.serialize_scalars(F, flat(F, a)).hex()
    assert hx(got["point"]) == want["linking"]["point"]
    assert hx(got["evaluations"]) == want["linking"]["evaluations"]
    assert hx(got["challenges"]) == want["linking"]["challenges"]
    proof = [flat(F, r) for r in got["sumcheck"]]
    assert orc.serialize_sumcheck_proof(F, proof).hex() == want["linking"]["proof"]
    for h in ins + outs + [m]:
        h.free()
    owner.free()
    tr.free()
    for c in counts:
        c.free()


@pytest.mark.gpu
@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("with_sum,with_weight,kind,bits,right_shift,max_bit_size,shape", [
    (False, False, "relu", 8, 12, 40, (3, 5, 6)),      # two zeroing chunks: degree 6 under the third eq table
    (True, True, "relu", 8, 12, 30, (2, 9, 12)),       # one zeroing chunk, the sum tied too, a weight table
    (True, False, "relu", 10, 13, 23, (7, 33)),        # no zeroing chunk, 2^9 entries
    (False, True, "exp", 8, 10, 34, (2, 6, 6)),        # a table over non-positive inputs
])
def test_linking_sumcheck_normalisation(dpb, ctx, prover, F, with_sum, with_weight, kind, bits, right_shift, max_bit_size,
                                        shape):
    rng = np.random.default_rng(9985 + bits)
    sign, table_out, n_cols = value_table(kind, bits)
    t = draw_tensor(rng, shape, sign, max_bit_size, 3)
    o_ci = orc.ChunkingInfo(right_shift, bits, sign, max_bit_size)
    w = orc.LookupOpWitness(o_ci, 3, 0, t, table_out, n_cols)
    out_min, out_max = int(table_out[0]), int(table_out[-1])
    dims = [1 << max(d - 1, 0).bit_length() for d in shape]
    total, n2d = sum(d.bit_length() - 1 for d in dims), sum(d.bit_length() - 1 for d in dims[-2:])
    slices = int(np.prod(shape[:-2])) if len(shape) > 2 else 1
    P = 1 << n2d
    rand = lambda: F.random_table_fast(rng, P) if F is orc.FrField else F.random_table(rng, P)
    extra = [rand() for _ in range(2 * slices)]
    weight = rand() if with_weight else None
    o_mles = [F.table_from_i64(c) for c in w.output_columns()] + extra
    claim_point = [F.random_scalar(rng) for _ in range(total)]
    logup_point = [F.random_scalar(rng) for _ in range(n2d)]
    o_tr = orc.Transcript(F)
    want = orc.lookup_linking_prove(F, o_tr, orc.VARIANT_NORMALISATION, o_ci, out_min, out_max, shape, o_mles, claim_point,
                                    logup_point, normalised_sum=with_sum, weight=weight)
    fam = family_dtype(dpb, F)
    ci = dpb.ChunkingInfo.new(right_shift, bits, sign, max_bit_size)
    up = lambda m: ctx.upload(np.ascontiguousarray(m), dpb.dtype_of_array(m, F.name))
    d_mles = [up(m) for m in o_mles]
    d_weight = up(weight) if with_weight else None
    tr = prover.Blake3Transcript(fam)
    variant = prover.VARIANT_NORMALISATION_WITH_SUM if with_sum else prover.VARIANT_NORMALISATION
    got = prover.lookup_linking_prove(ctx, tr, variant, ci, out_min, out_max, shape, d_mles,
                                      orc.scalars_to_array(F, claim_point), orc.scalars_to_array(F, logup_point),
                                      weight=d_weight)
    assert flat(F, got["challenges"]) == want["challenges"]
    assert flat(F, got["sumcheck"]) == [e for r in want["sumcheck"] for e in r]
    assert flat(F, got["point"]) == want["point"]
    assert flat(F, got["evaluations"]) == want["evaluations"]
    if with_weight:
        assert flat(F, got["weight_eval"]) == [want["weight_eval"]]
    assert tr.state() == (o_tr.state, o_tr.round)
    if not with_weight:  # a weight table belongs to this variant only
        with pytest.raises(dpb.DpbError):
            prover.lookup_linking_prove(ctx, tr, prover.VARIANT_STANDARD, ci, out_min, out_max, shape,
                                        d_mles[:len(w.output_columns())], orc.scalars_to_array(F, claim_point),
                                        orc.scalars_to_array(F, logup_point), weight=d_mles[0])
    for m in d_mles + ([d_weight] if d_weight else []):
        m.free()
    tr.free()
