"""The whole path of one dense + ReLU layer at the sizes of the two-layer MLP configuration (input 1 x 1024 int8,
weights 1024 x 1024 int8, int32 bias, ReLU through a 12-bit lookup table), every step on the device and checked
against the oracle, each step's output feeding the next:

  einsum axis fixing -> dense sumcheck (n = 10) -> lookup witness of the rescaled pre-activations (chunk columns,
  per-table counts) -> multiplicities -> batched logup-GKR over the three tables (2^16, 2^16 and 2^12 rows) and
  over the three lookups into them (2^10 each) -> linking sumcheck.

The inputs are seeded synthetic integers of the configuration's shapes and ranges."""
import importlib

import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import family_dtype, gpu_sumcheck_prove

pytestmark = pytest.mark.gpu

FIELDS = [orc.FrField, orc.GlField]


@pytest.fixture(scope="module")
def prover(dpb):
    return importlib.import_module("deep_prove_b200.prover")


def flat(F, arr):
    return orc.array_to_scalars(F, np.asarray(arr).reshape(-1, F.elem_words))


@pytest.mark.parametrize("F", FIELDS)
def test_dense_relu_layer_of_the_mlp(dpb, ctx, prover, F):
    rng = np.random.default_rng(0)
    d_in = d_out = 1024
    x = rng.integers(-128, 128, size=(1, d_in), dtype=np.int64)
    w = rng.integers(-128, 128, size=(d_in, d_out), dtype=np.int64)
    b = rng.integers(-(1 << 15), 1 << 15, size=d_out, dtype=np.int64)
    y = x @ w + b                                   # pre-activations, |y| < 2^25
    fam = family_dtype(dpb, F)
    base = dpb.FR if F is orc.FrField else dpb.GL_BASE
    S_ = lambda p: orc.scalars_to_array(F, p)
    T = F.table_from_i64

    # ---- dense layer: claim on y at r_out  =  sum_c x(c) W~(c, r_out) + b~(r_out)
    r_out = [F.random_scalar(rng) for _ in range(10)]
    O, C = dpb.AXIS_OUTER, dpb.AXIS_CONTRACTED
    w_owner, w_tabs = ctx.einsum_fix_axes(fam, w, (C, O), [None, S_(r_out)])
    x_tab = ctx.upload_i64(x.reshape(-1), base)     # a single row: nothing to bind on the input's side
    o_w = orc.mles_from_tensor(F, w, (orc.AXIS_CONTRACTED, orc.AXIS_OUTER), [None, r_out])[0]
    o_x = T(x.reshape(-1))
    assert np.array_equal(w_tabs[0].to_host(), o_w)
    terms = {(0, 1): F.one}
    want = orc.sumcheck_prove(F, 10, [o_x, o_w], terms, orc.Transcript(F))
    got = gpu_sumcheck_prove(dpb, ctx, F, 10, [x_tab, w_tabs[0]], terms, orc.Transcript(F))
    assert got == want
    y_claim = orc.evaluate(F, T(y.reshape(-1)), r_out)
    assert F.add(orc.extract_sum(F, got[0]), orc.evaluate(F, T(b), r_out)) == y_claim

    # ---- ReLU with requantisation through lookups: (y + 2^12) >> 13 into a 12-bit signed table
    bits, right_shift, max_bit_size, fpm = 12, 13, 28, 1
    lo, hi = orc.table_input_range(bits, orc.SIGN_MIXED)
    relu_in = np.arange(lo, hi + 1, dtype=np.int64)
    relu_out = np.clip(relu_in, 0, hi)
    o_ci = orc.ChunkingInfo(right_shift, bits, orc.SIGN_MIXED, max_bit_size)
    ci = dpb.ChunkingInfo.new(right_shift, bits, orc.SIGN_MIXED, max_bit_size)
    assert (o_ci.n_shifted, o_ci.n_zeroing) == (1, 1)
    o_wit = orc.LookupOpWitness(o_ci, fpm, 0, y, relu_out, 2)
    counts = [dpb.LookupCounts(ctx, n) for n in (16, bits, 16, 16)]
    wit_owner, ins, outs = dpb.lookup_witness(ctx, fam, ci, fpm, 0, y, relu_out, 2, counts)
    for got_col, col in zip(ins + outs, o_wit.input_columns() + o_wit.output_columns()):
        assert np.array_equal(got_col.to_host(), T(col))
    shifted, value_in, zero_in = ins
    value_out, zero_out = outs
    act = np.clip((y + (1 << 12)) >> 13, 0, hi)     # what the layer outputs
    assert np.array_equal(value_out.to_host(), T(act.reshape(-1)))  # nothing clamps at these magnitudes

    # ---- multiplicities, and the batched logup-GKR proof over lookups and tables
    o_counts = o_wit.get_counts()
    shift_col = orc.merged_table_column(16, orc.SIGN_POSITIVE, None)
    relu_col = orc.merged_table_column(bits, orc.SIGN_MIXED, relu_out)
    sz_in = np.arange(-(1 << 15), 1 << 15, dtype=np.int64)
    sz_out = np.sign(sz_in)
    sz_col = orc.merged_table_column(16, orc.SIGN_MIXED, sz_out)
    o_mult = [orc.table_multiplicities(F, shift_col, o_counts[0]), orc.table_multiplicities(F, relu_col, o_counts[1]),
              orc.table_multiplicities(F, sz_col, o_counts[3])]
    d_mult = [counts[0].multiplicities(fam), counts[1].multiplicities(fam), counts[3].multiplicities(fam)]
    for gm, om in zip(d_mult, o_mult):
        assert F.table_to_ints(gm.to_host()) == orc.array_to_scalars(F, om)
    chal = [(F.random_scalar(rng), F.random_scalar(rng)) for _ in range(3)]  # (constant, separator) per table
    S1 = lambda v: orc.scalars_to_array(F, [v])
    o_cols = o_wit.input_columns() + o_wit.output_columns()
    o_inputs = [
        orc.LogUpInput(F, 1, [T(np.arange(1 << 16, dtype=np.int64))], *chal[0], mult=T_base(F, o_mult[0])),
        orc.LogUpInput(F, 1, [T(sz_in), T(sz_out)], *chal[2], mult=T_base(F, o_mult[2])),
        orc.LogUpInput(F, 1, [T(relu_in), T(relu_out)], *chal[1], mult=T_base(F, o_mult[1])),
        orc.LogUpInput(F, 0, [T(o_cols[0])], *chal[0], columns_per_instance=1),
        orc.LogUpInput(F, 0, [T(o_cols[1]), T(o_cols[3])], *chal[1], columns_per_instance=2),
        orc.LogUpInput(F, 0, [T(o_cols[2]), T(o_cols[4])], *chal[2], columns_per_instance=2),
    ]
    up = lambda a: ctx.upload_i64(np.ascontiguousarray(a, dtype=np.int64), base)
    tables = [up(np.arange(1 << 16)), up(sz_in), up(sz_out), up(relu_in), up(relu_out)]
    d_inputs = [
        prover.LogUpInput.new_table([tables[0]], d_mult[0], S1(chal[0][0]), S1(chal[0][1])),
        prover.LogUpInput.new_table([tables[1], tables[2]], d_mult[2], S1(chal[2][0]), S1(chal[2][1])),
        prover.LogUpInput.new_table([tables[3], tables[4]], d_mult[1], S1(chal[1][0]), S1(chal[1][1])),
        prover.LogUpInput.new_lookup([shifted], S1(chal[0][0]), S1(chal[0][1]), 1),
        prover.LogUpInput.new_lookup([value_in, value_out], S1(chal[1][0]), S1(chal[1][1]), 2),
        prover.LogUpInput.new_lookup([zero_in, zero_out], S1(chal[2][0]), S1(chal[2][1]), 2),
    ]
    # a batch holds one kind of input (prover.rs:95-140): the tables' batch, then the lookups' batch
    res = []
    for lo_i, hi_i, kinds in ((0, 3, [(0, 1, 1, 15), (2, 2, 1, 15), (1, 2, 1, 11)]),
                              (3, 6, [(0, 1, 0, 9), (1, 2, 0, 9), (2, 2, 0, 9)])):
        o_tr = orc.Transcript(F)
        w_proof = orc.logup_batch_prove(F, o_inputs[lo_i:hi_i], o_tr)
        d_tr = prover.Blake3Transcript(fam)
        assert prover.new_batch_multiple_sizes_prove(ctx, d_inputs[lo_i:hi_i], d_tr) == orc.serialize_logup_proof(F, w_proof)
        assert d_tr.state() == (o_tr.state, o_tr.round)
        instances = [dict(constant=chal[t][0], sep=chal[t][1], num_columns=nc, kind=kind, num_vars=nv)
                     for t, nc, kind, nv in kinds]
        res.append(orc.logup_batch_verify(F, w_proof, instances, orc.Transcript(F)))
    # per table: its fraction and its lookups' fraction cancel (zkml/src/iop/verifier.rs:543-584)
    for tab, look in ((0, 0), (1, 2), (2, 1)):
        n1, d1 = res[0]["numerators"][tab], res[0]["denominators"][tab]
        n2, d2 = res[1]["numerators"][look], res[1]["denominators"][look]
        assert F.add(F.mul(n1, d2), F.mul(n2, d1)) == F.zero and F.mul(d1, d2) != F.zero

    # ---- linking sumcheck: the activation's claim and the lookup columns' claims in one sumcheck
    r_act = [F.random_scalar(rng) for _ in range(10)]
    logup_point = [F.random_scalar(rng) for _ in range(10)]
    o_tr2, d_tr2 = orc.Transcript(F), prover.Blake3Transcript(fam)
    o_mles = [T(c) for c in o_wit.output_columns()]
    w_link = orc.lookup_linking_prove(F, o_tr2, orc.VARIANT_STANDARD, o_ci, 0, hi, y.shape, o_mles, r_act, logup_point)
    g_link = prover.lookup_linking_prove(ctx, d_tr2, prover.VARIANT_STANDARD, ci, 0, hi, y.shape, outs, S_(r_act),
                                         S_(logup_point))
    assert flat(F, g_link["sumcheck"]) == [e for r in w_link["sumcheck"] for e in r]
    assert flat(F, g_link["point"]) == w_link["point"] and flat(F, g_link["evaluations"]) == w_link["evaluations"]
    assert d_tr2.state() == (o_tr2.state, o_tr2.round)
    s = w_link["challenges"][0]
    want_sum = F.add(orc.evaluate(F, T(act.reshape(-1)), r_act),
                     F.add(F.mul(s, orc.evaluate(F, o_mles[0], logup_point)),
                           F.mul(F.mul(s, s), orc.evaluate(F, o_mles[1], logup_point))))
    assert orc.extract_sum(F, w_link["sumcheck"]) == want_sum


def T_base(F, table):
    """The oracle's multiplicity table in the layout its logup code takes (base elements for Goldilocks)."""
    t = np.asarray(table)
    return t[:, 0].copy() if F is orc.GlField and t.ndim == 2 else t
