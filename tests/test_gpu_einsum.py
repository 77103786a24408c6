"""GPU parity of the einsum axis fixing (dpb_einsum_fix_axes) against the
oracle's restatement of FixedAxesMapping::mles_from_tensor
(zkml/src/layers/einsum/axis.rs:1142-1234), and a dense-layer sumcheck built on
it as EinSum::prove_internal does (zkml/src/layers/einsum/prove.rs:144-190)."""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import family_dtype, gpu_sumcheck_prove

pytestmark = pytest.mark.gpu

FIELDS = [orc.FrField, orc.GlField]
C, O, S = orc.AXIS_CONTRACTED, orc.AXIS_OUTER, orc.AXIS_STACKED

CASES = [
    ((24, 40), (O, C)),          # activations [seq, in]: bind seq, keep the contraction axis
    ((40, 24), (C, O)),          # weights [in, out]: bind the innermost axis (warp-per-output path)
    ((3, 8, 5), (S, O, C)),      # per-head tensor: stacked heads, bound rows
    ((3, 5, 8), (S, C, O)),      # stacked heads, bound innermost axis
    ((6, 4, 7), (O, C, O)),      # two bound axes around a kept one (strided contraction)
    ((5, 9), (C, C)),            # nothing bound: widening and padding only (45 -> 64)
    ((2, 3, 4, 5), (S, O, S, C)),
    ((16,), (O,)),               # everything bound: a single constant
]


def points_for(F, rng, shape, kinds):
    return [[F.random_scalar(rng) for _ in range(max(s - 1, 0).bit_length())] if k == O else None
            for s, k in zip(shape, kinds)]


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("shape,kinds", CASES)
def test_fix_axes_matches_oracle(dpb, ctx, F, shape, kinds):
    rng = np.random.default_rng(hash((shape, kinds)) % 2**32)
    t = rng.integers(-2048, 2048, size=shape, dtype=np.int64)
    pts = points_for(F, rng, shape, kinds)
    want = orc.mles_from_tensor(F, t, kinds, pts)
    owner, views = ctx.einsum_fix_axes(family_dtype(dpb, F), t, kinds,
                                       [orc.scalars_to_array(F, p) if p is not None else None for p in pts])
    assert len(views) == len(want)
    for v, w in zip(views, want):
        assert v.len == w.shape[0]
        assert (v.to_host().reshape(w.shape) == w).all()
        v.free()
    owner.free()
    # the same from a tensor that is already on the device
    owner, views = ctx.einsum_fix_axes(family_dtype(dpb, F), None, kinds,
                                       [orc.scalars_to_array(F, p) if p is not None else None for p in pts],
                                       device_tensor=ctx.upload_tensor_i64(t))
    for v, w in zip(views, want):
        assert (v.to_host().reshape(w.shape) == w).all()
        v.free()
    owner.free()


@pytest.mark.parametrize("F", FIELDS)
def test_fix_axes_full_range_entries(dpb, ctx, F):
    """Entries over the whole int64 range (both 32-bit halves of the magnitude in use, both signs, the extremes):
    the contraction adds integer * weight products up unreduced, so the wide cases must be exact too."""
    rng = np.random.default_rng(4242)
    shape, kinds = (37, 20), (O, C)
    t = rng.integers(-2**63, 2**63 - 1, size=shape, dtype=np.int64)
    t[0, 0], t[1, 0], t[2, 0], t[3, 0] = -2**63, 2**63 - 1, 0, -1
    pts = points_for(F, rng, shape, kinds)
    want = orc.mles_from_tensor(F, t, kinds, pts)
    for k2, t2 in ((kinds, t), ((C, O), np.ascontiguousarray(t.T))):
        pts2 = pts if k2 == kinds else pts[::-1]
        want = orc.mles_from_tensor(F, t2, k2, pts2)
        owner, views = ctx.einsum_fix_axes(family_dtype(dpb, F), t2, k2,
                                           [orc.scalars_to_array(F, p) if p is not None else None for p in pts2])
        for v, w in zip(views, want):
            assert (v.to_host().reshape(w.shape) == w).all()
            v.free()
        owner.free()


@pytest.mark.parametrize("F", FIELDS)
def test_dense_layer_sumcheck(dpb, ctx, F):
    """y = x W with x [seq, in], W [in, out]: the claim y~(r_seq, r_out) equals
    sum_c x~(r_seq, c) W~(c, r_out); fix the outer axes, run the sumcheck over
    the contraction axis, compare with the oracle and check the claim."""
    rng = np.random.default_rng(77)
    seq, d_in, d_out = 12, 48, 20
    x = rng.integers(-128, 128, size=(seq, d_in), dtype=np.int64)
    w = rng.integers(-128, 128, size=(d_in, d_out), dtype=np.int64)
    y = x @ w
    r_seq = [F.random_scalar(rng) for _ in range(4)]
    r_out = [F.random_scalar(rng) for _ in range(5)]
    S_ = lambda p: orc.scalars_to_array(F, p)
    fam = family_dtype(dpb, F)
    lo, lv = ctx.einsum_fix_axes(fam, x, (O, C), [S_(r_seq), None])
    ro, rv = ctx.einsum_fix_axes(fam, w, (C, O), [None, S_(r_out)])
    o_l = orc.mles_from_tensor(F, x, (O, C), [r_seq, None])[0]
    o_r = orc.mles_from_tensor(F, w, (C, O), [None, r_out])[0]
    n = 6  # 48 -> 64 entries
    terms = {(0, 1): F.one}
    want = orc.sumcheck_prove(F, n, [o_l, o_r], terms, orc.Transcript(F))
    got = gpu_sumcheck_prove(dpb, ctx, F, n, [lv[0], rv[0]], terms, orc.Transcript(F))
    assert got == want
    # the claimed sum is the MLE of y (padded) at (r_out, r_seq): columns are the low variables
    ypad = np.zeros((16, 32), dtype=np.int64)
    ypad[:seq, :d_out] = y
    claim = orc.evaluate(F, F.table_from_i64(ypad.reshape(-1)), r_out + r_seq)
    assert orc.extract_sum(F, got[0]) == claim


def test_fix_axes_errors(dpb, ctx):
    F = orc.FrField
    t = np.ones((4, 6), dtype=np.int64)
    short = orc.scalars_to_array(F, [F.one, F.one])  # 2 variables cannot cover 6 entries
    with pytest.raises(dpb.DpbError) as e:
        ctx.einsum_fix_axes(dpb.FR, t, (C, O), [None, short])
    assert e.value.code == dpb.EINVAL
    with pytest.raises(dpb.DpbError) as e:
        ctx.einsum_fix_axes(dpb.FR, t, (C, 7), [None, None])
    assert e.value.code == dpb.EINVAL


@pytest.mark.parametrize("F", FIELDS)
def test_einsum_prove_matches_oracle(dpb, ctx, F):
    """dpb_einsum_prove (axis fixing, stacking coefficients, batching challenge, sumcheck, input claims and, with two
    outputs, the merging sumcheck over the padded left tensor) byte for byte against the restated
    EinSum::prove_internal, with host and device tensors; the transcripts end in the same state."""
    import importlib
    from tests.test_oracle_pins import _padded_mle, einsum_cases
    prover = importlib.import_module("deep_prove_b200.prover")
    fam = family_dtype(dpb, F)
    rng = np.random.default_rng(33)

    def arr(p):
        return None if p is None else np.ascontiguousarray(orc.scalars_to_array(F, p), dtype=np.uint64).reshape(len(p), -1)
    for name, lhs, fixes, rhs, _, _ in einsum_cases(F, rng):
        for on_device in (False, True):
            To = orc.Transcript(F)
            want = orc.serialize_einsum_proof(F, orc.einsum_prove(F, To, lhs, fixes, rhs, lhs_padded=_padded_mle(F, lhs)))
            Tg = prover.Blake3Transcript(fam)
            dev = (lambda t: ctx.upload_tensor_i64(np.ascontiguousarray(t, dtype=np.int64))) if on_device else (lambda t: None)
            lops = [prover.EinsumOperand(lhs, k, [arr(p) for p in pts], device_tensor=dev(lhs)) for k, pts in fixes]
            rops = [prover.EinsumOperand(t, k, [arr(p) for p in pts], device_tensor=dev(t)) for t, k, pts in rhs]
            padded = ctx.upload(np.asarray(_padded_mle(F, lhs)), fam if F is orc.FrField else dpb.GL_BASE) \
                if len(rhs) > 1 else None
            got = prover.einsum_prove(ctx, lops, rops, Tg, lhs_padded=padded)
            assert got == want, (name, on_device)
            assert Tg.state() == (To.state, To.round), name
    # an outer axis of more than one entry needs its point; the stacked axes must span the same number of tables
    x = np.ones((2, 2), dtype=np.int64)
    with pytest.raises(dpb.DpbError):
        prover.einsum_prove(ctx, [prover.EinsumOperand(x, (O, C), [None, None])],
                            [prover.EinsumOperand(x, (C, C), [None, None])], prover.Blake3Transcript(fam))
    one = arr([F.random_scalar(rng)])
    with pytest.raises(dpb.DpbError):
        prover.einsum_prove(ctx, [prover.EinsumOperand(x, (S, C), [one, None])],
                            [prover.EinsumOperand(x, (C, C), [None, None])], prover.Blake3Transcript(fam))
    with pytest.raises(ValueError):
        op = prover.EinsumOperand(x, (C, C), [None, None])
        prover.einsum_prove(ctx, [op], [op, op], prover.Blake3Transcript(fam))


@pytest.mark.parametrize("F", FIELDS)
def test_einsum_golden(dpb, ctx, F):
    """dpb_einsum_prove against the committed fixture (stacked heads; two outputs with the merging sumcheck)."""
    import importlib
    import json
    import os
    from tests.golden import make_golden
    prover = importlib.import_module("deep_prove_b200.prover")
    with open(os.path.join(os.path.dirname(__file__), "golden", f"oracle_{F.name}.json")) as f:
        want = json.load(f)["einsum"]
    fam = family_dtype(dpb, F)

    def arr(p):
        return None if p is None else np.ascontiguousarray(orc.scalars_to_array(F, p), dtype=np.uint64).reshape(len(p), -1)
    for g, w in zip(make_golden.golden_inputs(F, "einsum"), want):
        lops = [prover.EinsumOperand(g["lhs"], k, [arr(p) for p in pts]) for k, pts in g["fixes"]]
        rops = [prover.EinsumOperand(t, k, [arr(p) for p in pts]) for t, k, pts in g["rhs"]]
        dims = [1 << max(d - 1, 0).bit_length() for d in g["lhs"].shape]
        padded = np.zeros(dims, dtype=np.int64)
        padded[tuple(slice(0, d) for d in g["lhs"].shape)] = g["lhs"]
        pm = ctx.upload_ints(padded.reshape(-1), dpb.FR_I64 if F is orc.FrField else dpb.GL_I64)
        got = prover.einsum_prove(ctx, lops, rops, prover.Blake3Transcript(fam), lhs_padded=pm)
        assert got.hex() == w
