"""Large one-pass rounds over a program cut into segments (sc_round_seg): sumchecks whose term list falls apart
into independent parts over few tables each, at sizes where a round has more than 16384 pairs.  Everything is
compared bit for bit with the oracle, and with the unsegmented kernels of the same library (DPB_NO_SEGMENTS=1 is
read when a sumcheck begins)."""
import importlib
import os

import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import family_dtype, gpu_sumcheck_prove, upload

pytestmark = pytest.mark.gpu
FIELDS = [orc.FrField, orc.GlField]


@pytest.fixture(scope="module")
def prover(dpb):
    return importlib.import_module("deep_prove_b200.prover")


@pytest.mark.parametrize("F", FIELDS)
def test_independent_products_and_an_unused_table(dpb, ctx, F):
    """sum_i c_i a_i b_i + c a_0 over 2^16 entries, six pairs of tables plus one table no term uses (it is still
    bound every round: its final evaluation is checked), degree 2, not led by an eq table."""
    rng = np.random.default_rng(71)
    n, pairs = 16, 6
    tabs = [F.random_table_fast(rng, 1 << n) if F is orc.FrField else F.random_table(rng, 1 << n)
            for _ in range(2 * pairs + 1)]
    terms = {(2 * i, 2 * i + 1): F.random_scalar(rng) for i in range(pairs)}
    terms[(0,)] = F.random_scalar(rng)
    want = orc.sumcheck_prove(F, n, tabs, terms, orc.Transcript(F))
    mles = [upload(dpb, ctx, F, t) for t in tabs]
    got = gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F))
    assert got == want
    os.environ["DPB_NO_SEGMENTS"] = "1"
    try:
        assert gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F)) == want
    finally:
        del os.environ["DPB_NO_SEGMENTS"]


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("cpi", [1, 2])
def test_logup_batch_of_large_instances(dpb, ctx, prover, F, cpi):
    """Three lookup instances of 2^17 rows: the top layers' rounds run segmented and in split-eq form (one segment
    per instance, the integer leaf layer included); proof bytes equal the oracle's."""
    rng = np.random.default_rng(72 + cpi)
    rows, inst = 1 << 17, 3
    base = dpb.FR if F is orc.FrField else dpb.GL_BASE
    cols = [rng.integers(-(1 << 15), 1 << 15, size=rows, dtype=np.int64) for _ in range(inst * cpi)]
    cst, sep = F.random_scalar(rng), F.random_scalar(rng)
    S = lambda v: orc.scalars_to_array(F, [v])
    o_in = orc.LogUpInput(F, 0, [F.table_from_i64(c) for c in cols], cst, sep, columns_per_instance=cpi)
    want = orc.serialize_logup_proof(F, orc.logup_batch_prove(F, [o_in], orc.Transcript(F)))
    fam = family_dtype(dpb, F)
    for ints in (False, True):
        dev = [ctx.upload_ints(c, dpb.FR_I64 if F is orc.FrField else dpb.GL_I64) if ints else ctx.upload_i64(c, base)
               for c in cols]
        d_in = prover.LogUpInput.new_lookup(dev, S(cst), S(sep), cpi)
        assert prover.new_batch_multiple_sizes_prove(ctx, [d_in], prover.Blake3Transcript(fam)) == want, ints


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("ncols", [1, 2])
def test_table_instance_with_multiplicities(dpb, ctx, prover, F, ncols):
    """A table of 2^17 rows with one or two columns and its multiplicities (the numerators are tables too)."""
    rng = np.random.default_rng(75 + ncols)
    rows = 1 << 17
    base = dpb.FR if F is orc.FrField else dpb.GL_BASE
    t_in = np.arange(rows, dtype=np.int64) - rows // 2
    cols = [t_in, np.maximum(t_in, 0)][:ncols]
    mult = rng.integers(0, 50, size=rows, dtype=np.int64)
    cst, sep = F.random_scalar(rng), F.random_scalar(rng)
    S = lambda v: orc.scalars_to_array(F, [v])
    T = F.table_from_i64
    o_t = orc.LogUpInput(F, 1, [T(c) for c in cols], cst, sep, mult=T(mult))
    want = orc.serialize_logup_proof(F, orc.logup_batch_prove(F, [o_t], orc.Transcript(F)))
    d_t = prover.LogUpInput.new_table([ctx.upload_i64(c, base) for c in cols], ctx.upload_i64(mult, base), S(cst), S(sep))
    assert prover.new_batch_multiple_sizes_prove(ctx, [d_t], prover.Blake3Transcript(family_dtype(dpb, F))) == want


@pytest.mark.parametrize("F", FIELDS)
def test_many_instances_and_three_columns(dpb, ctx, prover, F):
    """70 single-column instances of 2^16 rows (more than 64: still the layer kernel) and one three-column instance
    (more columns than the layer kernel takes: the segmented kernel), each batch against the oracle."""
    rng = np.random.default_rng(79)
    rows = 1 << 16
    base = dpb.FR if F is orc.FrField else dpb.GL_BASE
    S = lambda v: orc.scalars_to_array(F, [v])
    fam = family_dtype(dpb, F)
    for n_cols, cpi in ((70, 1), (3, 3)):
        cols = [rng.integers(0, 1 << 12, size=rows, dtype=np.int64) for _ in range(n_cols)]
        cst, sep = F.random_scalar(rng), F.random_scalar(rng)
        o_in = orc.LogUpInput(F, 0, [F.table_from_i64(c) for c in cols], cst, sep, columns_per_instance=cpi)
        want = orc.serialize_logup_proof(F, orc.logup_batch_prove(F, [o_in], orc.Transcript(F)))
        d_in = prover.LogUpInput.new_lookup([ctx.upload_i64(c, base) for c in cols], S(cst), S(sep), cpi)
        assert prover.new_batch_multiple_sizes_prove(ctx, [d_in], prover.Blake3Transcript(fam)) == want, (n_cols, cpi)
