"""Sumchecks whose term lists are long (many logup instances in one batch, many tables): small rounds are spread
over the terms (sliced two-pass evaluation) instead of one thread walking the whole list per pair, the resident
kernel is not used, and a sumcheck may pass from split-eq rounds to those rounds half way.  All against the oracle."""
import importlib

import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import family_dtype, gpu_sumcheck_prove, upload

pytestmark = pytest.mark.gpu

FIELDS = [orc.FrField, orc.GlField]


@pytest.fixture(scope="module")
def prover(dpb):
    return importlib.import_module("deep_prove_b200.prover")


def random_terms(F, rng, k, n_terms, max_degree):
    terms = {}
    while len(terms) < n_terms:
        deg = int(rng.integers(1, max_degree + 1))
        m = tuple(sorted(int(x) for x in rng.integers(0, k, size=deg)))
        terms[m] = F.random_scalar(rng) if rng.integers(0, 4) else F.one
    return terms


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("k,n_terms,n", [(40, 60, 9), (150, 120, 7), (24, 200, 13)])
def test_long_term_lists(dpb, ctx, F, k, n_terms, n):
    rng = np.random.default_rng(8800 + k)
    sizes = [n if j % 3 else max(n - 2, 1) for j in range(k)]
    tabs = [F.random_table_fast(rng, 1 << s) for s in sizes]
    terms = random_terms(F, rng, k, n_terms, 3)
    want = orc.sumcheck_prove(F, n, tabs, terms, orc.Transcript(F))
    mles = [upload(dpb, ctx, F, t) for t in tabs]
    try:
        assert gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F)) == want
    finally:
        for m in mles:
            m.free()


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("n_inst,m", [(16, 7), (40, 6), (12, 14), (12, 16)])
def test_logup_batches_of_many_instances(dpb, ctx, prover, F, n_inst, m):
    """(12, 16): the top layers start with split-eq rounds (8192 pairs and more) and pass to the spread rounds, the
    eq tables being materialised on the way; (12, 14): spread from the first round; (40, 6): more tables than the
    one-pass rounds take."""
    rng = np.random.default_rng(8900 + n_inst)
    cols = [F.table_from_i64(rng.integers(0, 1 << 12, size=1 << m, dtype=np.int64)) for _ in range(2 * n_inst)]
    cst, sep = F.random_scalar(rng), F.random_scalar(rng)
    o_in = orc.LogUpInput(F, 0, cols, cst, sep, columns_per_instance=2)
    want = orc.serialize_logup_proof(F, orc.logup_batch_prove(F, [o_in], orc.Transcript(F)))
    S = lambda v: orc.scalars_to_array(F, [v])
    d_cols = [upload(dpb, ctx, F, c) for c in cols]
    d_in = prover.LogUpInput.new_lookup(d_cols, S(cst), S(sep), 2)
    tr = prover.Blake3Transcript(family_dtype(dpb, F))
    assert prover.new_batch_multiple_sizes_prove(ctx, [d_in], tr) == want
    tr.free()
    for c in d_cols:
        c.free()
