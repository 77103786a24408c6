"""The allocation-free entry point, dpb_product_round_noalloc.

It serves callers that cannot allocate device memory at the moment they call
(inside a region an outer runtime is recording, under a memory manager that
owns the whole device, or with a fixed device-memory budget).  It must return
exactly what the ordinary path returns for the first round of a product
sumcheck: exact field arithmetic, so the comparison is bit for bit.  The scratch
array it uses is shared by all calls and keeps the previous call's contents,
hence two calls in a row (different inputs) are checked.

This file sorts last on purpose: a run that stops at the first failure has
then already run every other test.
"""
import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import terms_array, upload

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("F", [orc.GlField, orc.FrField])
@pytest.mark.parametrize("k,n", [(3, 15), (2, 9), (4, 12)])
def test_no_alloc_round_matches_ordinary_path(dpb, ctx, F, k, n):
    rng = np.random.default_rng(700 + k + n)
    fam = dpb.FR if F is orc.FrField else dpb.GL_EXT
    out = ctx.alloc(fam, 8)  # caller-owned output buffer (k+1 <= 5 elements used)
    for call in range(2):
        tabs = [F.random_table_fast(rng, 1 << n) for _ in range(k)]
        mles = [upload(dpb, ctx, F, t) for t in tabs]
        sc = ctx.sumcheck(n, mles, terms_array(dpb, F, {tuple(range(k)): F.one}))
        want = sc.round(None)
        sc.free()
        dpb.product_round_noalloc(ctx.stream, mles[0].dtype, [m.device_ptr for m in mles], 1 << n, out.device_ptr)
        ctx.sync()
        got = out.to_host()[: k + 1]
        assert (got == want).all(), f"call {call}"
        # and both agree with the CPU oracle
        assert orc.array_to_scalars(F, got) == orc.sumcheck_round(F, n, tabs, {tuple(range(k)): F.one}, k)
        for m in mles:
            m.free()
    out.free()


def test_no_alloc_rejects_oversize_and_bad_arguments(dpb, ctx):
    F = orc.GlField
    rng = np.random.default_rng(1)
    m = [upload(dpb, ctx, F, F.random_table(rng, 16)) for _ in range(2)]
    out = ctx.alloc(dpb.GL_EXT, 4)
    ptrs = [x.device_ptr for x in m]
    with pytest.raises(dpb.DpbError, match="exceed this entry point's maximum"):
        dpb.product_round_noalloc(ctx.stream, dpb.GL_BASE, ptrs, 1 << 31, out.device_ptr)
    with pytest.raises(dpb.DpbError, match="table count"):
        dpb.product_round_noalloc(ctx.stream, dpb.GL_BASE, ptrs[:1], 16, out.device_ptr)
    with pytest.raises(dpb.DpbError, match="power of two"):
        dpb.product_round_noalloc(ctx.stream, dpb.GL_BASE, ptrs, 12, out.device_ptr)
    with pytest.raises(dpb.DpbError, match="aligned"):
        dpb.product_round_noalloc(ctx.stream, dpb.GL_BASE, [ptrs[0] + 8, ptrs[1]], 8, out.device_ptr)
