"""The last rounds of a sumcheck run in one resident kernel that trades round
sums for challenges with the host through mapped memory.  These tests pin
that path against the one-launch-per-round path and the oracle, and check the
ways out of the kernel that are not the normal one: a sumcheck that is dropped
half way, two sumchecks advanced in turns on one context, a host that is held
up past the kernel's bounded wait (the kernel returns and is started again), and
launches that block the host (the kernel leaves at once and rounds become
launches)."""
import time

import numpy as np
import pytest

from oracle import oracle as orc
from tests.helpers import gpu_sumcheck_prove, terms_array, upload

pytestmark = pytest.mark.gpu

FIELDS = [orc.FrField, orc.GlField]


def mixed_case(F, rng, n):
    sizes = [n, n, n - 1, max(n - 2, 1), n, 1]
    tabs = [F.random_table_fast(rng, 1 << s) for s in sizes]
    c = [F.random_scalar(rng) for _ in range(3)]
    terms = {(0, 1): c[0], (0, 2, 3): c[1], (4, 4, 1, 3, 5): c[2], (1, 4): F.one}
    return tabs, terms


@pytest.mark.parametrize("F", FIELDS)
@pytest.mark.parametrize("n", [1, 2, 5, 9, 12])
def test_resident_equals_launches_and_oracle(dpb, ctx, F, n):
    rng = np.random.default_rng(7000 + n)
    for tabs, terms in (mixed_case(F, rng, n) if n >= 3 else ([F.random_table_fast(rng, 1 << n)] * 2, {(0, 1): F.one}),
                        ([F.random_table_fast(rng, 1 << n) for _ in range(3)], {(0, 1, 2): F.one})):
        want = orc.sumcheck_prove(F, n, tabs, terms, orc.Transcript(F))
        mles = [upload(dpb, ctx, F, t) for t in tabs]
        try:
            ctx.resident_rounds(True)
            resident = gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F))
            ctx.resident_rounds(False)
            launches = gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F))
        finally:
            ctx.resident_rounds(True)
            for m in mles:
                m.free()
        assert resident == want
        assert launches == want


@pytest.mark.parametrize("F", FIELDS)
def test_dropped_sumcheck_releases_the_kernel(dpb, ctx, F):
    """Free after two rounds: the kernel is told to leave, and the next sumcheck gets it again."""
    rng = np.random.default_rng(7100)
    n = 6
    tabs, terms = mixed_case(F, rng, n)
    mles = [upload(dpb, ctx, F, t) for t in tabs]
    sc = ctx.sumcheck(n, mles, terms_array(dpb, F, terms))
    r = orc.scalars_to_array(F, [F.random_scalar(rng)])
    sc.round(None)
    sc.round(r)
    t0 = time.perf_counter()
    sc.free()
    assert time.perf_counter() - t0 < 1.0  # an abort, not the kernel's time-out
    want = orc.sumcheck_prove(F, n, tabs, terms, orc.Transcript(F))
    assert gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F)) == want


@pytest.mark.parametrize("F", FIELDS)
def test_two_sumchecks_in_turns(dpb, ctx, F):
    """Only one sumcheck of a context holds the resident kernel; the other one runs launches.  Neither waits on
    the other."""
    rng = np.random.default_rng(7200)
    n = 7
    cases = [mixed_case(F, rng, n), ([F.random_table_fast(rng, 1 << n) for _ in range(3)], {(0, 1, 2): F.one})]
    want = [orc.sumcheck_prove(F, n, tabs, terms, orc.Transcript(F)) for tabs, terms in cases]
    mles = [[upload(dpb, ctx, F, t) for t in tabs] for tabs, _ in cases]
    scs = [ctx.sumcheck(n, m, terms_array(dpb, F, terms)) for m, (_, terms) in zip(mles, cases)]
    trs = [orc.Transcript(F), orc.Transcript(F)]
    for q in range(2):
        trs[q].append_scalars([F.from_int(n), F.from_int(scs[q].degree)])
    proofs, points, r_arr = [[], []], [[], []], [None, None]
    for _ in range(n):
        for q in range(2):
            ev = orc.array_to_scalars(F, scs[q].round(r_arr[q]))
            trs[q].append_scalars(ev)
            r = trs[q].append_and_sample(orc.ROUND_LABEL)
            proofs[q].append(ev)
            points[q].append(r)
            r_arr[q] = orc.scalars_to_array(F, [r])
    for q in range(2):
        finals = orc.array_to_scalars(F, scs[q].finish(r_arr[q]))
        scs[q].free()
        assert (proofs[q], points[q], finals) == want[q]


@pytest.mark.parametrize("F", FIELDS)
def test_host_that_is_held_up(dpb, ctx, F):
    """The kernel's wait for a challenge is bounded: when the host takes longer (here: sleeps past a 200 ms limit,
    twice, and once more before the last challenge) the kernel returns, the next call starts it again where it
    stopped, and the proof is the same."""
    rng = np.random.default_rng(7300)
    n = 6
    tabs, terms = mixed_case(F, rng, n)
    want = orc.sumcheck_prove(F, n, tabs, terms, orc.Transcript(F))
    mles = [upload(dpb, ctx, F, t) for t in tabs]
    ctx.resident_rounds(True, wait_ms=200)
    try:
        sc = ctx.sumcheck(n, mles, terms_array(dpb, F, terms))
        tr = orc.Transcript(F)
        tr.append_scalars([F.from_int(n), F.from_int(sc.degree)])
        proof, point, r_arr = [], [], None
        for i in range(n):
            if i in (1, 4):
                time.sleep(0.5)  # well past the 200 ms the kernel waits
            ev = orc.array_to_scalars(F, sc.round(r_arr))
            tr.append_scalars(ev)
            r = tr.append_and_sample(orc.ROUND_LABEL)
            proof.append(ev)
            point.append(r)
            r_arr = orc.scalars_to_array(F, [r])
        time.sleep(0.5)
        finals = orc.array_to_scalars(F, sc.finish(r_arr))
        sc.free()
    finally:
        ctx.resident_rounds(True, wait_ms=1000)
    assert (proof, point, finals) == want


@pytest.mark.parametrize("detect_at_init", [True, False])
def test_blocking_launches_fall_back_to_one_launch_per_round(detect_at_init):
    """With launches that block the host (CUDA_LAUNCH_BLOCKING=1; a profiler that serialises kernels behaves the
    same) the resident kernel cannot talk to the host.  The context sees the setting when it is created and never
    starts the kernel; with that check switched off (DPB_ASSUME_ASYNC_LAUNCHES=1) the kernel itself notices
    within 50 ms, leaves, and the context runs one launch per round from then on.  Results are unchanged and
    nothing waits for a time-out."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = r"""
import sys, time
sys.path.insert(0, {root!r}); sys.path.insert(0, {root!r} + '/tests')
import numpy as np
from conftest import load_package
from oracle import oracle as orc
from tests.helpers import gpu_sumcheck_prove, upload
dpb = load_package()
ctx = dpb.Context(0)
F = orc.GlField
rng = np.random.default_rng(7400)
n = 7
tabs = [F.random_table_fast(rng, 1 << n) for _ in range(3)]
terms = {{(0, 1, 2): F.one}}
want = orc.sumcheck_prove(F, n, tabs, terms, orc.Transcript(F))
mles = [upload(dpb, ctx, F, t) for t in tabs]
t0 = time.perf_counter()
for _ in range(3):
    assert gpu_sumcheck_prove(dpb, ctx, F, n, mles, terms, orc.Transcript(F)) == want
assert time.perf_counter() - t0 < 3.0
print('FALLBACK-OK')
""".format(root=root)
    env = dict(os.environ, CUDA_LAUNCH_BLOCKING="1")
    if not detect_at_init:
        env["DPB_ASSUME_ASYNC_LAUNCHES"] = "1"
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=300)
    assert "FALLBACK-OK" in out.stdout, out.stdout + out.stderr
