"""Device memory management of a context: tables are cut out of arenas the library keeps (device_alloc /
device_free in csrc/api_core.cu).  Live tables must keep their contents whatever is freed, allocated or trimmed around
them."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_tables_survive_churn_and_trim(dpb):
    ctx = dpb.Context(0)
    try:
        rng = np.random.default_rng(123)
        live = {}

        def add(i):
            n = 1 << int(rng.choice([0, 3, 7, 10, 14, 17, 20, 21, 23]))
            a = rng.integers(0, 2**63, size=n, dtype=np.uint64) % np.uint64(0xFFFFFFFF00000001)
            live[i] = (ctx.upload(a, dpb.GL_BASE), a)

        def check_all():
            for m, a in live.values():
                assert np.array_equal(m.to_host().reshape(-1), a)

        for i in range(96):
            add(i)
        check_all()
        for i in rng.choice(96, size=48, replace=False):
            live.pop(int(i))[0].free()
        for i in range(96, 160):
            add(i)
        check_all()
        ctx.trim()  # unused arenas go back; live tables stay where they are
        check_all()
        # a block of its own (2 GiB and more), freed and asked for again
        big = ctx.upload(np.zeros(1 << 28, dtype=np.uint64), dpb.GL_BASE)
        big.free()
        big = ctx.upload(np.ones(1 << 28, dtype=np.uint64), dpb.GL_BASE)
        assert int(big.to_host()[-1]) == 1
        big.free()
        check_all()
        for m, _ in live.values():
            m.free()
    finally:
        ctx.close()
