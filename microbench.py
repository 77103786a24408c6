"""Times the other pieces of the path on one GPU (the sumcheck itself is
bench.py's job): eq tables, fix_high / fix_low, the logup fraction tree, the
batched logup-GKR prover, einsum axis fixing and the generic (term-list)
sumcheck.  Prints one line per measurement with the algorithmic bytes it is
divided by, so each figure can be read against the HBM peak.

    python microbench.py [--field fr|gl] [--log2 22] [--reps 5]
    python microbench.py --lookup [--field ..] [--log2 ..]   only the lookup witness lines
    python microbench.py --mlp          one dense + ReLU layer of the MLP configuration, per step
    python microbench.py --issue-rate   field products per second the integer pipes deliver (dpb_issue_rate_probe)
    python microbench.py --msm          commit throughput (BN254 G1 multi-scalar multiplication)
    python microbench.py --latency      small sumchecks, one C call per proof, both fields,
                                                        with the resident last-rounds kernel and with one launch per round
"""
import argparse
import importlib
import importlib.util
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def load():
    name = "deep_prove_b200"
    if name not in sys.modules:
        pkg = os.path.join(HERE, "deep-prove_b200")
        spec = importlib.util.spec_from_file_location(name, os.path.join(pkg, "__init__.py"),
                                                      submodule_search_locations=[pkg])
        mod = importlib.util.module_from_spec(spec)
        sys.modules[name] = mod
        spec.loader.exec_module(mod)
    return sys.modules[name], importlib.import_module(name + ".prover")


def timed(ctx, fn, reps):
    fn()
    ctx.sync()
    best = 1e30
    for _ in range(reps):
        t0 = time.perf_counter()
        r = fn()
        ctx.sync()
        best = min(best, time.perf_counter() - t0)
        del r
    return best


def issue_rate(dpb, ctx):
    """The probes of csrc/issue_rate.cu: chains of the round kernels' own product routines on register operands.
    Cycles are per warp instruction stream per SM sub-partition at the SM clock read from nvidia-smi."""
    import subprocess
    try:
        mhz = float(subprocess.run(["nvidia-smi", "-i", "0", "--query-gpu=clocks.max.sm", "--format=csv,noheader,nounits"],
                                   capture_output=True, text=True).stdout.split()[0])
    except (OSError, IndexError, ValueError):
        mhz = 1965.0
    sms = 148
    names = ["32x32->64 multiply-add (64-bit addend, carry)", "BN254 Montgomery product (frw::mul)",
             "BN254 product by a per-launch constant (frw::mul_fixed)", "Goldilocks lazy multiply-accumulate (glw::acc_mac)",
             "Goldilocks product with reduction (glw::mul)"]
    print(f"# issue-rate probes, {sms} SMs x 4 sub-partitions, cycles at the maximum SM clock {mhz:.0f} MHz")
    print("# (a lower bound on cycles when the clock under load is lower; each probe: 4 blocks of 256 threads per SM)")
    for kind, name in enumerate(names):
        best = 0.0
        for _ in range(3):
            ops, ms = ctx.issue_rate(kind, 8192)
            best = max(best, ops)
        cyc = sms * 4 * mhz * 1e6 / (best / 32)
        print(f"{name:58s} {best / 1e9:10.2f} G/s   {cyc:8.1f} cycles per warp-wide operation per sub-partition")


def msm_bench(dpb, ctx):
    """Commit throughput: one MSM over 2^n G1 points, full-width field scalars and 32-bit integer tables."""
    import importlib
    pcs = importlib.import_module("deep_prove_b200.pcs")
    rng = np.random.default_rng(3)
    print("# dpb_msm_g1: one commitment over 2^n points (mean of 5 after a warm-up), milliseconds and M points/s")
    for n in (16, 18, 20):
        N = 1 << n
        bases = pcs.G1Bases.synthetic(ctx, N, 1)  # the multiples 1 G .. N G of the generator, made on the device
        t = rng.integers(0, 2**64, size=(N, 4), dtype=np.uint64)
        t[:, 3] &= np.uint64((1 << 60) - 1)
        tabs = {"field scalars (254 bits)": ctx.upload(t, dpb.FR),
                "int32 table (quantised tensor)": ctx.upload_ints(rng.integers(-2**31, 2**31, size=N, dtype=np.int64), dpb.FR_I32),
                "int32 table of 16-bit values (lookup column)": ctx.upload_ints(rng.integers(0, 2**16, size=N, dtype=np.int64), dpb.FR_I32)}
        for name, m in tabs.items():
            pcs.msm(ctx, bases, m)
            ctx.sync()
            t0 = time.perf_counter()
            for _ in range(5):
                pcs.msm(ctx, bases, m)
            ctx.sync()
            dt = (time.perf_counter() - t0) / 5
            print(f"2^{n} {name:46s} {dt * 1e3:9.3f} ms  {N / dt / 1e6:9.1f} M points/s")
            m.free()
        bases.free()


def latency(dpb, prover, ctx):
    """Time per proof of f*g*h over 2^n entries through dpb_prove_sumcheck (transcript in the library's C++)."""
    import ctypes
    rng = np.random.default_rng(1)
    lib = dpb.lib
    print("# product sumcheck f*g*h, one C call per proof (mean of 50), microseconds")
    for field in ("gl", "fr"):
        fr = field == "fr"
        fam, base, w = (dpb.FR, dpb.FR, 4) if fr else (dpb.GL_EXT, dpb.GL_BASE, 2)
        for resident in (True, False):
            ctx.resident_rounds(resident)
            for n in (4, 8, 12, 16, 20):
                if fr:
                    tabs = rng.integers(0, 2**64, size=(3, 1 << n, 4), dtype=np.uint64)
                    tabs[:, :, 3] &= np.uint64((1 << 60) - 1)
                else:
                    tabs = rng.integers(0, 2**64 - 2**32 + 1, size=(3, 1 << n), dtype=np.uint64)
                mles = [ctx.upload(tabs[j], base) for j in range(3)]
                terms = dpb.make_terms([(dpb.one_bytes(fam), [0, 1, 2])], bytes)
                hs = (ctypes.c_void_p * 3)(*[m.h for m in mles])
                evals = np.zeros((n, 4, w), dtype=np.uint64)
                point = np.zeros((n, w), dtype=np.uint64)
                finals = np.zeros((3, w), dtype=np.uint64)
                deg = ctypes.c_uint32()
                tr = prover.Blake3Transcript(fam)
                eb, pb, fb = dpb._buf(evals), dpb._buf(point), dpb._buf(finals)

                def go():
                    return lib.dpb_prove_sumcheck(ctx.h, n, hs, 3, terms, len(terms), tr.h, eb, n * 4, pb, fb,
                                                  ctypes.byref(deg))
                for _ in range(5):
                    dpb.check(go())
                ctx.sync()
                t0 = time.perf_counter()
                for _ in range(50):
                    go()
                ctx.sync()
                dt = (time.perf_counter() - t0) / 50
                mode = "resident last rounds" if resident else "one launch per round"
                print(f"{field}  n={n:2d}  {mode:22s} {dt * 1e6:8.1f}")
                tr.free()
                for m in mles:
                    m.free()
    ctx.resident_rounds(True)


def lookup(dpb, prover, ctx, rng, args, fam, s0, s1, report):
    """Lookup witness generation: a GELU-like lookup over 2^n rescaled values on the device."""
    n, N = args.log2, 1 << args.log2
    # 12-bit two-column table, shift 16, 44-bit values: 1 + 1 + 1 input columns and 1 + 1 output columns per entry
    lk_bits, lk_shift, lk_max = 12, 16, 44
    ci = dpb.ChunkingInfo.new(lk_shift, lk_bits, dpb.SIGN_MIXED, lk_max)
    rows = 1 << (n // 2)
    # activations with a bell shape: about one rescaled value in a hundred falls outside the table's range
    tens = np.rint(rng.standard_normal((rows, N // rows)) * ((1 << 27) / 181 / 2.6)).astype(np.int64)
    dt = ctx.upload_tensor_i64(tens)
    tab_out = np.clip(np.arange(-(1 << (lk_bits - 1)), 1 << (lk_bits - 1), dtype=np.int64), 0, None)
    d_tab = ctx.upload_tensor_i64(tab_out)
    cnt = [dpb.LookupCounts(ctx, b) for b in (16, lk_bits, 16, 16)]
    n_cols = ci.n_shifted_chunks + 1 + ci.n_zeroing_chunks + 1 + ci.n_zeroing_chunks

    def witness(counts):
        owner, ins, outs = dpb.lookup_witness(ctx, fam, ci, 181, 0, None, tab_out, 2, counts, device_tensor=dt,
                                              device_table=d_tab)
        for h in ins + outs:
            h.free()
        return owner

    t = timed(ctx, lambda: witness(cnt).free(), args.reps)
    report(f"lookup witness 2^{n}, {n_cols} columns, counted", t, N * 8 + n_cols * N * s0)
    t = timed(ctx, lambda: witness((None,) * 4).free(), args.reps)
    report("  the same without the counters", t, N * 8 + n_cols * N * s0)
    t = timed(ctx, lambda: cnt[0].multiplicities(fam).free(), args.reps)
    report("  multiplicities of a 2^16-row table", t, (1 << 16) * (8 + s0))
    for h in cnt:
        h.free()

    # the linking sumcheck over that witness (one slice of 2^n entries): value output, zeroing output and the two
    # eq tables, degree 4; bytes = the sumcheck traffic of the four tables (eq tables counted as tables)
    owner, ins, outs = dpb.lookup_witness(ctx, fam, ci, 181, 0, None, tab_out, 2, device_tensor=dt, device_table=d_tab)
    w = 4 if fam == dpb.FR else 2
    claim_pt = rng.integers(0, 2**62, size=(n, w), dtype=np.uint64)
    logup_pt = rng.integers(0, 2**62, size=(n, w), dtype=np.uint64)

    def linking():
        tr = prover.Blake3Transcript(fam)
        out = prover.lookup_linking_prove(ctx, tr, prover.VARIANT_STANDARD, ci, 0, (1 << (lk_bits - 1)) - 1, tens.shape, outs,
                                          claim_pt, logup_pt)
        tr.free()
        return out

    t = timed(ctx, linking, max(1, args.reps // 2))
    report(f"lookup linking sumcheck 2^{n}, {len(outs)} + 2 tables", t, (len(outs) * (2 * s0 + 2 * s1) + 2 * 4 * s1) * N)
    for h in ins + outs:
        h.free()
    owner.free()


def mlp_layer(dpb, prover, ctx):
    """Time of every step of one dense + ReLU layer of the two-layer MLP configuration (input 1 x 1024 int8, weights
    1024 x 1024 int8, ReLU through a 12-bit lookup), tensors resident on the device, transcript in the library."""
    rng = np.random.default_rng(0)
    print("# dense + ReLU layer of the MLP configuration, per step (best of 20), microseconds")
    for field in ("fr", "gl"):
        fam, base, w = (dpb.FR, dpb.FR, 4) if field == "fr" else (dpb.GL_EXT, dpb.GL_BASE, 2)
        x = rng.integers(-128, 128, size=(1, 1024), dtype=np.int64)
        wt = rng.integers(-128, 128, size=(1024, 1024), dtype=np.int64)
        y = x @ wt + rng.integers(-(1 << 15), 1 << 15, size=1024, dtype=np.int64)
        pt = rng.integers(0, 2**62, size=(10, w), dtype=np.uint64)
        d_w, d_y = ctx.upload_tensor_i64(wt), ctx.upload_tensor_i64(y)
        x_tab = ctx.upload_i64(x.reshape(-1), base)
        K = (dpb.AXIS_CONTRACTED, dpb.AXIS_OUTER)
        steps = []

        def step(name, fn, keep=False):
            out = fn()
            ctx.sync()
            best = 1e30
            for _ in range(20):
                t0 = time.perf_counter()
                r = fn()
                ctx.sync()
                best = min(best, time.perf_counter() - t0)
                if not keep:
                    release(r)
            steps.append((name, best))
            return out

        def release(r):
            if isinstance(r, (list, tuple)):
                for q in r:
                    release(q)
            elif hasattr(r, "free"):
                r.free()

        def fix_axes():
            owner, views = ctx.einsum_fix_axes(fam, None, K, [None, pt], device_tensor=d_w)
            return [views, owner]

        (w_views, w_owner) = step("einsum fix_axes W[1024,1024]", fix_axes, keep=True)
        terms = dpb.make_terms([(dpb.one_bytes(fam), [0, 1])], bytes)

        def dense():
            tr = prover.Blake3Transcript(fam)
            st = prover.IOPProverState.prove(ctx, 10, [x_tab, w_views[0]], terms, tr)
            tr.free()
            return st

        step("dense sumcheck, 2^10", dense)
        ci = dpb.ChunkingInfo.new(13, 12, dpb.SIGN_MIXED, 28)
        relu_in = np.arange(-2048, 2048, dtype=np.int64)
        relu_out = np.clip(relu_in, 0, None)
        d_tab = ctx.upload_tensor_i64(relu_out)
        cnt = [dpb.LookupCounts(ctx, b) for b in (16, 12, 16, 16)]

        def witness():
            owner, ins, outs = dpb.lookup_witness(ctx, fam, ci, 1, 0, None, relu_out, 2, cnt, device_tensor=d_y,
                                                  device_table=d_tab)
            return [ins, outs, owner]

        ins, outs, wit_owner = step("lookup witness, 2^10 entries, 5 columns", witness, keep=True)
        mult = step("multiplicities, 3 tables", lambda: [cnt[0].multiplicities(fam), cnt[1].multiplicities(fam),
                                                         cnt[3].multiplicities(fam)], keep=True)
        up = lambda a: ctx.upload_i64(np.ascontiguousarray(a, dtype=np.int64), base)
        sz_in = np.arange(-(1 << 15), 1 << 15, dtype=np.int64)
        tabs = [up(np.arange(1 << 16)), up(sz_in), up(np.sign(sz_in)), up(relu_in), up(relu_out)]
        ch = rng.integers(0, 2**62, size=(6, w), dtype=np.uint64)
        t_inputs = [prover.LogUpInput.new_table([tabs[0]], mult[0], ch[0], ch[1]),
                    prover.LogUpInput.new_table([tabs[1], tabs[2]], mult[2], ch[4], ch[5]),
                    prover.LogUpInput.new_table([tabs[3], tabs[4]], mult[1], ch[2], ch[3])]
        l_inputs = [prover.LogUpInput.new_lookup([ins[0]], ch[0], ch[1], 1),
                    prover.LogUpInput.new_lookup([ins[1], outs[0]], ch[2], ch[3], 2),
                    prover.LogUpInput.new_lookup([ins[2], outs[1]], ch[4], ch[5], 2)]

        def logup(inputs):
            tr = prover.Blake3Transcript(fam)
            out = prover.new_batch_multiple_sizes_prove(ctx, inputs, tr)
            tr.free()
            return out

        step("logup-GKR, tables 2^16 + 2^16 + 2^12", lambda: logup(t_inputs))
        step("logup-GKR, 3 lookups of 2^10", lambda: logup(l_inputs))

        def linking():
            tr = prover.Blake3Transcript(fam)
            out = prover.lookup_linking_prove(ctx, tr, prover.VARIANT_STANDARD, ci, 0, 2047, (1, 1024), outs, pt, pt)
            tr.free()
            return out

        step("linking sumcheck, 2^10", linking)
        for name, t in steps:
            print(f"{field}  {name:44s} {t * 1e6:9.1f}")
        print(f"{field}  {'layer total':44s} {sum(t for _, t in steps) * 1e6:9.1f}")


def lookup_layer_logup(dpb, prover, ctx, field):
    """The logup-GKR call of one lookup layer at the GELU size of GPT-2 (512 x 3072 entries, 12-bit table: one
    shifted-chunk instance and two two-column instances of 2^21 rows): wall time, where the host's time goes
    (dpb_trace_*), and the round kernels by (kernel, round, size) with launches timed one by one (dpb_profile_*;
    the resident last-rounds kernel is off while profiling, so its rounds appear as launches)."""
    import importlib
    wl = importlib.import_module("deep_prove_b200.workloads")
    be = wl.GpuBackend(dpb, prover, ctx, field)
    rng = np.random.default_rng(0)
    T = be.new_transcript()
    bits = 12
    spec = wl.LookupSpec("gelu", bits, right_shift=bits + 1, max_bit_size=2 * bits + 4, sign=wl.SIGN_MIXED)
    chal = {k: tuple(be.squeeze(T, 2)) for k in ("shift", "gelu", "zero", "signed")}
    sign, table_out, n_cols = wl.value_table("gelu", bits)
    t = wl.draw_tensor(rng, (512, 3072), spec)
    wit = be.lookup_witness(be.tensor(t), t.shape, spec, table_out, n_cols, [None] * 4)
    ins, outs, n_sh, n_z = wit["ins"], wit["outs"], wit["n_shifted"], wit["n_zeroing"]
    groups = {"shift": ins[:n_sh], "gelu": [ins[n_sh], outs[0]], "zero": [], "signed": []}
    for z in range(n_z):
        groups["signed" if z == n_z - 1 else "zero"] += [ins[n_sh + 1 + z], outs[1 + z]]
    inputs = [("lookup", groups[k], cpi, None, chal[k][0], chal[k][1])
              for k, cpi in (("shift", 1), ("gelu", 2), ("zero", 2), ("signed", 2)) if groups[k]]
    print(f"# {field}: instances (columns, columns per instance): {[(len(i[1]), i[2]) for i in inputs]}")
    for _ in range(3):
        be.logup(T, inputs)
    ctx.sync()
    t0 = time.perf_counter()
    for _ in range(5):
        be.logup(T, inputs)
    ctx.sync()
    print(f"wall per call {(time.perf_counter() - t0) / 5 * 1e3:.3f} ms")
    dpb.trace(True)
    be.logup(T, inputs)
    ctx.sync()
    tr = dpb.trace_read()
    dpb.trace(False)
    for k, (ms, calls) in sorted(tr.items(), key=lambda kv: -kv[1][0]):
        print(f"   host phase {k:36s} {ms:8.3f} ms  {calls} calls")
    ctx.profile(True)
    be.logup(T, inputs)
    ctx.sync()
    ctx.profile(False)
    prof = ctx.profile_read()
    print(f"round kernels, one launch per round: {sum(e['total_ms'] for e in prof):.3f} ms in "
          f"{sum(e['launches'] for e in prof)} launches")
    for e in sorted(prof, key=lambda e: -e["total_ms"])[:16]:
        per = e["total_ms"] / e["launches"]
        print(f"   {e['kernel']:34s} round {e['round']:2d} x{e['launches']:2d} {e['total_ms']:8.3f} ms "
              f"{e['alg_bytes_per_launch'] / 1e6:9.2f} MB {e['alg_bytes_per_launch'] / 1e6 / max(per, 1e-9):8.1f} GB/s")
    small = [e for e in prof if e["alg_bytes_per_launch"] < 4e6]
    print(f"   launches under 4 MB: {sum(e['launches'] for e in small)} launches, {sum(e['total_ms'] for e in small):.3f} ms")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--field", default="fr", choices=["fr", "gl"])
    ap.add_argument("--log2", type=int, default=22)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--latency", action="store_true")
    ap.add_argument("--msm", action="store_true", help="commit (G1 multi-scalar multiplication) throughput")
    ap.add_argument("--issue-rate", action="store_true", help="the integer pipes' product rates (dpb_issue_rate_probe)")
    ap.add_argument("--lookup", action="store_true", help="only the lookup witness lines")
    ap.add_argument("--mlp", action="store_true", help="the steps of one dense + ReLU layer of the MLP configuration")
    ap.add_argument("--lookup-layer-logup", action="store_true",
                    help="the logup-GKR call of a GELU-sized lookup layer: wall, host phases, round kernels")
    args = ap.parse_args()
    dpb, prover = load()
    ctx = dpb.Context(0)
    if args.issue_rate:
        issue_rate(dpb, ctx)
        ctx.close()
        return
    if args.msm:
        msm_bench(dpb, ctx)
        ctx.close()
        return
    if args.latency:
        latency(dpb, prover, ctx)
        ctx.close()
        return
    if args.mlp:
        mlp_layer(dpb, prover, ctx)
        ctx.close()
        return
    if args.lookup_layer_logup:
        lookup_layer_logup(dpb, prover, ctx, args.field)
        ctx.close()
        return
    rng = np.random.default_rng(0)
    n, N = args.log2, 1 << args.log2
    fr = args.field == "fr"
    base, fam, w = (dpb.FR, dpb.FR, 4) if fr else (dpb.GL_BASE, dpb.GL_EXT, 2)
    s0, s1 = (32, 32) if fr else (8, 16)
    one = np.frombuffer(dpb.one_bytes(fam), dtype=np.uint64)

    def table(m):
        if fr:
            t = rng.integers(0, 2**64, size=(m, 4), dtype=np.uint64)
            t[:, 3] &= np.uint64((1 << 60) - 1)
            return t
        return rng.integers(0, 2**64 - 2**32 + 1, size=m, dtype=np.uint64)

    def chal(k):
        return table(k) if fr else np.stack([table(k), table(k)], axis=1)

    def report(name, seconds, nbytes):
        print(f"{name:44s} {seconds * 1e3:9.3f} ms  {nbytes / 1e9:8.3f} GB  {nbytes / seconds / 1e9:8.1f} GB/s")

    if args.lookup:
        lookup(dpb, prover, ctx, rng, args, fam, s0, s1, report)
        ctx.close()
        return
    print(f"# field={args.field} log2={n} (one B200, best of {args.reps}, wall clock around a stream sync)")
    pt = chal(n)
    t = timed(ctx, lambda: ctx.eq_table(fam, pt).free(), args.reps)
    report(f"eq_table 2^{n}", t, N * s1)

    m = ctx.upload(table(N), base)
    for k in (1, 10, n):
        t = timed(ctx, lambda: ctx.fix_low(m, pt[:k]).free(), args.reps)
        report(f"fix_low  k={k}", t, N * s0 + (N >> k) * s1)
        t = timed(ctx, lambda: ctx.fix_high(m, pt[:k]).free(), args.reps)
        report(f"fix_high k={k}", t, N * s0 + (N >> k) * s1)

    cols = [ctx.upload(table(N), base) for _ in range(2)]
    c, sep = chal(1)[0], chal(1)[0]
    t = timed(ctx, lambda: ctx.logup(dpb.LOGUP_LOOKUP, cols[:1], c, sep).free(), args.reps)
    report("logup tree, lookup, 1 column", t, (1 + 4) * N * s1 if fr else N * s0 + 4 * N * s1)
    t = timed(ctx, lambda: ctx.logup(dpb.LOGUP_LOOKUP, cols, c, sep).free(), args.reps)
    report("logup tree, lookup, 2 columns", t, 2 * N * s0 + 4 * N * s1)

    def logup_prove(columns, cpi):
        tr = prover.Blake3Transcript(fam)
        inp = prover.LogUpInput.new_lookup(columns, c, sep, cpi)
        out = prover.new_batch_multiple_sizes_prove(ctx, [inp], tr)
        tr.free()
        return out

    t = timed(ctx, lambda: logup_prove(cols, 1), max(1, args.reps // 2))
    # tree build for both instances + one sumcheck per level over 4 tables per instance + eq
    tree = 2 * (N * s0 + 4 * N * s1)
    sc = sum((4 * 2 + 1) * (4 * s1) * (1 << v) for v in range(1, n)) // 2
    report(f"logup-GKR batch prove, 2 x 2^{n} lookups", t, tree + sc)

    # a batch of many small instances (softmax chunks x lookups per chunk): 36 two-column lookups of 2^12, whose
    # long term list is spread over threads in the small rounds
    many = [ctx.upload(table(1 << 12), base) for _ in range(72)]

    def logup_many():
        tr = prover.Blake3Transcript(fam)
        out = prover.new_batch_multiple_sizes_prove(ctx, [prover.LogUpInput.new_lookup(many, c, sep, 2)], tr)
        tr.free()
        return out

    t = timed(ctx, logup_many, max(1, args.reps // 2))
    m12 = 1 << 12
    report("logup-GKR batch prove, 36 x 2 columns x 2^12", t,
           36 * (2 * m12 * s0 + 4 * m12 * s1) + sum((4 * 36 + 1) * (4 * s1) * (1 << v) for v in range(1, 12)) // 2)
    for h in many:
        h.free()

    # generic sumcheck: two product terms with coefficients over four tables (einsum-like shape)
    tabs = [ctx.upload(table(N), base) for _ in range(4)]
    cb = chal(2)
    terms = dpb.make_terms([(cb[0].tobytes(), [0, 1]), (cb[1].tobytes(), [2, 3])], bytes)

    def generic():
        tr = prover.Blake3Transcript(fam)
        st = prover.IOPProverState.prove(ctx, n, tabs, terms, tr)
        tr.free()
        return st

    t = timed(ctx, generic, max(1, args.reps // 2))
    report(f"generic sumcheck, 4 tables, 2 terms, 2^{n}", t, 4 * (2 * s0 + 2 * s1) * N)

    x = rng.integers(-2048, 2048, size=(512, 768), dtype=np.int64)
    wt = rng.integers(-2048, 2048, size=(768, 3072), dtype=np.int64)
    p9, p12 = chal(9), chal(12)
    K = (dpb.AXIS_OUTER, dpb.AXIS_CONTRACTED)
    t = timed(ctx, lambda: [h.free() for h in ctx.einsum_fix_axes(fam, x, K, [p9, None])[1]], args.reps)
    report("einsum fix_axes x[512,768], bind rows", t, x.size * 8)
    K2 = (dpb.AXIS_CONTRACTED, dpb.AXIS_OUTER)
    t = timed(ctx, lambda: [h.free() for h in ctx.einsum_fix_axes(fam, wt, K2, [None, p12])[1]], args.reps)
    report("einsum fix_axes W[768,3072], bind columns", t, wt.size * 8)
    dx, dw = ctx.upload_tensor_i64(x), ctx.upload_tensor_i64(wt)
    t = timed(ctx, lambda: [h.free() for h in ctx.einsum_fix_axes(fam, None, K, [p9, None], device_tensor=dx)[1]], args.reps)
    report("  the same, tensor already on the device", t, x.size * 8)
    t = timed(ctx, lambda: [h.free() for h in ctx.einsum_fix_axes(fam, None, K2, [None, p12], device_tensor=dw)[1]], args.reps)
    report("  the same, tensor already on the device", t, wt.size * 8)

    lookup(dpb, prover, ctx, rng, args, fam, s0, s1, report)

    # claim batching of the opening proof: many committed polynomials of mixed sizes, one claim each, all
    # zero-padded to the largest; bytes = sumcheck traffic of every polynomial and its eq table at its own size
    sizes = [min(n, 16)] * 64 + [min(n, 12)] * 192 + [n] * 4
    polys, nbytes = [], 0
    for m in sizes:
        tab = ctx.upload(table(1 << m), base)
        polys.append(prover.CommittedPoly([tab], [(chal(m), chal(1)[0])]))
        nbytes += ((2 * s0 + 2 * s1) + 4 * s1) * (1 << m)

    def claims():
        tr = prover.Blake3Transcript(fam)
        out = prover.claims_batching_prove(ctx, tr, polys, with_rlc=False)
        tr.free()
        return out

    t = timed(ctx, claims, max(1, args.reps // 2))
    report(f"claim batching, {len(sizes)} polys up to 2^{n}", t, nbytes)
    mles = [p.chunks[0] for p in polys]
    cf = chal(len(mles))
    t = timed(ctx, lambda: dpb.linear_combination(ctx, mles, cf).free(), args.reps)
    report(f"linear combination of {len(mles)} polys", t, sum((1 << m) * s0 for m in sizes) + (1 << n) * s1)
    ctx.close()


if __name__ == "__main__":
    main()
