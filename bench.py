"""Benchmark of the sumcheck hot path on B200.

Workload: the standalone sumcheck microbenchmark — prove sum_x f(x) g(x) h(x)
over three random multilinear tables of 2^n Goldilocks base-field values, the
verifier challenges being quadratic-extension elements drawn from the host
transcript.  One "step" is one complete proof (all n rounds).  The metric is
sumcheck GB/s: algorithmic bytes B_alg = k (2 s0 + 2 s1) 2^n = 144 * 2^n (k = 3
tables, s0 = 8 B before and s1 = 16 B after the first fold) divided by the time
of a whole proof, host transcript turn-arounds included.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--log2-size n] [--field gl|fr]
    python bench.py --impl reference ...   times the CPU restatement of the same prover

Prints one JSON line (see the keys below).  Inputs are seeded synthetic data.
"""
import argparse
import importlib
import json
import os
import statistics
import subprocess
import sys
import tempfile
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GL_MOD = 2**64 - 2**32 + 1
FALLBACK_HBM_GBS = 6650.0

def load_ncu_traffic():
    """DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) per table entry of a launch's input, taken from an
    ncu capture at a smaller size; traffic grows in proportion to the entries processed, so a full launch is the
    figure times its input entries.  Keyed by (field, profile label of the kernel, round)."""
    path = os.path.join(ROOT, "profiles", "ncu_dram_traffic.json")
    try:
        with open(path) as f:
            rows = json.load(f)["kernels"]
    except (OSError, ValueError, KeyError):
        return {}
    return {(r["field"], r["kernel"], r["round"]): (r["dram_read_bytes"] + r["dram_write_bytes"]) / r["input_entries"]
            for r in rows}


def alg_bytes(field, n, k=3):
    s0, s1 = (8, 16) if field == "gl" else (32, 32)
    return k * (2 * s0 + 2 * s1) * (1 << n)


def load_peak():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    return FALLBACK_HBM_GBS, "fallback (6.65 TB/s)"


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("timestamp,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
         "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
         "clocks_event_reasons.sw_power_cap")

    def __init__(self, device):
        self.device = device
        self.proc = None
        self.path = None
        self.window = None

    def mark(self, t0, t1):
        """Wall-clock bounds (time.time()) of the timed region; samples outside are dropped when enough lie inside."""
        self.window = (t0, t1)

    def start(self):
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.device), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=open(self.path, "w"), stderr=subprocess.DEVNULL)
        except OSError:
            self.proc = None

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        import datetime
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = []
        with open(self.path) as f:
            for line in f:
                parts = [x.strip() for x in line.split(",")]
                if len(parts) < 9:
                    continue
                try:
                    ts = datetime.datetime.strptime(parts[0], "%Y/%m/%d %H:%M:%S.%f").timestamp()
                    rows.append((ts, float(parts[1]), float(parts[2]),
                                 [n for n, v in zip(names, parts[5:9]) if v.lower().startswith("active")]))
                except ValueError:
                    continue
        os.unlink(self.path)
        scope = "warm-up, timed and profiled steps (all under the same load)"
        if self.window:
            inside = [r for r in rows if self.window[0] - 0.05 <= r[0] <= self.window[1] + 0.05]
            if len(inside) >= 3:
                rows, scope = inside, "timed steps"
        sm, mx = [r[1] for r in rows], [r[2] for r in rows]
        reasons = sorted({n for r in rows for n in r[3]})
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": reasons, "samples": len(sm), "window": scope}


def host_tables(field, n, seed, pinned):
    """Three seeded tables of 2^n entries in host memory (pinned when asked)."""
    import torch
    N = 1 << n
    words = 1 if field == "gl" else 4
    t = torch.empty((3, N, words), dtype=torch.int64, pin_memory=pinned)
    a = t.numpy().view(np.uint64)
    rng = np.random.default_rng(seed)
    chunk = 1 << 22
    for j in range(3):
        for off in range(0, N, chunk):
            m = min(chunk, N - off)
            if field == "gl":
                a[j, off:off + m, 0] = rng.integers(0, GL_MOD, size=m, dtype=np.uint64)
            else:
                blk = rng.integers(0, 2**64, size=(m, 4), dtype=np.uint64)
                blk[:, 3] &= np.uint64((1 << 60) - 1)  # below the modulus: valid Montgomery residues
                a[j, off:off + m] = blk
    return t, (a[:, :, 0] if field == "gl" else a)


def cpu_prove(orc, F, n, tabs):
    return orc.sumcheck_prove(F, n, tabs, {(0, 1, 2): F.one}, orc.Transcript(F))


def cpu_setup():
    """The oracle tuned for this host's CPU and on every core this process may use (a launcher such as
    torch.distributed.run exports OMP_NUM_THREADS=1, which would turn the baseline into one core)."""
    from oracle import oracle as orc
    native = orc.use_native_build()
    cores = orc.set_num_threads()
    return orc, cores, native


def cpu_baseline(field, n_sample, seed):
    """The CPU restatement (oracle) of the same prover on the host cores.  Also returns the tables and the proof
    of the sample, for the parity check of the GPU path."""
    orc, cores, native = cpu_setup()
    F = orc.GlField if field == "gl" else orc.FrField
    if field != "gl":
        n_sample = min(n_sample, 22)  # BN254 on the host: 32-byte elements and a slower product
    rng = np.random.default_rng(seed)
    tabs = [F.random_table_fast(rng, 1 << n_sample) for _ in range(3)]
    cpu_prove(orc, F, min(n_sample, 16), [t[: 1 << min(n_sample, 16)] for t in tabs])  # warm up threads
    # whole proofs, one after the other, until about ten seconds of CPU work have been timed
    reps, t0 = 0, time.perf_counter()
    while reps < 16 and (reps == 0 or time.perf_counter() - t0 < 10.0):
        proof = cpu_prove(orc, F, n_sample, tabs)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    rec = {"value": alg_bytes(field, n_sample) / dt / 1e9, "unit": "GB/s", "cores": cores,
           "kind": "port", "seconds": dt * reps, "march_native": native,
           "sample": f"{reps} full proofs at 2^{n_sample} entries per table (same shape and field, smaller size), "
                     "mean; C/OpenMP restatement of the prover, not the reference's Rust binary"}
    return rec, (F, n_sample, tabs, proof)


def metric_name(field):
    return "sumcheck_GBps_" + ("goldilocks" if field == "gl" else "bn254")


def workload_config(field, n, n_gpus):
    name = "Goldilocks base tables, Ext2 challenges" if field == "gl" else "BN254 Fr"
    in_bytes = 3 * (1 << (n - (n_gpus.bit_length() - 1))) * (8 if field == "gl" else 32)  # per GPU
    l2 = ("inputs per step exceed the 126 MB L2; no flush needed" if in_bytes > 126e6
          else "inputs fit in the 126 MB L2: a small-size run, not a roofline measurement")
    return {"workload": f"standalone sumcheck microbench f*g*h, 2^{n} entries per table, {name} "
                        "(BASELINE.json configs[1])",
            "log2_size": n, "field": field, "tables": 3, "degree": 3, "sharding": f"top log2({n_gpus}) variables",
            "l2": l2}


def run_reference(args):
    """The reference arm: the CPU prover of the same workload on the host cores.  At one GPU each step is one full
    proof at the workload's own size; at N GPUs the workload is 2^(n + log2 N) entries per table, and each step
    proves the 2^n entries one GPU holds (a bounded sample, stated in cpu_baseline.sample; throughput in GB/s does
    not depend on the size on the CPU)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    orc, cores, native = cpu_setup()
    world = int(os.environ.get("WORLD_SIZE", str(args.gpus)))
    n_global = args.log2_size + world.bit_length() - 1
    F = orc.GlField if args.field == "gl" else orc.FrField
    n_s = min(args.log2_size, args.ref_max_log2 if args.field == "gl" else min(args.ref_max_log2, 24))
    rng = np.random.default_rng(args.seed)
    tabs = [F.random_table_fast(rng, 1 << n_s) for _ in range(3)]
    for _ in range(args.warmup):
        cpu_prove(orc, F, n_s, tabs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_prove(orc, F, n_s, tabs)
    dt = (time.perf_counter() - t0) / args.steps
    val = alg_bytes(args.field, n_s) / dt / 1e9
    if n_s == n_global:
        sample = f"each step is one full proof of the workload (2^{n_s} entries per table)"
    else:
        sample = (f"each step is one full proof at 2^{n_s} entries per table, a bounded sample of the "
                  f"2^{n_global} workload; GB/s does not depend on the size on the CPU")
    print(json.dumps({
        "impl": "reference", "metric": metric_name(args.field), "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u64" if args.field == "gl" else "u256", "data": "synthetic",
        "config": workload_config(args.field, n_global, world),
        "sample_log2_size": n_s,
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample,
                         "march_native": native, "omp_num_threads_env": os.environ.get("OMP_NUM_THREADS")},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's Rust prover cannot be built here (no Rust toolchain, dp-crypto not vendored); "
                "this is the C/OpenMP restatement in oracle/ on the host cores",
    }))


def proof_scalars(orc, F, st):
    """(rounds, point, final evaluations) of a proof from the library as the oracle's scalars."""
    flat = lambda a: orc.array_to_scalars(F, np.asarray(a).reshape(-1, F.elem_words))
    return flat(st.proof), flat(st.collect_raw_challenges()), flat(st.get_mle_flatten_final_evaluations())


def parity_check(dpb, prover, ctx, field, case, world, rank, dist):
    """Outside the timed region: the GPU path proves seeded tables the oracle has proved and the proofs must be
    equal (rounds, point, final evaluations).  One GPU: the 2^26 sample of the CPU baseline.  Several GPUs: every
    rank proves its shard of a 2^(22 + log2 N) sumcheck, all ranks' proofs must be equal and rank 0 compares them
    with the oracle's proof of the whole tables."""
    from oracle import oracle as orc
    base_dtype = dpb.GL_BASE if field == "gl" else dpb.FR
    fam = dpb.GL_EXT if field == "gl" else dpb.FR
    terms = dpb.make_terms([(dpb.one_bytes(fam), [0, 1, 2])], bytes)
    if world == 1:
        F, n, tabs, want = case
        mles = [ctx.upload(t, base_dtype) for t in tabs]
        t = prover.Blake3Transcript(fam)
        st = prover.IOPProverState.prove(ctx, n, mles, terms, t)
        t.free()
        for m in mles:
            m.free()
        got = proof_scalars(orc, F, st)
        ok = got[0] == [e for r in want[0] for e in r] and got[1] == want[1] and got[2] == want[2]
        return {"log2": n, "ok": bool(ok), "against": "oracle proof of the same seeded tables (rounds, point, finals)"}
    F = orc.GlField if field == "gl" else orc.FrField
    c = world.bit_length() - 1
    n = 22 + c
    rng = np.random.default_rng(12345)
    tabs = [F.random_table_fast(rng, 1 << n) for _ in range(3)]
    per = 1 << (n - c)
    mles = [ctx.upload(np.ascontiguousarray(t[rank * per:(rank + 1) * per]), base_dtype) for t in tabs]
    t = prover.Blake3Transcript(fam)
    st = prover.IOPProverState.prove(ctx, n, mles, terms, t, sharded=True)
    t.free()
    for m in mles:
        m.free()
    got = proof_scalars(orc, F, st)
    everyone = [None] * world
    dist.all_gather_object(everyone, got)
    if rank != 0:
        return None
    orc.set_num_threads()
    want = cpu_prove(orc, F, n, tabs)
    same = all(g == everyone[0] for g in everyone)
    ok = same and got[0] == [e for r in want[0] for e in r] and got[1] == want[1] and got[2] == want[2]
    return {"log2": n, "ok": bool(ok), "ranks_agree": bool(same),
            "against": "oracle proof of the whole seeded tables; every rank's proof equal to rank 0's"}


def device_random_fr(ctx, dpb, torch, n, seed, device):
    """Three BN254 tables of 2^n entries made on the device (random limbs below the modulus, taken as Montgomery
    residues): the BN254 record needs no host copy of its 6 GiB of inputs."""
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    keep, mles = [], []
    for _ in range(3):
        t = torch.randint(-2**63, 2**63 - 1, (1 << n, 4), dtype=torch.int64, device=device, generator=g)
        t[:, 3] &= (1 << 60) - 1
        keep.append(t)
        mles.append(ctx.wrap_device(t.data_ptr(), dpb.FR, 1 << n))
    torch.cuda.synchronize()
    return keep, mles


def bn254_record(dpb, prover, ctx, torch, stream, device, steps, n):
    """The same f*g*h shape over BN254 Fr, the reference's own field: whole-proof GB/s, per-round kernels, and the
    binding bound.  These rounds are bound by 32-bit multiply-add issue, not by HBM: the roofline entry compares
    the field products per second of the top kernel with what dpb_issue_rate_probe measures on this GPU."""
    keep, mles = device_random_fr(ctx, dpb, torch, n, 99, device)
    terms = dpb.make_terms([(dpb.one_bytes(dpb.FR), [0, 1, 2])], bytes)

    def step():
        t = prover.Blake3Transcript(dpb.FR)
        st = prover.IOPProverState.prove(ctx, n, mles, terms, t)
        t.free()
        return st

    for _ in range(3):
        step()
    ctx.sync()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    ctx.sync()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    ctx.profile(True)
    for _ in range(min(steps, 5)):
        step()
    ctx.sync()
    ctx.profile(False)
    prof = ctx.profile_read()
    mul_rate, _ = ctx.issue_rate(ctx.PROBE_FR_MUL)
    fixed_rate, _ = ctx.issue_rate(ctx.PROBE_FR_MUL_FIXED)
    mad_rate, _ = ctx.issue_rate(ctx.PROBE_WIDE_MAD)
    kernels = []
    for e in sorted(prof, key=lambda e: e["round"])[:6]:
        per_ms = e["total_ms"] / e["launches"]
        pairs = 1 << (n - e["round"] - 1)
        # round 0: samples at 0, 1, inf, -1 of a product of three = 8 products per pair;
        # later rounds: 6 folds by the challenge (precomputed rows) + 3 samples x 2 products
        floor_s = pairs * (8 / mul_rate if e["round"] == 0 else 6 / fixed_rate + 6 / mul_rate)
        kernels.append({"kernel": e["kernel"], "round": e["round"], "ms_per_launch": per_ms,
                        "GBps": e["alg_bytes_per_launch"] / (per_ms * 1e-3) / 1e9,
                        "products_per_pair": 8 if e["round"] == 0 else 12,
                        "frac_of_multiplier_floor": floor_s / (per_ms * 1e-3)})
    top = max(kernels, key=lambda k: k["ms_per_launch"]) if kernels else None
    peak, _ = load_peak()
    rec = {"workload": f"f*g*h, 2^{n} entries per table, BN254 Fr (the reference's field), tables made on the device",
           "log2_size": n, "value": alg_bytes("fr", n) / (ms * 1e-3) / 1e9, "unit": "GB/s", "ms_per_step": ms,
           "steps": steps, "frac_of_hbm_peak": alg_bytes("fr", n) / (ms * 1e-3) / 1e9 / peak, "kernels": kernels,
           "issue_rate_probe": {"fr_products_per_s": mul_rate, "fr_fixed_products_per_s": fixed_rate,
                                "wide_multiply_adds_per_s": mad_rate}}
    if top:
        ach = (1 << (n - top["round"] - 1)) * top["products_per_pair"] / (top["ms_per_launch"] * 1e-3)
        rec["roofline"] = {"bound": "imad", "kernel": top["kernel"], "round": top["round"],
                           "achieved": ach, "unit": "field products/s",
                           "peak": mul_rate if top["round"] == 0 else 12 / (6 / fixed_rate + 6 / mul_rate),
                           "frac": top["frac_of_multiplier_floor"],
                           "peak_source": "dpb_issue_rate_probe on this GPU (chains of the kernels' own product "
                                          "routines on register operands)"}
    for m in mles:
        m.free()
    del keep
    torch.cuda.empty_cache()
    # the same proof over 32-bit integer tables (quantised tensors and lookup columns are small integers): round 0 in
    # integer arithmetic, round 1 folds integers; algorithmic bytes with s0 = 4
    g = torch.Generator(device=device)
    g.manual_seed(7)
    ints = [torch.randint(-2**31, 2**31 - 1, (1 << n,), dtype=torch.int32, device=device, generator=g) for _ in range(3)]
    imles = [ctx.wrap_device(t.data_ptr(), dpb.FR_I32, 1 << n) for t in ints]
    torch.cuda.synchronize()

    def istep():
        t = prover.Blake3Transcript(dpb.FR)
        st = prover.IOPProverState.prove(ctx, n, imles, terms, t)
        t.free()
        return st

    for _ in range(3):
        istep()
    ctx.sync()
    e0.record(stream)
    for _ in range(steps):
        istep()
    e1.record(stream)
    ctx.sync()
    torch.cuda.synchronize()
    ims = e0.elapsed_time(e1) / steps
    ctx.profile(True)
    for _ in range(min(steps, 5)):
        istep()
    ctx.sync()
    ctx.profile(False)
    iprof = sorted(ctx.profile_read(), key=lambda e: e["round"])[:3]
    ibytes = 3 * (2 * 4 + 2 * 32) * (1 << n)
    rec["int32_tables"] = {
        "workload": f"f*g*h, 2^{n} int32 entries per table (DPB_FR_I32), BN254 Fr",
        "ms_per_step": ims, "speedup_over_field_tables": ms / ims,
        "value": ibytes / (ims * 1e-3) / 1e9, "unit": "GB/s",
        "alg_bytes": "k (2*4 + 2*32) 2^n: 4-byte entries before the first fold, 32-byte after",
        "kernels": [{"kernel": e["kernel"], "round": e["round"], "ms_per_launch": e["total_ms"] / e["launches"],
                     "GBps": e["alg_bytes_per_launch"] / (e["total_ms"] / e["launches"] * 1e-3) / 1e9} for e in iprof]}
    for m in imles:
        m.free()
    del ints
    torch.cuda.empty_cache()
    return rec


def strong_record(dpb, prover, ctx, torch, dist, stream, mles, terms, fam, n, world, rank, steps):
    """Strong scaling of the fixed 2^n proof: all ranks prove ONE sumcheck of 2^n entries per table, each holding
    2^(n - log2 N); rank 0 also proves a 2^n sumcheck alone in the same run, the N = 1 time of the ratio."""
    c = world.bit_length() - 1
    per = 1 << (n - c)
    views = [m.view(0, per) for m in mles]

    def timed(fn, reps):
        for _ in range(2):
            fn()
        dist.barrier()
        ctx.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(reps):
            fn()
        e1.record(stream)
        ctx.sync()
        torch.cuda.synchronize()
        tt = torch.tensor([e0.elapsed_time(e1) / reps], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        return float(tt.item())

    def sharded():
        t = prover.Blake3Transcript(fam)
        prover.IOPProverState.prove(ctx, n, views, terms, t, sharded=True)
        t.free()

    ms_n = timed(sharded, steps)
    ctx.profile(True)
    for _ in range(3):
        sharded()
    ctx.sync()
    ctx.profile(False)
    prof = ctx.profile_read()
    kernel_ms = sum(e["total_ms"] / 3 for e in prof)
    ms_1 = None
    if rank == 0:
        def alone():
            t = prover.Blake3Transcript(fam)
            prover.IOPProverState.prove(ctx, n, mles, terms, t)
            t.free()
        for _ in range(2):
            alone()
        ctx.sync()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        for _ in range(steps):
            alone()
        e1.record(stream)
        ctx.sync()
        torch.cuda.synchronize()
        ms_1 = e0.elapsed_time(e1) / steps
    dist.barrier()
    for v in views:
        v.free()
    if rank != 0:
        return None
    return {"workload": f"one f*g*h proof of 2^{n} entries per table over {world} GPUs (2^{n - c} per GPU)",
            "ms_per_proof": ms_n, "ms_per_proof_one_gpu_same_run": ms_1, "speedup": ms_1 / ms_n,
            "GBps": alg_bytes("gl" if fam == dpb.GL_EXT else "fr", n) / (ms_n * 1e-3) / 1e9,
            "local_rounds": n - c, "exchanges_per_proof": n - c + 1,
            "split_ms": {"round_kernels": kernel_ms, "exchange_launch_host": max(ms_n - kernel_ms, 0.0)},
            "limiter": "per-round turn-around (launch, exchange of the partial sums between the hosts, transcript) "
                       "of the local rounds plus the replicated last log2(N) rounds; the kernels scale with 1/N"}


def logup_spread_record(dpb, prover, ctx, torch, dist, world, rank, steps, seed):
    """A logup-GKR batch spread over the GPUs by instance (dpb_logup_batch_prove_partial): 24 two-column lookup
    instances of 2^18 rows (two attention layers' worth of softmax columns), BN254, integer columns resident on the
    device; instance j lives on rank j mod N.  Rank 0 also proves the whole batch alone in the same run, and the
    bytes of the two proofs are compared."""
    import numpy as np
    total, rows = 24, 1 << 18
    rng = np.random.default_rng(seed + 5)
    cst, sep = [rng.integers(1, 2**62, size=4, dtype=np.uint64) for _ in range(2)]
    cst[3] = sep[3] = 0
    cols = [[rng.integers(-(1 << 11), 1 << 11, size=rows, dtype=np.int64) for _ in range(2)] for _ in range(total)]

    def lookups(idx):
        dev = [ctx.upload_ints(c, dpb.FR_I64) for j in idx for c in cols[j]]
        return prover.LogUpInput.new_lookup(dev, cst.reshape(1, 4), sep.reshape(1, 4), 2), dev

    mine, mine_dev = lookups([j for j in range(total) if j % world == rank])

    def spread():
        t = prover.Blake3Transcript(dpb.FR)
        out = prover.new_batch_multiple_sizes_prove(ctx, [mine], t, partial=True)
        t.free()
        return out

    def wall(fn, reps, collective):
        for _ in range(2):
            got = fn()
        if collective:
            dist.barrier()
        ctx.sync()
        t0 = time.perf_counter()
        for _ in range(reps):
            got = fn()
        ctx.sync()
        dt = (time.perf_counter() - t0) / reps * 1e3
        if collective:
            tt = torch.tensor([dt], device="cuda")
            dist.all_reduce(tt, op=dist.ReduceOp.MAX)
            dt = float(tt.item())
        return dt, got

    ms_n, got = wall(spread, steps, True)
    ms_1, equal = None, None
    if rank == 0:
        whole, whole_dev = lookups(range(total))

        def alone():
            t = prover.Blake3Transcript(dpb.FR)
            out = prover.new_batch_multiple_sizes_prove(ctx, [whole], t)
            t.free()
            return out
        ms_1, want = wall(alone, steps, False)
        equal = want == got
        for m in whole_dev:
            m.free()
    dist.barrier()
    for m in mine_dev:
        m.free()
    if rank != 0:
        return None
    return {"workload": f"logup-GKR batch of {total} two-column lookup instances of 2^18 rows, BN254, over {world} GPUs "
                        f"({total // world} instances per GPU)",
            "ms_per_proof": ms_n, "ms_per_proof_one_gpu_same_run": ms_1, "speedup": ms_1 / ms_n,
            "proof_equals_single_gpu": equal,
            "timing": "wall clock around the call between device synchronisations, max over ranks",
            "exchanges": "per round the partial sums (shared host segment), per layer the final evaluations (NCCL)"}


def workload_record(dpb, prover, ctx, args):
    """The GPT-2-small seq-512 path workload (deep-prove_b200/workloads.py) over BN254, tensors resident on the
    device: tokens/s = sequence length / time of the path's calls, the reference's definition of token/sec
    (zkml/src/bin/bench/llm.rs:345-355) applied to the path instead of to prove_full.  The CPU restatement walks
    a bounded sample of the same call list (one block at a reduced shape) and the GPU walks that sample too."""
    wl = importlib.import_module("deep_prove_b200.workloads")
    shape = wl.GPT2_SMALL
    ctx.trim()
    # warm-up: one whole walk, so that kernels are loaded and the stream-ordered memory pool has grown to the
    # walk's largest allocation (the claim batching's fold buffers); a prover process is in this state after its
    # first proof
    wl.run_transformer_path(dpb, prover, ctx, shape, field="fr", seed=args.seed + 1, with_commit=True)
    dpb.trace(True)
    got = wl.run_transformer_path(dpb, prover, ctx, shape, field="fr", seed=args.seed, with_commit=True)
    phases = {k: {"ms": v[0], "calls": v[1]} for k, v in sorted(dpb.trace_read().items(), key=lambda kv: -kv[1][0])[:12]}
    dpb.trace(False)
    rec = {"workload": "GPT-2-small (12 layers, d_model 768, 12 heads, FFN 3072, vocab 50257), 512 tokens: every "
                       "sumcheck / fold / logup-GKR call of the forward graph, BN254 Fr, seeded synthetic integer "
                       "tensors resident on the device (BASELINE.json configs[2] shapes)",
           "field": "bn254", "ms": got["seconds"] * 1e3, "tokens_per_s": got["tokens_per_s"],
           "by_kind_ms": {k: v * 1e3 for k, v in sorted(got["by_kind"].items(), key=lambda kv: -kv[1])},
           "calls": got["calls"], "wall_seconds_with_input_generation": got["wall_seconds"],
           "host_phases_ms": phases,
           "witness_commit": {
               "ms": got["commit_seconds"] * 1e3,
               "what": "every lookup layer's witness columns committed: one BN254 G1 multi-scalar multiplication "
                       "per chunk of at most 2^20 evaluations against device-made stand-in bases "
                       "(zkml/src/lookup/context.rs:420-422); not part of the path, reported beside it",
               "tokens_per_s_path_plus_witness_commit": shape.seq / (got["seconds"] + got["commit_seconds"])},
           "timing": "wall clock per call with a device synchronisation on both sides, summed; generation and upload "
                     "of the synthetic tensors are outside",
           "excludes": "inference, HyperKZG opening and host orchestration of the reference's prove_full; the "
                       "reference's published 1.12 tokens/s (24-core EPYC, whole prover) is a different scope"}
    # the same walk over Goldilocks (base tables, extension challenges): the field of the standalone benchmark
    wl.run_transformer_path(dpb, prover, ctx, shape, field="gl", seed=args.seed + 1)
    gl = wl.run_transformer_path(dpb, prover, ctx, shape, field="gl", seed=args.seed)
    rec["goldilocks"] = {"ms": gl["seconds"] * 1e3, "tokens_per_s": gl["tokens_per_s"],
                         "by_kind_ms": {k: v * 1e3 for k, v in sorted(gl["by_kind"].items(), key=lambda kv: -kv[1])}}
    sample = wl.CPU_SAMPLE
    gpu_s = wl.run_transformer_path(dpb, prover, ctx, sample, field="fr", seed=args.seed)
    gpu_s = wl.run_transformer_path(dpb, prover, ctx, sample, field="fr", seed=args.seed)
    rec["cpu_sample"] = {"shape": "one block, seq 128, d_model 192, 4 heads x 48, FFN 768, vocab 4000, 10-bit tables",
                         "gpu_ms": gpu_s["seconds"] * 1e3, "gpu_tokens_per_s": gpu_s["tokens_per_s"]}
    if not args.no_cpu_baseline:
        from oracle.path_backend import OracleBackend
        orc, cores, native = cpu_setup()
        t0 = time.perf_counter()
        want, timer = wl.transformer_path(OracleBackend("fr"), sample, seed=args.seed)
        cpu_s = sum(timer.by_kind.values())
        rec["cpu_sample"].update({
            "cpu_ms": cpu_s * 1e3, "cpu_tokens_per_s": sample.seq / cpu_s, "cores": cores, "kind": "port",
            "cpu_wall_seconds": time.perf_counter() - t0,
            "payloads_equal": [r for r in gpu_s["records"]] == want,
            "note": "the CPU restatement keeps its protocol logic in Python (big integers) over C/OpenMP round "
                    "kernels, so it understates a compiled CPU prover; it is the checker, timed as it is"})
    return rec


def more_workloads(dpb, prover, ctx, args, which):
    """The other model configurations BASELINE.json names, walked like the GPT-2 one: the dense network
    (configs[0]; "tokens" are input rows), the Gemma-3-1B-style model (configs[3]) and two Llama-2-7B-style blocks
    (configs[4]), each on ONE GPU.  Warm-up: one whole walk (three for the dense network), which also grows the
    stream-ordered memory pool to the walk's largest working set (the claim batching: one eq table per committed
    chunk polynomial, tens of GB at these sizes) as a prover process has it after its first proof."""
    import torch
    wl = importlib.import_module("deep_prove_b200.workloads")
    table = {"mlp": (wl.MLP_2LAYER, "BASELINE.json configs[0] shapes: 1 x 1024 input, 1024 x 1024 and 1024 x 10 weights, "
                                    "ReLU through a lookup, argmax"),
             "gemma3_1b_seq512": (wl.GEMMA3_1B, "BASELINE.json configs[3] shapes: 26 layers, d_model 1152, 4 query heads / "
                                                "1 KV head x 256, GeGLU 6912, RoPE, vocab 262144, 512 tokens"),
             "llama2_7b_2blocks_seq1024": (wl.LLAMA2_7B_2BLOCKS, "BASELINE.json configs[4] shapes: 2 blocks, d_model 4096, 32 "
                                                                 "heads x 128, SwiGLU 11008, RoPE, vocab 32000, 1024 tokens; "
                                                                 "walked on one GPU")}
    out = {}
    for key in which:
        shape, what = table[key]
        ctx.trim()  # every workload starts from an empty pool, like a prover process started for that model
        try:
            if isinstance(shape, wl.MlpShape):
                for i in range(3):
                    wl.run_transformer_path(dpb, prover, ctx, shape, field="fr", seed=args.seed + 1 + i)
            else:
                wl.run_transformer_path(dpb, prover, ctx, shape, field="fr", seed=args.seed + 1)
            got = wl.run_transformer_path(dpb, prover, ctx, shape, field="fr", seed=args.seed)
        except Exception as e:  # a walk that does not fit this GPU's memory must not take the whole line with it
            out[key] = {"workload": what, "error": f"{type(e).__name__}: {e}"[:300]}
            continue
        free_b, total_b = torch.cuda.mem_get_info()
        out[key] = {"workload": what + "; every sumcheck / fold / logup-GKR call of the forward graph, BN254 Fr, seeded "
                                       "synthetic integer tensors resident on the device",
                    "field": "bn254", "ms": got["seconds"] * 1e3, "tokens_per_s": got["tokens_per_s"],
                    "by_kind_ms": {k: v * 1e3 for k, v in sorted(got["by_kind"].items(), key=lambda kv: -kv[1])},
                    "calls": got["calls"], "wall_seconds_with_input_generation": got["wall_seconds"],
                    "device_memory_held_after_GB": (total_b - free_b) / 1e9}
    return out


def run_only(args):
    """One sub-record of the default line by itself (one GPU)."""
    import torch
    from __graft_entry__ import load_package
    dpb = load_package()
    prover = importlib.import_module("deep_prove_b200.prover")
    torch.cuda.set_device(0)
    device = torch.device("cuda", 0)
    ctx = dpb.Context(0)
    stream = torch.cuda.ExternalStream(ctx.stream, device=device)
    if args.only == "bn254":
        rec = bn254_record(dpb, prover, ctx, torch, stream, device, min(args.steps, 10), args.bn254_log2)
    elif args.only == "workload":
        rec = workload_record(dpb, prover, ctx, args)
    else:
        rec = more_workloads(dpb, prover, ctx, args, [args.only])[args.only]
    print(json.dumps({args.only: rec}))


def run_ours(args):
    import torch
    import torch.distributed as dist
    from __graft_entry__ import load_package
    dpb = load_package()
    prover = importlib.import_module("deep_prove_b200.prover")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    field, n = args.field, args.log2_size
    base_dtype = dpb.GL_BASE if field == "gl" else dpb.FR
    fam = dpb.GL_EXT if field == "gl" else dpb.FR
    ctx = dpb.Context(local_rank)
    stream = torch.cuda.ExternalStream(ctx.stream, device=device)

    if world > 1:
        # the library's own communicator; torch.distributed only carries the 128-byte id
        box = [dpb.comm_unique_id() if rank == 0 else None]
        dist.broadcast_object_list(box, src=0)
        ctx.comm_init(box[0], rank, world)
    exchange = None
    if world > 1:
        exchange = ("per-round sums through a shared host segment every rank's kernel writes and every host polls"
                    if ctx.comm_shared_exchange() else "per-round sums through ncclAllGather + copy to the host")
    sharded = world > 1
    log2_world = world.bit_length() - 1
    n_global = n + log2_world  # weak scaling: every rank holds a 2^n shard of a 2^(n + log2 G) hypercube

    pinned, host = host_tables(field, n, args.seed + rank, pinned=True)
    mles = [ctx.upload(host[j], base_dtype) for j in range(3)]
    terms = dpb.make_terms([(dpb.one_bytes(fam), [0, 1, 2])], bytes)

    def step_device():
        t = prover.Blake3Transcript(fam)
        st = prover.IOPProverState.prove(ctx, n_global, mles, terms, t, sharded=sharded)
        t.free()
        return st

    def step_e2e():
        ms = [ctx.upload(host[j], base_dtype) for j in range(3)]
        t = prover.Blake3Transcript(fam)
        st = prover.IOPProverState.prove(ctx, n_global, ms, terms, t, sharded=sharded)
        t.free()
        for m in ms:
            m.free()
        return st

    def barrier():
        if world > 1:
            dist.barrier()
        ctx.sync()
        torch.cuda.synchronize()

    # ---- device-resident throughput
    sampler = ClockSampler(local_rank)
    sampler.start()  # before the warm-up: nvidia-smi takes a moment to deliver its first sample
    for _ in range(args.warmup):
        step_device()
    barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = ctx.sumcheck_launches()
    wall0 = time.time()
    e0.record(stream)
    for _ in range(args.steps):
        st = step_device()
    e1.record(stream)
    barrier()
    sampler.mark(wall0, time.time())
    launches = ctx.sumcheck_launches() - launches0
    ms_total = e0.elapsed_time(e1)
    # per-kernel CUDA-event times: the same steps once more with the library's per-round events on
    # (they cost about 10 us per round, so they stay out of the timed region above)
    ctx.profile(True)
    for _ in range(min(args.steps, 20)):
        st = step_device()
    barrier()
    ctx.profile(False)
    clocks = sampler.stop()
    if world > 1:
        tt = torch.tensor([ms_total], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        ms_total = float(tt.item())
    ms_step = ms_total / args.steps
    value = alg_bytes(field, n_global) / (ms_step * 1e-3) / 1e9
    prof = ctx.profile_read()

    # ---- end to end: host buffers in, proof out, copies inside the timed region
    e2e_steps = min(args.steps, 20)
    for _ in range(min(args.warmup, 2)):
        step_e2e()
    barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        st = step_e2e()
    barrier()
    e2e_s = (time.perf_counter() - t0) / e2e_steps
    words = 2 if field == "gl" else 4
    h2d = world * 3 * (1 << n) * (8 if field == "gl" else 32)
    d2h = (n_global * 4 + n_global + 3) * words * 8

    strong = None
    if world > 1:
        tt = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_s = float(tt.item())
        if not args.no_strong:
            strong = strong_record(dpb, prover, ctx, torch, dist, stream, mles, terms, fam, n, world, rank,
                                   min(args.steps, 20))
            spread = logup_spread_record(dpb, prover, ctx, torch, dist, world, rank, min(args.steps, 10), args.seed)
            if strong is not None:
                strong["logup_batch"] = spread
    # ---- parity of the timed path against the oracle, outside the timed region
    cpu_rec, case = None, None
    if world == 1 and not args.no_cpu_baseline:
        cpu_rec, case = cpu_baseline(field, args.cpu_sample_log2, args.seed)
    parity = None
    if case is not None or world > 1:
        parity = parity_check(dpb, prover, ctx, field, case, world, rank, dist)
    case = None
    # ---- the same shape over BN254 (one GPU; the Goldilocks buffers are released first)
    bn254 = None
    if world == 1 and field == "gl" and not args.no_bn254:
        for m in mles:
            m.free()
        mles = []
        del pinned, host
        bn254 = bn254_record(dpb, prover, ctx, torch, stream, device, min(args.steps, 10), args.bn254_log2)
    workloads = None
    if world == 1 and not args.no_workload:
        for m in mles:
            m.free()
        mles = []
        which = [w for w in args.workloads.split(",") if w]
        workloads = {}
        if "gpt2_seq512" in which:
            workloads["gpt2_seq512"] = workload_record(dpb, prover, ctx, args)
        workloads.update(more_workloads(dpb, prover, ctx, args, [w for w in which if w != "gpt2_seq512"]))
    if world > 1:
        ctx.comm_free()
        dist.barrier()
        dist.destroy_process_group()
    if rank != 0:
        return
    peak, peak_src = load_peak()
    top = max(prof, key=lambda e: e["total_ms"]) if prof else None
    roofline = None
    if top:
        per_launch_ms = top["total_ms"] / top["launches"]
        ach = top["alg_bytes_per_launch"] / (per_launch_ms * 1e-3) / 1e9
        traffic = None
        per_entry = load_ncu_traffic().get((field, top["kernel"], top["round"]))
        if per_entry is not None:
            traffic = per_entry * 3 * (1 << (n - max(top["round"] - 1, 0)))
        roofline = {"bound": "hbm", "achieved": ach, "peak": peak, "unit": "GB/s", "frac": ach / peak,
                    "traffic": traffic, "kernel": top["kernel"], "round": top["round"],
                    "launch_ms": per_launch_ms, "alg_bytes_per_launch": top["alg_bytes_per_launch"],
                    "peak_source": peak_src}
    kernels = [{"kernel": e["kernel"], "round": e["round"], "launches": e["launches"],
                "ms_per_launch": e["total_ms"] / e["launches"],
                "GBps": e["alg_bytes_per_launch"] / (e["total_ms"] / e["launches"] * 1e-3) / 1e9}
               for e in sorted(prof, key=lambda e: e["round"])[:6]]
    out = {
        "metric": metric_name(field), "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "u64" if field == "gl" else "u256", "data": "synthetic",
        "config": dict(workload_config(field, n_global, world), **({"exchange": exchange} if exchange else {})),
        "frac_of_hbm_peak": value / (peak * world),
        "roofline": roofline,
        "kernels": kernels,
        "e2e": {"value": alg_bytes(field, n_global) / e2e_s / 1e9, "unit": "GB/s", "h2d_bytes_per_step": h2d,
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_s * 1e3, "steps": e2e_steps},
        # counted by the library on rank 0 over the timed steps (every rank launches the same kernels): one
        # launch per large round, one resident kernel for the last rounds and the final evaluations
        "gpu_launches": launches * world,
        "clocks": clocks,
        "parity_checked": parity,
    }
    if cpu_rec is not None:
        out["cpu_baseline"] = cpu_rec
    if bn254 is not None:
        out["bn254"] = bn254
    if strong is not None:
        out["strong"] = strong
    if workloads is not None:
        out["workloads"] = workloads
    print(json.dumps(out))
    if parity is not None and not parity["ok"]:
        sys.exit("parity check failed: the GPU proof differs from the oracle's")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--log2-size", type=int, default=28)
    ap.add_argument("--field", default="gl", choices=["gl", "fr"])
    ap.add_argument("--cpu-sample-log2", type=int, default=26)
    ap.add_argument("--ref-max-log2", type=int, default=28,
                    help="largest table the reference arm proves per step (it proves min(log2-size, this))")
    ap.add_argument("--bn254-log2", type=int, default=26)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-bn254", action="store_true")
    ap.add_argument("--no-strong", action="store_true")
    ap.add_argument("--no-workload", action="store_true", help="skip the model-shaped path workloads")
    ap.add_argument("--workloads", default="gpt2_seq512,mlp,llama2_7b_2blocks_seq1024,gemma3_1b_seq512",
                    help="which path workloads the default line walks (comma-separated)")
    ap.add_argument("--only", default=None,
                    choices=["bn254", "workload", "mlp", "gemma3_1b_seq512", "llama2_7b_2blocks_seq1024"],
                    help="run one sub-record alone and print it (profiling captures of its kernels)")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    elif args.only:
        run_only(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
