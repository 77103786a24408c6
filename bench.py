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

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) per table entry of a
# launch's input, from the ncu capture at 2^24 summarised in
# profiles/sumcheck_goldilocks_product3_2p24_fused_rounds.md.  Traffic grows in
# proportion to the entries processed, so a full launch is this figure times
# its input entries.  Keyed by (field, profile label, round).
NCU_TRAFFIC_BYTES_PER_INPUT_ENTRY = {
    ("gl", "fused_eval0<base>", 0): (402.744064e6 + 6.582016e6) / (3 << 24),
    ("gl", "fused_fold_eval<base>", 1): (402.845952e6 + 359.348736e6) / (3 << 24),
    ("gl", "fused_fold_eval", 2): (402.789632e6 + 169.018880e6) / (3 << 23),
}


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


def cpu_baseline(field, n_sample, seed):
    """The CPU restatement (oracle) of the same prover on the host cores."""
    from oracle import oracle as orc
    F = orc.GlField if field == "gl" else orc.FrField
    if field != "gl":
        n_sample = min(n_sample, 22)  # BN254 on the host: 32-byte elements and a slower product
    rng = np.random.default_rng(seed)
    tabs = [F.random_table_fast(rng, 1 << n_sample) for _ in range(3)]
    cpu_prove(orc, F, min(n_sample, 16), [t[: 1 << min(n_sample, 16)] for t in tabs])  # warm up threads
    # whole proofs, one after the other, until about ten seconds of CPU work have been timed
    reps, t0 = 0, time.perf_counter()
    while reps < 16 and (reps == 0 or time.perf_counter() - t0 < 10.0):
        cpu_prove(orc, F, n_sample, tabs)
        reps += 1
    dt = (time.perf_counter() - t0) / reps
    return {"value": alg_bytes(field, n_sample) / dt / 1e9, "unit": "GB/s", "cores": orc.lib().orc_num_threads(),
            "kind": "port", "seconds": dt * reps,
            "sample": f"{reps} full proofs at 2^{n_sample} entries per table (same shape and field, smaller size), "
                      "mean; C/OpenMP restatement of the prover, not the reference's Rust binary"}


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
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from oracle import oracle as orc
    F = orc.GlField if args.field == "gl" else orc.FrField
    n_s = args.cpu_sample_log2 if args.field == "gl" else min(args.cpu_sample_log2, 22)
    rng = np.random.default_rng(args.seed)
    tabs = [F.random_table_fast(rng, 1 << n_s) for _ in range(3)]
    for _ in range(args.warmup):
        cpu_prove(orc, F, n_s, tabs)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_prove(orc, F, n_s, tabs)
    dt = (time.perf_counter() - t0) / args.steps
    val = alg_bytes(args.field, n_s) / dt / 1e9
    cores = orc.lib().orc_num_threads()
    sample = (f"each step is one full proof at 2^{n_s} entries per table (bounded sample of the 2^{args.log2_size} "
              "workload; throughput is size-independent on the CPU)")
    print(json.dumps({
        "impl": "reference", "metric": metric_name(args.field), "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "u64" if args.field == "gl" else "u256", "data": "synthetic",
        "config": workload_config(args.field, args.log2_size, args.gpus),
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's Rust prover cannot be built here (no Rust toolchain, dp-crypto not vendored); "
                "this is the C/OpenMP restatement in oracle/ on the host cores",
    }))


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
    field, n = args.field, args.log2_size
    base_dtype = dpb.GL_BASE if field == "gl" else dpb.FR
    fam = dpb.GL_EXT if field == "gl" else dpb.FR
    ctx = dpb.Context(local_rank)
    stream = torch.cuda.ExternalStream(ctx.stream, device=torch.device("cuda", local_rank))

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
    for _ in range(args.steps):
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
    for _ in range(min(args.warmup, 2)):
        step_e2e()
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        st = step_e2e()
    barrier()
    e2e_s = (time.perf_counter() - t0) / args.steps
    words = 2 if field == "gl" else 4
    h2d = world * 3 * (1 << n) * (8 if field == "gl" else 32)
    d2h = (n_global * 4 + n_global + 3) * words * 8

    if world > 1:
        tt = torch.tensor([e2e_s], device="cuda")
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        e2e_s = float(tt.item())
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
        per_entry = NCU_TRAFFIC_BYTES_PER_INPUT_ENTRY.get((field, top["kernel"], top["round"]))
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
                "d2h_bytes_per_step": d2h, "ms_per_step": e2e_s * 1e3},
        # counted by the library on rank 0 over the timed steps (every rank launches the same kernels): one
        # launch per large round, one resident kernel for the last rounds and the final evaluations
        "gpu_launches": launches * world,
        "clocks": clocks,
    }
    if world == 1 and not args.no_cpu_baseline:
        out["cpu_baseline"] = cpu_baseline(field, args.cpu_sample_log2, args.seed)
    print(json.dumps(out))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--log2-size", type=int, default=28)
    ap.add_argument("--field", default="gl", choices=["gl", "fr"])
    ap.add_argument("--cpu-sample-log2", type=int, default=26)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    if args.warmup < 3:
        args.warmup = 3
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
