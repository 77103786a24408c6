"""Child process of the multi-rank tests (one process per rank).

mode "gpu":  the library's sharded sumcheck on GPU `rank` over its own NCCL
             communicator; the 128-byte id travels through a file.
mode "cpu":  the same sharding protocol emulated with the CPU oracle over a
             torch.distributed gloo group — rounds on the rank's shard, partial
             evaluations all-gathered and added mod p, identical transcripts,
             one-entry shards gathered for the tail.  Covers the host-side logic
             of the N > 1 path without GPUs.
Each rank writes its proof to <out>.<rank>.json; the parent test compares them
with the single-process oracle proof of the whole tables.
"""
import json
import os
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from oracle import oracle as orc  # noqa: E402


def full_tables(F, n, seed, k=3):
    rng = np.random.default_rng(seed)
    return [F.random_table_fast(rng, 1 << n) for _ in range(k)]


def shard(t, rank, world):
    m = t.shape[0] // world
    return np.ascontiguousarray(t[rank * m:(rank + 1) * m])


def run_gpu(field, n, seed, rank, world, out):
    from tests.conftest import load_package
    import importlib
    dpb = load_package()
    prover = importlib.import_module("deep_prove_b200.prover")
    F = orc.FIELDS[field]
    ctx = dpb.Context(rank)
    id_path = out + ".id"
    if rank == 0:
        uid = dpb.comm_unique_id()
        with open(id_path + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(id_path + ".tmp", id_path)
    else:
        t0 = time.time()
        while not os.path.exists(id_path):
            if time.time() - t0 > 60:
                raise SystemExit("rank 0 never published the communicator id")
            time.sleep(0.01)
        with open(id_path, "rb") as f:
            uid = f.read()
    ctx.comm_init(uid, rank, world)
    tabs = [shard(t, rank, world) for t in full_tables(F, n, seed)]
    base = dpb.FR if field == "fr" else dpb.GL_BASE
    fam = dpb.FR if field == "fr" else dpb.GL_EXT
    mles = [ctx.upload(t, base) for t in tabs]
    terms = dpb.make_terms([(F.one, [0, 1, 2])], F.to_native)
    st = prover.IOPProverState.prove(ctx, n, mles, terms, prover.Blake3Transcript(fam), sharded=True)
    flat = lambda a: orc.serialize_scalars(F, orc.array_to_scalars(F, np.asarray(a).reshape(-1, F.elem_words))).hex()
    res = dict(proof=flat(st.proof), point=flat(st.collect_raw_challenges()),
               finals=flat(st.get_mle_flatten_final_evaluations()), shared_exchange=ctx.comm_shared_exchange())
    ctx.comm_free()
    ctx.close()
    with open(f"{out}.{rank}.json", "w") as f:
        json.dump(res, f)


def linking_case(F, n, seed):
    """Tables and terms of the shape of a linking / hadamard sumcheck: an eq table as a factor of every term."""
    rng = np.random.default_rng(seed + 1000)
    tabs = [F.random_table_fast(rng, 1 << n) for _ in range(3)]
    point = [F.random_scalar(rng) for _ in range(n)]
    c = [F.random_scalar(rng) for _ in range(2)]
    terms = {(3, 0, 1): F.one, (3, 1, 2, 2): c[0], (3, 0): c[1]}
    return tabs, point, terms


def run_gpu_eq(field, n, seed, rank, world, out):
    """The library's sharded sumcheck over a term list with an eq factor; every rank builds only its shard of the
    eq table (dpb_eq_table_shard)."""
    from tests.conftest import load_package
    import importlib
    dpb = load_package()
    prover = importlib.import_module("deep_prove_b200.prover")
    F = orc.FIELDS[field]
    ctx = dpb.Context(rank)
    id_path = out + ".id"
    if rank == 0:
        uid = dpb.comm_unique_id()
        with open(id_path + ".tmp", "wb") as f:
            f.write(uid)
        os.replace(id_path + ".tmp", id_path)
    else:
        t0 = time.time()
        while not os.path.exists(id_path):
            if time.time() - t0 > 60:
                raise SystemExit("rank 0 never published the communicator id")
            time.sleep(0.01)
        with open(id_path, "rb") as f:
            uid = f.read()
    ctx.comm_init(uid, rank, world)
    tabs, point, terms = linking_case(F, n, seed)
    base = dpb.FR if field == "fr" else dpb.GL_BASE
    fam = dpb.FR if field == "fr" else dpb.GL_EXT
    mles = [ctx.upload(shard(t, rank, world), base) for t in tabs]
    eq = ctx.eq_table_shard(fam, orc.scalars_to_array(F, point))
    want_eq = shard(orc.eq_evals(F, point), rank, world)
    assert (eq.to_host() == want_eq).all(), "eq shard differs from the slice of the whole eq table"
    arr = dpb.make_terms([(c, list(m)) for m, c in sorted(terms.items())], F.to_native)
    st = prover.IOPProverState.prove(ctx, n, mles + [eq], arr, prover.Blake3Transcript(fam), sharded=True)
    flat = lambda a: orc.serialize_scalars(F, orc.array_to_scalars(F, np.asarray(a).reshape(-1, F.elem_words))).hex()
    res = dict(proof=flat(st.proof), point=flat(st.collect_raw_challenges()),
               finals=flat(st.get_mle_flatten_final_evaluations()))
    ctx.comm_free()
    ctx.close()
    with open(f"{out}.{rank}.json", "w") as f:
        json.dump(res, f)


def run_cpu(field, n, seed, rank, world, out):
    import torch
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    F = orc.FIELDS[field]
    c = world.bit_length() - 1
    n_loc = n - c
    cur = [shard(t, rank, world) for t in full_tables(F, n, seed)]
    terms = {(0, 1, 2): F.one}
    d = 3
    tr = orc.Transcript(F)
    tr.append_scalars([F.from_int(n), F.from_int(d)])
    proof, point = [], []

    def exchange(arr):
        t = torch.from_numpy(np.ascontiguousarray(arr).view(np.int64).copy())
        outs = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(outs, t)
        return [o.numpy().view(np.uint64).reshape(arr.shape) for o in outs]

    for i in range(n_loc):
        part = orc.scalars_to_array(F, orc.sumcheck_round(F, n_loc - i, cur, terms, d))
        parts = [orc.array_to_scalars(F, p) for p in exchange(part)]
        evals = [F.zero] * (d + 1)
        for p in parts:
            evals = [F.add(a, b) for a, b in zip(evals, p)]
        tr.append_scalars(evals)
        r = tr.append_and_sample(orc.ROUND_LABEL)
        proof.append(evals)
        point.append(r)
        cur = [orc.fold_low(F, t, r) for t in cur]
    # every table is down to one entry per rank: gather them into 2^c-entry tables
    mine = np.concatenate([orc._widen(F, t) for t in cur], axis=0)
    gathered = exchange(mine)
    tail = [np.stack([g[j] for g in gathered]) for j in range(len(cur))]
    for i in range(c):
        evals = orc.sumcheck_round(F, c - i, tail, terms, d)
        tr.append_scalars(evals)
        r = tr.append_and_sample(orc.ROUND_LABEL)
        proof.append(evals)
        point.append(r)
        tail = [orc.fold_low(F, t, r) for t in tail]
    finals = [orc.array_to_scalars(F, t)[0] for t in tail]
    hx = lambda v: orc.serialize_scalars(F, v).hex()
    with open(f"{out}.{rank}.json", "w") as f:
        json.dump(dict(proof=orc.serialize_sumcheck_proof(F, proof).hex(), point=hx(point), finals=hx(finals)), f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    mode, field, n, seed, rank, world, out = sys.argv[1:8]
    {"gpu": run_gpu, "gpu_eq": run_gpu_eq, "cpu": run_cpu}[mode](field, int(n), int(seed), int(rank), int(world), out)
