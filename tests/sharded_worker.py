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


def logup_batch_case(F, n, seed, world):
    """A batch of lookups to spread over `world` ranks: per rank two two-column instances of 2^n rows and one
    single-column instance of 2^(n-2) rows.  Returns per rank its list of (columns, columns per instance, constant,
    separator) and the same instances in the order of the whole batch (local instance i of rank g at i * world + g)."""
    rng = np.random.default_rng(seed)
    cst = [F.random_scalar(rng), F.random_scalar(rng)]
    sep = [F.random_scalar(rng), F.random_scalar(rng)]
    per_rank = []
    for _ in range(world):
        two = [rng.integers(-(1 << 11), 1 << 11, size=1 << n, dtype=np.int64) for _ in range(4)]
        one = [rng.integers(0, 1 << 16, size=1 << (n - 2), dtype=np.int64)]
        per_rank.append([(two, 2, cst[0], sep[0]), (one, 1, cst[1], sep[1])])
    whole = []
    for cols_i, (cpi, c, s) in ((0, (2, cst[0], sep[0])), (1, (1, cst[1], sep[1]))):
        merged = []
        n_inst = len(per_rank[0][cols_i][0]) // cpi
        for i in range(n_inst):
            for g in range(world):
                merged += per_rank[g][cols_i][0][i * cpi:(i + 1) * cpi]
        whole.append((merged, cpi, c, s))
    return per_rank, whole


def run_gpu_logup(field, n, seed, rank, world, out):
    """dpb_logup_batch_prove_partial: every rank proves its own instances; all ranks return the whole batch's proof."""
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
    per_rank, whole = logup_batch_case(F, n, seed, world)
    base = dpb.FR if field == "fr" else dpb.GL_BASE
    fam = dpb.FR if field == "fr" else dpb.GL_EXT
    S = lambda v: orc.scalars_to_array(F, [v])

    def inputs(groups):
        return [prover.LogUpInput.new_lookup([ctx.upload_i64(c, base) for c in cols], S(c0), S(s0), cpi)
                for cols, cpi, c0, s0 in groups]
    got = prover.new_batch_multiple_sizes_prove(ctx, inputs(per_rank[rank]), prover.Blake3Transcript(fam), partial=True)
    res = dict(proof=got.hex())
    if rank == 0:
        # the same batch on this GPU alone
        res["single_gpu_equal"] = prover.new_batch_multiple_sizes_prove(ctx, inputs(whole), prover.Blake3Transcript(fam)) == got
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


def run_cpu_logup(field, n, seed, rank, world, out):
    """The protocol of dpb_logup_batch_prove_partial emulated with the CPU oracle over a gloo group: every rank
    holds its own instances (trees, layer tables), computes its part of each round's sums, and the ranks exchange
    the trees' outputs, the per-round sums and each layer's final evaluations; identical transcripts."""
    import torch
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    F = orc.FIELDS[field]
    per_rank, _ = logup_batch_case(F, n, seed, world)
    inputs = [orc.LogUpInput(F, 0, [F.table_from_i64(c) for c in cols], c0, s0, columns_per_instance=cpi)
              for cols, cpi, c0, s0 in per_rank[rank]]

    def gather(scalars):
        """rank-ordered lists of every rank's scalars"""
        arr = np.ascontiguousarray(orc.scalars_to_array(F, list(scalars)), dtype=np.uint64)
        t = torch.from_numpy(arr.view(np.int64).copy())
        outs = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(outs, t)
        return [orc.array_to_scalars(F, o.numpy().view(np.uint64).reshape(arr.shape)) for o in outs]

    T = orc.Transcript(F)
    circuits = [c for i in inputs for c in i.make_new_circuits()]
    total_layers = max(c.num_vars() for c in circuits)
    sizes = sorted({c.num_vars() for c in circuits}, reverse=True)
    by_size = {s: [c for c in circuits if c.num_vars() == s] for s in sizes}
    all_out = gather([e for c in circuits for e in c.outputs()])
    circuit_outputs = [all_out[q][4 * i:4 * i + 4] for i in range(len(circuits)) for q in range(world)]
    T.append_scalars([F.from_int(len(circuits) * world)])
    for o in circuit_outputs:
        T.append_scalars(o)
    rho = T.append_and_sample(b"initial_batching")
    alpha = T.append_and_sample(b"initial_alpha")
    lam = T.append_and_sample(b"initial_lambda")
    point = [rho]
    sumcheck_proofs, round_evaluations = [], []
    for v in range(1, total_layers + 1):
        remaining = total_layers - (v - 1)
        joining = [e for i, c in enumerate(circuits) if c.num_vars() == remaining
                   for q in range(world) for e in circuit_outputs[i * world + q]]
        wit_evals = (round_evaluations[-1] if round_evaluations else []) + joining
        tables, eq_tables, group_exprs, counts = [], [], [], []
        claim_expr = orc.Expr.const(F.zero)
        layer_count, wit_off = 0, 0
        for size in sizes:
            if size < remaining:
                continue
            mult = orc.Expr.const(F.from_int(1 << (total_layers - size)))
            layer_vars = size - remaining + 1
            group = orc.Expr.const(F.zero)
            for c in by_size[size]:
                for q in range(world):
                    sc, cl, nw = c.layer_exprs(layer_vars, layer_count, wit_off)
                    layer_count += 1
                    claim_expr = claim_expr + mult * cl
                    if q != rank:
                        continue
                    tables += c.layer_tables(layer_vars)
                    wit_off += nw
                    group = group + sc
                counts.append(nw)
            eq_tables.append(orc.eq_evals(F, point[len(point) - layer_vars:]))
            group_exprs.append(group)
        T.append_scalars([orc.eval_expr(F, claim_expr, wit_evals, [alpha, lam, rho])])
        full = orc.Expr.const(F.zero)
        for i, g in enumerate(group_exprs):
            full = full + g * orc.Expr.wit(wit_off + i)
        terms = orc.expr_to_terms(F, full, [alpha, lam])
        # the sumcheck over this rank's terms, round sums added over the ranks
        d = orc.terms_degree(terms)
        cur = tables + eq_tables
        nv = [orc.table_len(t).bit_length() - 1 for t in cur]
        T.append_scalars([F.from_int(v), F.from_int(d)])
        proof, pt = [], []
        for i in range(v):
            left = v - i
            evals = [F.zero] * (d + 1)
            for part in gather(orc.sumcheck_round(F, left, cur, terms, d)):
                evals = [F.add(a, b) for a, b in zip(evals, part)]
            T.append_scalars(evals)
            r = T.append_and_sample(orc.ROUND_LABEL)
            proof.append(evals)
            pt.append(r)
            for j in range(len(cur)):
                if nv[j] >= left:
                    cur[j] = orc.fold_low(F, cur[j], r)
                    nv[j] -= 1
        finals = [orc.array_to_scalars(F, orc._widen(F, t))[0] for t in cur]
        parts = gather(finals[:wit_off])
        evals, at = [], 0
        for nw in counts:
            for q in range(world):
                evals += parts[q][at:at + nw]
            at += nw
        rho = T.append_and_sample(b"logup_batching")
        if v != total_layers:
            alpha = T.append_and_sample(b"logup_alpha")
            lam = T.append_and_sample(b"logup_lambda")
        point = pt + [rho]
        sumcheck_proofs.append(proof)
        round_evaluations.append(evals)
    output_claims, ncols, nvars, skip = [], [], [], 0
    last = round_evaluations[-1]
    for c in circuits:
        for q in range(world):
            k = c.final_eval_count()
            ev = c.combine_final_evals(last[skip:skip + k], rho)
            skip += k
            output_claims += [(point[len(point) - (c.num_vars() + 1):], e) for e in ev]
            ncols.append(len(c.columns))
            nvars.append(c.num_vars())
    got = dict(sumcheck_proofs=sumcheck_proofs, round_evaluations=round_evaluations, output_claims=output_claims,
               circuit_outputs=circuit_outputs, proof_type=0, num_vars_per_instance=nvars,
               num_denominator_columns_per_instance=ncols)
    with open(f"{out}.{rank}.json", "w") as f:
        json.dump(dict(proof=orc.serialize_logup_proof(F, got).hex()), f)
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    mode, field, n, seed, rank, world, out = sys.argv[1:8]
    {"gpu": run_gpu, "gpu_eq": run_gpu_eq, "gpu_logup": run_gpu_logup, "cpu": run_cpu,
     "cpu_logup": run_cpu_logup}[mode](field, int(n), int(seed), int(rank), int(world), out)
