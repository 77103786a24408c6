"""Multi-rank sumcheck: the hypercube is sharded on its top log2(G) variables,
each rank folds its shard locally and contributes its partial round
evaluations through an all-gather; all ranks must produce the proof a single
process produces for the whole tables."""
import json
import os
import socket
import subprocess
import sys
import tempfile

import pytest

from oracle import oracle as orc
from tests import sharded_worker as W

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def launch(mode, field, n, seed, world, extra_env=None):
    tmp = tempfile.mkdtemp()
    out = os.path.join(tmp, "res")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(free_port()), OMP_NUM_THREADS="2",
               NCCL_NVLS_ENABLE="0")
    env.update(extra_env or {})
    procs = [subprocess.Popen([sys.executable, os.path.join(ROOT, "tests", "sharded_worker.py"), mode, field, str(n),
                               str(seed), str(r), str(world), out], env=env, cwd=ROOT,
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT) for r in range(world)]
    logs = []
    for p in procs:
        try:
            o, _ = p.communicate(timeout=300)
        except subprocess.TimeoutExpired:
            p.kill()
            o, _ = p.communicate()
        logs.append(o.decode(errors="replace"))
    for r, p in enumerate(procs):
        assert p.returncode == 0, f"rank {r} failed:\n{logs[r][-3000:]}"
    return [json.load(open(f"{out}.{r}.json")) for r in range(world)]


def oracle_proof(F, n, seed):
    tabs = W.full_tables(F, n, seed)
    proof, point, finals = orc.sumcheck_prove(F, n, tabs, {(0, 1, 2): F.one}, orc.Transcript(F))
    hx = lambda v: orc.serialize_scalars(F, v).hex()
    return dict(proof=orc.serialize_sumcheck_proof(F, proof).hex(), point=hx(point), finals=hx(finals))


@pytest.mark.parametrize("field", ["gl", "fr"])
@pytest.mark.parametrize("world,n", [(2, 7), (4, 6)])
def test_sharding_protocol_on_cpu_gloo(field, world, n):
    """world_size > 1 on CPU: gloo ranks run the sharding protocol with the oracle."""
    want = oracle_proof(orc.FIELDS[field], n, 11)
    for got in launch("cpu", field, n, 11, world):
        assert got == want


@pytest.mark.gpu
@pytest.mark.parametrize("field", ["gl", "fr"])
@pytest.mark.parametrize("n", [4, 14])
@pytest.mark.parametrize("exchange", ["shared", "nccl"])
def test_sharded_sumcheck_on_gpus(field, n, exchange):
    """The library's sharded path on as many GPUs as the box has (2, 4 or 8), with the per-round sums exchanged
    through the shared host segment and through ncclAllGather."""
    import torch
    g = torch.cuda.device_count()
    world = 8 if g >= 8 else 4 if g >= 4 else 2 if g >= 2 else 0
    if world == 0:
        pytest.skip("needs at least 2 GPUs")
    want = oracle_proof(orc.FIELDS[field], n, 12)
    env = {"DPB_NO_SHARED_EXCHANGE": "1"} if exchange == "nccl" else {}
    for got in launch("gpu", field, n, 12, world, env):
        shared = got.pop("shared_exchange")
        if exchange == "nccl":
            assert not shared
        assert got == want


@pytest.mark.gpu
@pytest.mark.parametrize("field", ["gl", "fr"])
@pytest.mark.parametrize("n", [5, 13])
def test_sharded_sumcheck_with_an_eq_factor_on_gpus(field, n):
    """A term list of the linking / hadamard shape (every term led by an eq table, a squared factor, coefficients)
    sharded over the GPUs of the box: each rank builds only its shard of the eq table (dpb_eq_table_shard, checked
    against the slice of the whole table) and all ranks produce the oracle's proof of the whole tables."""
    import torch
    g = torch.cuda.device_count()
    world = 8 if g >= 8 else 4 if g >= 4 else 2 if g >= 2 else 0
    if world == 0:
        pytest.skip("needs at least 2 GPUs")
    F = orc.FIELDS[field]
    tabs, point, terms = W.linking_case(F, n, 21)
    proof, pt, finals = orc.sumcheck_prove(F, n, tabs + [orc.eq_evals(F, point)], terms, orc.Transcript(F))
    hx = lambda v: orc.serialize_scalars(F, v).hex()
    want = dict(proof=orc.serialize_sumcheck_proof(F, proof).hex(), point=hx(pt), finals=hx(finals))
    for got in launch("gpu_eq", field, n, 21, world):
        assert got == want


@pytest.mark.gpu
@pytest.mark.parametrize("field", ["gl", "fr"])
@pytest.mark.parametrize("n", [6, 16])
def test_logup_batch_spread_over_gpus(field, n):
    """dpb_logup_batch_prove_partial: the instances of a batch (two sizes, one- and two-column lookups) spread over
    the GPUs of the box.  Every rank returns the same bytes, equal to the oracle's proof of the whole batch and to
    the single-GPU proof; n = 16 reaches the segmented one-pass rounds, n = 6 runs in the resident kernel's range
    (which partial sumchecks do not use)."""
    import torch
    g = torch.cuda.device_count()
    world = 8 if g >= 8 else 4 if g >= 4 else 2 if g >= 2 else 0
    if world == 0:
        pytest.skip("needs at least 2 GPUs")
    F = orc.FIELDS[field]
    _, whole = W.logup_batch_case(F, n, 31, world)
    o_in = [orc.LogUpInput(F, 0, [F.table_from_i64(c) for c in cols], c0, s0, columns_per_instance=cpi)
            for cols, cpi, c0, s0 in whole]
    want = orc.serialize_logup_proof(F, orc.logup_batch_prove(F, o_in, orc.Transcript(F))).hex()
    for r, got in enumerate(launch("gpu_logup", field, n, 31, world)):
        assert got["proof"] == want, f"rank {r}"
        if r == 0:
            assert got["single_gpu_equal"]


@pytest.mark.parametrize("field", ["gl", "fr"])
@pytest.mark.parametrize("world", [2, 4])
def test_logup_batch_spread_protocol_on_cpu_gloo(field, world):
    """The protocol of the instance-spread logup prover with gloo ranks on CPU: every rank ends with the oracle's
    proof of the whole batch (local instance i of rank g at position i * world + g)."""
    F = orc.FIELDS[field]
    _, whole = W.logup_batch_case(F, 5, 41, world)
    o_in = [orc.LogUpInput(F, 0, [F.table_from_i64(c) for c in cols], c0, s0, columns_per_instance=cpi)
            for cols, cpi, c0, s0 in whole]
    want = orc.serialize_logup_proof(F, orc.logup_batch_prove(F, o_in, orc.Transcript(F))).hex()
    for r, got in enumerate(launch("cpu_logup", field, 5, 41, world)):
        assert got["proof"] == want, f"rank {r}"
