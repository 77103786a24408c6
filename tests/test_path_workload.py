"""The transformer path workload (deep-prove_b200/workloads.py): the same walk of sumcheck / fold / logup-GKR calls
on the CPU restatement (oracle/path_backend.py) and on the GPU library, compared call by call.

CPU part: the walk itself (call list, shapes, determinism) on the oracle backend.  GPU part: every call's payload
(round messages, points, final evaluations, logup proofs, batching challenges) and the transcript's final state are
equal between the two backends, for BN254 and for Goldilocks, at a reduced shape with every call of the full
graph: embeddings, positions, one block (two normalisations, QKV / QK^T / AV / output / FFN einsums with stacked
heads, attention mask, softmax, GELU, three requantisations, two claim merges), final normalisation, LM head,
argmax range check and linking, the tables' logup proof and the claim batching over every committed polynomial."""
import importlib

import pytest

from oracle.path_backend import OracleBackend


@pytest.fixture(scope="module")
def wl(dpb):
    return importlib.import_module("deep_prove_b200.workloads")


def load_workloads_without_gpu():
    """The walk is plain Python over a backend; it loads without the CUDA library."""
    import importlib.util
    import os
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    name = "_dpb_workloads_cpu"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(root, "deep-prove_b200", "workloads.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


EXPECTED_KINDS = {"einsum": 7, "logup": 10, "linking": 8, "same_poly": 2, "attention_mask": 1, "embeddings": 1,
                  "positional": 1, "argmax_linking": 1, "claim_batching": 1, "state": 1}


def test_walk_on_the_cpu_backend_is_complete_and_deterministic():
    wl = load_workloads_without_gpu()
    a, timer = wl.transformer_path(OracleBackend("fr"), wl.TINY, seed=3)
    b, _ = wl.transformer_path(OracleBackend("fr"), wl.TINY, seed=3)
    assert a == b
    kinds = {}
    for _, kind, payload in a:
        kinds[kind] = kinds.get(kind, 0) + 1
        assert isinstance(payload, bytes) and len(payload) > 0
    assert kinds == EXPECTED_KINDS
    c, _ = wl.transformer_path(OracleBackend("fr"), wl.TINY, seed=4)
    assert [r[0] for r in c] == [r[0] for r in a] and c != a
    # every kind of call was timed
    assert {"einsum", "lookup_witness", "lookup_logup", "lookup_linking", "same_poly",
            "attention_mask", "embeddings", "positional", "argmax_logup", "argmax_linking", "tables_logup",
            "claim_batching"} == set(timer.by_kind)


def test_gpt2_shape_call_sizes():
    """The sizes the GPT-2-small configuration (12 layers, d_model 768, FFN 3072, vocab 50257, 512 tokens) gives the calls: contraction over
    768 -> 10 variables, 3072 -> 12, head dimension 64 -> 6, sequence 512 -> 9; softmax slices of 2^18, GELU 2^21,
    normalisation 2^19, logits 2^25, embeddings 2^26."""
    wl = load_workloads_without_gpu()
    g = wl.GPT2_SMALL
    lg = wl.ceil_log2
    assert (lg(g.d_model), lg(g.ffn), lg(g.head_dim), lg(g.seq)) == (10, 12, 6, 9)
    assert 2 * lg(g.seq) == 18 and lg(g.seq) + lg(g.ffn) == 21 and lg(g.seq) + lg(g.d_model) == 19
    assert lg(g.seq) + lg(g.vocab) == 25 and lg(g.vocab) + lg(g.d_model) == 26


@pytest.mark.gpu
@pytest.mark.parametrize("field", ["fr", "gl"])
@pytest.mark.parametrize("int_tables", [True, False])
def test_gpu_walk_equals_the_cpu_walk(dpb, ctx, wl, field, int_tables):
    """int_tables: the integer tensors stay integers on the device (the default) or become field tables at upload."""
    prover = importlib.import_module("deep_prove_b200.prover")
    want, _ = wl.transformer_path(OracleBackend(field), wl.TINY, seed=7)
    got = wl.run_transformer_path(dpb, prover, ctx, wl.TINY, field=field, seed=7, int_tables=int_tables)
    assert [r[:2] for r in got["records"]] == [r[:2] for r in want]
    for (name, kind, g), (_, _, w) in zip(got["records"], want):
        assert g == w, f"{name} ({kind}) differs from the CPU restatement"
    assert got["tokens_per_s"] > 0 and set(got["by_kind"]) == set(got["calls"])


def test_variant_walks_on_the_cpu_backend():
    """The gated / rotary / grouped-query block (Gemma- and Llama-style) and the dense network: the calls each adds."""
    wl = load_workloads_without_gpu()
    rec, timer = wl.transformer_path(OracleBackend("fr"), wl.TINY_GLU_ROPE, seed=3)
    names = [r[0] for r in rec]
    assert "block0.rope_q" in names and "block0.rope_k" in names and "block0.ffn_gate" in names
    assert "block0.glu.linking" in names and "positional" not in names
    assert "rope" in timer.by_kind and timer.calls["rope"] == 2
    rec, timer = wl.mlp_path(OracleBackend("gl"), wl.TINY_MLP, seed=3)
    assert [r[1] for r in rec] == ["einsum", "logup", "linking", "einsum", "logup", "argmax_linking", "logup",
                                   "claim_batching", "state"]


@pytest.mark.gpu
@pytest.mark.parametrize("field", ["fr", "gl"])
@pytest.mark.parametrize("shape", ["TINY_GLU_ROPE", "TINY_MLP"])
def test_gpu_variant_walks_equal_the_cpu_walks(dpb, ctx, wl, field, shape):
    """Gated FFN (GLU linking), rotary positions on Q and K, grouped-query attention; the dense network."""
    prover = importlib.import_module("deep_prove_b200.prover")
    shape = getattr(wl, shape)
    if isinstance(shape, wl.MlpShape):
        want, _ = wl.mlp_path(OracleBackend(field), shape, seed=11)
    else:
        want, _ = wl.transformer_path(OracleBackend(field), shape, seed=11)
    got = wl.run_transformer_path(dpb, prover, ctx, shape, field=field, seed=11)
    assert [r[:2] for r in got["records"]] == [r[:2] for r in want]
    for (name, kind, g), (_, _, w) in zip(got["records"], want):
        assert g == w, f"{name} ({kind}) differs from the CPU restatement"


@pytest.mark.gpu
@pytest.mark.parametrize("field", ["fr", "gl"])
def test_rope_permuted_eq(dpb, ctx, field):
    """dpb_rope_permuted_eq against the restated RopeLayout::permuted_eq_poly, both layouts."""
    import numpy as np
    from oracle import oracle as orc
    F = orc.FrField if field == "fr" else orc.GlField
    fam = dpb.FR if field == "fr" else dpb.GL_BASE
    rng = np.random.default_rng(5)
    point = [F.random_scalar(rng) for _ in range(7)]
    pt = np.ascontiguousarray(orc.scalars_to_array(F, point), dtype=np.uint64)
    eq = ctx.eq_table(fam, pt)
    want_eq = orc.eq_evals(F, point)
    for layout, row in ((0, 0), (1, 16), (1, 128)):
        got = dpb.rope_permuted_eq(ctx, eq, layout, row).to_host()
        want = np.asarray(orc.rope_permuted_eq(F, want_eq, layout, row), dtype=np.uint64)
        assert np.array_equal(got.reshape(want.shape), want)
    with pytest.raises(dpb.DpbError):
        dpb.rope_permuted_eq(ctx, eq, 1, 6)  # does not divide 128


@pytest.mark.gpu
def test_gpu_walk_two_blocks_without_head(dpb, ctx, wl):
    """Two blocks, nothing after them: the counters and kept witness columns of a longer walk."""
    prover = importlib.import_module("deep_prove_b200.prover")
    want, _ = wl.transformer_path(OracleBackend("fr"), wl.TINY, seed=9, blocks=2, with_final=False)
    got = wl.run_transformer_path(dpb, prover, ctx, wl.TINY, field="fr", seed=9, blocks=2, with_final=False)
    assert [r for r in got["records"]] == want


@pytest.mark.gpu
def test_gpu_walk_with_witness_commitments(dpb, ctx, wl):
    """The walk with every lookup layer's witness columns committed (one G1 multi-scalar multiplication per chunk):
    the commitments equal the CPU restatement's, which gets each of them from ONE scalar multiplication because the
    synthetic bases are consecutive multiples of the generator."""
    prover = importlib.import_module("deep_prove_b200.prover")
    want, _ = wl.transformer_path(OracleBackend("fr"), wl.TINY, seed=5, with_final=False, with_commit=True)
    got = wl.run_transformer_path(dpb, prover, ctx, wl.TINY, field="fr", seed=5, with_final=False, with_commit=True)
    assert got["records"] == want
    assert sum(1 for r in want if r[1] == "commit") == 7 and got["commit_seconds"] > 0
