"""The headers as a C compiler sees them: a small C program is compiled with gcc against include/*.h and linked with
libdpb.so.  It reports the size and field offsets of every struct that crosses the boundary, which must agree with
the ctypes definitions the Python face uses (a drift between header and binding would otherwise go unseen), and on
a GPU it proves one six-variable sumcheck through the C ABI alone and prints the round messages, which must equal
the oracle's."""
import ctypes
import importlib
import json
import os
import subprocess
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

C_SOURCE = r'''
#include <stddef.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include "dpb.h"
#include "dpb_prover.h"

#define SZ(T) printf("\"%s\": {\"size\": %zu", #T, sizeof(T))
#define OFF(T, f) printf(", \"%s\": %zu", #f, offsetof(T, f))
#define END() printf("}")

static void layouts(void) {
    printf("{");
    SZ(dpb_term); OFF(dpb_term, coeff); OFF(dpb_term, n_factors); OFF(dpb_term, idx); END(); printf(", ");
    SZ(dpb_profile_entry); OFF(dpb_profile_entry, kernel); OFF(dpb_profile_entry, round);
    OFF(dpb_profile_entry, launches); OFF(dpb_profile_entry, total_ms); OFF(dpb_profile_entry, alg_bytes_per_launch);
    END(); printf(", ");
    SZ(dpb_chunking_info); OFF(dpb_chunking_info, offset); OFF(dpb_chunking_info, value_chunk_offset);
    OFF(dpb_chunking_info, shifted_chunk_multiplier); OFF(dpb_chunking_info, top_zeroing_chunk_offset); END(); printf(", ");
    SZ(dpb_expr_node); OFF(dpb_expr_node, op); OFF(dpb_expr_node, a); OFF(dpb_expr_node, b); OFF(dpb_expr_node, c0);
    OFF(dpb_expr_node, c1); END(); printf(", ");
    SZ(dpb_committed_poly); OFF(dpb_committed_poly, chunks); OFF(dpb_committed_poly, n_chunks);
    OFF(dpb_committed_poly, n_claims); OFF(dpb_committed_poly, claim_points); OFF(dpb_committed_poly, claim_evals);
    END(); printf(", ");
    SZ(dpb_logup_input); OFF(dpb_logup_input, kind); OFF(dpb_logup_input, columns); OFF(dpb_logup_input, n_columns);
    OFF(dpb_logup_input, columns_per_instance); OFF(dpb_logup_input, multiplicities);
    OFF(dpb_logup_input, constant_challenge); OFF(dpb_logup_input, column_separation_challenge); END(); printf(", ");
    SZ(dpb_einsum_operand); OFF(dpb_einsum_operand, tensor); OFF(dpb_einsum_operand, tensor_on_device);
    OFF(dpb_einsum_operand, rank); OFF(dpb_einsum_operand, shape); OFF(dpb_einsum_operand, axis_kind);
    OFF(dpb_einsum_operand, axis_points); OFF(dpb_einsum_operand, axis_point_len); END();
    printf("}\n");
}

/* One sumcheck of f*g over 2^6 Goldilocks base entries, challenges fixed to 3 + 5X: every call checked. */
static int prove(void) {
    dpb_ctx* ctx = NULL;
    if (dpb_init(0, &ctx) != DPB_OK) { fprintf(stderr, "init: %s\n", dpb_last_error()); return 2; }
    unsigned long long f[64], g[64];
    for (int i = 0; i < 64; i++) { f[i] = 1000003ull * (i + 1) + 7; g[i] = 0xFFFFFFFF00000001ull - 1 - 17ull * i; }
    dpb_mle *mf = NULL, *mg = NULL;
    if (dpb_mle_from_host(ctx, DPB_GL_BASE, f, 64, DPB_FORM_NATIVE, &mf) != DPB_OK ||
        dpb_mle_from_host(ctx, DPB_GL_BASE, g, 64, DPB_FORM_NATIVE, &mg) != DPB_OK) {
        fprintf(stderr, "upload: %s\n", dpb_last_error()); return 2;
    }
    dpb_term term;
    memset(&term, 0, sizeof term);
    term.coeff[0] = 1;  /* one in the Goldilocks extension: (1, 0) */
    term.n_factors = 2;
    term.idx[0] = 0; term.idx[1] = 1;
    dpb_mle* tabs[2] = {mf, mg};
    dpb_sc* sc = NULL;
    if (dpb_sumcheck_begin(ctx, 6, tabs, 2, &term, 1, &sc) != DPB_OK) { fprintf(stderr, "begin: %s\n", dpb_last_error()); return 2; }
    unsigned long long r[2] = {3, 5}, ev[3 * 2], fin[2 * 2];
    printf("[");
    for (int i = 0; i < 6; i++) {
        unsigned n = 0;
        if (dpb_sumcheck_round(sc, i ? r : NULL, ev, &n) != DPB_OK || n != 3) { fprintf(stderr, "round: %s\n", dpb_last_error()); return 2; }
        for (int x = 0; x < 6; x++) printf("%s%llu", (i || x) ? ", " : "", ev[x]);
    }
    if (dpb_sumcheck_finish(sc, r, fin) != DPB_OK) { fprintf(stderr, "finish: %s\n", dpb_last_error()); return 2; }
    for (int x = 0; x < 4; x++) printf(", %llu", fin[x]);
    printf("]\n");
    dpb_sumcheck_free(sc);
    dpb_mle_free(mf); dpb_mle_free(mg);
    dpb_shutdown(ctx);
    return 0;
}

int main(int argc, char** argv) {
    if (argc > 1 && strcmp(argv[1], "prove") == 0) return prove();
    layouts();
    return 0;
}
'''


@pytest.fixture(scope="module")
def c_program(tmp_path_factory):
    d = tmp_path_factory.mktemp("abi_c")
    src, exe = d / "abi.c", d / "abi"
    src.write_text(C_SOURCE)
    lib_dir = os.path.join(ROOT, "deep-prove_b200")
    cmd = ["gcc", "-std=c99", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"), str(src), "-o", str(exe),
           "-L", lib_dir, "-ldpb", f"-Wl,-rpath,{lib_dir}", "-Wl,--allow-shlib-undefined"]
    r = subprocess.run(cmd, capture_output=True, text=True)
    assert r.returncode == 0, r.stdout + r.stderr
    return str(exe)


def run(exe, *args):
    env = dict(os.environ)
    env["LD_LIBRARY_PATH"] = "/usr/local/cuda/lib64:" + env.get("LD_LIBRARY_PATH", "")
    r = subprocess.run([exe, *args], capture_output=True, text=True, env=env, timeout=120)
    assert r.returncode == 0, r.stdout + r.stderr
    return json.loads(r.stdout)


def ctypes_layout(T, fields):
    out = {"size": ctypes.sizeof(T)}
    for f in fields:
        out[f] = getattr(T, f).offset
    return out


def test_headers_compile_as_c_and_layouts_match_the_bindings(dpb, c_program):
    prover = importlib.import_module("deep_prove_b200.prover")
    got = run(c_program)
    assert got["dpb_term"] == ctypes_layout(dpb.Term, ["coeff", "n_factors", "idx"])
    assert got["dpb_profile_entry"] == ctypes_layout(dpb.ProfileEntry, ["kernel", "round", "launches", "total_ms",
                                                                        "alg_bytes_per_launch"])
    assert got["dpb_chunking_info"] == ctypes_layout(dpb.ChunkingInfo, ["offset", "value_chunk_offset",
                                                                        "shifted_chunk_multiplier",
                                                                        "top_zeroing_chunk_offset"])
    assert got["dpb_expr_node"] == ctypes_layout(prover.ExprNode, ["op", "a", "b", "c0", "c1"])
    assert got["dpb_committed_poly"] == ctypes_layout(prover.CommittedPolyStruct, ["chunks", "n_chunks", "n_claims",
                                                                                   "claim_points", "claim_evals"])
    assert got["dpb_logup_input"] == ctypes_layout(prover.LogupInputStruct, ["kind", "columns", "n_columns",
                                                                             "columns_per_instance", "multiplicities",
                                                                             "constant_challenge",
                                                                             "column_separation_challenge"])
    assert got["dpb_einsum_operand"] == ctypes_layout(prover.EinsumOperandStruct, ["tensor", "tensor_on_device", "rank",
                                                                                   "shape", "axis_kind", "axis_points",
                                                                                   "axis_point_len"])


@pytest.mark.gpu
def test_a_sumcheck_through_the_c_abi_alone(c_program):
    """No Python between the caller and the library: the C program's round messages equal the oracle's."""
    from oracle import oracle as orc
    F = orc.GlField
    got = run(c_program, "prove")
    f = np.array([1000003 * (i + 1) + 7 for i in range(64)], dtype=np.uint64)
    g = np.array([orc.GL_MOD - 1 - 17 * i for i in range(64)], dtype=np.uint64)
    r = (3, 5)
    tabs, want = [f, g], []
    for i in range(6):
        want += [c for e in orc.sumcheck_round(F, 6 - i, tabs, {(0, 1): F.one}, 2) for c in e]
        tabs = [orc.fold_low(F, t, r) for t in tabs]
    want += [c for t in tabs for c in orc.array_to_scalars(F, t)[0]]
    assert got == want
