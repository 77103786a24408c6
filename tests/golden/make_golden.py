"""Generates the committed fixtures in this directory.

    python -m tests.golden.make_golden          (from the repository root)

blake3_kat.json  BLAKE3 digests of the specification's test-input pattern
                 (byte i = i mod 251) at several lengths, produced with the
                 `blake3` Python module (the reference implementation's
                 binding) — the known answers both BLAKE3 implementations in
                 this repository are checked against.
oracle_fr.json,  outputs of the CPU oracle on seeded inputs (hex of canonical
oracle_gl.json   encodings).  The reference itself cannot run here and holds no
                 golden proof, so these freeze the oracle — already pinned by
                 the reference's algebraic tests — as the byte-level target of
                 the CUDA path.
"""
import json
import os

import numpy as np

from oracle import oracle as orc

HERE = os.path.dirname(os.path.abspath(__file__))


def golden_inputs(F, name):
    """Seeded inputs shared by the generator and the GPU parity tests."""
    seed = {"prod3": 101, "hadamard": 102, "logup_lookup": 103, "logup_table": 104, "fix": 105,
            "mixed": 106, "claims": 107, "lookup": 108, "einsum": 109}[name]
    rng = np.random.default_rng(seed)
    if name == "prod3":
        n = 6
        return dict(n=n, tables=[F.random_table(rng, 1 << n) for _ in range(3)])
    if name == "hadamard":
        n = 5
        return dict(n=n, v1=F.random_table(rng, 1 << n), v2=F.random_table(rng, 1 << n),
                    point=[F.random_scalar(rng) for _ in range(n)])
    if name == "logup_lookup":
        out = []
        for m in (5, 4, 3):
            cols = [F.random_table(rng, 1 << m) for _ in range(2)]
            out.append(dict(columns=cols, constant=F.random_scalar(rng), sep=F.random_scalar(rng), cpi=1))
        return out
    if name == "logup_table":
        m = 4
        return dict(columns=[F.random_table(rng, 1 << m) for _ in range(2)],
                    mult=F.table_from_ints([int(x) for x in rng.integers(0, 5, size=1 << m)]),
                    constant=F.random_scalar(rng), sep=F.random_scalar(rng))
    if name == "fix":
        n = 7
        return dict(n=n, table=F.random_table(rng, 1 << n), point=[F.random_scalar(rng) for _ in range(n)])
    if name == "mixed":
        # tables of different sizes and a term list with coefficients (generic path)
        n = 6
        return dict(n=n, tables=[F.random_table(rng, 1 << n), F.random_table(rng, 1 << n),
                                 F.random_table(rng, 1 << (n - 2)), F.random_table(rng, 1 << (n - 2))],
                    coeffs=[F.random_scalar(rng) for _ in range(3)])
    if name == "lookup":
        # a signed lookup operation (8-bit table of ReLU shape, shift 12, 40-bit values: two zeroing chunks) over a
        # ragged rank-3 tensor, with the points of its linking sumcheck
        bits, shape = 8, (2, 3, 5)
        lo, hi = orc.table_input_range(bits, orc.SIGN_MIXED)
        t = rng.integers(-(1 << 36), 1 << 36, size=shape, dtype=np.int64)
        t.reshape(-1)[::2] >>= 20
        return dict(bits=bits, right_shift=12, max_bit_size=40, fpm=3, padding=1, tensor=t,
                    table_out=np.clip(np.arange(lo, hi + 1, dtype=np.int64), 0, hi), out_min=0, out_max=hi,
                    claim_point=[F.random_scalar(rng) for _ in range(2 + 3 + 1)],
                    logup_point=[F.random_scalar(rng) for _ in range(2 + 3)])
    if name == "einsum":
        # (left tensor, its fixes per output, right tensors with their fixes): stacked heads with one output, and one
        # left tensor with two right tensors (two outputs: the left claims are merged by a second sumcheck)
        C, O, S = orc.AXIS_CONTRACTED, orc.AXIS_OUTER, orc.AXIS_STACKED
        lg = lambda d: max(d - 1, 0).bit_length()
        pt = lambda d: [F.random_scalar(rng) for _ in range(lg(d))]
        q, k = rng.integers(-9, 9, (3, 5, 4)), rng.integers(-9, 9, (3, 6, 4))
        hp, sp, tp = pt(3), pt(5), pt(6)
        x, w, w2 = rng.integers(-99, 99, (6, 10)), rng.integers(-99, 99, (10, 5)), rng.integers(-99, 99, (10, 3))
        rp, cp, rp2, cp2 = pt(6), pt(5), pt(6), pt(3)
        return [dict(lhs=q, fixes=[((S, O, C), [hp, sp, None])], rhs=[(k, (S, O, C), [hp, tp, None])]),
                dict(lhs=x, fixes=[((O, C), [rp, None]), ((O, C), [rp2, None])],
                     rhs=[(w, (C, O), [None, cp]), (w2, (C, O), [None, cp2])])]
    if name == "claims":
        # committed polynomials (num_vars, chunks, claims): one unchunked with two claims, one in four chunks, one small
        polys = []
        for nv, nchunks, nclaims in ((5, 1, 2), (6, 4, 1), (3, 1, 1)):
            full = F.random_table(rng, 1 << nv)
            m = nv - (nchunks.bit_length() - 1)
            claims = []
            for _ in range(nclaims):
                pt = [F.random_scalar(rng) for _ in range(nv)]
                claims.append((pt, orc.evaluate(F, full, pt)))
            polys.append(orc.CommittedPoly([full[i << m:(i + 1) << m] for i in range(nchunks)], claims))
        return polys
    raise KeyError(name)


def mixed_terms(F, coeffs):
    return {(0, 1): coeffs[0], (0, 2, 3): coeffs[1], (1, 1, 3): coeffs[2], (2,): F.one}


def generate(F):
    hx = lambda vals: orc.serialize_scalars(F, vals).hex()
    out = {}
    t = orc.Transcript(F, b"m2vec")
    t.append_scalars([F.from_int(7), F.neg(F.one)])
    out["transcript"] = hx([t.append_and_sample(b"initial_alpha"), t.challenge_scalar(), t.challenge_scalar()])

    g = golden_inputs(F, "prod3")
    proof, point, finals = orc.sumcheck_prove(F, g["n"], g["tables"], {(0, 1, 2): F.one}, orc.Transcript(F))
    out["prod3"] = dict(proof=orc.serialize_sumcheck_proof(F, proof).hex(), point=hx(point), finals=hx(finals))

    g = golden_inputs(F, "mixed")
    proof, point, finals = orc.sumcheck_prove(F, g["n"], g["tables"], mixed_terms(F, g["coeffs"]), orc.Transcript(F))
    out["mixed"] = dict(proof=orc.serialize_sumcheck_proof(F, proof).hex(), point=hx(point), finals=hx(finals))

    g = golden_inputs(F, "hadamard")
    pr = orc.hadamard_prove(F, orc.Transcript(F), g["point"], g["v1"], g["v2"])
    out["hadamard"] = dict(proof=orc.serialize_sumcheck_proof(F, pr["sumcheck"]).hex(), point=hx(pr["point"]),
                           claims=hx(pr["individual_claim"]))

    g = golden_inputs(F, "logup_lookup")
    inputs = [orc.LogUpInput(F, 0, i["columns"], i["constant"], i["sep"], columns_per_instance=i["cpi"]) for i in g]
    out["logup_lookup"] = orc.serialize_logup_proof(F, orc.logup_batch_prove(F, inputs, orc.Transcript(F))).hex()

    g = golden_inputs(F, "logup_table")
    inp = orc.LogUpInput(F, 1, g["columns"], g["constant"], g["sep"], mult=g["mult"])
    out["logup_table"] = orc.serialize_logup_proof(F, orc.logup_batch_prove(F, [inp], orc.Transcript(F))).hex()

    pr = orc.claims_batching_prove(F, golden_inputs(F, "claims"), orc.Transcript(F))
    out["claims"] = dict(proof=orc.serialize_sumcheck_proof(F, pr["sumcheck"]).hex(), point=hx(pr["point"]),
                         evals=hx(pr["sumcheck_evals"]), rlc_challenges=hx(pr["rlc_challenges"]),
                         rlc=hx(orc.array_to_scalars(F, pr["rlc"])))

    g = golden_inputs(F, "lookup")
    ci = orc.ChunkingInfo(g["right_shift"], g["bits"], orc.SIGN_MIXED, g["max_bit_size"])
    wit = orc.LookupOpWitness(ci, g["fpm"], g["padding"], g["tensor"], g["table_out"], 2)
    cols = wit.input_columns() + wit.output_columns()
    counts = wit.get_counts()
    link = orc.lookup_linking_prove(F, orc.Transcript(F), orc.VARIANT_STANDARD, ci, g["out_min"], g["out_max"],
                                    g["tensor"].shape, [F.table_from_i64(c) for c in wit.output_columns()],
                                    g["claim_point"], g["logup_point"])
    out["lookup"] = dict(
        columns=[[int(v) for v in c] for c in cols],
        counts=[sorted([int(k), int(v)] for k, v in d.items()) for d in counts],
        multiplicities=hx(orc.array_to_scalars(F, orc.table_multiplicities(
            F, orc.merged_table_column(g["bits"], orc.SIGN_MIXED, g["table_out"]), counts[1]))),
        linking=dict(proof=orc.serialize_sumcheck_proof(F, link["sumcheck"]).hex(), point=hx(link["point"]),
                     evaluations=hx(link["evaluations"]), challenges=hx(link["challenges"])))

    out["einsum"] = []
    for g in golden_inputs(F, "einsum"):
        dims = [1 << max(d - 1, 0).bit_length() for d in g["lhs"].shape]
        padded = np.zeros(dims, dtype=np.int64)
        padded[tuple(slice(0, d) for d in g["lhs"].shape)] = g["lhs"]
        pr = orc.einsum_prove(F, orc.Transcript(F), g["lhs"], g["fixes"], g["rhs"],
                              lhs_padded=F.table_from_i64(padded.reshape(-1)))
        out["einsum"].append(orc.serialize_einsum_proof(F, pr).hex())

    g = golden_inputs(F, "fix")
    out["eq"] = hx(orc.array_to_scalars(F, orc.eq_evals(F, g["point"][:4])))
    out["fix_high3"] = hx(orc.array_to_scalars(F, orc.fix_high_variables(F, g["table"], g["point"][:3])))
    out["fix_low3"] = hx(orc.array_to_scalars(F, orc.fix_low_variables(F, g["table"], g["point"][:3])))
    out["evaluate"] = hx([orc.evaluate(F, g["table"], g["point"])])
    return out


def blake3_kat():
    import blake3
    return {str(n): blake3.blake3(bytes(i % 251 for i in range(n))).hexdigest()
            for n in (0, 1, 2, 63, 64, 65, 127, 128, 1023, 1024, 1025, 2048, 2049, 3072, 3073, 4096, 4097, 5120, 8192)}


if __name__ == "__main__":
    with open(os.path.join(HERE, "blake3_kat.json"), "w") as f:
        json.dump(blake3_kat(), f, indent=1)
    for F in (orc.FrField, orc.GlField):
        with open(os.path.join(HERE, f"oracle_{F.name}.json"), "w") as f:
            json.dump(generate(F), f, indent=1)
    print("fixtures written to", HERE)
