"""CPU backend of the path workloads (deep-prove_b200/workloads.py): every call of the walk restated on the oracle.

TEST INFRASTRUCTURE ONLY, like the rest of oracle/: the tests run the same walk on this backend and on the GPU
library and compare every call's payload byte for byte, and bench.py times this backend on a bounded sample of the
walk as the CPU baseline.  Nothing in the shipped library imports it.

Scalars are the oracle's (Python ints for BN254, pairs for the Goldilocks extension); tables are numpy arrays in
the library's layouts.  Payloads are the native little-endian words of every scalar in the order the GPU backend
exports them, so equal protocol outputs give equal bytes.
"""
import numpy as np

from . import oracle as orc


class _Expr:
    def __init__(self, e):
        self.e = e

    def __add__(self, o): return _Expr(self.e + o.e)
    def __sub__(self, o): return _Expr(self.e - o.e)
    def __mul__(self, o): return _Expr(self.e * o.e)


class _Counts:
    def __init__(self, bits):
        self.bits = bits
        self.d = {}

    def add(self, other):
        for k, c in other.items():
            self.d[k] = self.d.get(k, 0) + c


class OracleBackend:
    def __init__(self, field="fr"):
        self.F = orc.FrField if field == "fr" else orc.GlField
        self.name = field

    # -- plumbing
    def sync(self):
        pass

    def free(self, *handles):
        pass

    def keep(self, h):
        pass

    def release(self):
        pass

    def export(self, scalars):
        return np.ascontiguousarray(orc.scalars_to_array(self.F, list(scalars)), dtype=np.uint64).tobytes()

    # -- transcript and scalars
    def new_transcript(self):
        return orc.Transcript(self.F)

    def transcript_state(self, T):
        return bytes(T.state) + int(T.round).to_bytes(4, "little")

    def squeeze(self, T, m):
        return [T.challenge_scalar() for _ in range(m)]

    def scalar(self, x):
        return self.F.from_int(x)

    def inv2(self):
        return self.F.inv(self.F.from_int(2))

    # -- commitments: the synthetic bases are the multiples 1 G, 2 G, ... of the generator, so
    # sum_i s_i * (i + 1) G = (sum_i s_i (i + 1) mod r) G: one scalar multiplication checks a whole MSM
    def commit_setup(self, n):
        return n

    def commit(self, srs, tables):
        from . import g1
        if self.F is not orc.FrField:
            raise ValueError("commitments are over BN254")
        out = b""
        for t in tables:
            vals = self.F.table_to_ints(t)
            assert len(vals) <= srs
            k = sum(v * (i + 1) for i, v in enumerate(vals)) % g1.R_ORDER
            x, y = g1.boundary(g1.mul(k, g1.GENERATOR))
            out += int(x).to_bytes(32, "little") + int(y).to_bytes(32, "little")
        return out

    # -- tables
    def int_table(self, arr):
        return self.F.table_from_i64(np.ascontiguousarray(arr, dtype=np.int64))

    def tensor(self, arr):
        return np.ascontiguousarray(arr, dtype=np.int64)

    def num_vars(self, table):
        return orc.table_len(table).bit_length() - 1

    def chunks(self, table, n_chunks):
        per = orc.table_len(table) // n_chunks
        return [table[i * per:(i + 1) * per] for i in range(n_chunks)]

    def einsum_prove(self, T, lhs, lhs_shape, lhs_kinds, lhs_points, rhs, rhs_shape, rhs_kinds, rhs_points):
        got = orc.einsum_prove(self.F, T, lhs.reshape(lhs_shape), [(tuple(lhs_kinds), list(lhs_points))],
                               [(rhs.reshape(rhs_shape), tuple(rhs_kinds), list(rhs_points))])
        return orc.serialize_einsum_proof(self.F, got)

    def fix_axes(self, tensor, kinds, points):
        return None, orc.mles_from_tensor(self.F, tensor, tuple(kinds), list(points))

    def eq_table(self, point):
        return orc.eq_evals(self.F, list(point))

    def eq_values(self, point):
        return orc.array_to_scalars(self.F, orc.eq_evals(self.F, list(point)))

    def fix_low(self, table, point):
        return orc.fix_low_variables(self.F, table, list(point))

    def fix_high(self, table, point):
        return orc.fix_high_variables(self.F, table, list(point))

    def permuted_eq(self, eq):
        return orc.rope_permuted_eq(self.F, eq)

    def evaluate(self, table, point):
        return orc.evaluate(self.F, table, list(point))

    # -- sumchecks
    def _payload(self, proof, point, finals):
        return self.export([e for r in proof for e in r]) + self.export(point) + self.export(finals)

    def sumcheck(self, T, n, tables, terms):
        td = {}
        for c, idx in terms:
            key = tuple(idx)
            val = self.F.one if c is None else c
            td[key] = self.F.add(td[key], val) if key in td else val
        proof, point, finals = orc.sumcheck_prove(self.F, n, list(tables), td, T)
        return self._payload(proof, point, finals), point, finals

    def wit(self, i):
        return _Expr(orc.Expr.wit(i))

    def const(self, c):
        return _Expr(orc.Expr.const(c))

    def chal(self, i):
        return _Expr(orc.Expr.chal(i, 1, self.F.one, self.F.zero))

    def expr_sumcheck(self, T, n, tables, expr, challenges):
        terms = orc.expr_to_terms(self.F, expr.e, list(challenges))
        proof, point, finals = orc.sumcheck_prove(self.F, n, list(tables), terms, T)
        return self._payload(proof, point, finals), point, finals

    def same_poly(self, T, table, points):
        F = self.F
        # same_poly::Prover::prove takes (point, eval) claims; the evaluations do not enter the prover's messages
        got = orc.same_poly_prove(F, T, table, [(list(p), F.zero) for p in points])
        return self.export([e for r in got["sumcheck"] for e in r]) + self.export(got["point"]) + self.export([got["eval"]])

    # -- lookups
    def new_counts(self, bits):
        return _Counts(bits)

    def count_rows(self, counts, rows):
        keys, n = np.unique(np.asarray(rows, dtype=np.int64), return_counts=True)
        counts.add(dict(zip(keys.tolist(), n.tolist())))

    def lookup_witness(self, tensor, shape, spec, table_out, n_cols, counts):
        info = orc.ChunkingInfo(spec.right_shift, spec.bits, spec.sign, spec.max_bit_size, spec.n_value)
        w = orc.LookupOpWitness(info, spec.fpm, spec.padding, tensor.reshape(shape), table_out, n_cols)
        for c, d in zip(counts, w.get_counts()):
            c.add(d)
        T_ = self.F.table_from_i64
        return dict(owner=None, ins=[T_(c) for c in w.input_columns()], outs=[T_(c) for c in w.output_columns()],
                    n_shifted=info.n_shifted, n_zeroing=info.n_zeroing)

    def multiplicities(self, counts, table_cols, sign):
        F = self.F
        if len(table_cols) == 1:
            merged = np.asarray(table_cols[0], dtype=np.int64)
        else:
            merged = np.asarray(table_cols[0], dtype=np.int64) + orc.COLUMN_SEPARATOR * np.asarray(table_cols[1], dtype=np.int64)
        m = orc.table_multiplicities(F, merged, counts.d)
        t = np.asarray(m)
        return t[:, 0].copy() if F is orc.GlField and t.ndim == 2 else t

    def logup(self, T, inputs):
        F = self.F
        arr = []
        for kind, cols, cpi, mult, cst, sep in inputs:
            if kind == "lookup":
                arr.append(orc.LogUpInput(F, 0, list(cols), cst, sep, columns_per_instance=cpi))
            else:
                arr.append(orc.LogUpInput(F, 1, list(cols), cst, sep, mult=mult))
        return orc.serialize_logup_proof(F, orc.logup_batch_prove(F, arr, T))

    def linking(self, T, variant, spec, out_min, out_max, shape, mles, claim_point, logup_point, weight):
        F = self.F
        info = orc.ChunkingInfo(spec.right_shift, spec.bits, spec.sign, spec.max_bit_size, spec.n_value)
        with_sum = variant == 4
        v = orc.VARIANT_NORMALISATION if variant in (3, 4) else variant
        got = orc.lookup_linking_prove(F, T, v, info, out_min, out_max, tuple(shape), list(mles), list(claim_point),
                                       list(logup_point), normalised_sum=with_sum, weight=weight)
        payload = self.export([e for r in got["sumcheck"] for e in r]) + self.export(got["point"]) + \
            self.export(got["evaluations"]) + self.export(got["challenges"])
        if got["weight_eval"] is not None:
            payload += self.export([got["weight_eval"]])
        return payload

    def claims_batching(self, T, polys):
        F = self.F
        cps = [orc.CommittedPoly(list(chunks), [(list(pt), ev) for pt, ev in claims]) for chunks, claims in polys]
        got = orc.claims_batching_prove(F, cps, T)
        return self.export([e for r in got["sumcheck"] for e in r]) + self.export(got["point"]) + \
            self.export(got["sumcheck_evals"]) + self.export(got["rlc_challenges"])
