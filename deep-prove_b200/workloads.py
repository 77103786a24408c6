"""Path workloads: the sumcheck / fold / logup-GKR calls that proving a transformer's forward graph makes, at the
model's shapes, over seeded synthetic integer tensors.

What a workload is.  The reference's prover walks the model graph backwards and, per layer, calls into the path this
library implements: einsum layers fix axes and run one sumcheck (zkml/src/layers/einsum/prove.rs:46-334); lookup
layers (requantisation, activation, softmax, normalisation) generate a lookup witness, run a batched logup-GKR proof
over their lookups and one linking sumcheck (zkml/src/lookup/operation/generic_prove.rs:66-343); the attention mask,
the logits' argmax, the embeddings and the positional layer each run a sumcheck of their own
(zkml/src/layers/transformer/attention_mask/prove.rs:60-140, logits.rs:531-670, embeddings.rs:395-445,
positional/absolute.rs:290-330); claims on one tensor are merged by same_poly (zkml/src/iop/same_poly.rs:84-114); at
the end come the tables' logup-GKR proof (zkml/src/iop/prover.rs:220-274) and the claim-batching sumcheck over every
committed polynomial (zkml/src/poly_commit/prover.rs:140-255).  `transformer_path` makes exactly these calls, in
forward order, with the tensor shapes of the configuration it is given.

What it is not.  It does not run inference: tensors are seeded random integers of each tensor's shape and bit width,
not the activations of a real forward pass, and claim points are squeezed from the transcript instead of being handed
from layer to layer.  The work per call depends on shapes, table sizes and term structure, not on the values, so the
time of the walk is the time of the path for that model; the polynomial-commitment scheme (HyperKZG commit / open),
which the reference's end-to-end prove time includes, is not part of the path and is not included.

The walk is written against a small backend interface so that the same call list runs on the GPU library
(`GpuBackend`, below) and on a CPU restatement used by the tests; every call returns a byte string (`payload`) that
must be equal between backends.
"""
import time
from dataclasses import dataclass

import numpy as np

AX_CONTRACTED, AX_OUTER, AX_STACKED = 0, 1, 2
SIGN_POSITIVE, SIGN_NEGATIVE, SIGN_MIXED = 0, 1, 2
VARIANT_STANDARD, VARIANT_GLU, VARIANT_SOFTMAX, VARIANT_NORMALISATION, VARIANT_NORMALISATION_WITH_SUM = 0, 1, 2, 3, 4


@dataclass(frozen=True)
class TransformerShape:
    """A decoder-only transformer as far as the path needs to know it."""
    name: str
    layers: int
    seq: int
    d_model: int
    heads: int
    head_dim: int
    ffn: int
    vocab: int
    table_bits: int = 12        # activation / requantisation tables (ZKML_BIT_LEN's default, quantization/mod.rs:28-33)
    commit_chunk_log2: int = 20  # committed polynomials are cut into chunks of at most 2^20 (poly_commit/context.rs:103-118)
    range_check_chunks: int = 2  # 16-bit chunks of the logits' max - logit difference (logits.rs:286-298)
    kv_heads: int = 0            # 0: as many as query heads; fewer: grouped-query attention (K and V shared by groups)
    glu: bool = False            # gated feed-forward (GeGLU / SwiGLU): two up projections and a GLU linking sumcheck
    rope: bool = False           # rotary positions on Q and K per block instead of one absolute-position layer


@dataclass(frozen=True)
class MlpShape:
    """A dense network: layer widths, ReLU through a lookup after every layer but the last, argmax at the end."""
    name: str
    widths: tuple
    batch: int = 1
    table_bits: int = 12
    commit_chunk_log2: int = 20
    range_check_chunks: int = 2


GPT2_SMALL = TransformerShape("gpt2-small", layers=12, seq=512, d_model=768, heads=12, head_dim=64, ffn=3072,
                              vocab=50257)
# BASELINE.json configs[3]: 26 layers, d_model 1152, 4 query heads / 1 KV head, head_dim 256, GeGLU 6912, RMSNorm,
# RoPE, vocab 262144, 512 tokens
GEMMA3_1B = TransformerShape("gemma3-1b-style", layers=26, seq=512, d_model=1152, heads=4, head_dim=256, ffn=6912,
                             vocab=262144, kv_heads=1, glu=True, rope=True)
# BASELINE.json configs[4]: two blocks of d_model 4096, 32 heads x 128, SwiGLU 11008, RMSNorm, RoPE, vocab 32000,
# 1024 tokens
LLAMA2_7B_2BLOCKS = TransformerShape("llama2-7b-style-2-blocks", layers=2, seq=1024, d_model=4096, heads=32,
                                     head_dim=128, ffn=11008, vocab=32000, glu=True, rope=True)
# BASELINE.json configs[0]: input 1 x 1024, 1024 x 1024 and 1024 x 10 weights, ReLU through a lookup, argmax
MLP_2LAYER = MlpShape("mlp-1024-1024-10", widths=(1024, 1024, 10))
# the same graphs at sizes a CPU restatement proves in seconds: every call of the walk, one block
TINY = TransformerShape("tiny", layers=1, seq=24, d_model=48, heads=3, head_dim=16, ffn=80, vocab=200, table_bits=8,
                        commit_chunk_log2=8, range_check_chunks=2)
TINY_GLU_ROPE = TransformerShape("tiny-glu-rope-gqa", layers=1, seq=20, d_model=40, heads=4, head_dim=8, ffn=56,
                                 vocab=150, table_bits=8, commit_chunk_log2=8, kv_heads=2, glu=True, rope=True)
TINY_MLP = MlpShape("tiny-mlp", widths=(48, 40, 10), table_bits=8, commit_chunk_log2=8)


# one block at a size the CPU restatement walks in some tens of seconds: the bounded sample bench.py times on the host
CPU_SAMPLE = TransformerShape("cpu-sample", layers=1, seq=128, d_model=192, heads=4, head_dim=48, ffn=768, vocab=4000,
                              table_bits=10, commit_chunk_log2=14, range_check_chunks=2)


def ceil_log2(x):
    return max(int(x) - 1, 0).bit_length()


def table_input_range(bits, sign):
    """Table::min_input_value / max_input_value (zkml/src/lookup/table/mod.rs:126-142)."""
    if sign == SIGN_POSITIVE:
        return 0, (1 << bits) - 1
    if sign == SIGN_MIXED:
        return -(1 << (bits - 1)), (1 << (bits - 1)) - 1
    return -(1 << bits) + 1, 0


@dataclass(frozen=True)
class LookupSpec:
    """One lookup operation's decomposition (ChunkingInfo::new, decomposer.rs:182-249) and its value table."""
    table: str          # key of the value table: "requant", "gelu", "exp", "norm"
    bits: int
    right_shift: int
    max_bit_size: int
    sign: int
    n_value: int = 1
    fpm: int = 1        # fixed-point multiplier applied before the decomposition
    padding: int = 0


def value_table(table, bits):
    """(sign, output column over the table's input range or None for a one-column table, columns).  The output
    columns are integer stand-ins of the right shape: the reference computes them once per table in float
    arithmetic (tabletype.rs:83-125); they are data to the path, not part of it."""
    if table == "requant":
        return SIGN_MIXED, None, 1
    if table in ("gelu", "norm", "relu"):
        lo, hi = table_input_range(bits, SIGN_MIXED)
        x = np.arange(lo, hi + 1, dtype=np.int64)
        # gelu-like: x * sigmoid(1.702 x) at the table's scale, rounded; norm: a plain clamp at zero
        if table == "gelu":
            s = np.float64(1 << (bits - 3))
            out = np.rint(x / (1.0 + np.exp(-1.702 * x / s))).astype(np.int64)
        else:
            out = np.clip(x, 0, hi)
        return SIGN_MIXED, out, 2
    if table == "exp":
        lo, hi = table_input_range(bits, SIGN_NEGATIVE)
        x = np.arange(lo, hi + 1, dtype=np.int64)
        out = np.rint(np.exp(x.astype(np.float64) / np.float64(1 << (bits - 3))) * np.float64(1 << 20)).astype(np.int64)
        out[0] = 0
        return SIGN_NEGATIVE, out, 2
    raise ValueError(table)


def draw_tensor(rng, shape, spec):
    """Seeded integers that fit the operation's declared size after its fixed-point multiplier."""
    big = max((1 << (spec.max_bit_size - 2)) // spec.fpm, 2)
    if spec.sign == SIGN_MIXED:
        t = rng.integers(-big, big, size=shape, dtype=np.int64)
    elif spec.sign == SIGN_POSITIVE:
        t = rng.integers(0, big, size=shape, dtype=np.int64)
    else:
        t = -rng.integers(0, big, size=shape, dtype=np.int64)
    return t


class PathTimer:
    """Wall time per kind of call, with a device synchronisation on both sides when the backend has a device."""

    def __init__(self, be):
        self.be, self.by_kind, self.calls = be, {}, {}

    def __call__(self, kind):
        timer = self

        class _Span:
            def __enter__(self):
                timer.be.sync()
                self.t0 = time.perf_counter()

            def __exit__(self, *exc):
                timer.be.sync()
                dt = time.perf_counter() - self.t0
                timer.by_kind[kind] = timer.by_kind.get(kind, 0.0) + dt
                timer.calls[kind] = timer.calls.get(kind, 0) + 1
                return False
        return _Span()


class PathWalk:
    """The calls of the path, one method per kind of layer, over one backend and one transcript.  A model's walk
    (transformer_path, mlp_path) strings them together in forward order; `records` collects (name, kind, payload)."""

    TABLE_KEYS = ["shift", "zero", "signed", "requant", "gelu", "exp", "norm", "relu"]

    def __init__(self, be, bits, commit_chunk_log2, range_check_chunks, seed, with_commit):
        self.be, self.bits, self.chunk_log2, self.range_chunks = be, bits, commit_chunk_log2, range_check_chunks
        self.rng = np.random.default_rng(seed)
        self.T = be.new_transcript()
        self.timer = PathTimer(be)
        self.rec = []
        self.with_commit = with_commit
        # per-table logup challenges (ChallengeStorage, zkml/src/iop/mod.rs:174-187) and lookup counters
        self.chal = {k: tuple(be.squeeze(self.T, 2)) for k in self.TABLE_KEYS}
        self.counts = {"shift": be.new_counts(16), "zero": be.new_counts(16), "signed": be.new_counts(16)}
        for k in ("requant", "gelu", "exp", "norm", "relu"):
            self.counts[k] = be.new_counts(bits)
        self.used_tables = set()
        self.committed = []  # (name, table handle, entries): everything the claim batching at the end opens
        self.srs = be.commit_setup(1 << commit_chunk_log2) if with_commit else None
        self.act_bits = bits + 2
        self.specs = {
            "requant": LookupSpec("requant", bits, right_shift=bits + 1, max_bit_size=2 * bits + 4, sign=SIGN_MIXED),
            "gelu": LookupSpec("gelu", bits, right_shift=bits + 1, max_bit_size=2 * bits + 4, sign=SIGN_MIXED),
            "relu": LookupSpec("relu", bits, right_shift=bits + 1, max_bit_size=2 * bits + 4, sign=SIGN_MIXED),
            "exp": LookupSpec("exp", bits, right_shift=bits - 2, max_bit_size=2 * bits + 10, sign=SIGN_NEGATIVE),
            "norm": LookupSpec("norm", bits, right_shift=bits, max_bit_size=2 * bits + 2, sign=SIGN_MIXED),
        }

    # ------------------------------------------------------------------ synthetic data
    def small(self, shape_):
        return self.rng.integers(-(1 << (self.act_bits - 1)), 1 << (self.act_bits - 1), size=shape_, dtype=np.int64)

    def weights(self, shape_):
        return self.rng.integers(-(1 << (self.bits - 1)), 1 << (self.bits - 1), size=shape_, dtype=np.int64)

    def draw(self, shape_, table):
        return draw_tensor(self.rng, shape_, self.specs[table])

    def commit_weight(self, name, w):
        """A weight matrix as a committed polynomial: padded to powers of two per dimension."""
        dims = [1 << ceil_log2(d) for d in w.shape]
        padded = np.zeros(dims, dtype=np.int64)
        padded[tuple(slice(0, d) for d in w.shape)] = w
        self.committed.append((name, self.be.int_table(padded.reshape(-1)), padded.size))

    # ------------------------------------------------------------------ the calls
    def einsum(self, name, lhs, lhs_kinds, rhs, rhs_kinds):
        """EinSum::prove_internal (zkml/src/layers/einsum/prove.rs:48-335) with one right tensor: the outer axes of
        both tensors are bound to (squeezed stand-ins for) the output claim's coordinates, the stacked axes (heads)
        share one point that gives the stacking coefficients, and the sumcheck runs over the contracted axis."""
        be, T, lg = self.be, self.T, ceil_log2
        lhs_dev, rhs_dev = be.tensor(lhs), be.tensor(rhs)  # resident before the clock starts
        # the output claim's coordinates: stand-ins, drawn before the clock starts
        lp = [be.squeeze(T, lg(d)) if k != AX_CONTRACTED else None for d, k in zip(lhs.shape, lhs_kinds)]
        stacked = [p for p, k in zip(lp, lhs_kinds) if k == AX_STACKED]
        rp = []
        for d, k in zip(rhs.shape, rhs_kinds):
            rp.append(stacked.pop(0) if k == AX_STACKED else be.squeeze(T, lg(d)) if k == AX_OUTER else None)
        with self.timer("einsum"):
            payload = be.einsum_prove(T, lhs_dev, lhs.shape, lhs_kinds, lp, rhs_dev, rhs.shape, rhs_kinds, rp)
        self.rec.append((name, "einsum", payload))

    def lookup_layer(self, name, tensor, table, variant=VARIANT_STANDARD, weight=None, glu=False):
        """prove_lookup_op: witness columns -> batched logup-GKR over the lookups -> linking sumcheck."""
        be, T, lg, spec = self.be, self.T, ceil_log2, self.specs[table]
        sign, table_out, n_cols = value_table(spec.table, spec.bits)
        self.used_tables.update(("shift", "zero", "signed", table))
        tensor_dev = be.tensor(tensor)
        with self.timer("lookup_witness"):
            cs = [self.counts["shift"], self.counts[table], self.counts["zero"], self.counts["signed"]]
            wit = be.lookup_witness(tensor_dev, tensor.shape, spec, table_out, n_cols, cs)
            ins, outs = wit["ins"], wit["outs"]
        slices = int(np.prod(tensor.shape[:-2])) if tensor.ndim > 2 else 1
        n_sh, n_z = wit["n_shifted"], wit["n_zeroing"]
        per_in = n_sh + (spec.n_value if n_cols != 1 else 0) + n_z
        per_out = spec.n_value + n_z
        signed = sign == SIGN_MIXED
        groups = {"shift": [], table: [], "zero": [], "signed": []}
        for c in range(slices):
            i0, o0 = c * per_in, c * per_out
            groups["shift"] += ins[i0:i0 + n_sh]
            for v in range(spec.n_value):
                if n_cols != 1:
                    groups[table] += [ins[i0 + n_sh + v], outs[o0 + v]]
                else:
                    groups[table] += [outs[o0 + v]]
            zi0 = i0 + n_sh + (spec.n_value if n_cols != 1 else 0)
            for z in range(n_z):
                key = "signed" if (signed and z == n_z - 1) else "zero"
                groups[key] += [ins[zi0 + z], outs[o0 + spec.n_value + z]]
        inputs = []
        for key, cpi in (("shift", 1), (table, 2 if n_cols != 1 else 1), ("zero", 2), ("signed", 2)):
            if groups[key]:
                inputs.append(("lookup", groups[key], cpi, None, self.chal[key][0], self.chal[key][1]))
        with self.timer("lookup_logup"):
            self.rec.append((name + ".logup", "logup", be.logup(T, inputs)))
        dims = [1 << lg(d) for d in tensor.shape]
        total = sum(lg(d) for d in dims)
        n2d = sum(lg(d) for d in dims[-2:]) if tensor.ndim > 1 else lg(dims[-1])
        if table_out is None:
            out_min, out_max = table_input_range(spec.bits, sign)
        else:
            out_min, out_max = int(table_out[0]), int(table_out[-1])
        mles = list(outs)
        extra_owner = []
        P = 1 << n2d
        if variant in (VARIANT_NORMALISATION, VARIANT_NORMALISATION_WITH_SUM):
            # one input table and one scaling table per slice (variant.rs:288-346)
            for _ in range(2 * slices):
                tab = be.int_table(self.small(P))
                extra_owner.append(tab)
                mles.append(tab)
        if glu:
            # the gate's partner: one witness table per slice multiplies the looked-up value (variant.rs:229-287)
            variant = VARIANT_GLU
            for _ in range(slices):
                tab = be.int_table(self.small(P))
                extra_owner.append(tab)
                mles.append(tab)
        claim_point = be.squeeze(T, total)
        logup_point = be.squeeze(T, n2d)
        with self.timer("lookup_linking"):
            payload = be.linking(T, variant, spec, out_min, out_max, tensor.shape, mles, claim_point, logup_point, weight)
        self.rec.append((name + ".linking", "linking", payload))
        # the witness columns are committed polynomials: they are opened at the end
        for j, col in enumerate(ins + outs):
            self.committed.append((f"{name}.w{j}", col, 1 << n2d))
        if self.with_commit:
            n_chunks = 1 << max(n2d - self.chunk_log2, 0)
            with self.timer("witness_commit"):
                chunks = [c_ for col in ins + outs for c_ in be.chunks(col, n_chunks)]
                self.rec.append((name + ".commit", "commit", be.commit(self.srs, chunks)))
        be.free(*extra_owner)
        be.keep(wit["owner"])

    def same_poly(self, name, n_entries, n_claims):
        """Claims on one tensor merged into one (flatten_and_merge_claims, iop/prover.rs:1064-1101)."""
        be, T = self.be, self.T
        tab = be.int_table(self.small(n_entries))
        with self.timer("same_poly"):
            pts = [be.squeeze(T, ceil_log2(n_entries)) for _ in range(n_claims)]
            self.rec.append((name, "same_poly", be.same_poly(T, tab, pts)))
        be.free(tab)

    def attention_mask(self, name, batch, seq):
        """AttentionMask::prove_internal: eq * row_lt * col_lt * sum_j chi_j (mask * in_j + NEG (1 - mask)),
        tables eq, mask, row_lt, col_lt, then one input table per head (attention_mask/mod.rs:115-159)."""
        be, T, lg = self.be, self.T, ceil_log2
        ps = 1 << lg(seq)
        n = 2 * lg(seq)
        i = np.arange(ps)
        mask = (i[None, :] <= i[:, None]).astype(np.int64)           # lower triangular
        row_lt = np.repeat((i < seq).astype(np.int64), ps)
        col_lt = np.tile((i < seq).astype(np.int64), ps)
        fixed = [be.int_table(mask.reshape(-1)), be.int_table(row_lt), be.int_table(col_lt)]
        fixed += [be.int_table(self.small(ps * ps)) for _ in range(batch)]
        with self.timer("attention_mask"):
            tabs = [be.eq_table(be.squeeze(T, n))] + fixed
            chi = be.eq_values(be.squeeze(T, lg(batch)))[:batch] if batch > 1 else [be.scalar(1)]
            neg = be.const(be.scalar(-(1 << (2 * self.bits))))
            lead = be.wit(0) * (be.wit(2) * be.wit(3))
            one_minus = be.const(be.scalar(1)) - be.wit(1)
            e_ = None
            for j in range(batch):
                term = lead * be.chal(j) * (be.wit(1) * be.wit(4 + j) + neg * one_minus)
                e_ = term if e_ is None else e_ + term
            payload, point, finals = be.expr_sumcheck(T, n, tabs, e_, chi)
        self.rec.append((name, "attention_mask", payload))
        be.free(*tabs)

    def embeddings(self, wte, V, e):
        """Embeddings::prove: bind the column variables of the padded matrix, then sum_v onehot(v) * E(v)
        (transformer/embeddings.rs:395-445)."""
        be, T, lg = self.be, self.T, ceil_log2
        pv, pe = wte.shape
        wte_tab = be.int_table(wte.reshape(-1))
        self.committed.append(("wte", wte_tab, wte.size))
        one_hot = be.int_table(self.rng.integers(0, 3, size=pv, dtype=np.int64))
        with self.timer("embeddings"):
            col_point = be.squeeze(T, lg(pe))
            fixed = be.fix_low(wte_tab, col_point)
            payload, point, finals = be.sumcheck(T, lg(pv), [one_hot, fixed], [(None, [0, 1])])
            self.rec.append(("embeddings", "embeddings", payload))
        be.free(fixed, one_hot)

    def positional(self, e):
        """Positional (absolute): fixed_positional * lt * column_eq over the embedding columns
        (positional/absolute.rs:290-330)."""
        be, T, lg = self.be, self.T, ceil_log2
        ps_ = 1 << lg(e)
        tabs = [be.int_table(self.small(ps_)), be.int_table((np.arange(ps_) < e).astype(np.int64))]
        with self.timer("positional"):
            tabs.append(be.eq_table(be.squeeze(T, lg(ps_))))
            payload, point, finals = be.sumcheck(T, lg(ps_), tabs, [(None, [0, 1, 2])])
            self.rec.append(("positional", "positional", payload))
        be.free(*tabs)

    def rope(self, name, heads, seq, dh):
        """Rotary positions (positional/rope.rs:526-590): bind the head variables of the input (fix_high), then
        input * lt * (eq * cos + permuted_eq * sin) over the (position, head dimension) variables."""
        be, T, lg = self.be, self.T, ceil_log2
        ph, ps_, pd = 1 << lg(heads), 1 << lg(seq), 1 << lg(dh)
        n = lg(ps_) + lg(pd)
        x = np.zeros((ph, ps_, pd), dtype=np.int64)
        x[:heads, :seq, :dh] = self.small((heads, seq, dh))
        inp = be.int_table(x.reshape(-1))
        cos, sin = be.int_table(self.small(ps_ * pd)), be.int_table(self.small(ps_ * pd))
        lt = be.int_table(np.repeat((np.arange(ps_) < seq).astype(np.int64), pd))
        with self.timer("rope"):
            fix_point = be.squeeze(T, lg(ph))
            beta = be.squeeze(T, n)
            fixed = be.fix_high(inp, fix_point) if lg(ph) else inp
            eq = be.eq_table(beta)
            peq = be.permuted_eq(eq)
            tabs = [fixed, cos, sin, eq, peq, lt]
            expr = be.wit(0) * be.wit(5) * (be.wit(3) * be.wit(1) + be.wit(4) * be.wit(2))
            payload, point, finals = be.expr_sumcheck(T, n, tabs, expr, [])
        self.rec.append((name, "rope", payload))
        be.free(inp, cos, sin, lt, eq, peq)
        if lg(ph):
            be.free(fixed)

    def argmax(self, rows, V):
        """Logits (argmax): the range check of max - logit over range_check_chunks 16-bit chunks, then the linking
        sumcheck  sum_eq (max - C onehot input) + chi input_eq lt (max - input)   (logits.rs:531-670)."""
        be, T, lg, rng = self.be, self.T, ceil_log2, self.rng
        ps_, pv_ = 1 << lg(rows), 1 << lg(V)
        n = lg(ps_) + lg(pv_)
        logits = self.small((ps_, pv_))
        logits[:, V:] = 0
        arg = logits[:, :V].argmax(axis=1)
        one_hot = np.zeros((ps_, pv_), dtype=np.int64)
        one_hot[np.arange(ps_), arg] = 1
        mx = np.repeat(logits[np.arange(ps_), arg], pv_)
        lt = np.tile((np.arange(pv_) < V).astype(np.int64), ps_)
        diff = (mx - logits.reshape(-1)) * lt          # max - logit, zero in the padding
        chunk_ints = [(diff >> (16 * c_)) & 0xFFFF for c_ in range(self.range_chunks)]
        cols = [be.int_table(c_) for c_ in chunk_ints]
        self.used_tables.add("shift")
        with self.timer("argmax_logup"):
            for c_ in chunk_ints:
                be.count_rows(self.counts["shift"], c_)
            self.rec.append(("argmax.logup", "logup",
                             be.logup(T, [("lookup", cols, 1, None, self.chal["shift"][0], self.chal["shift"][1])])))
        tabs = [be.int_table(logits.reshape(-1)), be.int_table(mx), be.int_table(one_hot.reshape(-1)), None, None,
                be.int_table(lt)]
        del diff, chunk_ints, logits, one_hot, mx, lt
        with self.timer("argmax_linking"):
            row_point = be.squeeze(T, lg(ps_))
            sum_eq_point = [be.inv2()] * lg(pv_) + list(row_point)
            tabs[3] = be.eq_table(sum_eq_point)
            tabs[4] = be.eq_table(be.squeeze(T, n))
            C = be.const(be.scalar(pv_))
            first = be.wit(3) * (be.wit(1) - C * be.wit(2) * be.wit(0))
            second = be.wit(4) * be.wit(5) * (be.wit(1) - be.wit(0))
            expr = first + be.chal(0) * second
            payload, point, finals = be.expr_sumcheck(T, n, tabs, expr, be.squeeze(T, 1))
            self.rec.append(("argmax.linking", "argmax_linking", payload))
        for c_ in cols:
            self.committed.append(("argmax.chunk", c_, ps_ * pv_))
        be.free(*tabs)

    def tables_logup(self):
        """prove_tables (zkml/src/iop/prover.rs:220-274): one logup-GKR batch over every table that was looked up,
        with the multiplicities the lookups left in the counters."""
        be, T, bits = self.be, self.T, self.bits
        t16 = np.arange(1 << 16, dtype=np.int64)
        s16 = np.arange(-(1 << 15), 1 << 15, dtype=np.int64)
        table_cols = {"shift": [t16], "zero": [t16, (t16 == 0).astype(np.int64)], "signed": [s16, np.sign(s16)]}
        for key in ("requant", "gelu", "exp", "norm", "relu"):
            sign, out, n_cols = value_table(key, bits)
            lo, hi = table_input_range(bits, sign)
            ins_ = np.arange(lo, hi + 1, dtype=np.int64)
            table_cols[key] = [ins_] if out is None else [ins_, out]
        keys = [k for k in self.TABLE_KEYS if k in self.used_tables]
        dev_cols = {key: [be.int_table(c_) for c_ in table_cols[key]] for key in keys}
        owners, inputs = [], []
        with self.timer("tables_logup"):
            for key in keys:
                mult = be.multiplicities(self.counts[key], table_cols[key], None)
                owners += dev_cols[key] + [mult]
                inputs.append(("table", dev_cols[key], len(dev_cols[key]), mult, self.chal[key][0], self.chal[key][1]))
            # a batch is ordered by non-increasing size (prover.rs:95-140)
            inputs.sort(key=lambda i_: -be.num_vars(i_[1][0]))
            self.rec.append(("tables.logup", "logup", be.logup(T, inputs)))
        be.free(*owners)

    def claim_batching(self):
        """CommitmentProver::claims_batching_sumcheck + the linear combination over every committed polynomial
        (zkml/src/poly_commit/prover.rs:113-131, 140-255), one claim per polynomial."""
        be, T = self.be, self.T
        # the claims themselves stand in for what the layers' proofs hand on: drawn before the clock starts
        polys = []
        for name, tab, entries in self.committed:
            nv = ceil_log2(entries)
            n_chunks = 1 << max(nv - self.chunk_log2, 0)
            point = be.squeeze(T, nv)
            ev = be.squeeze(T, 1)[0]
            polys.append((be.chunks(tab, n_chunks), [(point, ev)]))
        with self.timer("claim_batching"):
            self.rec.append(("claim_batching", "claim_batching", be.claims_batching(T, polys)))

    def finish(self):
        be = self.be
        self.rec.append(("transcript", "state", be.transcript_state(self.T)))
        be.free(self.srs)
        be.release()
        return self.rec, self.timer


def transformer_path(be, shape, seed=0, blocks=None, with_final=True, with_commit=False):
    """Walks the path calls of `shape` on backend `be`.  Returns (records, timer): records is a list of
    (name, kind, payload bytes); timer.by_kind holds seconds per kind of call.  `blocks` limits the number of
    transformer blocks walked (default: all); `with_final=False` leaves out everything after the last block.
    with_commit: every lookup layer also commits to its witness columns (one multi-scalar multiplication per
    chunk of at most 2^commit_chunk_log2 evaluations, zkml/src/lookup/context.rs:420-422), timed as its own kind
    "witness_commit": the commitment scheme's share of a proof, next to the path's."""
    w = PathWalk(be, shape.table_bits, shape.commit_chunk_log2, shape.range_check_chunks, seed, with_commit)
    s, e, h, dh, f, V = shape.seq, shape.d_model, shape.heads, shape.head_dim, shape.ffn, shape.vocab
    kv = shape.kv_heads or h
    lg = ceil_log2
    n_blocks = shape.layers if blocks is None else blocks
    O, C, S = AX_OUTER, AX_CONTRACTED, AX_STACKED

    def gamma_table():
        return be.int_table(np.tile(np.pad(w.weights(e), (0, (1 << lg(e)) - e)), 1 << lg(s)))

    wte = None
    if with_final:
        pv, pe = 1 << lg(V), 1 << lg(e)
        wte = np.zeros((pv, pe), dtype=np.int64)
        wte[:V, :e] = w.weights((V, e))
        w.embeddings(wte, V, e)
        if not shape.rope:
            w.positional(e)

    for b in range(n_blocks):
        pre = f"block{b}."
        x = w.small((s, e))
        gamma = gamma_table()
        w.lookup_layer(pre + "norm1", w.draw((s, e), "norm"), "norm", VARIANT_NORMALISATION, gamma)
        qkv_cols = (h + 2 * kv) * dh
        w_qkv = w.weights((e, qkv_cols))
        w.commit_weight(pre + "w_qkv", w_qkv)
        w.einsum(pre + "qkv", x, (O, C), w_qkv, (C, O))
        w.lookup_layer(pre + "qkv.requant", w.draw((s, qkv_cols), "requant"), "requant")
        if shape.rope:
            w.rope(pre + "rope_q", h, s, dh)
            w.rope(pre + "rope_k", kv, s, dh)
        # grouped-query attention: every K / V head serves h // kv query heads; the proof sees them repeated
        q = w.small((h, s, dh))
        k_ = np.repeat(w.small((kv, s, dh)), h // kv, axis=0)
        v_ = np.repeat(w.small((kv, s, dh)), h // kv, axis=0)
        w.einsum(pre + "qk", q, (S, O, C), k_, (S, O, C))
        w.attention_mask(pre + "mask", h, s)
        w.lookup_layer(pre + "softmax", w.draw((h, s, s), "exp"), "exp", VARIANT_SOFTMAX)
        w.einsum(pre + "av", w.small((h, s, s)), (S, O, C), v_, (S, C, O))
        w.lookup_layer(pre + "av.requant", w.draw((s, h * dh), "requant"), "requant")
        w_o = w.weights((h * dh, e))
        w.commit_weight(pre + "w_o", w_o)
        w.einsum(pre + "out", w.small((s, h * dh)), (O, C), w_o, (C, O))
        w.same_poly(pre + "residual1", (1 << lg(s)) * (1 << lg(e)), 2)
        w.lookup_layer(pre + "norm2", w.draw((s, e), "norm"), "norm", VARIANT_NORMALISATION, gamma)
        w_up = w.weights((e, f))
        w.commit_weight(pre + "w_up", w_up)
        w.einsum(pre + "ffn_up", x, (O, C), w_up, (C, O))
        if shape.glu:
            w_gate = w.weights((e, f))
            w.commit_weight(pre + "w_gate", w_gate)
            w.einsum(pre + "ffn_gate", x, (O, C), w_gate, (C, O))
            w.lookup_layer(pre + "glu", w.draw((s, f), "gelu"), "gelu", glu=True)
        else:
            w.lookup_layer(pre + "gelu", w.draw((s, f), "gelu"), "gelu")
        w_down = w.weights((f, e))
        w.commit_weight(pre + "w_down", w_down)
        w.einsum(pre + "ffn_down", w.small((s, f)), (O, C), w_down, (C, O))
        w.lookup_layer(pre + "ffn_down.requant", w.draw((s, e), "requant"), "requant")
        w.same_poly(pre + "residual2", (1 << lg(s)) * (1 << lg(e)), 2)
        be.free(gamma)

    if with_final:
        gamma = gamma_table()
        w.lookup_layer("norm_f", w.draw((s, e), "norm"), "norm", VARIANT_NORMALISATION, gamma)
        be.free(gamma)
        w.einsum("lm_head", w.small((s, e)), (O, C), wte[:V, :e].T.copy(), (C, O))
        w.argmax(s, V)
        w.tables_logup()
        w.claim_batching()
    return w.finish()


def mlp_path(be, shape, seed=0, with_commit=False):
    """The dense network (a 2-layer MLP with ReLU through a lookup and an argmax output): per layer the einsum's axis fixing and sumcheck, then
    (all but the last layer) ReLU with requantisation through a lookup: witness, logup-GKR, linking sumcheck; at the
    end the argmax, the tables' logup proof and the claim batching."""
    w = PathWalk(be, shape.table_bits, shape.commit_chunk_log2, shape.range_check_chunks, seed, with_commit)
    O, C = AX_OUTER, AX_CONTRACTED
    widths = shape.widths
    for i in range(len(widths) - 1):
        x = w.small((shape.batch, widths[i]))
        wt = w.weights((widths[i], widths[i + 1]))
        w.commit_weight(f"layer{i}.w", wt)
        w.einsum(f"layer{i}.dense", x, (O, C), wt, (C, O))
        if i < len(widths) - 2:
            w.lookup_layer(f"layer{i}.relu", w.draw((shape.batch, widths[i + 1]), "relu"), "relu")
    w.argmax(shape.batch, widths[-1])
    w.tables_logup()
    w.claim_batching()
    return w.finish()


# ------------------------------------------------------------------------------ GPU backend
class _Expr:
    """Expression wrapper of the GPU backend over prover.Expression."""

    def __init__(self, e):
        self.e = e

    def __add__(self, o): return _Expr(self.e + o.e)
    def __sub__(self, o): return _Expr(self.e - o.e)
    def __mul__(self, o): return _Expr(self.e * o.e)


class GpuBackend:
    """The walk's calls on the GPU library: every method is one or a few C-ABI calls (device tensors stay on the
    device; the transcript and the expression algebra run in the library's host code)."""

    def __init__(self, dpb, prover, ctx, field="fr", int_tables=True):
        self.dpb, self.prover, self.ctx = dpb, prover, ctx
        # int_tables: integer tensors (weights, activations, fixed 0/1 tables) stay 32- or 64-bit integers on the
        # device instead of being converted to field elements at upload; every result is the same
        self.int_tables = int_tables
        self.i32 = dpb.FR_I32 if field == "fr" else dpb.GL_I32
        self.i64 = dpb.FR_I64 if field == "fr" else dpb.GL_I64
        self.fam = dpb.FR if field == "fr" else dpb.GL_EXT
        self.base = dpb.FR if field == "fr" else dpb.GL_BASE
        self.w = dpb.elem_words(self.fam)
        self.name = field
        self._kept = []
        self._one = np.frombuffer(dpb.one_bytes(self.fam), dtype=np.uint64).copy()

    # -- plumbing
    def sync(self):
        self.ctx.sync()

    def free(self, *handles):
        for h in handles:
            if h is None:
                continue
            if isinstance(h, tuple):  # device tensor (mle, shape)
                h[0].free()
            else:
                h.free()

    def keep(self, h):
        self._kept.append(h)

    def release(self):
        for h in self._kept:
            self.free(h)
        self._kept = []

    def export(self, arr):
        return np.ascontiguousarray(arr, dtype=np.uint64).tobytes()

    # -- transcript and scalars
    def new_transcript(self):
        return self.prover.Blake3Transcript(self.fam)

    def transcript_state(self, T):
        st, rnd = T.state()
        return st + int(rnd).to_bytes(4, "little")

    def squeeze(self, T, m):
        return [T.challenge_scalar() for _ in range(m)]

    def scalar(self, x):
        """A small integer as a challenge element."""
        t = self.ctx.upload_i64(np.array([x, 0], dtype=np.int64), self.base)
        v = t.to_host()
        t.free()
        out = np.zeros(self.w, dtype=np.uint64)
        row = np.asarray(v).reshape(2, -1)[0]
        out[: row.size] = row
        return out

    def inv2(self):
        if not hasattr(self, "_inv2"):
            # 1/2 = (p + 1) / 2 as a table entry: evaluate the table [0, 1] at ... needs no inversion:
            # eq((1/2)) cannot be formed without it, so it is computed once on the host with Python integers
            if self.name == "fr":
                p = 21888242871839275222246405745257275088548364400416034343698204186575808495617
                val = ((p + 1) // 2 * (1 << 256)) % p
                self._inv2 = np.frombuffer(val.to_bytes(32, "little"), dtype=np.uint64).copy()
            else:
                p = 2**64 - 2**32 + 1
                self._inv2 = np.array([(p + 1) // 2, 0], dtype=np.uint64)
        return self._inv2

    def _pt(self, point):
        return np.ascontiguousarray(np.stack(point) if len(point) else np.zeros((0, self.w), np.uint64), dtype=np.uint64)

    # -- commitments
    def commit_setup(self, n):
        import importlib
        self.pcs = importlib.import_module("deep_prove_b200.pcs")
        return self.pcs.G1Bases.synthetic(self.ctx, n, 1)

    def commit(self, srs, tables):
        pts = self.pcs.batch_commit(self.ctx, srs, tables)
        return b"".join(int(x).to_bytes(32, "little") + int(y).to_bytes(32, "little") for x, y in pts)

    # -- tables
    def int_table(self, arr):
        a = np.ascontiguousarray(arr, dtype=np.int64)
        if not self.int_tables:
            return self.ctx.upload_i64(a, self.base)
        fits32 = a.size == 0 or (int(a.min()) >= -2**31 and int(a.max()) < 2**31)
        return self.ctx.upload_ints(a, self.i32 if fits32 else self.i64)

    def tensor(self, arr):
        return self.ctx.upload_tensor_i64(arr)

    def num_vars(self, table):
        return int(table.len).bit_length() - 1

    def chunks(self, table, n_chunks):
        if n_chunks == 1:
            return [table]
        per = table.len // n_chunks
        views = [table.view(i * per, per) for i in range(n_chunks)]
        self._kept += views
        return views

    def einsum_prove(self, T, lhs, lhs_shape, lhs_kinds, lhs_points, rhs, rhs_shape, rhs_kinds, rhs_points):
        pt = lambda ps: [self._pt(p) if p is not None else None for p in ps]
        lo = self.prover.EinsumOperand(None, lhs_kinds, pt(lhs_points), device_tensor=lhs)
        ro = self.prover.EinsumOperand(None, rhs_kinds, pt(rhs_points), device_tensor=rhs)
        payload = self.prover.einsum_prove(self.ctx, [lo], [ro], T)
        lhs[0].free()
        rhs[0].free()
        return payload

    def fix_axes(self, tensor, kinds, points):
        pts = [self._pt(p) if p is not None else None for p in points]
        owner, tabs = self.ctx.einsum_fix_axes(self.fam, None, kinds, pts, device_tensor=tensor)
        tensor[0].free()
        return owner, tabs

    def eq_table(self, point):
        return self.ctx.eq_table(self.fam, self._pt(point))

    def eq_values(self, point):
        t = self.eq_table(point)
        v = t.to_host().reshape(-1, self.w)
        t.free()
        return [v[i].copy() for i in range(v.shape[0])]

    def fix_low(self, table, point):
        return self.ctx.fix_low(table, self._pt(point))

    def fix_high(self, table, point):
        return self.ctx.fix_high(table, self._pt(point))

    def permuted_eq(self, eq):
        return self.dpb.rope_permuted_eq(self.ctx, eq)

    def evaluate(self, table, point):
        return self.ctx.evaluate(table, self._pt(point))

    # -- sumchecks
    def _prove(self, T, n, tables, term_array):
        st = self.prover.IOPProverState.prove(self.ctx, n, tables, term_array, T)
        point = [r.copy() for r in st.collect_raw_challenges()]
        finals = [r.copy() for r in st.get_mle_flatten_final_evaluations()]
        payload = self.export(st.proof) + self.export(st.collect_raw_challenges()) + \
            self.export(st.get_mle_flatten_final_evaluations())
        return payload, point, finals

    def sumcheck(self, T, n, tables, terms):
        arr = self.dpb.make_terms([(self._one if c is None else c, idx) for c, idx in terms],
                                  lambda c: np.ascontiguousarray(c, dtype=np.uint64).tobytes())
        return self._prove(T, n, tables, arr)

    def wit(self, i):
        return _Expr(self.prover.Expression.WitIn(i))

    def const(self, c):
        return _Expr(self.prover.Expression.Constant(np.ascontiguousarray(c, dtype=np.uint64).tobytes()))

    def chal(self, i):
        zero = np.zeros(self.w, dtype=np.uint64).tobytes()
        return _Expr(self.prover.Expression.Challenge(i, 1, self._one.tobytes(), zero))

    def expr_sumcheck(self, T, n, tables, expr, challenges):
        ch = self._pt(challenges)
        arr = expr.e.to_terms(self.fam, ch)
        return self._prove(T, n, tables, arr)

    def same_poly(self, T, table, points):
        evals, point, ev = self.prover.same_poly_prove(self.ctx, T, table, np.stack([self._pt(p) for p in points]))
        return self.export(evals) + self.export(point) + self.export(ev)

    # -- lookups
    def new_counts(self, bits):
        c = self.dpb.LookupCounts(self.ctx, bits)
        self._kept.append(c)
        return c

    def count_rows(self, counts, rows):
        """Lookups without a decomposition (the logits layer's range-check chunks)."""
        counts.add_rows(rows)

    def lookup_witness(self, tensor, shape, spec, table_out, n_cols, counts):
        info = self.dpb.ChunkingInfo.new(spec.right_shift, spec.bits, spec.sign, spec.max_bit_size, spec.n_value)
        owner, ins, outs = self.dpb.lookup_witness(self.ctx, self.i64 if self.int_tables else self.fam, info, spec.fpm,
                                                   spec.padding, None, table_out, n_cols, counts, device_tensor=tensor)
        tensor[0].free()
        return dict(owner=owner, ins=ins, outs=outs, n_shifted=info.n_shifted_chunks, n_zeroing=info.n_zeroing_chunks)

    def multiplicities(self, counts, table_cols, sign):
        return counts.multiplicities(self.fam)

    def logup(self, T, inputs):
        P = self.prover
        arr = []
        for kind, cols, cpi, mult, cst, sep in inputs:
            if kind == "lookup":
                arr.append(P.LogUpInput.new_lookup(cols, cst, sep, cpi))
            else:
                arr.append(P.LogUpInput.new_table(cols, mult, cst, sep))
        return P.new_batch_multiple_sizes_prove(self.ctx, arr, T)

    def linking(self, T, variant, spec, out_min, out_max, shape, mles, claim_point, logup_point, weight):
        info = self.dpb.ChunkingInfo.new(spec.right_shift, spec.bits, spec.sign, spec.max_bit_size, spec.n_value)
        got = self.prover.lookup_linking_prove(self.ctx, T, variant, info, out_min, out_max, tuple(shape), mles,
                                               self._pt(claim_point), self._pt(logup_point), weight=weight)
        payload = self.export(got["sumcheck"]) + self.export(got["point"]) + self.export(got["evaluations"]) + \
            self.export(got["challenges"])
        if got["weight_eval"] is not None:
            payload += self.export(got["weight_eval"])
        return payload

    def claims_batching(self, T, polys):
        P = self.prover
        cps = [P.CommittedPoly(chunks, [(self._pt(pt), np.asarray(ev, dtype=np.uint64)) for pt, ev in claims])
               for chunks, claims in polys]
        got = P.claims_batching_prove(self.ctx, T, cps, with_rlc=True)
        payload = self.export(got["sumcheck"]) + self.export(got["point"]) + self.export(got["sumcheck_evals"]) + \
            self.export(got["rlc_challenges"])
        got["rlc"].free()
        return payload


def run_transformer_path(dpb, prover, ctx, shape=GPT2_SMALL, field="fr", seed=0, blocks=None, with_final=True,
                         int_tables=True, with_commit=False):
    """One walk on the GPU (a TransformerShape or an MlpShape).  Returns dict(seconds, tokens_per_s, by_kind, calls,
    records); `seconds` and `tokens_per_s` count the path's calls only, `commit_seconds` is the witness
    commitments' time (with_commit).  For an MlpShape "tokens" are input rows."""
    be = GpuBackend(dpb, prover, ctx, field, int_tables)
    ctx.sync()
    t0 = time.perf_counter()
    if isinstance(shape, MlpShape):
        rec, timer = mlp_path(be, shape, seed, with_commit)
    else:
        rec, timer = transformer_path(be, shape, seed, blocks, with_final, with_commit)
    ctx.sync()
    wall = time.perf_counter() - t0
    commit_s = timer.by_kind.get("witness_commit", 0.0)
    path_s = sum(timer.by_kind.values()) - commit_s
    return dict(seconds=path_s, commit_seconds=commit_s, wall_seconds=wall,
                tokens_per_s=(shape.batch if isinstance(shape, MlpShape) else shape.seq) / path_s if path_s else None,
                by_kind=dict(timer.by_kind), calls=dict(timer.calls), records=rec)
