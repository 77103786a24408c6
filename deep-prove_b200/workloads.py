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


GPT2_SMALL = TransformerShape("gpt2-small", layers=12, seq=512, d_model=768, heads=12, head_dim=64, ffn=3072,
                              vocab=50257)
# the same graph at a size a CPU restatement proves in seconds: every call of the walk, one block
TINY = TransformerShape("tiny", layers=1, seq=24, d_model=48, heads=3, head_dim=16, ffn=80, vocab=200, table_bits=8,
                        commit_chunk_log2=8, range_check_chunks=2)


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
    if table in ("gelu", "norm"):
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


def transformer_path(be, shape, seed=0, blocks=None, with_final=True, with_commit=False):
    """Walks the path calls of `shape` on backend `be`.  Returns (records, timer): records is a list of
    (name, kind, payload bytes); timer.by_kind holds seconds per kind of call.  `blocks` limits the number of
    transformer blocks walked (default: all); `with_final=False` leaves out everything after the last block.
    with_commit: every lookup layer also commits to its witness columns (one multi-scalar multiplication per
    chunk of at most 2^commit_chunk_log2 evaluations, zkml/src/lookup/context.rs:420-422), timed as its own kind
    "witness_commit": the commitment scheme's share of a proof, next to the path's."""
    rng = np.random.default_rng(seed)
    T = be.new_transcript()
    timer = PathTimer(be)
    rec = []
    s, e, h, dh, f, V = shape.seq, shape.d_model, shape.heads, shape.head_dim, shape.ffn, shape.vocab
    bits = shape.table_bits
    lg = ceil_log2
    n_blocks = shape.layers if blocks is None else blocks

    # ---- per-table logup challenges (ChallengeStorage, zkml/src/iop/mod.rs:174-187) and lookup counters
    table_keys = ["shift", "zero", "signed", "requant", "gelu", "exp", "norm"]
    chal = {k: tuple(be.squeeze(T, 2)) for k in table_keys}
    counts = {"shift": be.new_counts(16), "zero": be.new_counts(16), "signed": be.new_counts(16)}
    for k in ("requant", "gelu", "exp", "norm"):
        counts[k] = be.new_counts(bits)
    committed = []  # (name, table handle, num entries): everything the claim batching at the end opens
    srs = be.commit_setup(1 << shape.commit_chunk_log2) if with_commit else None

    act_bits = bits + 2
    specs = {
        "requant": LookupSpec("requant", bits, right_shift=bits + 1, max_bit_size=2 * bits + 4, sign=SIGN_MIXED),
        "gelu": LookupSpec("gelu", bits, right_shift=bits + 1, max_bit_size=2 * bits + 4, sign=SIGN_MIXED),
        "exp": LookupSpec("exp", bits, right_shift=bits - 2, max_bit_size=2 * bits + 10, sign=SIGN_NEGATIVE),
        "norm": LookupSpec("norm", bits, right_shift=bits, max_bit_size=2 * bits + 2, sign=SIGN_MIXED),
    }

    def small(shape_):
        return rng.integers(-(1 << (act_bits - 1)), 1 << (act_bits - 1), size=shape_, dtype=np.int64)

    def weights(shape_):
        return rng.integers(-(1 << (bits - 1)), 1 << (bits - 1), size=shape_, dtype=np.int64)

    def commit_weight(name, w):
        """A weight matrix as a committed polynomial: padded to powers of two per dimension, as field elements."""
        dims = [1 << lg(d) for d in w.shape]
        padded = np.zeros(dims, dtype=np.int64)
        padded[tuple(slice(0, d) for d in w.shape)] = w
        committed.append((name, be.int_table(padded.reshape(-1)), padded.size))

    # ------------------------------------------------------------------ the calls
    def einsum(name, lhs, lhs_kinds, rhs, rhs_kinds):
        """EinSum::prove_internal: fix the outer axes of both tensors at the output claim's point, keep the
        stacked axes as one table each, sumcheck over the contracted axis
        sum_t coef_t * lhs_t * rhs_t with the stacking coefficients eq(r_stack, t) (einsum/axis.rs:1043-1062)."""
        lhs_dev, rhs_dev = be.tensor(lhs), be.tensor(rhs)  # resident before the clock starts
        with timer("einsum_fix_axes"):
            lp = [be.squeeze(T, lg(d)) if k == AX_OUTER else None for d, k in zip(lhs.shape, lhs_kinds)]
            rp = [be.squeeze(T, lg(d)) if k == AX_OUTER else None for d, k in zip(rhs.shape, rhs_kinds)]
            lt_owner, lt = be.fix_axes(lhs_dev, lhs_kinds, lp)
            rt_owner, rt = be.fix_axes(rhs_dev, rhs_kinds, rp)
        H = len(lt)
        assert len(rt) == H
        with timer("einsum_sumcheck"):
            if H > 1:
                coef = be.eq_values(be.squeeze(T, lg(H)))[:H]
            else:
                coef = [None]
            n = be.num_vars(lt[0])
            payload, point, finals = be.sumcheck(T, n, lt + rt, [(coef[t], [t, H + t]) for t in range(H)])
        rec.append((name, "einsum", payload))
        be.free(lt_owner, rt_owner)

    def lookup_layer(name, tensor, spec, variant=VARIANT_STANDARD, weight=None):
        """prove_lookup_op: witness columns -> batched logup-GKR over the lookups -> linking sumcheck."""
        sign, table_out, n_cols = value_table(spec.table, spec.bits)
        tensor_dev = be.tensor(tensor)
        with timer("lookup_witness"):
            cs = [counts["shift"], counts[spec.table], counts["zero"], counts["signed"]]
            wit = be.lookup_witness(tensor_dev, tensor.shape, spec, table_out, n_cols, cs)
            ins, outs = wit["ins"], wit["outs"]
        slices = int(np.prod(tensor.shape[:-2])) if tensor.ndim > 2 else 1
        n_sh, n_z = wit["n_shifted"], wit["n_zeroing"]
        per_in = n_sh + (spec.n_value if n_cols != 1 else 0) + n_z
        per_out = spec.n_value + n_z
        signed = sign == SIGN_MIXED
        groups = {"shift": [], spec.table: [], "zero": [], "signed": []}
        for c in range(slices):
            i0, o0 = c * per_in, c * per_out
            groups["shift"] += ins[i0:i0 + n_sh]
            for v in range(spec.n_value):
                if n_cols != 1:
                    groups[spec.table] += [ins[i0 + n_sh + v], outs[o0 + v]]
                else:
                    groups[spec.table] += [outs[o0 + v]]
            zi0 = i0 + n_sh + (spec.n_value if n_cols != 1 else 0)
            for z in range(n_z):
                key = "signed" if (signed and z == n_z - 1) else "zero"
                groups[key] += [ins[zi0 + z], outs[o0 + spec.n_value + z]]
        inputs = []
        for key, cpi in (("shift", 1), (spec.table, 2 if n_cols != 1 else 1), ("zero", 2), ("signed", 2)):
            if groups[key]:
                inputs.append(("lookup", groups[key], cpi, None, chal[key][0], chal[key][1]))
        with timer("lookup_logup"):
            rec.append((name + ".logup", "logup", be.logup(T, inputs)))
        dims = [1 << lg(d) for d in tensor.shape]
        total = sum(lg(d) for d in dims)
        n2d = sum(lg(d) for d in dims[-2:]) if tensor.ndim > 1 else lg(dims[-1])
        if table_out is None:
            out_min, out_max = table_input_range(spec.bits, sign)
        else:
            out_min, out_max = int(table_out[0]), int(table_out[-1])
        mles = list(outs)
        extra_owner = []
        if variant in (VARIANT_NORMALISATION, VARIANT_NORMALISATION_WITH_SUM):
            # one input table and one scaling table per slice (variant.rs:288-346)
            P = 1 << n2d
            for _ in range(2 * slices):
                tab = be.int_table(small(P))
                extra_owner.append(tab)
                mles.append(tab)
        with timer("lookup_linking"):
            claim_point = be.squeeze(T, total)
            logup_point = be.squeeze(T, n2d)
            payload = be.linking(T, variant, spec, out_min, out_max, tensor.shape, mles, claim_point, logup_point, weight)
        rec.append((name + ".linking", "linking", payload))
        # the witness columns are committed polynomials: they are opened at the end
        for j, col in enumerate(ins + outs):
            committed.append((f"{name}.w{j}", col, 1 << n2d))
        if with_commit:
            n_chunks = 1 << max(n2d - shape.commit_chunk_log2, 0)
            with timer("witness_commit"):
                chunks = [c_ for col in ins + outs for c_ in be.chunks(col, n_chunks)]
                rec.append((name + ".commit", "commit", be.commit(srs, chunks)))
        be.free(*extra_owner)
        be.keep(wit["owner"])

    def same_poly(name, n_entries, n_claims):
        """Two claims on the residual stream merged into one (flatten_and_merge_claims, iop/prover.rs:1064-1101)."""
        tab = be.int_table(small(n_entries))
        with timer("same_poly"):
            pts = [be.squeeze(T, lg(n_entries)) for _ in range(n_claims)]
            rec.append((name, "same_poly", be.same_poly(T, tab, pts)))
        be.free(tab)

    def expr_sumcheck(name, kind, n, tables, expr, challenges):
        with timer(kind):
            payload, point, finals = be.expr_sumcheck(T, n, tables, expr, challenges)
        rec.append((name, kind, payload))

    def attention_mask(name, batch, seq):
        """AttentionMask::prove_internal: eq * row_lt * col_lt * sum_j chi_j (mask * in_j + NEG (1 - mask)),
        tables eq, mask, row_lt, col_lt, then one input table per head (attention_mask/mod.rs:115-159)."""
        ps = 1 << lg(seq)
        n = 2 * lg(seq)
        i = np.arange(ps)
        mask = (i[None, :] <= i[:, None]).astype(np.int64)           # lower triangular
        row_lt = np.repeat((i < seq).astype(np.int64), ps)
        col_lt = np.tile((i < seq).astype(np.int64), ps)
        fixed = [be.int_table(mask.reshape(-1)), be.int_table(row_lt), be.int_table(col_lt)]
        fixed += [be.int_table(small(ps * ps)) for _ in range(batch)]
        with timer("attention_mask"):
            tabs = [be.eq_table(be.squeeze(T, n))] + fixed
            chi = be.eq_values(be.squeeze(T, lg(batch)))[:batch] if batch > 1 else [be.scalar(1)]
            neg = be.const(be.scalar(-(1 << (2 * bits))))
            lead = be.wit(0) * (be.wit(2) * be.wit(3))
            one_minus = be.const(be.scalar(1)) - be.wit(1)
            e_ = None
            for j in range(batch):
                term = lead * be.chal(j) * (be.wit(1) * be.wit(4 + j) + neg * one_minus)
                e_ = term if e_ is None else e_ + term
            payload, point, finals = be.expr_sumcheck(T, n, tabs, e_, chi)
        rec.append((name, "attention_mask", payload))
        be.free(*tabs)

    # ------------------------------------------------------------------ embeddings and positions
    if with_final:
        pv, pe = 1 << lg(V), 1 << lg(e)
        wte = np.zeros((pv, pe), dtype=np.int64)
        wte[:V, :e] = weights((V, e))
        wte_tab = be.int_table(wte.reshape(-1))
        committed.append(("wte", wte_tab, wte.size))
        one_hot = be.int_table(rng.integers(0, 3, size=pv, dtype=np.int64))
        with timer("embeddings"):
            # Embeddings::prove: bind the column variables of the padded matrix, then sum_v onehot(v) * E(v)
            col_point = be.squeeze(T, lg(pe))
            fixed = be.fix_low(wte_tab, col_point)
            payload, point, finals = be.sumcheck(T, lg(pv), [one_hot, fixed], [(None, [0, 1])])
            rec.append(("embeddings", "embeddings", payload))
        be.free(fixed, one_hot)
        # Positional (absolute): fixed_positional * lt * column_eq over the embedding columns
        ps_ = 1 << lg(e)
        tabs = [be.int_table(small(ps_)), be.int_table((np.arange(ps_) < e).astype(np.int64))]
        with timer("positional"):
            tabs.append(be.eq_table(be.squeeze(T, lg(ps_))))
            payload, point, finals = be.sumcheck(T, lg(ps_), tabs, [(None, [0, 1, 2])])
            rec.append(("positional", "positional", payload))
        be.free(*tabs)

    # ------------------------------------------------------------------ transformer blocks
    for b in range(n_blocks):
        pre = f"block{b}."
        x = small((s, e))
        gamma = be.int_table(np.tile(np.pad(weights(e), (0, (1 << lg(e)) - e)), 1 << lg(s)))
        lookup_layer(pre + "ln1", draw_tensor(rng, (s, e), specs["norm"]), specs["norm"], VARIANT_NORMALISATION, gamma)
        w_qkv = weights((e, 3 * e))
        commit_weight(pre + "w_qkv", w_qkv)
        einsum(pre + "qkv", x, (AX_OUTER, AX_CONTRACTED), w_qkv, (AX_CONTRACTED, AX_OUTER))
        lookup_layer(pre + "qkv.requant", draw_tensor(rng, (s, 3 * e), specs["requant"]), specs["requant"])
        q, k_, v_ = small((h, s, dh)), small((h, s, dh)), small((h, s, dh))
        einsum(pre + "qk", q, (AX_STACKED, AX_OUTER, AX_CONTRACTED), k_, (AX_STACKED, AX_OUTER, AX_CONTRACTED))
        attention_mask(pre + "mask", h, s)
        lookup_layer(pre + "softmax", draw_tensor(rng, (h, s, s), specs["exp"]), specs["exp"], VARIANT_SOFTMAX)
        a = small((h, s, s))
        einsum(pre + "av", a, (AX_STACKED, AX_OUTER, AX_CONTRACTED), v_, (AX_STACKED, AX_CONTRACTED, AX_OUTER))
        lookup_layer(pre + "av.requant", draw_tensor(rng, (s, e), specs["requant"]), specs["requant"])
        w_o = weights((e, e))
        commit_weight(pre + "w_o", w_o)
        einsum(pre + "out", x, (AX_OUTER, AX_CONTRACTED), w_o, (AX_CONTRACTED, AX_OUTER))
        same_poly(pre + "residual1", (1 << lg(s)) * (1 << lg(e)), 2)
        lookup_layer(pre + "ln2", draw_tensor(rng, (s, e), specs["norm"]), specs["norm"], VARIANT_NORMALISATION, gamma)
        w_up = weights((e, f))
        commit_weight(pre + "w_up", w_up)
        einsum(pre + "ffn_up", x, (AX_OUTER, AX_CONTRACTED), w_up, (AX_CONTRACTED, AX_OUTER))
        lookup_layer(pre + "gelu", draw_tensor(rng, (s, f), specs["gelu"]), specs["gelu"])
        w_down = weights((f, e))
        commit_weight(pre + "w_down", w_down)
        einsum(pre + "ffn_down", small((s, f)), (AX_OUTER, AX_CONTRACTED), w_down, (AX_CONTRACTED, AX_OUTER))
        lookup_layer(pre + "ffn_down.requant", draw_tensor(rng, (s, e), specs["requant"]), specs["requant"])
        same_poly(pre + "residual2", (1 << lg(s)) * (1 << lg(e)), 2)
        be.free(gamma)

    # ------------------------------------------------------------------ head
    if with_final:
        gamma = be.int_table(np.tile(np.pad(weights(e), (0, (1 << lg(e)) - e)), 1 << lg(s)))
        lookup_layer("ln_f", draw_tensor(rng, (s, e), specs["norm"]), specs["norm"], VARIANT_NORMALISATION, gamma)
        be.free(gamma)
        einsum("lm_head", small((s, e)), (AX_OUTER, AX_CONTRACTED), wte[:V, :e].T.copy(), (AX_CONTRACTED, AX_OUTER))
        # Logits (argmax): the range check of max - logit over range_check_chunks 16-bit chunks, then the linking
        # sumcheck  sum_eq (max - C onehot input) + chi input_eq lt (max - input)   (logits.rs:531-670)
        ps_, pv_ = 1 << lg(s), 1 << lg(V)
        n = lg(ps_) + lg(pv_)
        logits = small((ps_, pv_))
        logits[:, V:] = 0
        arg = logits[:, :V].argmax(axis=1)
        one_hot = np.zeros((ps_, pv_), dtype=np.int64)
        one_hot[np.arange(ps_), arg] = 1
        mx = np.repeat(logits[np.arange(ps_), arg], pv_)
        lt = np.tile((np.arange(pv_) < V).astype(np.int64), ps_)
        diff = (mx - logits.reshape(-1)) * lt          # max - logit, zero in the padding
        chunk_ints = [(diff >> (16 * c_)) & 0xFFFF for c_ in range(shape.range_check_chunks)]
        cols = [be.int_table(c_) for c_ in chunk_ints]
        with timer("argmax_logup"):
            for c_ in chunk_ints:
                be.count_rows(counts["shift"], c_)
            rec.append(("argmax.logup", "logup",
                        be.logup(T, [("lookup", cols, 1, None, chal["shift"][0], chal["shift"][1])])))
        tabs = [be.int_table(logits.reshape(-1)), be.int_table(mx), be.int_table(one_hot.reshape(-1)), None, None,
                be.int_table(lt)]
        del diff, chunk_ints
        with timer("argmax_linking"):
            row_point = be.squeeze(T, lg(ps_))
            sum_eq_point = [be.inv2()] * lg(pv_) + list(row_point)
            tabs[3] = be.eq_table(sum_eq_point)
            tabs[4] = be.eq_table(be.squeeze(T, n))
            C = be.const(be.scalar(pv_))
            first = be.wit(3) * (be.wit(1) - C * be.wit(2) * be.wit(0))
            second = be.wit(4) * be.wit(5) * (be.wit(1) - be.wit(0))
            expr = first + be.chal(0) * second
            payload, point, finals = be.expr_sumcheck(T, n, tabs, expr, be.squeeze(T, 1))
            rec.append(("argmax.linking", "argmax_linking", payload))
        for c_ in cols:
            committed.append(("argmax.chunk", c_, ps_ * pv_))
        be.free(*tabs)

        # ---------------------------------------------------------------- tables' logup-GKR (prove_tables)
        inputs = []
        t16 = np.arange(1 << 16, dtype=np.int64)
        s16 = np.arange(-(1 << 15), 1 << 15, dtype=np.int64)
        table_cols = {"shift": [t16], "zero": [t16, (t16 == 0).astype(np.int64)], "signed": [s16, np.sign(s16)]}
        for key in ("requant", "gelu", "exp", "norm"):
            sign, out, n_cols = value_table(key, bits)
            lo, hi = table_input_range(bits, sign)
            ins_ = np.arange(lo, hi + 1, dtype=np.int64)
            table_cols[key] = [ins_] if out is None else [ins_, out]
        owners = []
        dev_cols = {key: [be.int_table(c_) for c_ in table_cols[key]] for key in table_keys}
        with timer("tables_logup"):
            for key in table_keys:
                mult = be.multiplicities(counts[key], table_cols[key], value_table(key, bits)[0] if key in specs else None)
                owners += dev_cols[key] + [mult]
                inputs.append(("table", dev_cols[key], len(dev_cols[key]), mult, chal[key][0], chal[key][1]))
            # a batch is ordered by non-increasing size (prover.rs:95-140)
            inputs.sort(key=lambda i_: -be.num_vars(i_[1][0]))
            rec.append(("tables.logup", "logup", be.logup(T, inputs)))
        be.free(*owners)

        # ---------------------------------------------------------------- claim batching over every committed polynomial
        with timer("claim_batching"):
            polys = []
            cmax = shape.commit_chunk_log2
            for name, tab, entries in committed:
                nv = lg(entries)
                n_chunks = 1 << max(nv - cmax, 0)
                point = be.squeeze(T, nv)
                ev = be.squeeze(T, 1)[0]
                polys.append((be.chunks(tab, n_chunks), [(point, ev)]))
            rec.append(("claim_batching", "claim_batching", be.claims_batching(T, polys)))
    rec.append(("transcript", "state", be.transcript_state(T)))
    be.free(srs)
    be.release()
    return rec, timer


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
    """One walk on the GPU.  Returns dict(seconds, tokens_per_s, by_kind, calls, records); `seconds` and
    `tokens_per_s` count the path's calls only, `commit_seconds` is the witness commitments' time (with_commit)."""
    be = GpuBackend(dpb, prover, ctx, field, int_tables)
    ctx.sync()
    t0 = time.perf_counter()
    rec, timer = transformer_path(be, shape, seed, blocks, with_final, with_commit)
    ctx.sync()
    wall = time.perf_counter() - t0
    commit_s = timer.by_kind.get("witness_commit", 0.0)
    path_s = sum(timer.by_kind.values()) - commit_s
    return dict(seconds=path_s, commit_seconds=commit_s, wall_seconds=wall,
                tokens_per_s=shape.seq / path_s if path_s else None,
                by_kind=dict(timer.by_kind), calls=dict(timer.calls), records=rec)
