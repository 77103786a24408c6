"""Python face of the host-side prover layer (include/dpb_prover.h), with the
names the reference's callers use: Blake3Transcript, Expression,
IOPProverState.prove, hadamard / same_poly provers, LogUpInput and
new_batch_multiple_sizes_prove.  Everything here forwards to libdpb.so; the
transcript and the expression algebra run in its C++ host code, the rounds on
the GPU.
"""
import ctypes

import numpy as np

from . import (FR, GL_EXT, LOGUP_LOOKUP, LOGUP_TABLE, Term, _buf, _int, _pp, _u32, _vp, chal_dtype, check,
               elem_words, lib)


class ExprNode(ctypes.Structure):
    _fields_ = [("op", ctypes.c_uint32), ("a", ctypes.c_uint32), ("b", ctypes.c_uint32), ("pad", ctypes.c_uint32),
                ("c0", ctypes.c_uint8 * 32), ("c1", ctypes.c_uint8 * 32)]


class LogupInputStruct(ctypes.Structure):
    _fields_ = [("kind", ctypes.c_int), ("columns", _pp), ("n_columns", ctypes.c_uint32),
                ("columns_per_instance", ctypes.c_uint32), ("multiplicities", ctypes.c_void_p),
                ("constant_challenge", ctypes.c_void_p), ("column_separation_challenge", ctypes.c_void_p)]


class CommittedPolyStruct(ctypes.Structure):
    _fields_ = [("chunks", _pp), ("n_chunks", ctypes.c_uint32), ("n_claims", ctypes.c_uint32),
                ("claim_points", ctypes.c_void_p), ("claim_evals", ctypes.c_void_p)]


class EinsumOperandStruct(ctypes.Structure):
    _fields_ = [("tensor", ctypes.c_void_p), ("tensor_on_device", ctypes.c_int32), ("rank", ctypes.c_uint32),
                ("shape", ctypes.c_void_p), ("axis_kind", ctypes.c_void_p), ("axis_points", ctypes.c_void_p),
                ("axis_point_len", ctypes.c_void_p)]


_size_t = ctypes.c_size_t
PROVER_SIGNATURES = {
    "dpb_transcript_new": (_int, [_int, _vp, _size_t, _pp]),
    "dpb_transcript_clone": (_int, [_vp, _pp]),
    "dpb_transcript_free": (None, [_vp]),
    "dpb_transcript_append_scalars": (_int, [_vp, _vp, _u32]),
    "dpb_transcript_append_and_sample": (_int, [_vp, _vp, _size_t, _vp]),
    "dpb_transcript_challenge_scalar": (_int, [_vp, _vp]),
    "dpb_transcript_state": (_int, [_vp, _vp, ctypes.POINTER(_u32)]),
    "dpb_expr_to_terms": (_int, [_int, ctypes.POINTER(ExprNode), _u32, _vp, _u32, ctypes.POINTER(Term), _u32,
                                 ctypes.POINTER(_u32)]),
    "dpb_expr_eval": (_int, [_int, ctypes.POINTER(ExprNode), _u32, _vp, _u32, _vp, _u32, _vp]),
    "dpb_lookup_padding_evaluation": (_int, [_int, _vp, _vp, _u32, _vp, _u32, _vp]),
    "dpb_scalar_inverse": (_int, [_int, _vp, _vp]),
    "dpb_bias_evaluation": (_int, [_int, _vp, _u32, _vp, _vp, _vp, _u32, _vp, _vp, _vp, _u32, ctypes.POINTER(_u32)]),
    "dpb_prove_sumcheck": (_int, [_vp, _u32, _pp, _u32, ctypes.POINTER(Term), _u32, _vp, _vp, _u32, _vp, _vp,
                                  ctypes.POINTER(_u32)]),
    "dpb_prove_sumcheck_sharded": (_int, [_vp, _u32, _pp, _u32, ctypes.POINTER(Term), _u32, _vp, _vp, _u32, _vp, _vp,
                                          ctypes.POINTER(_u32)]),
    "dpb_hadamard_prove": (_int, [_vp, _vp, _vp, _vp, _u32, _vp, _vp, _vp, _vp]),
    "dpb_same_poly_prove": (_int, [_vp, _vp, _vp, _u32, _u32, _vp, _vp, _vp, _vp]),
    "dpb_claims_batching_prove": (_int, [_vp, ctypes.POINTER(CommittedPolyStruct), _u32, _vp, _vp, _u32, _vp,
                                         ctypes.POINTER(_u32), _vp, _u32, _vp, _pp]),
    "dpb_lookup_linking_prove": (_int, [_vp, _int, _vp, ctypes.c_int64, ctypes.c_int64, _vp, _u32, _pp, _u32, _vp, _u32, _vp,
                                        _u32, _vp, _vp, _u32, _vp, _vp, _vp, _u32, ctypes.POINTER(_u32),
                                        ctypes.POINTER(_u32), _vp, _vp]),
    "dpb_logup_batch_prove": (_int, [_vp, ctypes.POINTER(LogupInputStruct), _u32, _vp, _pp]),
    "dpb_logup_batch_prove_partial": (_int, [_vp, ctypes.POINTER(LogupInputStruct), _u32, _vp, _pp]),
    "dpb_logup_proof_serialize": (_int, [_vp, _vp, _size_t, ctypes.POINTER(_size_t)]),
    "dpb_logup_proof_free": (None, [_vp]),
    "dpb_einsum_prove": (_int, [_vp, ctypes.POINTER(EinsumOperandStruct), ctypes.POINTER(EinsumOperandStruct), _u32, _vp,
                                _vp, _pp]),
    "dpb_einsum_proof_serialize": (_int, [_vp, _vp, _size_t, ctypes.POINTER(_size_t)]),
    "dpb_einsum_proof_free": (None, [_vp]),
}
for _name, (_res, _args) in PROVER_SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def _scalars(a):
    return np.ascontiguousarray(a, dtype=np.uint64)


class Blake3Transcript:
    """Blake3Transcript::new(label); challenges are uint64 arrays in the
    library's challenge-element layout of `family_dtype` (GL_EXT or FR)."""

    def __init__(self, family_dtype, label=b"m2vec", _h=None):
        self.family = chal_dtype(family_dtype)
        self.words = elem_words(self.family)
        if _h is None:
            _h = ctypes.c_void_p()
            check(lib.dpb_transcript_new(self.family, label, len(label), ctypes.byref(_h)))
        self.h = _h

    def clone(self):
        h = ctypes.c_void_p()
        check(lib.dpb_transcript_clone(self.h, ctypes.byref(h)))
        return Blake3Transcript(self.family, _h=h)

    def append_scalars(self, scalars):
        s = _scalars(scalars).reshape(-1, self.words)
        check(lib.dpb_transcript_append_scalars(self.h, _buf(s) if s.size else None, s.shape[0]))

    def append_and_sample(self, label):
        out = np.zeros(self.words, dtype=np.uint64)
        check(lib.dpb_transcript_append_and_sample(self.h, label, len(label), _buf(out)))
        return out

    def challenge_scalar(self):
        out = np.zeros(self.words, dtype=np.uint64)
        check(lib.dpb_transcript_challenge_scalar(self.h, _buf(out)))
        return out

    def state(self):
        st = (ctypes.c_uint8 * 32)()
        rnd = ctypes.c_uint32()
        check(lib.dpb_transcript_state(self.h, st, ctypes.byref(rnd)))
        return bytes(st), rnd.value

    def free(self):
        if self.h:
            lib.dpb_transcript_free(self.h)
            self.h = None


class Expression:
    """dp_crypto::Expression: WitIn / Constant / Challenge closed under + - *
    and negation, kept as a postfix program for the C ABI.  Constants and
    challenge scalars are native challenge-element bytes."""
    WITIN, CONSTANT, CHALLENGE, ADD, SUB, MUL, NEG = range(7)

    def __init__(self, nodes):
        self.nodes = nodes

    @staticmethod
    def WitIn(i):
        return Expression([(Expression.WITIN, i, 0, b"", b"")])

    @staticmethod
    def Constant(c):
        return Expression([(Expression.CONSTANT, 0, 0, bytes(c), b"")])

    @staticmethod
    def Challenge(i, power, scalar, offset):
        return Expression([(Expression.CHALLENGE, i, power, bytes(scalar), bytes(offset))])

    def _bin(self, o, op):
        return Expression(self.nodes + o.nodes + [(op, 0, 0, b"", b"")])

    def __add__(self, o): return self._bin(o, Expression.ADD)
    def __sub__(self, o): return self._bin(o, Expression.SUB)
    def __mul__(self, o): return self._bin(o, Expression.MUL)
    def __neg__(self): return Expression(self.nodes + [(Expression.NEG, 0, 0, b"", b"")])

    def _array(self):
        arr = (ExprNode * len(self.nodes))()
        for i, (op, a, b, c0, c1) in enumerate(self.nodes):
            arr[i].op, arr[i].a, arr[i].b = op, a, b
            for j, v in enumerate(c0):
                arr[i].c0[j] = v
            for j, v in enumerate(c1):
                arr[i].c1[j] = v
        return arr

    def to_terms(self, family_dtype, challenges):
        """VirtualPolynomialsBuilder::to_virtual_polys: a ctypes array of Term."""
        ch = _scalars(challenges)
        n_ch = 0 if ch.size == 0 else ch.reshape(-1, elem_words(chal_dtype(family_dtype))).shape[0]
        arr = self._array()
        n = ctypes.c_uint32()
        check(lib.dpb_expr_to_terms(family_dtype, arr, len(arr), _buf(ch) if n_ch else None, n_ch, None, 0,
                                    ctypes.byref(n)))
        out = (Term * max(n.value, 1))()
        check(lib.dpb_expr_to_terms(family_dtype, arr, len(arr), _buf(ch) if n_ch else None, n_ch, out, n.value,
                                    ctypes.byref(n)))
        return (Term * n.value).from_buffer_copy(bytes(out)[:ctypes.sizeof(Term) * n.value]) if n.value else (Term * 0)()

    def evaluate(self, family_dtype, wit_evals, challenges):
        """eval_by_expr_with_instance"""
        w = elem_words(chal_dtype(family_dtype))
        we = _scalars(wit_evals).reshape(-1, w)
        ch = _scalars(challenges).reshape(-1, w)
        out = np.zeros(w, dtype=np.uint64)
        arr = self._array()
        check(lib.dpb_expr_eval(family_dtype, arr, len(arr), _buf(we) if we.size else None, we.shape[0],
                                _buf(ch) if ch.size else None, ch.shape[0], _buf(out)))
        return out


class IOPProverState:
    """Result of IOPProverState::prove: `proof` (round evaluations,
    [num_vars, degree+1, words]), collect_raw_challenges(),
    get_mle_flatten_final_evaluations()."""

    def __init__(self, proof, point, finals):
        self.proof, self._point, self._finals = proof, point, finals

    @staticmethod
    def prove(ctx, num_vars, mles, term_array, transcript, sharded=False):
        """sharded=True: `mles` are this rank's shards, num_vars counts all
        variables, and every rank of the context's communicator makes this call."""
        k = len(mles)
        w = elem_words(chal_dtype(mles[0].dtype))
        d = max(t.n_factors for t in term_array)
        hs = (ctypes.c_void_p * k)(*[m.h for m in mles])
        evals = np.zeros((num_vars, d + 1, w), dtype=np.uint64)
        point = np.zeros((num_vars, w), dtype=np.uint64)
        finals = np.zeros((k, w), dtype=np.uint64)
        deg = ctypes.c_uint32()
        fn = lib.dpb_prove_sumcheck_sharded if sharded else lib.dpb_prove_sumcheck
        check(fn(ctx.h, num_vars, hs, k, term_array, len(term_array), transcript.h, _buf(evals),
                                     num_vars * (d + 1), _buf(point), _buf(finals), ctypes.byref(deg)))
        return IOPProverState(evals, point, finals)

    def collect_raw_challenges(self):
        return self._point

    def get_mle_flatten_final_evaluations(self):
        return self._finals

    def extract_sum(self):
        raise NotImplementedError("add proof[0][0] and proof[0][1] in the field of your choice")


def lookup_padding_evaluation(family_dtype, padding_value, shape, point):
    """compute_lookup_padding_evaluation (zkml/src/lookup/operation/mod.rs:289-340); host arithmetic."""
    w = elem_words(chal_dtype(family_dtype))
    pv, pt = _scalars(padding_value).reshape(w), _scalars(point).reshape(-1, w)
    shp = (ctypes.c_uint64 * len(shape))(*shape)
    out = np.zeros(w, dtype=np.uint64)
    check(lib.dpb_lookup_padding_evaluation(family_dtype, _buf(pv), shp, len(shape), _buf(pt) if pt.size else None,
                                            pt.shape[0], _buf(out)))
    return out


def scalar_inverse(family_dtype, a):
    """dpb_scalar_inverse: 1 / a for a challenge element (0 -> 0)."""
    x = _scalars(a).reshape(elem_words(chal_dtype(family_dtype)))
    out = np.zeros_like(x)
    check(lib.dpb_scalar_inverse(family_dtype, _buf(x), _buf(out)))
    return out


def bias_evaluation(family_dtype, output_shape, axis_in_bias, bias_axis_position, point, bias_eval):
    """AxesMapping::compute_bias_evaluation (zkml/src/layers/einsum/axis.rs:655-720) -> (evaluation, bias point)."""
    w = elem_words(chal_dtype(family_dtype))
    pt, be = _scalars(point).reshape(-1, w), _scalars(bias_eval).reshape(w)
    rank = len(output_shape)
    shp = (ctypes.c_uint64 * rank)(*output_shape)
    pres = (ctypes.c_uint8 * rank)(*[1 if a else 0 for a in axis_in_bias])
    pos = (ctypes.c_uint32 * rank)(*[int(p) for p in bias_axis_position])
    out = np.zeros(w, dtype=np.uint64)
    bp = np.zeros((max(pt.shape[0], 1), w), dtype=np.uint64)
    n = ctypes.c_uint32()
    check(lib.dpb_bias_evaluation(family_dtype, shp, rank, pres, pos, _buf(pt) if pt.size else None, pt.shape[0], _buf(be),
                                  _buf(out), _buf(bp), bp.shape[0], ctypes.byref(n)))
    return out, bp[: n.value]


def hadamard_prove(ctx, transcript, claim_point, v1, v2):
    """zkml/src/layers/hadamard.rs:93-131 -> (round evals [n,4,w], point [n,w], claims [2,w])"""
    p = _scalars(claim_point)
    w = elem_words(chal_dtype(v1.dtype))
    p = p.reshape(-1, w)
    n = p.shape[0]
    evals = np.zeros((n, 4, w), dtype=np.uint64)
    point = np.zeros((n, w), dtype=np.uint64)
    claims = np.zeros((2, w), dtype=np.uint64)
    check(lib.dpb_hadamard_prove(ctx.h, v1.h, v2.h, _buf(p), n, transcript.h, _buf(evals), _buf(point), _buf(claims)))
    return evals, point, claims


def same_poly_prove(ctx, transcript, poly, points):
    """zkml/src/iop/same_poly.rs:84-114; points: [n_claims, n, w]"""
    w = elem_words(chal_dtype(poly.dtype))
    p = _scalars(points).reshape(len(points), -1, w)
    m, n = p.shape[0], p.shape[1]
    evals = np.zeros((n, 3, w), dtype=np.uint64)
    point = np.zeros((n, w), dtype=np.uint64)
    ev = np.zeros(w, dtype=np.uint64)
    check(lib.dpb_same_poly_prove(ctx.h, poly.h, _buf(p), m, n, transcript.h, _buf(evals), _buf(point), _buf(ev)))
    return evals, point, ev


VARIANT_STANDARD, VARIANT_GLU, VARIANT_SOFTMAX, VARIANT_NORMALISATION, VARIANT_NORMALISATION_WITH_SUM = 0, 1, 2, 3, 4


def lookup_linking_prove(ctx, transcript, variant, info, table_min_output, table_max_output, shape, mles,
                         last_claim_point, logup_point, weight=None):
    """LookupInputConfig::prove_linking_sumcheck (zkml/src/lookup/operation/inputs/proving.rs:26-114), Standard and
    GLU variants.  info: ChunkingInfo; shape: the operation's unpadded input shape; mles: the witness tables in
    the expression's order; points: [coords, w].  Returns dict(sumcheck [n, d+1, w], point [n, w],
    evaluations [len(mles), w], challenges [1 + slices (+ the variant's own), w], weight_eval [w] or None).
    weight: the Normalisation variant's weight table (an Mle) or None."""
    w = elem_words(chal_dtype(mles[0].dtype))
    cp, lp = _scalars(last_claim_point).reshape(-1, w), _scalars(logup_point).reshape(-1, w)
    n = lp.shape[0]
    rank = len(shape)
    shp = (ctypes.c_uint64 * rank)(*shape)
    slices = 1
    for d in shape[:-2]:
        slices *= d
    hs = (ctypes.c_void_p * len(mles))(*[m.h for m in mles])
    cap = n * 9  # degree at most 8 factors per term
    evals = np.zeros((cap, w), dtype=np.uint64)
    point = np.zeros((n, w), dtype=np.uint64)
    finals = np.zeros((len(mles), w), dtype=np.uint64)
    chal = np.zeros((3 + slices, w), dtype=np.uint64)
    weight_eval = np.zeros(w, dtype=np.uint64)
    n_chal, degree = ctypes.c_uint32(), ctypes.c_uint32()
    check(lib.dpb_lookup_linking_prove(ctx.h, variant, ctypes.byref(info), table_min_output, table_max_output, shp, rank, hs,
                                       len(mles), _buf(cp), cp.shape[0], _buf(lp), n, transcript.h, _buf(evals), cap,
                                       _buf(point), _buf(finals), _buf(chal), 3 + slices, ctypes.byref(n_chal),
                                       ctypes.byref(degree), weight.h if weight is not None else None, _buf(weight_eval)))
    d = degree.value
    return dict(sumcheck=evals[: n * (d + 1)].reshape(n, d + 1, w), point=point, evaluations=finals,
                challenges=chal[: n_chal.value], weight_eval=weight_eval if weight is not None else None)


class CommittedPoly:
    """A committed polynomial as its chunk tables (a power of two of them, equal lengths) and the claims
    (point, eval) to batch for it (zkml/src/poly_commit/mod.rs:32-93)."""

    def __init__(self, chunks, claims):
        self.chunks = list(chunks)
        self.claims = list(claims)


def claims_batching_prove(ctx, transcript, polys, with_rlc=True):
    """CommitmentProver::claims_batching_sumcheck and the random linear combination that follows it
    (zkml/src/poly_commit/prover.rs:113-131, 140-255).
    Returns dict(sumcheck [n,3,w], point [n,w], sumcheck_evals [chunks,w], rlc_challenges, rlc Mle)."""
    from . import Mle
    w = elem_words(chal_dtype(polys[0].chunks[0].dtype))
    arr = (CommittedPolyStruct * len(polys))()
    keep = []
    total_chunks, max_vars = 0, 0
    for i, p in enumerate(polys):
        hs = (ctypes.c_void_p * len(p.chunks))(*[m.h for m in p.chunks])
        pts = _scalars([c[0] for c in p.claims]).reshape(len(p.claims), -1, w) if p.claims else np.zeros((0, 0, w), np.uint64)
        evs = _scalars([c[1] for c in p.claims]).reshape(len(p.claims), w) if p.claims else np.zeros((0, w), np.uint64)
        keep += [hs, pts, evs]
        arr[i].chunks = hs
        arr[i].n_chunks = len(p.chunks)
        arr[i].n_claims = len(p.claims)
        arr[i].claim_points = pts.ctypes.data if p.claims else None
        arr[i].claim_evals = evs.ctypes.data if p.claims else None
        total_chunks += len(p.chunks)
        max_vars = max(max_vars, int(p.chunks[0].len).bit_length() - 1)
    evals = np.zeros((max_vars, 3, w), dtype=np.uint64)
    point = np.zeros((max_vars, w), dtype=np.uint64)
    sc_evals = np.zeros((total_chunks, w), dtype=np.uint64)
    chal = np.zeros((total_chunks, w), dtype=np.uint64)
    nv = ctypes.c_uint32()
    h = ctypes.c_void_p()
    check(lib.dpb_claims_batching_prove(ctx.h, arr, len(polys), transcript.h, _buf(evals), max_vars * 3, _buf(point),
                                        ctypes.byref(nv), _buf(sc_evals), total_chunks,
                                        _buf(chal) if with_rlc else None, ctypes.byref(h) if with_rlc else None))
    assert nv.value == max_vars
    return dict(sumcheck=evals, point=point, sumcheck_evals=sc_evals, rlc_challenges=chal if with_rlc else None,
                rlc=Mle(ctx, h) if with_rlc else None)


class LogUpInput:
    """zkml/src/lookup/logup_gkr/structs.rs:138-231"""

    def __init__(self, kind, columns, constant, sep, columns_per_instance=1, multiplicities=None):
        self.kind, self.columns, self.mult = kind, list(columns), multiplicities
        self.constant, self.sep = _scalars(constant), _scalars(sep)
        self.cpi = columns_per_instance

    @staticmethod
    def new_lookup(columns, constant, sep, columns_per_instance):
        return LogUpInput(LOGUP_LOOKUP, columns, constant, sep, columns_per_instance)

    @staticmethod
    def new_table(columns, multiplicities, constant, sep):
        return LogUpInput(LOGUP_TABLE, columns, constant, sep, len(columns), multiplicities)


def new_batch_multiple_sizes_prove(ctx, inputs, transcript, partial=False):
    """zkml/src/lookup/logup_gkr/prover.rs:91-344.  Returns the flat canonical
    encoding of the LogUpBatchProof (see include/dpb_prover.h).  partial: `inputs` are this rank's instances of a
    batch spread over the communicator's ranks (dpb_logup_batch_prove_partial); the proof is the whole batch's."""
    arr = (LogupInputStruct * max(len(inputs), 1))()
    keep = []
    for i, inp in enumerate(inputs):
        hs = (ctypes.c_void_p * len(inp.columns))(*[m.h for m in inp.columns])
        keep.append(hs)
        arr[i].kind = inp.kind
        arr[i].columns = hs
        arr[i].n_columns = len(inp.columns)
        arr[i].columns_per_instance = inp.cpi
        arr[i].multiplicities = inp.mult.h if inp.mult is not None else None
        arr[i].constant_challenge = inp.constant.ctypes.data
        arr[i].column_separation_challenge = inp.sep.ctypes.data
    h = ctypes.c_void_p()
    fn = lib.dpb_logup_batch_prove_partial if partial else lib.dpb_logup_batch_prove
    check(fn(ctx.h, arr, len(inputs), transcript.h, ctypes.byref(h)))
    try:
        n = ctypes.c_size_t()
        check(lib.dpb_logup_proof_serialize(h, None, 0, ctypes.byref(n)))
        buf = (ctypes.c_uint8 * n.value)()
        check(lib.dpb_logup_proof_serialize(h, buf, n.value, ctypes.byref(n)))
        return bytes(buf)
    finally:
        lib.dpb_logup_proof_free(h)


class EinsumOperand:
    """One tensor of an einsum and what happens to its axes (dpb_einsum_operand).  tensor: int64 ndarray (unpadded)
    or, with device_tensor = ctx.upload_tensor_i64(...), a tensor already on the device; kinds[a] in AXIS_*;
    points[a]: challenge elements uint64[len, words] for outer and stacked axes, None for contracted ones."""

    def __init__(self, tensor, kinds, points, device_tensor=None):
        if device_tensor is not None:
            mle, shape = device_tensor
            self._keep = [mle]
            self.ptr, self.on_device = lib.dpb_mle_device_ptr(mle.h), 1
        else:
            t = np.ascontiguousarray(tensor, dtype=np.int64)
            shape = t.shape
            self._keep = [t]
            self.ptr, self.on_device = t.ctypes.data, 0
        rank = len(shape)
        self.shape = (ctypes.c_uint64 * rank)(*shape)
        self.kinds = (ctypes.c_uint8 * rank)(*kinds)
        pts = [np.ascontiguousarray(p, dtype=np.uint64) if p is not None else None for p in points]
        self._keep.append(pts)
        self.points = (ctypes.c_void_p * rank)(*[p.ctypes.data if p is not None and p.size else None for p in pts])
        self.lens = (ctypes.c_uint32 * rank)(*[0 if p is None or not p.size else p.shape[0] for p in pts])
        self.rank = rank

    def fill(self, s):
        s.tensor, s.tensor_on_device, s.rank = self.ptr, self.on_device, self.rank
        s.shape = ctypes.cast(self.shape, ctypes.c_void_p)
        s.axis_kind = ctypes.cast(self.kinds, ctypes.c_void_p)
        s.axis_points = ctypes.cast(self.points, ctypes.c_void_p)
        s.axis_point_len = ctypes.cast(self.lens, ctypes.c_void_p)


def einsum_prove(ctx, lhs_fixes, rhs, transcript, lhs_padded=None):
    """EinSum::prove_internal (zkml/src/layers/einsum/prove.rs:48-335) below the axis mapping: lhs_fixes[i] is the
    left tensor with output i's fixes, rhs[i] the right tensor of output i (EinsumOperand each); lhs_padded (an
    Mle, the left tensor padded to powers of two per axis) is needed when there are several outputs.  Returns the
    flat canonical encoding of the proof (see include/dpb_prover.h)."""
    n = len(rhs)
    if len(lhs_fixes) != n:
        raise ValueError("one fix of the left tensor per right tensor")
    la, ra = (EinsumOperandStruct * n)(), (EinsumOperandStruct * n)()
    for i in range(n):
        lhs_fixes[i].fill(la[i])
        rhs[i].fill(ra[i])
    h = ctypes.c_void_p()
    check(lib.dpb_einsum_prove(ctx.h, la, ra, n, lhs_padded.h if lhs_padded is not None else None, transcript.h,
                               ctypes.byref(h)))
    try:
        sz = ctypes.c_size_t()
        check(lib.dpb_einsum_proof_serialize(h, None, 0, ctypes.byref(sz)))
        buf = (ctypes.c_uint8 * sz.value)()
        check(lib.dpb_einsum_proof_serialize(h, buf, sz.value, ctypes.byref(sz)))
        return bytes(buf)
    finally:
        lib.dpb_einsum_proof_free(h)
