"""ctypes binding of libdpb.so, the C-ABI library of the B200 sumcheck /
multilinear-fold / logup-GKR back end (declarations: include/dpb.h).

The directory name is not a Python identifier; load it by path under the name
`deep_prove_b200` (tests/conftest.py and bench.py show how).  There is no CPU
path: importing works without a GPU (so the exported symbols can be checked),
but creating a Context raises when no CUDA device is usable, and a missing
library raises at import.
"""
import ctypes
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "libdpb.so")

GL_BASE, GL_EXT, FR = 0, 1, 2
GL_I64, GL_I32, FR_I64, FR_I32 = 3, 4, 5, 6  # integer tables (the integers themselves, 8 or 4 bytes per entry)
INT_DTYPES = {GL_I64: np.int64, GL_I32: np.int32, FR_I64: np.int64, FR_I32: np.int32}
FORM_NATIVE, FORM_CANONICAL, FORM_I64 = 0, 1, 2
LOGUP_LOOKUP, LOGUP_TABLE = 0, 1
AXIS_CONTRACTED, AXIS_OUTER, AXIS_STACKED = 0, 1, 2
MAX_FACTORS = 8

OK, EINVAL, ENOMEM, ECUDA, ETIMEOUT, ESTATE, ENCCL = 0, -1, -2, -3, -4, -5, -6


class DpbError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"dpb error {code}: {msg}")
        self.code = code


if not os.path.exists(LIB_PATH):
    raise ImportError(
        f"{LIB_PATH} is missing: build it with `python deep-prove_b200/build.py` "
        "(nvcc, sm_100a). There is no fallback implementation.")

lib = ctypes.CDLL(LIB_PATH)


class Term(ctypes.Structure):
    _fields_ = [("coeff", ctypes.c_uint8 * 32), ("n_factors", ctypes.c_uint32),
                ("idx", ctypes.c_uint16 * MAX_FACTORS)]


class ProfileEntry(ctypes.Structure):
    _fields_ = [("kernel", ctypes.c_char * 48), ("round", ctypes.c_uint32), ("launches", ctypes.c_uint32),
                ("total_ms", ctypes.c_double), ("alg_bytes_per_launch", ctypes.c_uint64)]


_vp, _u32, _u64, _int = ctypes.c_void_p, ctypes.c_uint32, ctypes.c_uint64, ctypes.c_int
_pp = ctypes.POINTER(ctypes.c_void_p)

SIGNATURES = {
    "dpb_comm_shared_exchange": (_int, [_vp]),
    "dpb_resident_rounds": (_int, [_vp, _int, _u32]),
    "dpb_sumcheck_launches": (_u64, [_vp]),
    "dpb_trim": (_int, [_vp]),
    "dpb_mle_evaluate_many": (_int, [_vp, _pp, _u32, _vp, _u32, _vp]),
    "dpb_issue_rate_probe": (_int, [_vp, _int, _u32, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)]),
    "dpb_trace_enable": (_int, [_int]),
    "dpb_trace_read": (_int, [ctypes.c_char_p, ctypes.c_size_t, ctypes.POINTER(ctypes.c_size_t)]),
    "dpb_profile_enable": (_int, [_vp, _int]),
    "dpb_profile_read": (_int, [_vp, ctypes.POINTER(ProfileEntry), _u32, ctypes.POINTER(_u32)]),
    "dpb_init": (_int, [_int, _pp]),
    "dpb_shutdown": (None, [_vp]),
    "dpb_last_error": (ctypes.c_char_p, []),
    "dpb_sync": (_int, [_vp]),
    "dpb_stream": (_vp, [_vp]),
    "dpb_mle_from_host": (_int, [_vp, _int, _vp, _u64, _int, _pp]),
    "dpb_mle_from_device": (_int, [_vp, _int, _vp, _u64, _pp]),
    "dpb_mle_alloc": (_int, [_vp, _int, _u64, _pp]),
    "dpb_mle_free": (_int, [_vp]),
    "dpb_mle_to_host": (_int, [_vp, _vp, _u64, _int]),
    "dpb_mle_len": (_u64, [_vp]),
    "dpb_mle_dtype": (_int, [_vp]),
    "dpb_mle_device_ptr": (_vp, [_vp]),
    "dpb_mle_view": (_int, [_vp, _u64, _u64, _pp]),
    "dpb_mle_zero_padded": (_int, [_vp, _pp]),
    "dpb_eq_tables": (_int, [_vp, _int, _vp, ctypes.POINTER(_u32), _u32, _pp, _pp]),
    "dpb_linear_combination": (_int, [_vp, _pp, _vp, _u32, _pp]),
    "dpb_eq_table": (_int, [_vp, _int, _vp, _u32, _pp]),
    "dpb_fix_high": (_int, [_vp, _vp, _vp, _u32, _pp]),
    "dpb_fix_low": (_int, [_vp, _vp, _vp, _u32, _pp]),
    "dpb_rope_permuted_eq": (_int, [_vp, _vp, _int, _u64, _pp]),
    "dpb_mle_evaluate": (_int, [_vp, _vp, _vp, _u32, _vp]),
    "dpb_sumcheck_begin": (_int, [_vp, _u32, _pp, _u32, ctypes.POINTER(Term), _u32, _pp]),
    "dpb_sumcheck_degree": (_u32, [_vp]),
    "dpb_sumcheck_round": (_int, [_vp, _vp, _vp, ctypes.POINTER(_u32)]),
    "dpb_sumcheck_finish": (_int, [_vp, _vp, _vp]),
    "dpb_sumcheck_free": (None, [_vp]),
    "dpb_logup_build": (_int, [_vp, _int, _pp, _u32, _vp, _vp, _vp, _pp]),
    "dpb_logup_num_levels": (_u32, [_vp]),
    "dpb_logup_level": (_int, [_vp, _u32, _pp]),
    "dpb_logup_outputs": (_int, [_vp, _vp]),
    "dpb_logup_outputs_batch": (_int, [_pp, _u32, _vp]),
    "dpb_logup_free": (None, [_vp]),
    "dpb_product_round_noalloc": (_int, [_vp, _int, _pp, _u32, _u64, _vp]),
    "dpb_einsum_fix_axes": (_int, [_vp, _int, _vp, _int, _vp, _vp, _pp, _vp, _u32, _pp, _pp, _u32, ctypes.POINTER(_u32)]),
    "dpb_chunking_info_new": (_int, [_u32, _u32, _int, _u32, _u32, _vp]),
    "dpb_lookup_counts_new": (_int, [_vp, _u32, _pp]),
    "dpb_lookup_counts_to_host": (_int, [_vp, _vp, _u64]),
    "dpb_lookup_counts_free": (None, [_vp]),
    "dpb_lookup_multiplicities": (_int, [_vp, _vp, _int, _pp]),
    "dpb_lookup_counts_add_rows": (_int, [_vp, _vp, _vp, _int, _u64]),
    "dpb_lookup_witness": (_int, [_vp, _int, _vp, ctypes.c_int64, ctypes.c_int64, _vp, _int, _vp, _u32, _vp, _int, _u32,
                                  _vp, _vp, _vp, _vp, _pp, _pp, _u32, ctypes.POINTER(_u32), _pp, _u32, ctypes.POINTER(_u32)]),
    "dpb_eq_table_shard": (_int, [_vp, _int, _vp, _u32, _pp]),
    "dpb_comm_unique_id": (_int, [_vp]),
    "dpb_comm_init": (_int, [_vp, _vp, _int, _int]),
    "dpb_comm_rank": (_int, [_vp]),
    "dpb_comm_size": (_int, [_vp]),
    "dpb_comm_free": (_int, [_vp]),
    "dpb_sumcheck_begin_sharded": (_int, [_vp, _u32, _pp, _u32, ctypes.POINTER(Term), _u32, _pp]),
    "dpb_sumcheck_begin_partial": (_int, [_vp, _u32, _pp, _u32, ctypes.POINTER(Term), _u32, _pp]),
}

COMM_ID_BYTES = 128


def trace(on):
    """dpb_trace_enable: host-side phase timers of the whole-protocol entry points."""
    check(lib.dpb_trace_enable(1 if on else 0))


def trace_read():
    """{phase: (milliseconds, calls)} since trace(True)."""
    n = ctypes.c_size_t()
    check(lib.dpb_trace_read(None, 0, ctypes.byref(n)))
    buf = ctypes.create_string_buffer(n.value)
    check(lib.dpb_trace_read(buf, n.value, ctypes.byref(n)))
    out = {}
    for line in buf.value.decode().splitlines():
        name, ms, calls = line.split("\t")
        out[name] = (float(ms), int(calls))
    return out


def comm_unique_id():
    """dpb_comm_unique_id: 128 bytes to hand to every rank's Context.comm_init."""
    buf = (ctypes.c_uint8 * COMM_ID_BYTES)()
    check(lib.dpb_comm_unique_id(buf))
    return bytes(buf)


def _bind():
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args


_bind()


def check(rc):
    if rc != OK:
        raise DpbError(rc, lib.dpb_last_error().decode(errors="replace"))


def elem_words(dtype):
    """64-bit words per entry of a field layout (integer layouts are described by INT_DTYPES)."""
    return {GL_BASE: 1, GL_EXT: 2, FR: 4}[dtype]


def chal_dtype(dtype):
    return FR if dtype in (FR, FR_I64, FR_I32) else GL_EXT


FR_MODULUS = 21888242871839275222246405745257275088548364400416034343698204186575808495617


def one_bytes(dtype):
    """The field's one as native challenge-element bytes (Fr: Montgomery form)."""
    if dtype == FR:
        return ((1 << 256) % FR_MODULUS).to_bytes(32, "little")
    return (1).to_bytes(8, "little") + bytes(8)


def _buf(a):
    return ctypes.c_void_p(a.ctypes.data)


def dtype_of_array(a, family):
    """family 'gl': uint64[n] -> base, uint64[n,2] -> extension; 'fr': uint64[n,4]."""
    a = np.asarray(a)
    if family == "fr":
        return FR
    return GL_BASE if a.ndim == 1 else GL_EXT


class Context:
    """One GPU, one stream (dpb_init / dpb_shutdown)."""

    def __init__(self, device=0):
        h = ctypes.c_void_p()
        check(lib.dpb_init(device, ctypes.byref(h)))
        self.h = h
        self.device = device

    def close(self):
        if self.h:
            lib.dpb_shutdown(self.h)
            self.h = None

    def trim(self):
        """dpb_trim: kept device memory goes back to the pool and the pool's unused memory to the device."""
        check(lib.dpb_trim(self.h))

    def sync(self):
        check(lib.dpb_sync(self.h))

    @property
    def stream(self):
        return lib.dpb_stream(self.h)

    def comm_init(self, unique_id, rank, nranks):
        """Joins the NCCL communicator of sharded sumchecks (collective over all ranks)."""
        buf = (ctypes.c_uint8 * COMM_ID_BYTES).from_buffer_copy(unique_id)
        check(lib.dpb_comm_init(self.h, buf, rank, nranks))

    def comm_free(self):
        check(lib.dpb_comm_free(self.h))

    def comm_shared_exchange(self):
        """True when sharded rounds exchange their sums through the shared host segment, False for ncclAllGather."""
        return bool(lib.dpb_comm_shared_exchange(self.h))

    def resident_rounds(self, enable=True, wait_ms=0):
        """Last rounds in one resident kernel (default) or one launch per round; wait_ms bounds the kernel's waits
        for a challenge (a kernel that returned is started again by the next call)."""
        check(lib.dpb_resident_rounds(self.h, 1 if enable else 0, int(wait_ms)))

    def sumcheck_launches(self):
        return int(lib.dpb_sumcheck_launches(self.h))

    PROBE_WIDE_MAD, PROBE_FR_MUL, PROBE_FR_MUL_FIXED, PROBE_GL_MAC, PROBE_GL_MUL = range(5)

    def issue_rate(self, kind, iters=4096):
        """dpb_issue_rate_probe: (operations per second, milliseconds of the timed launch)."""
        ops, ms = ctypes.c_double(), ctypes.c_double()
        check(lib.dpb_issue_rate_probe(self.h, kind, iters, ctypes.byref(ops), ctypes.byref(ms)))
        return ops.value, ms.value

    def profile(self, on):
        check(lib.dpb_profile_enable(self.h, 1 if on else 0))

    def profile_read(self):
        n = ctypes.c_uint32()
        check(lib.dpb_profile_read(self.h, None, 0, ctypes.byref(n)))
        arr = (ProfileEntry * max(n.value, 1))()
        check(lib.dpb_profile_read(self.h, arr, n.value, ctypes.byref(n)))
        return [dict(kernel=arr[i].kernel.decode(), round=arr[i].round, launches=arr[i].launches,
                     total_ms=arr[i].total_ms, alg_bytes_per_launch=arr[i].alg_bytes_per_launch)
                for i in range(n.value)]

    # ---- tables
    def upload(self, array, dtype, form=FORM_NATIVE):
        a = np.ascontiguousarray(array)
        n = a.shape[0]
        h = ctypes.c_void_p()
        check(lib.dpb_mle_from_host(self.h, dtype, _buf(a), n, form, ctypes.byref(h)))
        return Mle(self, h)

    def upload_ints(self, array, dtype):
        """An integer table (GL_I64 / GL_I32 / FR_I64 / FR_I32): the integers stay integers on the device."""
        a = np.ascontiguousarray(array, dtype=INT_DTYPES[dtype])
        h = ctypes.c_void_p()
        check(lib.dpb_mle_from_host(self.h, dtype, _buf(a), a.size, FORM_NATIVE, ctypes.byref(h)))
        return Mle(self, h)

    def upload_i64(self, array, dtype):
        a = np.ascontiguousarray(array, dtype=np.int64)
        h = ctypes.c_void_p()
        check(lib.dpb_mle_from_host(self.h, dtype, _buf(a), a.size, FORM_I64, ctypes.byref(h)))
        return Mle(self, h)

    def alloc(self, dtype, n):
        h = ctypes.c_void_p()
        check(lib.dpb_mle_alloc(self.h, dtype, n, ctypes.byref(h)))
        return Mle(self, h)

    def wrap_device(self, dev_ptr, dtype, n):
        h = ctypes.c_void_p()
        check(lib.dpb_mle_from_device(self.h, dtype, ctypes.c_void_p(dev_ptr), n, ctypes.byref(h)))
        return Mle(self, h)

    def eq_table(self, family_dtype, point_array):
        """point_array: challenge elements, uint64[m, words]"""
        p = np.ascontiguousarray(point_array, dtype=np.uint64)
        m = p.shape[0] if p.size else 0
        h = ctypes.c_void_p()
        check(lib.dpb_eq_table(self.h, family_dtype, _buf(p) if m else None, m, ctypes.byref(h)))
        return Mle(self, h)

    def eq_table_shard(self, family_dtype, point_array):
        """dpb_eq_table_shard: this rank's slice of the eq table of the point."""
        p = np.ascontiguousarray(point_array, dtype=np.uint64)
        m = p.shape[0] if p.size else 0
        h = ctypes.c_void_p()
        check(lib.dpb_eq_table_shard(self.h, family_dtype, _buf(p) if m else None, m, ctypes.byref(h)))
        return Mle(self, h)

    def fix_high(self, mle, point_array):
        p = np.ascontiguousarray(point_array, dtype=np.uint64)
        h = ctypes.c_void_p()
        check(lib.dpb_fix_high(self.h, mle.h, _buf(p), p.shape[0], ctypes.byref(h)))
        return Mle(self, h)

    def fix_low(self, mle, point_array):
        p = np.ascontiguousarray(point_array, dtype=np.uint64)
        h = ctypes.c_void_p()
        check(lib.dpb_fix_low(self.h, mle.h, _buf(p), p.shape[0], ctypes.byref(h)))
        return Mle(self, h)

    def evaluate(self, mle, point_array):
        p = np.ascontiguousarray(point_array, dtype=np.uint64)
        n = p.shape[0] if p.size else 0
        out = np.zeros(elem_words(chal_dtype(mle.dtype)), dtype=np.uint64)
        check(lib.dpb_mle_evaluate(self.h, mle.h, _buf(p) if n else None, n, _buf(out)))
        return out

    def upload_tensor_i64(self, tensor):
        """An int64 tensor kept on the device as raw 64-bit words, for einsum_fix_axes(device_tensor=...)."""
        t = np.ascontiguousarray(tensor, dtype=np.int64)
        n = 1
        while n < t.size:
            n *= 2
        flat = np.zeros(n, dtype=np.uint64)
        flat[: t.size] = t.reshape(-1).view(np.uint64)
        return self.upload(flat, GL_BASE), tuple(t.shape)

    def einsum_fix_axes(self, family_dtype, tensor, kinds, points, device_tensor=None):
        """dpb_einsum_fix_axes.  tensor: int64 ndarray (unpadded); kinds[a] in
        AXIS_*; points[a]: challenge elements uint64[len, words] for outer axes,
        None otherwise.  device_tensor = upload_tensor_i64(...) uses a tensor that
        is already on the device instead.  Returns (owner, [views])."""
        if device_tensor is not None:
            mle, tshape = device_tensor
            t = None
        else:
            t = np.ascontiguousarray(tensor, dtype=np.int64)
            tshape = t.shape
        rank = len(tshape)
        shape = (ctypes.c_uint64 * rank)(*tshape)
        kd = (ctypes.c_uint8 * rank)(*kinds)
        keep = [np.ascontiguousarray(p, dtype=np.uint64) if p is not None else None for p in points]
        pts = (ctypes.c_void_p * rank)(*[k.ctypes.data if k is not None and k.size else None for k in keep])
        lens = (ctypes.c_uint32 * rank)(*[0 if k is None else (k.shape[0] if k.size else 0) for k in keep])
        cap = 1
        for a in range(rank):
            if kinds[a] == AXIS_STACKED:
                cap *= tshape[a]
        views = (ctypes.c_void_p * cap)()
        owner = ctypes.c_void_p()
        n = ctypes.c_uint32()
        src = _buf(t) if t is not None else ctypes.c_void_p(lib.dpb_mle_device_ptr(mle.h))
        check(lib.dpb_einsum_fix_axes(self.h, family_dtype, src, 0 if t is not None else 1, shape, kd, pts, lens, rank,
                                      ctypes.byref(owner), views, cap, ctypes.byref(n)))
        return Mle(self, owner), [Mle(self, ctypes.c_void_p(views[i])) for i in range(n.value)]

    def sumcheck(self, num_vars, mles, terms, sharded=False):
        return Sumcheck(self, num_vars, mles, terms, sharded)

    def logup(self, kind, columns, constant, sep, mult=None):
        return Logup(self, kind, columns, constant, sep, mult)


SIGN_POSITIVE, SIGN_NEGATIVE, SIGN_MIXED = 0, 1, 2


class ChunkingInfo(ctypes.Structure):
    """dpb_chunking_info, built by dpb_chunking_info_new (ChunkingInfo::new of the reference)."""
    _fields_ = [("right_shift", _u32), ("value_chunk_bits", _u32), ("n_value_chunks", _u32), ("n_shifted_chunks", _u32),
                ("n_zeroing_chunks", _u32), ("table_sign", ctypes.c_int32), ("offset", ctypes.c_int64),
                ("value_chunk_offset", ctypes.c_int64), ("shifted_chunk_multiplier", ctypes.c_int64),
                ("top_zeroing_chunk_offset", ctypes.c_int64)]

    @classmethod
    def new(cls, right_shift, table_bits, table_sign, max_bit_size, n_value_chunks=1):
        ci = cls()
        check(lib.dpb_chunking_info_new(right_shift, table_bits, table_sign, max_bit_size, n_value_chunks, ctypes.byref(ci)))
        return ci


class LookupCounts:
    """dpb_lookup_counts: per-row lookup counters of one table, on the device."""

    def __init__(self, ctx, table_bits):
        self.ctx, self.bits = ctx, table_bits
        self.h = ctypes.c_void_p()
        check(lib.dpb_lookup_counts_new(ctx.h, table_bits, ctypes.byref(self.h)))

    def to_host(self):
        out = np.empty(1 << self.bits, dtype=np.uint64)
        check(lib.dpb_lookup_counts_to_host(self.h, _buf(out), out.size))
        return out

    def add_rows(self, rows):
        """dpb_lookup_counts_add_rows: rows is an int64 array of row indices (host memory)."""
        r = np.ascontiguousarray(rows, dtype=np.int64)
        check(lib.dpb_lookup_counts_add_rows(self.ctx.h, self.h, _buf(r), 0, r.size))

    def multiplicities(self, family_dtype):
        h = ctypes.c_void_p()
        check(lib.dpb_lookup_multiplicities(self.ctx.h, self.h, family_dtype, ctypes.byref(h)))
        return Mle(self.ctx, h)

    def free(self):
        if self.h:
            lib.dpb_lookup_counts_free(self.h)
            self.h = None


def lookup_witness(ctx, family_dtype, info, fixed_point_multiplier, padding_value, tensor, value_table_outputs,
                   num_value_columns, counts=(None, None, None, None), device_tensor=None, device_table=None):
    """dpb_lookup_witness.  tensor: int64 ndarray (unpadded), or device_tensor = ctx.upload_tensor_i64(...);
    value_table_outputs: int64 array over the value table's inputs, or None for a one-column table;
    counts: LookupCounts for the shift-check, value, zero-check and signed zero-check tables (None: not counted);
    device_table = ctx.upload_tensor_i64(value_table_outputs) uses an output column that is already on the device.
    Returns (owner, input columns, output columns)."""
    if device_tensor is not None:
        mle, tshape = device_tensor
        src, on_dev = ctypes.c_void_p(lib.dpb_mle_device_ptr(mle.h)), 1
    else:
        t = np.ascontiguousarray(tensor, dtype=np.int64)
        tshape, src, on_dev = t.shape, _buf(t), 0
    rank = len(tshape)
    shape = (ctypes.c_uint64 * rank)(*tshape)
    slices = 1
    for d in tshape[:-2]:
        slices *= d
    cap = slices * 12
    ins, outs = (ctypes.c_void_p * cap)(), (ctypes.c_void_p * cap)()
    n_in, n_out, owner = ctypes.c_uint32(), ctypes.c_uint32(), ctypes.c_void_p()
    tab = None if value_table_outputs is None else np.ascontiguousarray(value_table_outputs, dtype=np.int64)
    if device_table is not None:
        tab_ptr, tab_dev = ctypes.c_void_p(lib.dpb_mle_device_ptr(device_table[0].h)), 1
    else:
        tab_ptr, tab_dev = (_buf(tab) if tab is not None else None), 0
    hs = [c.h if c is not None else None for c in counts]
    check(lib.dpb_lookup_witness(ctx.h, family_dtype, ctypes.byref(info), fixed_point_multiplier, padding_value, src, on_dev,
                                 shape, rank, tab_ptr, tab_dev, num_value_columns, hs[0], hs[1],
                                 hs[2], hs[3], ctypes.byref(owner), ins, cap, ctypes.byref(n_in), outs, cap,
                                 ctypes.byref(n_out)))
    return (Mle(ctx, owner), [Mle(ctx, ctypes.c_void_p(ins[i])) for i in range(n_in.value)],
            [Mle(ctx, ctypes.c_void_p(outs[i])) for i in range(n_out.value)])


def product_round_noalloc(stream, dtype, table_ptrs, length, out_ptr):
    """dpb_product_round_noalloc: first sumcheck round of a product of tables
    for callers that may not allocate device memory.  `table_ptrs` and
    `out_ptr` are device addresses the caller owns; the kernel is queued on
    `stream` (a cudaStream_t value) and the caller synchronises."""
    k = len(table_ptrs)
    arr = (ctypes.c_void_p * k)(*table_ptrs)
    check(lib.dpb_product_round_noalloc(ctypes.c_void_p(stream), dtype, arr, k, length, ctypes.c_void_p(out_ptr)))


class Mle:
    """A multilinear table on the device (dpb_mle)."""

    def __init__(self, ctx, h):
        self.ctx, self.h = ctx, h

    @property
    def len(self):
        return lib.dpb_mle_len(self.h)

    @property
    def dtype(self):
        return lib.dpb_mle_dtype(self.h)

    @property
    def device_ptr(self):
        return lib.dpb_mle_device_ptr(self.h)

    def to_host(self, form=FORM_NATIVE, n=None):
        n = self.len if n is None else n
        if self.dtype in INT_DTYPES:
            out = np.empty(n, dtype=INT_DTYPES[self.dtype])
            check(lib.dpb_mle_to_host(self.h, _buf(out), n, FORM_NATIVE))
            return out
        w = elem_words(self.dtype)
        out = np.empty((n, w) if w > 1 else (n,), dtype=np.uint64)
        check(lib.dpb_mle_to_host(self.h, _buf(out), n, form))
        return out

    def view(self, offset, n):
        h = ctypes.c_void_p()
        check(lib.dpb_mle_view(self.h, offset, n, ctypes.byref(h)))
        return Mle(self.ctx, h)

    def zero_padded(self):
        """A view that a sumcheck over more variables treats as zero above this table's length."""
        h = ctypes.c_void_p()
        check(lib.dpb_mle_zero_padded(self.h, ctypes.byref(h)))
        return Mle(self.ctx, h)

    def free(self):
        if self.h:
            lib.dpb_mle_free(self.h)
            self.h = None


def eq_tables(ctx, family_dtype, points):
    """One eq table per point (a list of [m_t, w] arrays) in a single call.  Returns (owner, [tables]): the tables
    are views into the owner's memory; free the owner last."""
    n = len(points)
    nv = (ctypes.c_uint32 * n)(*[int(np.asarray(p).shape[0]) for p in points])
    w = elem_words(chal_dtype(family_dtype))
    flat = np.ascontiguousarray(np.concatenate([np.asarray(p, dtype=np.uint64).reshape(-1, w) for p in points])
                                if n else np.zeros((0, w), np.uint64))
    owner = ctypes.c_void_p()
    outs = (ctypes.c_void_p * n)()
    check(lib.dpb_eq_tables(ctx.h, family_dtype, _buf(flat), nv, n, ctypes.byref(owner), outs))
    return Mle(ctx, owner), [Mle(ctx, ctypes.c_void_p(outs[i])) for i in range(n)]


def evaluate_many(ctx, mles, point_array):
    """dpb_mle_evaluate_many: every table (zero-padded to the point's number of variables) at one point."""
    p = np.ascontiguousarray(point_array, dtype=np.uint64)
    n = len(mles)
    w = elem_words(chal_dtype(mles[0].dtype))
    hs = (ctypes.c_void_p * n)(*[m.h for m in mles])
    out = np.zeros((n, w), dtype=np.uint64)
    check(lib.dpb_mle_evaluate_many(ctx.h, hs, n, _buf(p) if p.size else None, p.shape[0] if p.size else 0, _buf(out)))
    return out


ROPE_ADJACENT, ROPE_ROTATE_HALF = 0, 1


def rope_permuted_eq(ctx, eq, layout=ROPE_ADJACENT, row_size=0):
    """RopeLayout::permuted_eq_poly (zkml/src/layers/transformer/positional/rope.rs:238-258) of an eq table."""
    h = ctypes.c_void_p()
    check(lib.dpb_rope_permuted_eq(ctx.h, eq.h, layout, row_size, ctypes.byref(h)))
    return Mle(ctx, h)


def linear_combination(ctx, mles, coeffs):
    """DensePolynomial::linear_combination: sum_j coeffs[j] * mles[j]; shorter tables are zero-padded."""
    k = len(mles)
    hs = (ctypes.c_void_p * k)(*[m.h for m in mles])
    c = np.ascontiguousarray(coeffs, dtype=np.uint64)
    h = ctypes.c_void_p()
    check(lib.dpb_linear_combination(ctx.h, hs, _buf(c), k, ctypes.byref(h)))
    return Mle(ctx, h)


def make_terms(terms, coeff_bytes):
    """terms: list of (coeff, [table ids]); coeff_bytes(coeff) -> native bytes."""
    arr = (Term * len(terms))()
    for t, (c, idx) in enumerate(terms):
        raw = coeff_bytes(c)
        for i, b in enumerate(raw):
            arr[t].coeff[i] = b
        arr[t].n_factors = len(idx)
        if len(idx) > MAX_FACTORS:
            raise ValueError("too many factors")
        for j, v in enumerate(idx):
            arr[t].idx[j] = v
    return arr


class Sumcheck:
    """dpb_sumcheck_begin / round / finish."""

    def __init__(self, ctx, num_vars, mles, term_array, sharded=False):
        self.ctx = ctx
        k = len(mles)
        hs = (ctypes.c_void_p * k)(*[m.h for m in mles])
        h = ctypes.c_void_p()
        # sharded: True = this rank's slices of the tables; "partial" = this rank's part of the terms over whole tables
        begin = lib.dpb_sumcheck_begin_partial if sharded == "partial" else \
            lib.dpb_sumcheck_begin_sharded if sharded else lib.dpb_sumcheck_begin
        check(begin(ctx.h, num_vars, hs, k, term_array, len(term_array), ctypes.byref(h)))
        self.h = h
        self.k = k
        self.num_vars = num_vars
        self.words = elem_words(chal_dtype(mles[0].dtype))
        self.degree = lib.dpb_sumcheck_degree(h)
        self._out = np.zeros((self.degree + 1, self.words), dtype=np.uint64)

    def round(self, prev_challenge=None):
        n = ctypes.c_uint32()
        pc = None
        if prev_challenge is not None:
            self._pc = np.ascontiguousarray(prev_challenge, dtype=np.uint64)
            pc = _buf(self._pc)
        check(lib.dpb_sumcheck_round(self.h, pc, _buf(self._out), ctypes.byref(n)))
        return self._out.copy()

    def finish(self, last_challenge):
        lc = np.ascontiguousarray(last_challenge, dtype=np.uint64)
        out = np.zeros((self.k, self.words), dtype=np.uint64)
        check(lib.dpb_sumcheck_finish(self.h, _buf(lc), _buf(out)))
        return out

    def free(self):
        if self.h:
            lib.dpb_sumcheck_free(self.h)
            self.h = None


class Logup:
    """dpb_logup_build and accessors."""

    def __init__(self, ctx, kind, columns, constant, sep, mult=None):
        self.ctx = ctx
        k = len(columns)
        hs = (ctypes.c_void_p * k)(*[m.h for m in columns])
        c = np.ascontiguousarray(constant, dtype=np.uint64)
        s = np.ascontiguousarray(sep, dtype=np.uint64)
        h = ctypes.c_void_p()
        check(lib.dpb_logup_build(ctx.h, kind, hs, k, mult.h if mult is not None else None, _buf(c), _buf(s),
                                  ctypes.byref(h)))
        self.h = h
        self.words = elem_words(chal_dtype(columns[0].dtype))

    @property
    def num_levels(self):
        return lib.dpb_logup_num_levels(self.h)

    def level(self, l):
        out = (ctypes.c_void_p * 4)()
        check(lib.dpb_logup_level(self.h, l, out))
        return [Mle(self.ctx, ctypes.c_void_p(v)) for v in out]

    def outputs(self):
        out = np.zeros((4, self.words), dtype=np.uint64)
        check(lib.dpb_logup_outputs(self.h, _buf(out)))
        return out

    def free(self):
        if self.h:
            lib.dpb_logup_free(self.h)
            self.h = None
