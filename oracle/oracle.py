"""CPU oracle for the sumcheck / multilinear-fold / logup-GKR path.

TEST INFRASTRUCTURE ONLY.  Only the tests, the smoke check and the benchmark's
CPU-baseline legs may import this module; the library never does.

PARITY UNPINNED at the byte level (see the header of oracle.c): the
reference's sumcheck core and transcript live in the absent third-party crate
dp-crypto 0.1.0 (rev 22e8e93), and the reference ships no golden proof.  The
protocol logic below restates the reference's in-repo code step by step
(file:line beside each function, paths relative to the reference repository);
the heavy loops are in oracle.c (plain C + OpenMP), scalars are Python ints.

Conventions shared with the library:
  * tables are little-endian (bit i of the index = variable i,
    zkml/src/lib.rs:357-369); sumcheck round i binds variable i;
  * a round message is the round polynomial's evaluations at 0..=d;
  * the transcript is the BLAKE3 construction of `Transcript` below.
"""
import ctypes
import os
import subprocess

import numpy as np

from . import blake3_py

HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(HERE, "_build", "liboracle.so")

DT_GL_BASE, DT_GL_EXT, DT_FR = 0, 1, 2

FR_MOD = 21888242871839275222246405745257275088548364400416034343698204186575808495617
GL_MOD = 2**64 - 2**32 + 1
GL_NONRES = 7


def _cpu_tag():
    """Short tag of this host's instruction-set flags: a library tuned for one CPU is never loaded on another."""
    import hashlib
    flags = ""
    try:
        with open("/proc/cpuinfo") as f:
            for line in f:
                if line.startswith("flags"):
                    flags = line
                    break
    except OSError:
        pass
    return hashlib.sha1(flags.encode()).hexdigest()[:10]


def build(force=False, native=False):
    """Compiles oracle.c into oracle/_build/liboracle.so with gcc.  native=True builds a second library tuned for
    the CPU it is compiled on (-march=native), named after that CPU's flag set; it is what the timed CPU baseline
    uses, and it is compiled on the host that runs it."""
    src = os.path.join(HERE, "oracle.c")
    path = os.path.join(HERE, "_build", f"liboracle_native_{_cpu_tag()}.so") if native else LIB_PATH
    if not force and os.path.exists(path) and os.path.getmtime(path) >= os.path.getmtime(src):
        return path
    os.makedirs(os.path.dirname(path), exist_ok=True)
    flags = ["-O3", "-fopenmp", "-shared", "-fPIC"] + (["-march=native"] if native else [])
    tmp = f"{path}.{os.getpid()}.tmp"
    subprocess.run(["gcc", *flags, "-o", tmp, src], check=True)
    os.replace(tmp, path)
    return path


_lib = None


def lib():
    global _lib
    if _lib is None:
        _lib = ctypes.CDLL(build())
    return _lib


def use_native_build():
    """Switches this process to the -march=native library (timed CPU baseline); falls back to the portable one
    when the compiler is missing.  Returns True when the native library is in use."""
    global _lib
    try:
        _lib = ctypes.CDLL(build(native=True))
        return True
    except (OSError, subprocess.CalledProcessError):
        return False


def set_num_threads(n=None):
    """OpenMP threads of the C routines; default: every core this process may run on."""
    if n is None:
        n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().orc_set_num_threads(int(n))
    return lib().orc_num_threads()


class OrcTerm(ctypes.Structure):
    _fields_ = [("coeff", ctypes.c_uint8 * 32), ("n_factors", ctypes.c_uint32), ("idx", ctypes.c_uint16 * 8)]


def _ptr(a):
    return ctypes.c_void_p(a.ctypes.data)


# --------------------------------------------------------------------- fields
class FrField:
    """BN254 Fr.  Scalars are Python ints in [0, r); tables are uint64[n, 4]
    Montgomery limbs (the library's DPB_FR layout)."""
    name = "fr"
    chal_dtype = DT_FR
    elem_words = 4
    R = (1 << 256) % FR_MOD
    RINV = pow((1 << 256) % FR_MOD, -1, FR_MOD)

    zero, one = 0, 1

    @staticmethod
    def add(a, b): return (a + b) % FR_MOD
    @staticmethod
    def sub(a, b): return (a - b) % FR_MOD
    @staticmethod
    def mul(a, b): return (a * b) % FR_MOD
    @staticmethod
    def neg(a): return (-a) % FR_MOD
    @staticmethod
    def inv(a): return pow(a, -1, FR_MOD)
    @staticmethod
    def from_int(x): return x % FR_MOD

    @classmethod
    def pow(cls, a, e):
        return pow(a, e, FR_MOD)

    # scalar <-> native bytes (Montgomery limbs)
    @classmethod
    def to_native(cls, a):
        return ((a * cls.R) % FR_MOD).to_bytes(32, "little")

    @classmethod
    def from_native(cls, b):
        return (int.from_bytes(bytes(b), "little") * cls.RINV) % FR_MOD

    # scalar <-> canonical bytes (what ark_serialize writes: 32 bytes LE)
    @staticmethod
    def to_canonical(a):
        return int(a).to_bytes(32, "little")

    @classmethod
    def table_from_ints(cls, vals):
        buf = b"".join(cls.to_native(v % FR_MOD) for v in vals)
        return np.frombuffer(buf, dtype=np.uint64).reshape(-1, 4).copy()

    @classmethod
    def table_to_ints(cls, t):
        raw = np.ascontiguousarray(t).tobytes()
        return [cls.from_native(raw[i:i + 32]) for i in range(0, len(raw), 32)]

    @classmethod
    def table_from_i64(cls, x):
        x = np.ascontiguousarray(x, dtype=np.int64)
        out = np.empty((x.size, 4), dtype=np.uint64)
        lib().orc_fr_from_i64(_ptr(x), _ptr(out), ctypes.c_uint64(x.size))
        return out

    @classmethod
    def random_table(cls, rng, n):
        """n uniform elements (512 random bits reduced mod r)."""
        vals = [int.from_bytes(rng.bytes(64), "little") % FR_MOD for _ in range(n)]
        return cls.table_from_ints(vals)

    @classmethod
    def random_table_fast(cls, rng, n):
        """n pseudo-random elements for large tables: random limbs with the top
        limb masked below the modulus' top limb, taken as Montgomery residues."""
        t = rng.integers(0, 2**64, size=(n, 4), dtype=np.uint64)
        t[:, 3] &= np.uint64((1 << 60) - 1)
        return t

    @classmethod
    def random_scalar(cls, rng):
        return int.from_bytes(rng.bytes(64), "little") % FR_MOD

    @staticmethod
    def dtype_of(table):
        return DT_FR

    @classmethod
    def challenge_from_bytes(cls, b64):
        return int.from_bytes(b64, "little") % FR_MOD


class GlField:
    """Goldilocks with its quadratic extension X^2 = 7.  Scalars are (c0, c1)
    tuples; tables are uint64[n] (base) or uint64[n, 2] (extension)."""
    name = "gl"
    chal_dtype = DT_GL_EXT
    elem_words = 2
    zero, one = (0, 0), (1, 0)

    @staticmethod
    def add(a, b): return ((a[0] + b[0]) % GL_MOD, (a[1] + b[1]) % GL_MOD)
    @staticmethod
    def sub(a, b): return ((a[0] - b[0]) % GL_MOD, (a[1] - b[1]) % GL_MOD)
    @staticmethod
    def mul(a, b):
        return ((a[0] * b[0] + GL_NONRES * a[1] * b[1]) % GL_MOD, (a[0] * b[1] + a[1] * b[0]) % GL_MOD)
    @staticmethod
    def neg(a): return ((-a[0]) % GL_MOD, (-a[1]) % GL_MOD)
    @staticmethod
    def inv(a):
        n = pow((a[0] * a[0] - GL_NONRES * a[1] * a[1]) % GL_MOD, -1, GL_MOD)
        return ((a[0] * n) % GL_MOD, (-a[1] * n) % GL_MOD)
    @staticmethod
    def from_int(x): return (x % GL_MOD, 0)

    @classmethod
    def pow(cls, a, e):
        r = cls.one
        while e:
            if e & 1:
                r = cls.mul(r, a)
            a = cls.mul(a, a)
            e >>= 1
        return r

    @staticmethod
    def to_native(a):
        return int(a[0]).to_bytes(8, "little") + int(a[1]).to_bytes(8, "little")

    @staticmethod
    def from_native(b):
        b = bytes(b)
        return (int.from_bytes(b[:8], "little"), int.from_bytes(b[8:16], "little"))

    to_canonical = to_native

    @classmethod
    def table_from_ints(cls, vals):
        """vals: ints -> base table; tuples -> extension table."""
        if len(vals) and isinstance(vals[0], tuple):
            return np.array([[v[0] % GL_MOD, v[1] % GL_MOD] for v in vals], dtype=np.uint64).reshape(-1, 2)
        return np.array([v % GL_MOD for v in vals], dtype=np.uint64)

    @classmethod
    def table_to_ints(cls, t):
        t = np.asarray(t)
        if t.ndim == 1:
            return [(int(v), 0) for v in t]
        return [(int(a), int(b)) for a, b in t]

    @classmethod
    def table_from_i64(cls, x):
        x = np.ascontiguousarray(x, dtype=np.int64)
        out = np.empty(x.size, dtype=np.uint64)
        lib().orc_gl_from_i64(_ptr(x), _ptr(out), ctypes.c_uint64(x.size))
        return out

    @classmethod
    def random_table(cls, rng, n):
        """n uniform base-field values by rejection sampling below p."""
        out = rng.integers(0, 2**64, size=n, dtype=np.uint64)
        while True:
            bad = out >= np.uint64(GL_MOD)
            k = int(bad.sum())
            if k == 0:
                return out
            out[bad] = rng.integers(0, 2**64, size=k, dtype=np.uint64)

    random_table_fast = random_table

    @classmethod
    def random_ext_table(cls, rng, n):
        return np.stack([cls.random_table(rng, n), cls.random_table(rng, n)], axis=1).copy()

    @classmethod
    def random_scalar(cls, rng):
        return (int.from_bytes(rng.bytes(16), "little") % GL_MOD, int.from_bytes(rng.bytes(16), "little") % GL_MOD)

    @staticmethod
    def dtype_of(table):
        return DT_GL_BASE if np.asarray(table).ndim == 1 else DT_GL_EXT

    @classmethod
    def challenge_from_bytes(cls, b64):
        return (int.from_bytes(b64[:16], "little") % GL_MOD, int.from_bytes(b64[32:48], "little") % GL_MOD)


FIELDS = {"fr": FrField, "gl": GlField}


def scalars_to_array(F, vals):
    buf = b"".join(F.to_native(v) for v in vals)
    return np.frombuffer(buf, dtype=np.uint64).reshape(-1, F.elem_words).copy()


def array_to_scalars(F, arr):
    raw = np.ascontiguousarray(arr).tobytes()
    w = F.elem_words * 8
    return [F.from_native(raw[i:i + w]) for i in range(0, len(raw), w)]


def table_len(t):
    return np.asarray(t).shape[0]


# ----------------------------------------------------------------- transcript
class Transcript:
    """Fiat-Shamir transcript over BLAKE3 with the method names the reference
    uses (`Blake3Transcript::new(b"m2vec")`, zkml/src/lib.rs:106-108;
    append_scalars / append_and_sample / challenge_scalar,
    zkml/src/lookup/logup_gkr/prover.rs:163-173).  The reference's byte format is
    defined in the absent dp-crypto crate; this one is the library's own:

      state_0      = BLAKE3("dpb-transcript-v1" || label)
      absorb(t, m) : state = BLAKE3(state || u32le(round) || u32le(len t) || t || m); round += 1
      append_scalars(v)      = absorb("scalars", u64le(len v) || canonical bytes of each v)
      append_and_sample(l)   = absorb("label", l); challenge_scalar()
      challenge_scalar()     = absorb("challenge", ""); 64 bytes = BLAKE3(state||0) || BLAKE3(state||1)
                               Fr: the 64 bytes as an LE integer mod r
                               Goldilocks ext: c0 = bytes[0:16] mod p, c1 = bytes[32:48] mod p
    """

    def __init__(self, F, label=b"m2vec", hash_fn=None):
        self.F = F
        self.h = hash_fn or blake3_py.blake3
        self.state = self.h(b"dpb-transcript-v1" + bytes(label))
        self.round = 0

    def clone(self):
        t = Transcript.__new__(Transcript)
        t.F, t.h, t.state, t.round = self.F, self.h, self.state, self.round
        return t

    def _absorb(self, tag, msg):
        self.state = self.h(self.state + self.round.to_bytes(4, "little") + len(tag).to_bytes(4, "little") + tag + msg)
        self.round += 1

    def append_scalars(self, vals):
        self._absorb(b"scalars", len(vals).to_bytes(8, "little") + b"".join(self.F.to_canonical(v) for v in vals))

    def challenge_scalar(self):
        self._absorb(b"challenge", b"")
        return self.F.challenge_from_bytes(self.h(self.state + b"\0") + self.h(self.state + b"\1"))

    def append_and_sample(self, label):
        self._absorb(b"label", bytes(label))
        return self.challenge_scalar()

    def read_challenges(self, n):
        """zkml/src/lib.rs:176-184"""
        return [self.challenge_scalar() for _ in range(n)]


# ----------------------------------------------------------------- expressions
class Expr:
    """dp_crypto::Expression as zkml uses it: WitIn(id), Constant(c),
    Challenge(id, pow, scalar, offset) = scalar * ch[id]^pow + offset, closed
    under + - * and negation (zkml/src/lookup/logup_gkr/circuit.rs:245-284)."""

    def __init__(self, kind, *args):
        self.kind, self.args = kind, args

    @staticmethod
    def wit(i): return Expr("wit", i)
    @staticmethod
    def const(c): return Expr("const", c)
    @staticmethod
    def chal(i, p, scalar, offset): return Expr("chal", i, p, scalar, offset)

    def __add__(self, o): return Expr("add", self, o)
    def __sub__(self, o): return Expr("add", self, Expr("neg", o))
    def __mul__(self, o): return Expr("mul", self, o)
    def __neg__(self): return Expr("neg", self)


def expr_to_terms(F, e, challenges):
    """Expands an expression into {sorted tuple of table ids: coefficient}
    (what VirtualPolynomialsBuilder::to_virtual_polys hands the prover)."""
    k = e.kind
    if k == "wit":
        return {(e.args[0],): F.one}
    if k == "const":
        return {(): e.args[0]} if e.args[0] != F.zero else {}
    if k == "chal":
        i, p, s, off = e.args
        v = F.add(F.mul(s, F.pow(challenges[i], p)), off)
        return {(): v} if v != F.zero else {}
    if k == "neg":
        return {m: F.neg(c) for m, c in expr_to_terms(F, e.args[0], challenges).items()}
    a = expr_to_terms(F, e.args[0], challenges)
    b = expr_to_terms(F, e.args[1], challenges)
    out = {}
    if k == "add":
        for src in (a, b):
            for m, c in src.items():
                out[m] = F.add(out.get(m, F.zero), c)
    elif k == "mul":
        for ma, ca in a.items():
            for mb, cb in b.items():
                m = tuple(sorted(ma + mb))
                out[m] = F.add(out.get(m, F.zero), F.mul(ca, cb))
    else:
        raise ValueError(k)
    return {m: c for m, c in out.items() if c != F.zero}


def eval_expr(F, e, wit_evals, challenges):
    """dp_crypto::utils::eval_by_expr_with_instance with only witness values
    and challenges populated (zkml/src/lookup/logup_gkr/prover.rs:50-57)."""
    k = e.kind
    if k == "wit":
        return wit_evals[e.args[0]]
    if k == "const":
        return e.args[0]
    if k == "chal":
        i, p, s, off = e.args
        return F.add(F.mul(s, F.pow(challenges[i], p)), off)
    if k == "neg":
        return F.neg(eval_expr(F, e.args[0], wit_evals, challenges))
    a = eval_expr(F, e.args[0], wit_evals, challenges)
    b = eval_expr(F, e.args[1], wit_evals, challenges)
    return F.add(a, b) if k == "add" else F.mul(a, b)


# ------------------------------------------------------------------- poly ops
def eq_evals(F, point):
    """dp_crypto::poly::eq::evals: eq(x, point) for all x, little-endian."""
    m = len(point)
    out = np.empty((1 << m, F.elem_words), dtype=np.uint64)
    pt = scalars_to_array(F, point) if m else np.zeros((1, F.elem_words), dtype=np.uint64)
    fn = lib().orc_eq_gl if F is GlField else lib().orc_eq_fr
    fn(_ptr(pt), ctypes.c_uint32(m), _ptr(out))
    return out


def identity_eval(F, r1, r2):
    """zkml/src/poly_commit/mod.rs:184-192"""
    acc = F.one
    for a, b in zip(r1, r2):
        acc = F.mul(acc, F.add(F.mul(a, b), F.mul(F.sub(F.one, a), F.sub(F.one, b))))
    return acc


def fold_low(F, table, r):
    """Binds variable 0 of `table` to r."""
    t = np.ascontiguousarray(table)
    n_out = t.shape[0] // 2
    out = np.empty((n_out, F.elem_words), dtype=np.uint64)
    rr = scalars_to_array(F, [r])
    fn = lib().orc_fold_gl if F is GlField else lib().orc_fold_fr
    fn(_ptr(t), ctypes.c_int(F.dtype_of(t)), ctypes.c_uint64(n_out), _ptr(rr), _ptr(out))
    return out


def fold_high(F, table, r):
    """Binds the top variable of `table` to r."""
    t = np.ascontiguousarray(table)
    n_out = t.shape[0] // 2
    out = np.empty((n_out, F.elem_words), dtype=np.uint64)
    rr = scalars_to_array(F, [r])
    fn = lib().orc_fold_high_gl if F is GlField else lib().orc_fold_high_fr
    fn(_ptr(t), ctypes.c_int(F.dtype_of(t)), ctypes.c_uint64(n_out), _ptr(rr), _ptr(out))
    return out


def fix_low_variables(F, table, point):
    """DensePolynomial::fix_low_variables: variable j := point[j], one pass
    per variable (zkml/src/layers/transformer/attention_mask/prove.rs:431-436)."""
    t = table
    for r in point:
        t = fold_low(F, t, r)
    return t


def rope_permuted_eq(F, eq, layout=0, row_size=0):
    """RopeLayout::permuted_eq_poly (zkml/src/layers/transformer/positional/rope.rs:238-258).  layout 0 (Adjacent):
    pairs (a, b) -> (b, -a).  layout 1 (RotateHalf): each row of row_size entries -> second half, then the negated
    first half."""
    v = array_to_scalars(F, eq)
    out = []
    if layout == 0:
        for i in range(0, len(v), 2):
            out += [v[i + 1], F.neg(v[i])]
    else:
        half = row_size // 2
        for r in range(0, len(v), row_size):
            row = v[r:r + row_size]
            out += row[half:] + [F.neg(e) for e in row[:half]]
    return scalars_to_array(F, out)


def fix_high_variables(F, table, point):
    """DensePolynomial::fix_high_variables: the top len(point) variables, with
    point[j] the value of variable n - len(point) + j
    (zkml/src/layers/transformer/attention_mask/prove.rs:419-426,
    zkml/src/tensor/mod.rs:1889-1895)."""
    t = table
    for r in reversed(point):
        t = fold_high(F, t, r)
    return t


def evaluate(F, table, point):
    """DensePolynomial::evaluate, little-endian (zkml/src/lib.rs:357-369)."""
    assert table_len(table) == 1 << len(point)
    if not point:
        return array_to_scalars(F, _widen(F, table))[0]
    return array_to_scalars(F, fix_low_variables(F, table, point))[0]


def _widen(F, table):
    t = np.asarray(table)
    if F is GlField and t.ndim == 1:
        return np.stack([t, np.zeros_like(t)], axis=1).copy()
    return t


# -------------------------------------------------------------------- sumcheck
def terms_degree(terms):
    return max(len(m) for m in terms)


def _terms_array(F, terms):
    items = sorted(terms.items())
    arr = (OrcTerm * len(items))()
    for t, (m, c) in enumerate(items):
        raw = F.to_native(c)
        for i, b in enumerate(raw):
            arr[t].coeff[i] = b
        arr[t].n_factors = len(m)
        for j, idx in enumerate(m):
            arr[t].idx[j] = idx
    return arr, len(items)


def sumcheck_round(F, vars_left, tables, terms, d):
    """Round polynomial evaluations at 0..=d over tables that have `vars_left`
    (or fewer) variables."""
    k = len(tables)
    tabs = [np.ascontiguousarray(t) for t in tables]
    # fast path: first round of a coefficient-one product of base tables
    if (F is GlField and len(terms) == 1 and all(t.ndim == 1 for t in tabs)
            and all(table_len(t) == 1 << vars_left for t in tabs)):
        (m, c), = terms.items()
        if c == F.one and sorted(m) == list(range(k)) and d == k:
            ptrs = (ctypes.c_void_p * k)(*[t.ctypes.data for t in tabs])
            out = np.empty((d + 1, 2), dtype=np.uint64)
            lib().orc_round_gl_base_product(ctypes.c_uint32(vars_left), ptrs, ctypes.c_uint32(k), _ptr(out))
            return array_to_scalars(F, out)
    ptrs = (ctypes.c_void_p * k)(*[t.ctypes.data for t in tabs])
    dts = (ctypes.c_int * k)(*[F.dtype_of(t) for t in tabs])
    tv = (ctypes.c_uint32 * k)(*[table_len(t).bit_length() - 1 for t in tabs])
    arr, n_terms = _terms_array(F, terms)
    out = np.empty((d + 1, F.elem_words), dtype=np.uint64)
    fn = lib().orc_round_gl if F is GlField else lib().orc_round_fr
    fn(ctypes.c_uint32(vars_left), ptrs, dts, tv, ctypes.c_uint32(k), arr, ctypes.c_uint32(n_terms),
       ctypes.c_uint32(d), _ptr(out))
    return array_to_scalars(F, out)


ROUND_LABEL = b"sumcheck_round"


def sumcheck_prove(F, num_vars, tables, terms, transcript, degree=None):
    """IOPProverState::prove as its call sites use it
    (zkml/src/layers/hadamard.rs:115-130): returns (proof, point, final_evals)
    with proof = list of per-round evaluation lists, point[j] the challenge of
    variable j (collect_raw_challenges) and final_evals[i] = table i at the
    point (get_mle_flatten_final_evaluations).  A table with fewer variables
    is a function of the last variables and starts folding when its turn comes."""
    d = degree if degree is not None else terms_degree(terms)
    cur = list(tables)
    nv = [table_len(t).bit_length() - 1 for t in cur]
    transcript.append_scalars([F.from_int(num_vars), F.from_int(d)])
    proof, point = [], []
    for i in range(num_vars):
        left = num_vars - i
        evals = sumcheck_round(F, left, cur, terms, d)
        transcript.append_scalars(evals)
        r = transcript.append_and_sample(ROUND_LABEL)
        proof.append(evals)
        point.append(r)
        for j in range(len(cur)):
            if nv[j] >= left:
                cur[j] = fold_low(F, cur[j], r)
                nv[j] -= 1
    finals = [array_to_scalars(F, _widen(F, t))[0] for t in cur]
    return proof, point, finals


def interpolate_eval(F, evals, r):
    """Value at r of the polynomial with the given values at 0..len-1."""
    n = len(evals)
    tot = F.zero
    for i in range(n):
        num, den = F.one, F.one
        for j in range(n):
            if j != i:
                num = F.mul(num, F.sub(r, F.from_int(j)))
                den = F.mul(den, F.sub(F.from_int(i), F.from_int(j)))
        tot = F.add(tot, F.mul(evals[i], F.mul(num, F.inv(den))))
    return tot


def sumcheck_verify(F, claimed_sum, proof, num_vars, degree, transcript):
    """IOPVerifierState::verify (zkml/src/lookup/logup_gkr/verifier.rs:186-191):
    returns (point, expected_evaluation)."""
    transcript.append_scalars([F.from_int(num_vars), F.from_int(degree)])
    claim = claimed_sum
    point = []
    assert len(proof) == num_vars
    for evals in proof:
        assert len(evals) == degree + 1
        if F.add(evals[0], evals[1]) != claim:
            raise ValueError("sumcheck round check failed")
        transcript.append_scalars(evals)
        r = transcript.append_and_sample(ROUND_LABEL)
        claim = interpolate_eval(F, evals, r)
        point.append(r)
    return point, claim


def extract_sum(F, proof):
    """IOPProof::extract_sum (zkml/src/layers/hadamard.rs:118)."""
    return F.add(proof[0][0], proof[0][1])


# ----------------------------------------------------------------- logup-GKR
def logup_next(F, kind, cols, mult, constant, sep):
    """One LogUpLayer::next_layer step (zkml/src/lookup/logup_gkr/circuit.rs:88-184).
    kind 0 lookup / 1 table: cols = denominator columns; kind 2: cols = [num, den]."""
    cols = [np.ascontiguousarray(c) for c in cols]
    half = table_len(cols[0]) // 2
    num = np.empty((half, F.elem_words), dtype=np.uint64)
    den = np.empty((half, F.elem_words), dtype=np.uint64)
    k = len(cols)
    ptrs = (ctypes.c_void_p * k)(*[c.ctypes.data for c in cols])
    dts = (ctypes.c_int * k)(*[F.dtype_of(c) for c in cols])
    cst = scalars_to_array(F, [constant if constant is not None else F.zero])
    sp = scalars_to_array(F, [sep if sep is not None else F.zero])
    m = np.ascontiguousarray(mult) if mult is not None else None
    fn = lib().orc_logup_next_gl if F is GlField else lib().orc_logup_next_fr
    fn(ctypes.c_int(kind), ptrs, dts, ctypes.c_uint32(k), _ptr(m) if m is not None else None,
       ctypes.c_int(F.dtype_of(m) if m is not None else 0), _ptr(cst), _ptr(sp), ctypes.c_uint64(half),
       _ptr(num), _ptr(den))
    return num, den


class LogUpCircuit:
    """LogUpCircuit::new (zkml/src/lookup/logup_gkr/circuit.rs:512-516): all
    levels, bottom to top.  levels[0] describes the input layer; levels[l] for
    l >= 1 are (num, den) arrays of 2^(m-l) entries."""

    def __init__(self, F, kind, columns, mult, constant, sep):
        self.F, self.kind = F, kind  # 0 lookup, 1 table
        self.columns, self.mult, self.constant, self.sep = columns, mult, constant, sep
        m = table_len(columns[0]).bit_length() - 1
        assert m >= 2
        self.m = m
        self.levels = [None]
        num, den = logup_next(F, kind, columns, mult, constant, sep)
        self.levels.append((num, den))
        while table_len(num) > 2:
            num, den = logup_next(F, 2, [num, den], None, None, None)
            self.levels.append((num, den))

    def num_vars(self):
        """circuit.rs:564-566: the input layer's num_vars = m - 1"""
        return self.m - 1

    def outputs(self):
        """circuit.rs:558-560: [num[0], num[1], den[0], den[1]] of the top level"""
        num, den = self.levels[-1]
        return array_to_scalars(self.F, num) + array_to_scalars(self.F, den)

    def final_eval_count(self):
        """circuit.rs:414-426"""
        return 2 * len(self.columns) + (2 if self.kind == 1 else 0)

    def layer_tables(self, layer_vars):
        """The MLEs LogUpLayer::layer_proving_info registers for the layer whose
        halves have `layer_vars` variables (circuit.rs:255-271, 298-353, 360-409)."""
        half = 1 << layer_vars
        if layer_vars == self.m - 1:  # the input layer
            lo = [np.ascontiguousarray(c[:half]) for c in self.columns]
            hi = [np.ascontiguousarray(c[half:]) for c in self.columns]
            if self.kind == 1:
                return [np.ascontiguousarray(self.mult[:half]), np.ascontiguousarray(self.mult[half:])] + lo + hi
            return lo + hi
        num, den = self.levels[self.m - 1 - layer_vars]
        return [num[:half], num[half:], den[:half], den[half:]]

    def layer_exprs(self, layer_vars, layer_count, wit0):
        """(sumcheck_expression, claim_expression, n_witnesses) of
        layer_proving_info (circuit.rs:231-412)."""
        F = self.F
        one, zero = F.one, F.zero
        W, C = Expr.wit, Expr.chal
        b = layer_count * 4
        claim = C(0, layer_count, one, zero) * (
            C(2, 1, one, zero) * (W(b + 1) - W(b)) + W(b)
            + C(1, 1, one, zero) * (C(2, 1, one, zero) * (W(b + 3) - W(b + 2)) + W(b + 2)))
        alpha_j = C(0, layer_count, one, zero)
        lam = C(1, 1, one, zero)
        if layer_vars != self.m - 1:
            n_lo, n_hi, d_lo, d_hi = W(wit0), W(wit0 + 1), W(wit0 + 2), W(wit0 + 3)
            sc = alpha_j * (n_lo * d_hi + n_hi * d_lo + lam * d_lo * d_hi)
            return sc, claim, 4
        ncol = len(self.columns)
        first = wit0 + (2 if self.kind == 1 else 0)
        d_lo, d_hi = Expr.const(self.constant), Expr.const(self.constant)
        pw = one
        for i in range(ncol):
            d_lo = d_lo + Expr.const(pw) * W(first + i)
            d_hi = d_hi + Expr.const(pw) * W(first + ncol + i)
            pw = F.mul(pw, self.sep)
        if self.kind == 1:
            sc = alpha_j * (W(wit0) * d_hi + W(wit0 + 1) * d_lo + lam * d_lo * d_hi)
            return sc, claim, 2 + 2 * ncol
        sc = alpha_j * (-d_hi - d_lo + lam * d_lo * d_hi)
        return sc, claim, 2 * ncol

    def combine_final_evals(self, evals, rho):
        """circuit.rs:442-500"""
        F = self.F
        ncol = len(self.columns)
        out = []
        if self.kind == 1:
            out.append(F.add(F.mul(rho, F.sub(evals[1], evals[0])), evals[0]))
            evals = evals[2:]
        lo, hi = evals[:ncol], evals[ncol:]
        out += [F.add(F.mul(rho, F.sub(h, l)), l) for l, h in zip(lo, hi)]
        return out


class LogUpInput:
    """zkml/src/lookup/logup_gkr/structs.rs:138-231.  kind 0 = Lookup with
    `columns_per_instance` columns per circuit, kind 1 = Table."""

    def __init__(self, F, kind, columns, constant, sep, columns_per_instance=None, mult=None):
        if not columns:
            raise ValueError("No column evals were provided for Lookup input")
        n = table_len(columns[0])
        if n & (n - 1) or n == 0:
            raise ValueError(f"Need a power of two number of evaluations got: {n}")
        if any(table_len(c) != n for c in columns):
            raise ValueError("All sets of evaluations should be the same length")
        if kind == 1 and table_len(mult) != n:
            raise ValueError("Multiplicities length was not equal to column evaluations length")
        self.F, self.kind, self.columns, self.constant, self.sep = F, kind, columns, constant, sep
        self.columns_per_instance = columns_per_instance if kind == 0 else len(columns)
        self.mult = mult

    def make_new_circuits(self):
        """structs.rs:241-272"""
        if self.kind == 1:
            return [LogUpCircuit(self.F, 1, self.columns, self.mult, self.constant, self.sep)]
        c = self.columns_per_instance
        return [LogUpCircuit(self.F, 0, self.columns[i:i + c], None, self.constant, self.sep)
                for i in range(0, len(self.columns), c)]


def logup_batch_prove(F, inputs, transcript):
    """new_batch_multiple_sizes_prove (zkml/src/lookup/logup_gkr/prover.rs:91-344).
    Returns a dict with the fields of LogUpBatchProof (structs.rs:555-578)."""
    if not inputs:
        raise ValueError("No inputs provided for LogUp")
    if any(i.kind != inputs[0].kind for i in inputs):
        raise ValueError("Not all proof types matched")
    circuits = [c for i in inputs for c in i.make_new_circuits()]
    for a, b in zip(circuits, circuits[1:]):
        if a.num_vars() < b.num_vars():
            raise ValueError("Circuits were not in decreasing size order")
    total_layers = max(c.num_vars() for c in circuits)
    sizes = sorted({c.num_vars() for c in circuits}, reverse=True)
    by_size = {s: [c for c in circuits if c.num_vars() == s] for s in sizes}
    circuit_outputs = [c.outputs() for c in circuits]

    transcript.append_scalars([F.from_int(len(circuits))])
    for o in circuit_outputs:
        transcript.append_scalars(o)
    rho = transcript.append_and_sample(b"initial_batching")
    alpha = transcript.append_and_sample(b"initial_alpha")
    lam = transcript.append_and_sample(b"initial_lambda")
    point = [rho]
    sumcheck_proofs, round_evaluations = [], []

    for v in range(1, total_layers + 1):
        remaining = total_layers - (v - 1)
        joining = [e for c in by_size.get(remaining, []) for e in c.outputs()]
        wit_evals = (round_evaluations[-1] if round_evaluations else []) + joining
        if not wit_evals:
            raise ValueError("Proving failed: No previous evals and no evals for this number of variables")
        tables, eq_tables, group_exprs = [], [], []
        claim_expr = Expr.const(F.zero)
        layer_count, wit_off = 0, 0
        for size in sizes:
            if size < remaining:
                continue
            mult = Expr.const(F.from_int(1 << (total_layers - size)))
            layer_vars = size - remaining + 1  # variables of this group's halves in this step
            group = Expr.const(F.zero)
            for c in by_size[size]:
                sc, cl, nw = c.layer_exprs(layer_vars, layer_count, wit_off)
                tables += c.layer_tables(layer_vars)
                layer_count += 1
                wit_off += nw
                group = group + sc
                claim_expr = claim_expr + mult * cl
            eq_tables.append(eq_evals(F, point[len(point) - layer_vars:]))
            group_exprs.append(group)
        current_claim = eval_expr(F, claim_expr, wit_evals, [alpha, lam, rho])
        transcript.append_scalars([current_claim])
        full = Expr.const(F.zero)
        for i, g in enumerate(group_exprs):
            full = full + g * Expr.wit(wit_off + i)
        terms = expr_to_terms(F, full, [alpha, lam])
        proof, point, finals = sumcheck_prove(F, v, tables + eq_tables, terms, transcript)
        evals = finals[:wit_off]
        rho = transcript.append_and_sample(b"logup_batching")
        if v != total_layers:
            alpha = transcript.append_and_sample(b"logup_alpha")
            lam = transcript.append_and_sample(b"logup_lambda")
        point = point + [rho]
        sumcheck_proofs.append(proof)
        round_evaluations.append(evals)

    output_claims, ncols = [], []
    skip = 0
    last = round_evaluations[-1]
    for c in circuits:
        n = c.final_eval_count()
        ev = c.combine_final_evals(last[skip:skip + n], rho)
        skip += n
        pt = point[len(point) - (c.num_vars() + 1):]
        output_claims += [(pt, e) for e in ev]
        ncols.append(len(c.columns))
    return dict(sumcheck_proofs=sumcheck_proofs, round_evaluations=round_evaluations,
                output_claims=output_claims, circuit_outputs=circuit_outputs, proof_type=inputs[0].kind,
                num_vars_per_instance=[c.num_vars() for c in circuits],
                num_denominator_columns_per_instance=ncols)


def _verifier_instance_exprs(F, inst, layer_count, wit0, is_final):
    """LogUpVerifierInstance::instance_expressions (structs.rs:427-553).
    inst = dict(constant, sep, num_columns, kind, num_vars)."""
    one, zero = F.one, F.zero
    W, C = Expr.wit, Expr.chal
    b = layer_count * 4
    claim = C(0, layer_count, one, zero) * (
        C(2, 1, one, zero) * (W(b + 1) - W(b)) + W(b)
        + C(1, 1, one, zero) * (C(2, 1, one, zero) * (W(b + 3) - W(b + 2)) + W(b + 2)))
    alpha_j, lam = C(0, layer_count, one, zero), C(1, 1, one, zero)
    if not is_final:
        sc = alpha_j * (W(wit0) * W(wit0 + 3) + W(wit0 + 1) * W(wit0 + 2) + lam * W(wit0 + 2) * W(wit0 + 3))
        return sc, claim, 4
    ncol = inst["num_columns"]
    first = wit0 + (2 if inst["kind"] == 1 else 0)
    d_lo, d_hi = Expr.const(inst["constant"]), Expr.const(inst["constant"])
    pw = one
    for i in range(ncol):
        d_lo = d_lo + Expr.const(pw) * W(first + i)
        d_hi = d_hi + Expr.const(pw) * W(first + ncol + i)
        pw = F.mul(pw, inst["sep"])
    if inst["kind"] == 1:
        return alpha_j * (W(wit0) * d_hi + W(wit0 + 1) * d_lo + lam * d_lo * d_hi), claim, 2 + 2 * ncol
    return alpha_j * (-d_hi - d_lo + lam * d_lo * d_hi), claim, 2 * ncol


def logup_batch_verify(F, proof, instances, transcript):
    """new_verify_logup_proof_multiple_sizes (zkml/src/lookup/logup_gkr/verifier.rs:77-256).
    Returns dict(output_claims, point, numerators, denominators); raises on failure."""
    transcript.append_scalars([F.from_int(len(instances))])
    for o in proof["circuit_outputs"]:
        transcript.append_scalars(o)
    numer = [F.add(F.mul(e[0], e[3]), F.mul(e[1], e[2])) for e in proof["circuit_outputs"]]
    denom = [F.mul(e[2], e[3]) for e in proof["circuit_outputs"]]
    out_by_size = {}
    for inst, o in zip(instances, proof["circuit_outputs"]):
        out_by_size.setdefault(inst["num_vars"], []).append(o)
    sizes = sorted({i["num_vars"] for i in instances}, reverse=True)
    total_layers = len(proof["sumcheck_proofs"])
    rho = transcript.append_and_sample(b"initial_batching")
    alpha = transcript.append_and_sample(b"initial_alpha")
    lam = transcript.append_and_sample(b"initial_lambda")
    point = [rho]
    for i, (sc_proof, round_evals) in enumerate(zip(proof["sumcheck_proofs"], proof["round_evaluations"])):
        remaining = total_layers - i
        joining = [e for o in out_by_size.get(remaining, []) for e in o]
        wit_evals = (proof["round_evaluations"][i - 1] if i else []) + joining
        layer_count, wit_off = 0, 0
        claim_expr = Expr.const(F.zero)
        group_exprs, eq_points = [], []
        for size in sizes:
            if size < remaining:
                continue
            mult = Expr.const(F.from_int(1 << (total_layers - size)))
            group = Expr.const(F.zero)
            cur_vars = size + 1 - remaining
            for inst in instances:
                if inst["num_vars"] == size:
                    sc, cl, nw = _verifier_instance_exprs(F, inst, layer_count, wit_off, i + 1 == total_layers)
                    layer_count += 1
                    wit_off += nw
                    group = group + sc
                    claim_expr = claim_expr + mult * cl
            eq_points.append(point[len(point) - cur_vars:])
            group_exprs.append(group)
        current_claim = eval_expr(F, claim_expr, wit_evals, [alpha, lam, rho])
        transcript.append_scalars([current_claim])
        cur_point, expected = sumcheck_verify(F, current_claim, sc_proof, i + 1, 3, transcript)
        rho = transcript.append_and_sample(b"logup_batching")
        full = Expr.const(F.zero)
        for g_i, g in enumerate(group_exprs):
            full = full + g * Expr.wit(wit_off + g_i)
        eq_vals = [identity_eval(F, cur_point[len(cur_point) - len(p):], p) for p in eq_points]
        calc = eval_expr(F, full, list(round_evals) + eq_vals, [alpha, lam])
        if i + 1 != total_layers:
            alpha = transcript.append_and_sample(b"logup_alpha")
            lam = transcript.append_and_sample(b"logup_lambda")
        if calc != expected:
            raise ValueError(f"LogUp Verifier error at round {i}")
        point = cur_point + [rho]
    last = proof["round_evaluations"][-1]
    skip, claims = 0, []
    for inst in instances:
        ncol = inst["num_columns"]
        n = 2 * ncol + (2 if inst["kind"] == 1 else 0)
        ev = last[skip:skip + n]
        skip += n
        pt = point[len(point) - 1 - inst["num_vars"]:]
        if inst["kind"] == 1:
            claims.append((pt, F.add(F.mul(rho, F.sub(ev[1], ev[0])), ev[0])))
            ev = ev[2:]
        claims += [(pt, F.add(F.mul(rho, F.sub(h, l)), l)) for l, h in zip(ev[:ncol], ev[ncol:])]
    return dict(output_claims=claims, point=point, numerators=numer, denominators=denom)


# --------------------------------------------------------- layer-level provers
def hadamard_prove(F, transcript, claim_point, v1, v2):
    """zkml/src/layers/hadamard.rs:93-131: sum_x v1(x) v2(x) eq(r, x)."""
    beta = eq_evals(F, claim_point)
    terms = {(0, 1, 2): F.one}
    proof, point, finals = sumcheck_prove(F, len(claim_point), [v1, v2, beta], terms, transcript)
    return dict(sumcheck=proof, individual_claim=finals[:2], point=point)


def same_poly_prove(F, transcript, poly, claims):
    """same_poly::Prover::prove (zkml/src/iop/same_poly.rs:84-114):
    sum_x f(x) * sum_i a_i eq_i(x)."""
    chal = transcript.read_challenges(len(claims))
    betas = [eq_evals(F, pt) for pt, _ in claims]
    e = Expr.const(F.zero)
    for i in range(len(claims)):
        e = e + Expr.chal(i, 1, F.one, F.zero) * Expr.wit(1 + i)
    terms = expr_to_terms(F, Expr.wit(0) * e, chal)
    n = len(claims[0][0])
    proof, point, finals = sumcheck_prove(F, n, [poly] + betas, terms, transcript)
    return dict(sumcheck=proof, eval=finals[0], point=point, challenges=chal)


# ------------------------------------------------ claim batching (opening proof)
def zero_pad_table(F, table, num_vars):
    """DensePolynomial::zero_pad_num_vars, materialised: entries above the table's length are zero, i.e. the
    padded polynomial is p(x_0..x_{m-1}) * prod_{j >= m} (1 - x_j) (the verifier's formula for padded eq tables,
    zkml/src/poly_commit/verifier.rs:300-311, pins this convention)."""
    t = _widen(F, table)
    out = np.zeros((1 << num_vars, F.elem_words), dtype=np.uint64)
    out[: t.shape[0]] = t
    return out


def linear_combination(F, tables, coeffs):
    """DensePolynomial::linear_combination (zkml/src/poly_commit/prover.rs:122); shorter tables are zero-padded."""
    n = max(table_len(t) for t in tables)
    acc = [F.zero] * n
    for t, c in zip(tables, coeffs):
        for i, v in enumerate(array_to_scalars(F, _widen(F, t))):
            acc[i] = F.add(acc[i], F.mul(c, v))
    return scalars_to_array(F, acc)


class CommittedPoly:
    """A committed polynomial as its M = 2^b chunk tables of equal length (ChunkedCommitment,
    zkml/src/poly_commit/mod.rs:32-93) with the claims to batch for it."""

    def __init__(self, chunks, claims):
        self.chunks = chunks
        self.claims = claims  # [(point over chunk_vars + b coordinates, eval)]
        self.num_chunks = len(chunks)
        self.batch_vars = (self.num_chunks - 1).bit_length()
        assert 1 << self.batch_vars == self.num_chunks
        self.chunk_vars = (table_len(chunks[0]) - 1).bit_length()

    def eq_point_per_chunk(self, point):
        return point[: len(point) - self.batch_vars]

    def batching_coefficients_for_chunks(self, F, point):
        coords = point[len(point) - self.batch_vars:]
        return [identity_eval(F, coords, [F.from_int((i >> b) & 1) for b in range(self.batch_vars)])
                for i in range(self.num_chunks)]


def claims_batching_expression(F, polys, coeffs_per_poly):
    """build_sumcheck_expression (zkml/src/poly_commit/mod.rs:96-148)."""
    eq_offset = sum(p.num_chunks for p in polys)
    e = Expr.const(F.zero)
    total_terms = total_polys = 0
    for p, per_claim in zip(polys, coeffs_per_poly):
        for i, chunk_coeffs in enumerate(per_claim):
            inner = Expr.const(F.zero)
            for ci, c in enumerate(chunk_coeffs):
                inner = inner + Expr.const(c) * Expr.wit(total_polys + ci)
            e = e + Expr.chal(0, total_terms + i, F.one, F.zero) * inner * Expr.wit(total_terms + i + eq_offset)
        total_terms += len(per_claim)
        total_polys += p.num_chunks
    return e


def claims_batching_prove(F, polys, transcript):
    """CommitmentProver::claims_batching_sumcheck + the random linear combination that follows it
    (zkml/src/poly_commit/prover.rs:113-131, 140-255).  `polys` in the order the reference visits them
    (model commitments, then witness commitments)."""
    eq_tables, committed, coeffs_per_poly = [], [], []
    max_vars = 0
    for p in polys:
        per_claim = []
        for point, ev in p.claims:
            transcript.append_scalars([ev])
            eq_tables.append(eq_evals(F, p.eq_point_per_chunk(point)))
            per_claim.append(p.batching_coefficients_for_chunks(F, point))
        coeffs_per_poly.append(per_claim)
        committed.extend(p.chunks)
        max_vars = max(max_vars, p.chunk_vars)
    expr = claims_batching_expression(F, polys, coeffs_per_poly)
    challenge = transcript.append_and_sample(b"model_batching")
    terms = expr_to_terms(F, expr, [challenge])
    tables = [zero_pad_table(F, t, max_vars) for t in committed + eq_tables]
    proof, point, finals = sumcheck_prove(F, max_vars, tables, terms, transcript, degree=2)
    evals = finals[: len(committed)]
    transcript.append_scalars(point)
    transcript.append_scalars(evals)
    rlc_challenges = [transcript.challenge_scalar() for _ in committed]
    rlc = linear_combination(F, committed, rlc_challenges)
    return dict(sumcheck=proof, sumcheck_evals=evals, point=point, rlc_challenges=rlc_challenges, rlc=rlc)


def claims_batching_verify(F, proof, polys_info, transcript):
    """CommitmentVerifier::claims_batching_sumcheck (zkml/src/poly_commit/verifier.rs:203-330).
    polys_info: CommittedPoly objects whose chunks may be None (only sizes and claims are used)."""
    eq_points, evals, coeffs_per_poly = [], [], []
    max_vars = 0
    for p in polys_info:
        per_claim = []
        for point, ev in p.claims:
            transcript.append_scalars([ev])
            eq_points.append(p.eq_point_per_chunk(point))
            evals.append(ev)
            per_claim.append(p.batching_coefficients_for_chunks(F, point))
        coeffs_per_poly.append(per_claim)
        max_vars = max(max_vars, p.chunk_vars)
    expr = claims_batching_expression(F, polys_info, coeffs_per_poly)
    challenge = transcript.append_and_sample(b"model_batching")
    claimed, acc = F.zero, F.one
    for e in evals:
        claimed = F.add(claimed, F.mul(acc, e))
        acc = F.mul(acc, challenge)
    try:
        point, expected = sumcheck_verify(F, claimed, proof["sumcheck"], max_vars, 2, transcript)
    except ValueError:
        return False
    wit = list(proof["sumcheck_evals"])
    for eq_point in eq_points:
        v = identity_eval(F, point[: len(eq_point)], eq_point)
        for pcoord in point[len(eq_point):]:
            v = F.mul(v, F.sub(F.one, pcoord))
        wit.append(v)
    return eval_expr(F, expr, wit, [challenge]) == expected


# -------------------------------------------------------------- serialization
def serialize_scalars(F, vals):
    return b"".join(F.to_canonical(v) for v in vals)


def serialize_sumcheck_proof(F, proof):
    return b"".join(serialize_scalars(F, ev) for ev in proof)


def serialize_logup_proof(F, p):
    """A flat canonical encoding used to compare proofs byte for byte:
    u32 counts (LE) followed by canonical scalars, field order of
    LogUpBatchProof (zkml/src/lookup/logup_gkr/structs.rs:561-578)."""
    out = bytearray()
    u32 = lambda x: int(x).to_bytes(4, "little")
    out += u32(len(p["sumcheck_proofs"]))
    for sp in p["sumcheck_proofs"]:
        out += u32(len(sp))
        for ev in sp:
            out += u32(len(ev)) + serialize_scalars(F, ev)
    out += u32(len(p["round_evaluations"]))
    for ev in p["round_evaluations"]:
        out += u32(len(ev)) + serialize_scalars(F, ev)
    out += u32(len(p["output_claims"]))
    for pt, e in p["output_claims"]:
        out += u32(len(pt)) + serialize_scalars(F, pt) + serialize_scalars(F, [e])
    out += u32(len(p["circuit_outputs"]))
    for o in p["circuit_outputs"]:
        out += u32(len(o)) + serialize_scalars(F, o)
    out += u32(p["proof_type"])
    out += u32(len(p["num_vars_per_instance"]))
    for v in p["num_vars_per_instance"]:
        out += u32(v)
    out += u32(len(p["num_denominator_columns_per_instance"]))
    for v in p["num_denominator_columns_per_instance"]:
        out += u32(v)
    return bytes(out)


def serialize_einsum_proof(F, p):
    """The flat encoding of einsum_prove's result that the library's dpb_einsum_proof_serialize writes."""
    out = bytearray()
    u32 = lambda x: int(x).to_bytes(4, "little")

    def sumcheck(sp):
        b = u32(len(sp))
        for ev in sp:
            b += u32(len(ev)) + serialize_scalars(F, ev)
        return b

    def claim(c):
        return u32(len(c[0])) + serialize_scalars(F, c[0]) + serialize_scalars(F, [c[1]])
    out += u32(len(p["stacking_coeffs"])) + u32(len(p["stacking_coeffs"][0]))
    out += serialize_scalars(F, [p["batching_challenge"]])
    for cs in p["stacking_coeffs"]:
        out += serialize_scalars(F, cs)
    out += sumcheck(p["sumcheck"])
    out += u32(len(p["point"])) + serialize_scalars(F, p["point"])
    out += u32(len(p["evaluations"])) + serialize_scalars(F, p["evaluations"])
    for c in p["rhs_claims"]:
        out += claim(c)
    out += claim(p["lhs_claim"])
    if p["aggregation"] is None:
        out += u32(0)
    else:
        out += u32(1) + serialize_scalars(F, [p["aggregation"]["challenge"]]) + sumcheck(p["aggregation"]["sumcheck"])
    return bytes(out)


# ------------------------------------------------------------ einsum axis fixing
AXIS_CONTRACTED, AXIS_OUTER, AXIS_STACKED = 0, 1, 2


def mles_from_tensor(F, tensor_i64, kinds, points):
    """FixedAxesMapping::mles_from_tensor (zkml/src/layers/einsum/axis.rs:1142-1234),
    axis by axis from the innermost one as the reference does: an Outer axis is
    contracted against evals(point)[..size] (a plain dot product when nothing
    kept lies inside it, a strided one otherwise), Stacked and Contracted axes
    are kept; the result is cut into chunks of the contraction size, each
    zero-padded to a power of two.  Scalars are Python ints (small tensors only).
    Returns a list of tables (one per stacked index)."""
    shape = list(tensor_i64.shape)
    cur = [F.from_int(int(v)) for v in np.asarray(tensor_i64).reshape(-1)]
    chunk, contraction = 1, 1
    for axis in reversed(range(len(shape))):
        size = shape[axis]
        if kinds[axis] == AXIS_OUTER:
            beta = array_to_scalars(F, eq_evals(F, points[axis]))[:size]
            nxt = []
            for start in range(0, len(cur), chunk * size):
                full = cur[start:start + chunk * size]
                for i in range(chunk):
                    acc = F.zero
                    for b, v in zip(beta, full[i::chunk]):
                        acc = F.add(acc, F.mul(v, b))
                    nxt.append(acc)
            cur = nxt
        elif kinds[axis] == AXIS_STACKED:
            chunk *= size
        else:
            chunk *= size
            contraction *= size
    n_vars = max(contraction - 1, 0).bit_length()
    pad = (1 << n_vars) - contraction
    out = []
    for start in range(0, len(cur), contraction):
        vals = cur[start:start + contraction] + [F.zero] * pad
        out.append(scalars_to_array(F, vals))
    return out


def stacking_coefficients(F, shape, kinds, points):
    """FixedAxesMapping::lhs_fixes / stacking_coefficients (zkml/src/layers/einsum/axis.rs:1043-1062, 1077-1100):
    the product over the Stacked axes of evals(point)[..size], the FIRST stacked axis the slowest index."""
    acc = [F.one]
    for axis in reversed(range(len(shape))):
        if kinds[axis] != AXIS_STACKED:
            continue
        beta = array_to_scalars(F, eq_evals(F, points[axis]))[:shape[axis]]
        acc = [F.mul(a, b) for b in beta for a in acc]
    return acc


def reconstruct_full_point(kinds, points, sumcheck_point, padded_shape):
    """reconstruct_full_point (zkml/src/layers/einsum/prove.rs:338-361): the axes from last to first; Outer and
    Stacked axes give their own point, a Contracted axis the next ceil_log2(dim) sumcheck coordinates."""
    out, skip = [], 0
    for axis in reversed(range(len(kinds))):
        if kinds[axis] == AXIS_CONTRACTED:
            n = max(int(padded_shape[axis]) - 1, 0).bit_length()
            out += list(sumcheck_point[skip:skip + n])
            skip += n
        else:
            out += list(points[axis])
    return out


def einsum_prove(F, transcript, lhs, lhs_fixes, rhs, lhs_padded=None):
    """EinSum::prove_internal (zkml/src/layers/einsum/prove.rs:48-335) below the axis mapping and without biases
    (a bias claim is an evaluation, prove.rs:190-213; it does not touch the transcript).

    lhs: the left tensor (int64 array, unpadded); lhs_fixes[i] = (kinds, points) fixes it for output i;
    rhs[i] = (tensor, kinds, points) is the right tensor of output i.  Outer and Stacked axes carry points.
    The sumcheck proves  sum_i gamma^i sum_t coef_{i,t} lhs_{i,t} rhs_{i,t}  with gamma sampled under the label
    "batching_challenge" (prove.rs:157; expression: op_info.rs:159-195).  With more than one output the claims on
    the left tensor are merged by a second sumcheck  input * sum_i c^i eq_i  over the padded left tensor
    `lhs_padded` (prove.rs:260-288), c sampled under "input_batching_challenge"."""
    R = len(rhs)
    assert len(lhs_fixes) == R and R >= 1
    lhs = np.asarray(lhs, dtype=np.int64)
    lhs_tabs, coeffs = [], []
    for kinds, points in lhs_fixes:
        lhs_tabs.append(mles_from_tensor(F, lhs, tuple(kinds), list(points)))
        coeffs.append(stacking_coefficients(F, lhs.shape, kinds, points))
    rhs_tabs = [mles_from_tensor(F, np.asarray(t, dtype=np.int64), tuple(k), list(p)) for t, k, p in rhs]
    S = len(coeffs[0])
    assert all(len(t) == S for t in lhs_tabs + rhs_tabs)
    gamma = transcript.append_and_sample(b"batching_challenge")
    e = None
    for i in range(R):
        off, roff = i * S, R * S + i * S
        inner = Expr.const(coeffs[i][0]) * Expr.wit(off) * Expr.wit(roff)
        for j in range(1, S):
            inner = Expr.const(coeffs[i][j]) * Expr.wit(off + j) * Expr.wit(roff + j) + inner
        term = Expr.chal(0, i, F.one, F.zero) * inner
        e = term if e is None else e + term
    terms = expr_to_terms(F, e, [gamma])
    tables = [t for ts in lhs_tabs for t in ts] + [t for ts in rhs_tabs for t in ts]
    n = table_len(tables[0]).bit_length() - 1
    proof, point, finals = sumcheck_prove(F, n, tables, terms, transcript)

    def pad(shape):
        return [1 << max(int(d) - 1, 0).bit_length() for d in shape]

    def comb(c, ev):
        acc = F.zero
        for a, b in zip(c, ev):
            acc = F.add(acc, F.mul(a, b))
        return acc
    rhs_claims = []
    for i, (t, kinds, points) in enumerate(rhs):
        full = reconstruct_full_point(kinds, points, point, pad(np.asarray(t).shape))
        rhs_claims.append((full, comb(coeffs[i], finals[R * S + i * S:R * S + (i + 1) * S])))
    out = dict(batching_challenge=gamma, stacking_coeffs=coeffs, sumcheck=proof, point=point, evaluations=finals,
               rhs_claims=rhs_claims, aggregation=None)
    if R == 1:
        kinds, points = lhs_fixes[0]
        out["lhs_claim"] = (reconstruct_full_point(kinds, points, point, pad(lhs.shape)), comb(coeffs[0], finals[:S]))
        return out
    eqs = [eq_evals(F, reconstruct_full_point(k, p, point, pad(lhs.shape))) for k, p in lhs_fixes]
    c = transcript.append_and_sample(b"input_batching_challenge")
    agg = None
    for i in range(R):
        term = Expr.wit(0) * Expr.wit(i + 1) * Expr.chal(0, i, F.one, F.zero)
        agg = term if agg is None else agg + term
    nv = table_len(lhs_padded).bit_length() - 1
    a_proof, a_point, a_finals = sumcheck_prove(F, nv, [lhs_padded] + eqs, expr_to_terms(F, agg, [c]), transcript)
    out["aggregation"] = dict(challenge=c, sumcheck=a_proof, point=a_point)
    out["lhs_claim"] = (a_point, a_finals[0])
    return out


# ------------------------------------------------- lookup witness generation
SHIFT_CHECK_TABLE_BIT_SIZE = 16  # zkml/src/lookup/table/mod.rs:20-23
ZERO_CHECK_TABLE_BIT_SIZE = 16
COLUMN_SEPARATOR = 1 << 32       # zkml/src/lookup/context.rs:205
SIGN_POSITIVE, SIGN_NEGATIVE, SIGN_MIXED = 0, 1, 2


def table_input_range(table_bits, sign):
    """Table::min_input_value / max_input_value (zkml/src/lookup/table/mod.rs:126-142)."""
    if sign == SIGN_POSITIVE:
        return 0, (1 << table_bits) - 1
    if sign == SIGN_MIXED:
        return -(1 << (table_bits - 1)), (1 << (table_bits - 1)) - 1
    return -(1 << table_bits) + 1, 0


class ChunkingInfo:
    """ChunkingInfo::new (zkml/src/lookup/operation/decomposer.rs:182-249): how a rescaled value is cut into
    shifted chunks (the bits a right shift drops, 16 at a time), value chunks (looked up in the value table)
    and zeroing chunks (the bits above, 16 at a time)."""

    def __init__(self, right_shift, table_bits, sign, max_bit_size, n_value_chunks=1):
        if right_shift <= 0:
            raise ValueError("Right shift must be greater than zero to decompose value")
        self.right_shift, self.value_chunk_size, self.sign = right_shift, table_bits, sign
        self.n_value = n_value_chunks
        self.n_shifted = -(-right_shift // SHIFT_CHECK_TABLE_BIT_SIZE)
        self.n_zeroing = -(-max(max_bit_size - (right_shift + table_bits * n_value_chunks), 0) // ZERO_CHECK_TABLE_BIT_SIZE)
        rem = right_shift % SHIFT_CHECK_TABLE_BIT_SIZE
        self.shifted_chunk_multiplier = (1 << (SHIFT_CHECK_TABLE_BIT_SIZE - rem)) if rem else 1
        if sign == SIGN_MIXED:
            self.value_chunk_offset = 1 << (table_bits - 1)
            combined = 1 << (table_bits * n_value_chunks - 1)
            first = max(1 << (max_bit_size - 1), combined << right_shift)
            self.offset = first + (1 if self.n_zeroing > 0 else 0) * (combined << right_shift)
        else:
            self.value_chunk_offset = self.offset = 0
        if self.n_zeroing > 0 and sign == SIGN_MIXED:
            self.top_zeroing_chunk_offset = self.offset >> (
                right_shift + table_bits * n_value_chunks + (self.n_zeroing - 1) * ZERO_CHECK_TABLE_BIT_SIZE)
        else:
            self.top_zeroing_chunk_offset = 0
        self.is_signed = sign == SIGN_MIXED

    def rounding_constant(self):
        return 1 << (self.right_shift - 1)

    def decompose_input(self, values):
        """decompose_input (decomposer.rs:252-312) on an int64 array; returns (shifted, value, zeroing), each a
        list of int64 arrays."""
        v = np.asarray(values, dtype=np.int64)
        rem = v + self.offset if self.sign == SIGN_MIXED else (v.copy() if self.sign == SIGN_POSITIVE else -v)
        shifted, value, zeroing = [], [], []
        for i in range(self.n_shifted):
            if i != self.n_shifted - 1 or self.right_shift % SHIFT_CHECK_TABLE_BIT_SIZE == 0:
                shifted.append(rem & ((1 << SHIFT_CHECK_TABLE_BIT_SIZE) - 1))
                rem = rem >> SHIFT_CHECK_TABLE_BIT_SIZE
            else:
                size = self.right_shift % SHIFT_CHECK_TABLE_BIT_SIZE
                shifted.append((rem & ((1 << size) - 1)) * self.shifted_chunk_multiplier)
                rem = rem >> size
        for _ in range(self.n_value):
            c = rem & ((1 << self.value_chunk_size) - 1)
            value.append(c - self.value_chunk_offset if self.sign == SIGN_MIXED else (c if self.sign == SIGN_POSITIVE else -c))
            rem = rem >> self.value_chunk_size
        for i in range(self.n_zeroing):
            c = rem & ((1 << ZERO_CHECK_TABLE_BIT_SIZE) - 1)
            zeroing.append(c if (i != self.n_zeroing - 1 or not self.is_signed) else c - self.top_zeroing_chunk_offset)
            rem = rem >> ZERO_CHECK_TABLE_BIT_SIZE
        return shifted, value, zeroing

    def table_output(self, value, zeroing, value_outputs):
        """table_output (decomposer.rs:315-383): value chunks go through the value table (`value_outputs` = its
        output column over min..=max inputs, or None for a one-column table, whose output is its input), zeroing
        chunks through the zero-check table (1 at 0, else 0), the top chunk of a signed operation through the
        signed zero-check table (signum; an input outside -2^15..2^15-1 is an error)."""
        lo, hi = table_input_range(self.value_chunk_size, self.sign)
        outs = []
        for c in value:
            if c.size and (c.min() < lo or c.max() > hi):
                raise ValueError("value chunk outside its table")
            outs.append(c.copy() if value_outputs is None else np.asarray(value_outputs, dtype=np.int64)[c - lo])
        zouts = []
        for i, c in enumerate(zeroing):
            if self.is_signed and i == self.n_zeroing - 1:
                if c.size and (c.min() < -(1 << 15) or c.max() > (1 << 15) - 1):
                    raise ValueError("out of range for SignedZeroCheckTable")
                zouts.append(np.sign(c).astype(np.int64))
            else:
                zouts.append((c == 0).astype(np.int64))
        return outs, zouts

    def combine_input_claims(self, F, shifted, value, zeroing):
        """combine_input_claims (decomposer.rs:431-499) on field scalars: the rescaled input from its chunks."""
        acc = F.zero
        for j, c in enumerate(shifted):
            w = F.from_int(1 << (j * SHIFT_CHECK_TABLE_BIT_SIZE))
            if j != self.n_shifted - 1 or self.right_shift % SHIFT_CHECK_TABLE_BIT_SIZE == 0:
                acc = F.add(acc, F.mul(c, w))
            else:
                acc = F.add(acc, F.mul(F.mul(c, F.inv(F.from_int(self.shifted_chunk_multiplier))), w))
        comb = F.zero
        for j, c in enumerate(value):
            w = F.from_int(1 << (j * self.value_chunk_size))
            rec = F.add(c, F.from_int(self.value_chunk_offset)) if self.sign == SIGN_MIXED else (c if self.sign == SIGN_POSITIVE else F.neg(c))
            comb = F.add(comb, F.mul(rec, w))
        acc = F.add(acc, F.mul(comb, F.from_int(1 << self.right_shift)))
        for j, c in enumerate(zeroing):
            w = F.from_int(1 << (self.value_chunk_size * self.n_value + self.right_shift + j * ZERO_CHECK_TABLE_BIT_SIZE))
            if j != self.n_zeroing - 1 or not self.is_signed:
                acc = F.add(acc, F.mul(c, w))
            else:
                acc = F.add(acc, F.mul(F.add(c, F.from_int(self.top_zeroing_chunk_offset)), w))
        if self.sign == SIGN_MIXED:
            return F.sub(acc, F.from_int(self.offset))
        return acc if self.sign == SIGN_POSITIVE else F.neg(acc)


class LookupOpWitness:
    """LookupOp::generate_witness (zkml/src/lookup/operation/mod.rs:103-160) and LookupOpWitness
    (mod.rs:163-283).  `inputs[c]` / `outputs[c]` hold, for the c-th slice over the last two dimensions,
    (shifted, value, zeroing) and (value outputs, zeroing outputs)."""

    def __init__(self, info, fixed_point_multiplier, padding_value, tensor, value_outputs, num_value_columns):
        t = np.asarray(tensor, dtype=np.int64)
        if t.ndim < 1:
            raise ValueError("Input tensor must have rank at least 1")
        rows, cols = (1, t.shape[0]) if t.ndim == 1 else t.shape[-2:]
        prow, pcol = 1 << max(rows - 1, 0).bit_length(), 1 << max(cols - 1, 0).bit_length()
        rc = info.rounding_constant()
        self.info, self.num_value_columns = info, num_value_columns
        self.inputs, self.outputs = [], []
        for chunk in t.reshape(-1, rows, cols):
            padded = np.full((prow, pcol), padding_value * fixed_point_multiplier + rc, dtype=np.int64)
            padded[:rows, :cols] = chunk * fixed_point_multiplier + rc
            dec = info.decompose_input(padded.reshape(-1))
            self.inputs.append(dec)
            self.outputs.append(info.table_output(dec[1], dec[2], value_outputs))

    def input_columns(self):
        """input_mle_evals (mod.rs:269-274) with ChunkedInput::to_evals (decomposer.rs:71-87), as int64 arrays."""
        out = []
        for shifted, value, zeroing in self.inputs:
            out += list(shifted) + (list(value) if self.num_value_columns != 1 else []) + list(zeroing)
        return out

    def output_columns(self):
        """output_mle_evals (mod.rs:276-282)."""
        out = []
        for value_out, zero_out in self.outputs:
            out += list(value_out) + list(zero_out)
        return out

    def get_counts(self):
        """get_counts (mod.rs:193-267): how often each (merged) table row is looked up, for the shift-check table,
        the value table, the zero-check table and the signed zero-check table."""
        def count(arrays):
            d = {}
            for a in arrays:
                keys, n = np.unique(a, return_counts=True)
                for k, c in zip(keys.tolist(), n.tolist()):
                    d[k] = d.get(k, 0) + c
            return d
        sep = COLUMN_SEPARATOR
        shift = count([s for dec in self.inputs for s in dec[0]])
        if self.num_value_columns == 1:
            value = count([v for o in self.outputs for v in o[0]])
        else:
            value = count([vi + sep * vo for dec, o in zip(self.inputs, self.outputs) for vi, vo in zip(dec[1], o[0])])
        if not self.info.is_signed:
            zero = count([zi + sep * zo for dec, o in zip(self.inputs, self.outputs) for zi, zo in zip(dec[2], o[1])])
            signed = {}
        else:
            zero = count([zi + sep * zo for dec, o in zip(self.inputs, self.outputs) for zi, zo in zip(dec[2][:-1], o[1][:-1])])
            signed = count([zi + sep * zo for dec, o in zip(self.inputs, self.outputs) for zi, zo in zip(dec[2][-1:], o[1][-1:])])
        return [shift, value, zero, signed]


def merged_table_column(table_bits, sign, outputs):
    """Table::get_merged_table_columns (zkml/src/lookup/table/mod.rs:252-264): input + 2^32 * output per row
    (the input alone for a one-column table, `outputs` None)."""
    lo, hi = table_input_range(table_bits, sign)
    ins = np.arange(lo, hi + 1, dtype=np.int64)
    return ins if outputs is None else ins + COLUMN_SEPARATOR * np.asarray(outputs, dtype=np.int64)


def table_multiplicities(F, merged_column, counts):
    """The multiplicity polynomial of one table (zkml/src/lookup/context.rs:313-371): per row, the number of
    lookups of that row divided by the number of times the row occurs in the table."""
    col = [int(x) for x in merged_column]
    occurs = {}
    for x in col:
        occurs[x] = occurs.get(x, 0) + 1
    vals = []
    for x in col:
        if x in counts:
            inv = F.inv(F.from_int(occurs[x])) if occurs[x] != 1 else F.one
            vals.append(F.mul(F.from_int(counts[x]), inv))
        else:
            vals.append(F.zero)
    return scalars_to_array(F, vals)


# ------------------------------------------------ lookup linking sumcheck
VARIANT_STANDARD, VARIANT_GLU, VARIANT_SOFTMAX, VARIANT_NORMALISATION = 0, 1, 2, 3


def lookup_output_expressions(F, info, chunk, out_min, out_max):
    """LookupVariant::build_lookup_output_expressions (zkml/src/lookup/operation/variant.rs:73-226) with
    ValueExpression::new (variant.rs:467-510): (value, prod_selector, clamping_expression, sum,
    squared_clamping_expression) over the witnesses of one chunk, which are its value chunk outputs followed by its zeroing chunk outputs.  out_min / out_max are
    the value table's extreme outputs (Table::min_output_value / max_output_value)."""
    one, zero = F.one, F.zero
    ONE, bits, nz = Expr.const(one), info.value_chunk_size, info.n_zeroing
    sq_clamp = Expr.const(zero)  # only the signed case with zeroing chunks has one (variant.rs:163-170, 212-213)
    offset = chunk * (info.n_value + nz)
    if info.n_value == 1:
        value = Expr.wit(offset)
        total = Expr.wit(offset) * Expr.chal(0, 1, one, zero)
        wo, so = offset + 1, 2
    else:
        value = Expr.const(F.neg(F.from_int(1 << (info.n_value * bits - 1))))
        total = Expr.const(zero)
        for idx in range(info.n_value):
            c = Expr.wit(offset + idx)
            value = value + Expr.const(F.from_int(1 << (bits * idx))) * (c + Expr.const(F.from_int(1 << (bits - 1))))
            total = total + c * Expr.chal(0, idx + 1, one, zero)
        wo, so = offset + info.n_value, 1 + info.n_value
    if info.is_signed:
        prod = ONE
        for idx in range(max(nz - 1, 0)):
            c = Expr.wit(wo + idx)
            prod = prod * c
            total = total + c * Expr.chal(0, so + idx, one, zero)
        if info.n_value == 1:
            cmin, cmax = F.from_int(out_min), F.from_int(out_max)
        else:
            full = info.n_value * bits
            cmin, cmax = F.from_int(-(1 << (full - 1))), F.from_int((1 << (full - 1)) - 1)
        if nz != 0:
            last = Expr.wit(wo - 1 + nz)
            lower = prod
            one_minus_sq = ONE - last * last
            prod = prod * one_minus_sq
            total = total + last * Expr.chal(0, so - 1 + nz, one, zero)
            half = Expr.const(F.inv(F.from_int(2)))
            first = last * (last + ONE) * half + (one_minus_sq - lower * one_minus_sq)
            second = last * (last - ONE) * half
            clamp = first * Expr.const(cmax) + second * Expr.const(cmin)
            sq_clamp = first * Expr.const(cmax) * Expr.const(cmax) + second * Expr.const(cmin) * Expr.const(cmin)
        else:
            clamp = Expr.const(zero)
    else:
        prod = ONE
        for idx in range(nz):
            c = Expr.wit(wo + idx)
            prod = prod * c
            total = total + c * Expr.chal(0, so + idx, one, zero)
        if nz != 0:
            clamp = Expr.const(F.from_int(out_max if info.sign == SIGN_POSITIVE else out_min))
        else:
            clamp = ONE
    return value, prod, clamp, total, sq_clamp


def lookup_linking_expression(F, variant, total_chunks, info, out_min, out_max, final_dim_size=None,
                              normalised_sum=False, has_weight=False):
    """build_full_sumcheck_expression / sumcheck_expression_for_chunk (variant.rs:55-70, 229-287) for the Standard,
    GLU and Softmax variants: sum over chunks of
        challenge[1 + c] * (eq_out * P_c [* glu_witness_c] [+ 2^k challenge[1 + chunks] * eq_norm * P_c]
                            + eq_lookup * sum),   P_c = clamping + prod_selector * value,
    2^k the padded size of the last dimension.  Witness ids: the chunks' outputs, then (GLU) one witness per chunk,
    then eq_out, eq_lookup, (Softmax) eq_norm.
    Normalisation (variant.rs:288-346), two more witnesses per chunk (the chunk's input and its scaling):
        challenge[1 + c] * (eq_out [* weight] * P_c [+ 2^k nu^2 * eq_norm * P_c] + 2^k nu * eq_norm * Q_c
                            + eq_lookup * (sum + iota * input_c * scaling_c)),
    Q_c = squared clamping + prod_selector * value^2, nu = challenge[1 + chunks], iota = challenge[2 + chunks];
    witness ids: outputs, inputs per chunk, scalings per chunk, eq_out, eq_lookup, eq_norm, (weight)."""
    per = info.n_value + info.n_zeroing
    total_out = total_chunks * per
    extra = {VARIANT_GLU: 1, VARIANT_NORMALISATION: 2}.get(variant, 0)
    total_wit = total_out + total_chunks * extra
    eq_out, eq_lk = Expr.wit(total_wit), Expr.wit(total_wit + 1)
    e = Expr.const(F.zero)
    for c in range(total_chunks):
        value, prod, clamp, total, sq_clamp = lookup_output_expressions(F, info, c, out_min, out_max)
        prod_expression = clamp + prod * value
        if variant == VARIANT_NORMALISATION:
            norm_eq = Expr.wit(total_wit + 2)
            pow_two = F.from_int(1 << max(final_dim_size - 1, 0).bit_length())
            prod_squared = sq_clamp + prod * value * value
            lead = eq_out * Expr.wit(total_wit + 3) if has_weight else eq_out
            out_part = lead * prod_expression
            if normalised_sum:
                out_part = out_part + Expr.chal(1 + total_chunks, 2, pow_two, F.zero) * (norm_eq * prod_expression)
            inp = Expr.wit(total_out + c) * Expr.wit(total_out + total_chunks + c)
            e = e + Expr.chal(1 + c, 1, F.one, F.zero) * (
                out_part + Expr.chal(1 + total_chunks, 1, pow_two, F.zero) * (norm_eq * prod_squared)
                + eq_lk * (total + Expr.chal(2 + total_chunks, 1, F.one, F.zero) * inp))
            continue
        out_part = eq_out * prod_expression
        if variant == VARIANT_GLU:
            out_part = out_part * Expr.wit(total_out + c)
        if variant == VARIANT_SOFTMAX:
            pow_two = F.from_int(1 << max(final_dim_size - 1, 0).bit_length())
            out_part = out_part + Expr.chal(1 + total_chunks, 1, pow_two, F.zero) * (Expr.wit(total_wit + 2) * prod_expression)
        e = e + Expr.chal(1 + c, 1, F.one, F.zero) * (out_part + eq_lk * total)
    return e


def eq_point_and_batching_challenges(F, shape, point):
    """Shape::compute_eq_point_and_batching_challenges (zkml/src/shape.rs:565-610): the coordinates of the last
    two (padded) dimensions, and one coefficient per slice over them: the product of eq evaluations of the leading
    dimensions' coordinates, first dimension outermost, only the unpadded indices."""
    dims = [1 << max(d - 1, 0).bit_length() for d in shape]
    if len(point) != sum(d.bit_length() - 1 for d in dims):
        raise ValueError("Point length %d does not match total variables" % len(point))
    end, parts = len(point), []
    for d in dims:  # split_point (shape.rs:475-496): the first dimension takes the last coordinates
        start = end - (d.bit_length() - 1)
        parts.append(point[start:end])
        end = start
    skip = max(len(shape) - 2, 0)
    eq_point, chal = [], [F.one]
    for i, (p, size) in enumerate(zip(parts, shape)):
        if i < skip:
            ev = array_to_scalars(F, eq_evals(F, p))[:size]
            chal = [F.mul(c, e) for c in chal for e in ev]
        else:
            eq_point = list(p) + eq_point
    return eq_point, chal


def eval_zeroifier_mle(F, column_point, row_point):
    """eval_zeroifier_mle (zkml/src/lib.rs:131-138): the MLE of the matrix with ones where column <= row (indices
    little-endian) at (column_point, row_point).  With row_point the bits of n - 1 it is the "less than n"
    polynomial of a dimension of size n at column_point."""
    acc = F.one
    two = F.from_int(2)
    for c, r in zip(column_point, row_point):
        acc = F.add(F.mul(acc, F.add(F.sub(F.sub(F.one, c), r), F.mul(two, F.mul(c, r)))), F.mul(F.sub(F.one, c), r))
    return acc


def evaluate_dim_lt_poly(F, point, size):
    """evaluate_dim_lt_poly (zkml/src/lookup/operation/variant/verifying.rs:6-22)."""
    bits = max(size - 1, 0).bit_length()
    if len(point) != bits:
        raise ValueError("Row point length %d does not match unpadded seq len log2 %d" % (len(point), bits))
    return eval_zeroifier_mle(F, point, [F.from_int(((size - 1) >> b) & 1) for b in range(bits)])


def split_point(shape, point):
    """Shape::split_point (zkml/src/shape.rs:475-496) on the PADDED shape: one slice of coordinates per dimension,
    the last dimension taking the first coordinates."""
    dims = [1 << max(d - 1, 0).bit_length() for d in shape]
    if len(point) != sum(d.bit_length() - 1 for d in dims):
        raise ValueError("Point length %d does not match total variables" % len(point))
    end, parts = len(point), []
    for d in dims:
        start = end - (d.bit_length() - 1)
        parts.append(list(point[start:end]))
        end = start
    return parts


def broadcasting_evaluation(F, shape, dim_points, unbroadcast_shape):
    """Shape::broadcasting_evaluation (zkml/src/shape.rs:516-562): the product of the less-than polynomials of the
    dimensions that a tensor of shape `unbroadcast_shape` (size one there) is broadcast along."""
    if len(unbroadcast_shape) != len(shape) or len(dim_points) != len(shape):
        raise ValueError("shape ranks differ")
    ev = F.one
    for full, small, pt in zip(shape, unbroadcast_shape, dim_points):
        if small == 1:
            ev = F.mul(ev, eval_zeroifier_mle(F, pt, [F.from_int(((full - 1) >> b) & 1) for b in range(len(pt))]))
        elif small != full:
            raise ValueError("Dimension size %d does not match unbroadcasted dimension size %d" % (full, small))
    return ev


def compute_lookup_padding_evaluation(F, padding_value, shape, dim_points):
    """compute_lookup_padding_evaluation (zkml/src/lookup/operation/mod.rs:289-340): the evaluation of the tensor
    that is zero inside the unpadded last two dimensions and `padding_value` in their padding, repeated over the
    leading dimensions' unpadded indices."""
    rank = len(shape)
    is_pow2 = lambda d: d & (d - 1) == 0
    if all(is_pow2(d) for d in shape[max(rank - 2, 0):]):
        return F.zero
    unbroadcast = [1 if i < max(rank - 2, 0) else d for i, d in enumerate(shape)]
    leading = broadcasting_evaluation(F, shape, dim_points, unbroadcast)
    second_last, last = (shape[rank - 2], shape[rank - 1]) if rank >= 2 else (1, shape[0])
    last_lt = F.zero if is_pow2(last) else F.sub(F.one, evaluate_dim_lt_poly(F, dim_points[rank - 1], last))
    if second_last == 1 or is_pow2(second_last):
        ev = F.mul(leading, last_lt)
    else:
        sl = evaluate_dim_lt_poly(F, dim_points[rank - 2], second_last)
        ev = F.mul(leading, F.add(F.mul(sl, last_lt), F.sub(F.one, sl)))
    return F.mul(ev, padding_value)


def bias_evaluation_point(output_axes, bias_axes, claim_point):
    """AxesMapping::bias_evaluation_point (zkml/src/layers/einsum/axis.rs:583-637).  Axes are labels (one character
    each); claim_point holds one slice per output dimension (split_point order).  The bias's point is its
    dimensions' slices, last dimension first."""
    slices = [None] * len(bias_axes)
    for a in bias_axes:
        if a not in output_axes:
            raise ValueError("Bias tensor has an axis %s that is not present in the output tensor" % a)
    for pos, a in enumerate(output_axes):
        if a in bias_axes:
            slices[bias_axes.index(a)] = claim_point[pos]
    out = []
    for sl in reversed(slices):
        out += list(sl)
    return out


def compute_bias_evaluation(F, output_axes, bias_axes, claim_point, bias_eval, output_shape):
    """AxesMapping::compute_bias_evaluation (axis.rs:655-720): the bias's evaluation times the less-than polynomial
    of every output dimension the bias is broadcast along."""
    ev = bias_eval
    for pos, a in enumerate(output_axes):
        if a not in bias_axes:
            sl, size = claim_point[pos], output_shape[pos]
            ev = F.mul(ev, eval_zeroifier_mle(F, sl, [F.from_int(((size - 1) >> b) & 1) for b in range(len(sl))]))
    return ev, bias_evaluation_point(output_axes, bias_axes, claim_point)


def lookup_linking_prove(F, transcript, variant, info, out_min, out_max, shape, mles, last_claim_point, logup_point,
                         normalised_sum=False, weight=None):
    """LookupInputConfig::prove_linking_sumcheck (zkml/src/lookup/operation/inputs/proving.rs:26-114), Standard,
    GLU and Softmax variants, without a weight table.  `mles`: the witness tables in the expression's order.
    Returns the proof, the tables' evaluations at the sumcheck's point (eq tables left out), the point and the
    batching challenges.  Softmax squeezes one more challenge ("normalisation", variant.rs:363-379) and adds the
    eq table of the point (1/2, .., 1/2, logup point's coordinates above the last dimension's)
    (build_eq_polys, variant/proving.rs:225-253)."""
    eq_point, chal = eq_point_and_batching_challenges(F, shape, last_claim_point)
    sum_challenge = transcript.append_and_sample(b"sum")
    other = []
    if variant in (VARIANT_SOFTMAX, VARIANT_NORMALISATION):
        other.append(transcript.append_and_sample(b"normalisation"))
    if variant == VARIANT_NORMALISATION:
        other.append(transcript.append_and_sample(b"input"))
    total_chunks = len(chal)
    chal = [sum_challenge] + chal + other
    eqs = [eq_evals(F, eq_point), eq_evals(F, logup_point)]
    if variant in (VARIANT_SOFTMAX, VARIANT_NORMALISATION):
        fdv = max(shape[-1] - 1, 0).bit_length()
        eqs.append(eq_evals(F, [F.inv(F.from_int(2))] * fdv + list(logup_point[fdv:])))
    if weight is not None:
        eqs.append(weight)  # the weight table comes after the eq tables (inputs/proving.rs:66-68)
    expr = lookup_linking_expression(F, variant, total_chunks, info, out_min, out_max, shape[-1], normalised_sum,
                                     weight is not None)
    terms = expr_to_terms(F, expr, chal)
    proof, point, finals = sumcheck_prove(F, len(eq_point), list(mles) + eqs, terms, transcript)
    return dict(sumcheck=proof, evaluations=finals[:len(mles)], point=point, challenges=chal,
                weight_eval=finals[-1] if weight is not None else None)
