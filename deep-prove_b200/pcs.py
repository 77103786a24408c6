"""Python face of include/dpb_pcs.h: the SRS's G1 points on the device and the multi-scalar multiplication that a
HyperKZG commitment is (CommittedPolynomial::batch_commit, zkml/src/poly_commit/context.rs:56-90).  Points are
(x, y) pairs of Python integers; the point at infinity is (0, 0)."""
import ctypes

import numpy as np

from . import _buf, _int, _pp, _u32, _u64, _vp, check, lib

PCS_SIGNATURES = {
    "dpb_g1_bases_from_host": (_int, [_vp, _vp, _u64, _pp]),
    "dpb_g1_bases_synthetic": (_int, [_vp, _u64, _u32, _pp]),
    "dpb_g1_bases_len": (_u64, [_vp]),
    "dpb_g1_bases_free": (None, [_vp]),
    "dpb_msm_g1": (_int, [_vp, _vp, _vp, _vp]),
    "dpb_pcs_batch_commit": (_int, [_vp, _vp, _pp, _u32, _vp]),
}
for _name, (_res, _args) in PCS_SIGNATURES.items():
    _fn = getattr(lib, _name)
    _fn.restype = _res
    _fn.argtypes = _args


def points_to_array(points):
    """[(x, y), ...] -> uint64[n, 8]: canonical little-endian coordinates."""
    raw = b"".join(int(x).to_bytes(32, "little") + int(y).to_bytes(32, "little") for x, y in points)
    return np.frombuffer(raw, dtype=np.uint64).reshape(-1, 8).copy()


def array_to_points(arr):
    a = np.ascontiguousarray(arr, dtype=np.uint64).reshape(-1, 8)
    out = []
    for row in a:
        b = row.tobytes()
        out.append((int.from_bytes(b[:32], "little"), int.from_bytes(b[32:], "little")))
    return out


class G1Bases:
    """dpb_g1_bases: the points an MSM multiplies (HyperKZG's prover setup)."""

    def __init__(self, ctx, points, _h=None):
        self.ctx = ctx
        if _h is not None:
            self.h = _h
            return
        arr = points if isinstance(points, np.ndarray) else points_to_array(points)
        arr = np.ascontiguousarray(arr, dtype=np.uint64).reshape(-1, 8)
        self.h = ctypes.c_void_p()
        check(lib.dpb_g1_bases_from_host(ctx.h, _buf(arr), arr.shape[0], ctypes.byref(self.h)))

    @staticmethod
    def synthetic(ctx, n, first_multiple=1):
        """dpb_g1_bases_synthetic: point i = (first_multiple + i) * G, made on the device."""
        h = ctypes.c_void_p()
        check(lib.dpb_g1_bases_synthetic(ctx.h, n, first_multiple, ctypes.byref(h)))
        return G1Bases(ctx, None, _h=h)

    def __len__(self):
        return lib.dpb_g1_bases_len(self.h)

    def free(self):
        if self.h:
            lib.dpb_g1_bases_free(self.h)
            self.h = None


def msm(ctx, bases, scalars):
    """dpb_msm_g1 -> (x, y)"""
    out = np.zeros(8, dtype=np.uint64)
    check(lib.dpb_msm_g1(ctx.h, bases.h, scalars.h, _buf(out)))
    return array_to_points(out)[0]


def batch_commit(ctx, bases, polys):
    """dpb_pcs_batch_commit -> [(x, y)] per table"""
    hs = (ctypes.c_void_p * len(polys))(*[m.h for m in polys])
    out = np.zeros((max(len(polys), 1), 8), dtype=np.uint64)
    check(lib.dpb_pcs_batch_commit(ctx.h, bases.h, hs, len(polys), _buf(out)))
    return array_to_points(out[: len(polys)])
