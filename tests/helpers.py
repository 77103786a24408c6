"""Shared helpers of the GPU parity tests: drive the C-ABI sumcheck with the
oracle's transcript so that both sides see the same challenges."""
import numpy as np

from oracle import oracle as orc


def family_dtype(dpb, F):
    return dpb.FR if F is orc.FrField else dpb.GL_EXT


def upload(dpb, ctx, F, table):
    t = np.ascontiguousarray(table)
    return ctx.upload(t, dpb.dtype_of_array(t, F.name))


def terms_array(dpb, F, terms_dict):
    return dpb.make_terms([(c, list(m)) for m, c in sorted(terms_dict.items())], F.to_native)


def gpu_sumcheck_prove(dpb, ctx, F, num_vars, mles, terms_dict, transcript):
    """Same contract as oracle.sumcheck_prove, rounds computed on the GPU."""
    sc = ctx.sumcheck(num_vars, mles, terms_array(dpb, F, terms_dict))
    try:
        d = sc.degree
        transcript.append_scalars([F.from_int(num_vars), F.from_int(d)])
        proof, point = [], []
        r_arr = None
        for _ in range(num_vars):
            ev = orc.array_to_scalars(F, sc.round(r_arr))
            transcript.append_scalars(ev)
            r = transcript.append_and_sample(orc.ROUND_LABEL)
            proof.append(ev)
            point.append(r)
            r_arr = orc.scalars_to_array(F, [r])
        finals = orc.array_to_scalars(F, sc.finish(r_arr))
    finally:
        sc.free()
    return proof, point, finals
