/*
 * dpb_pcs.h -- the group arithmetic of the polynomial commitment's commit step.
 *
 * The reference commits to every witness and model polynomial with HyperKZG over BN254
 * (type Pcs = HyperKZG<Bn254>, zkml/src/bin/bench/llm.rs:34-39): a commitment to a multilinear polynomial is
 * the multi-scalar multiplication  sum_i evals[i] * G_i  of its evaluation table with the first len(evals) G1
 * points of the structured reference string.  CommittedPolynomial::batch_commit
 * (zkml/src/poly_commit/context.rs:56-90, called from zkml/src/lookup/context.rs:420-422) cuts every polynomial
 * into chunks of at most 2^20 evaluations and calls PCS::batch_commit on the chunks; the scheme itself lives in
 * dp-crypto's arkyper module (HyperKZG / HyperKZGGpu), whose source is not part of the reference tree.  What is
 * restated here is the published definition of the commit (the MSM).  The opening protocol (PCS::prove,
 * zkml/src/poly_commit/prover.rs:125-131) is not: its message order and transcript use are defined by the absent
 * source.
 *
 * Points cross the boundary as affine coordinates (x, y), each a 32-byte little-endian canonical integer below
 * the base-field modulus q (arkworks' Fq in canonical form); the point at infinity is (0, 0).
 */
#ifndef DPB_PCS_H
#define DPB_PCS_H

#include "dpb.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef struct dpb_g1_bases dpb_g1_bases;

/* The SRS's G1 points (HyperKZG's prover setup), kept on the device.  affine_xy: n points of 64 bytes.
 * Every point is checked to lie on y^2 = x^3 + 3 with coordinates below q; DPB_EINVAL otherwise. */
int dpb_g1_bases_from_host(dpb_ctx* ctx, const void* affine_xy, uint64_t n, dpb_g1_bases** out);
/* n valid, distinct points made on the device: point i = (first_multiple + i) * G for the generator G = (1, 2).
 * A stand-in for an SRS in benchmarks and tests (an MSM treats its points as opaque); no reference counterpart:
 * the reference loads or samples its setup on the host. */
int dpb_g1_bases_synthetic(dpb_ctx* ctx, uint64_t n, uint32_t first_multiple, dpb_g1_bases** out);
uint64_t dpb_g1_bases_len(const dpb_g1_bases* bases);
void dpb_g1_bases_free(dpb_g1_bases* bases);

/* sum_i scalars[i] * bases[i] over the table's len entries (len <= number of bases): one commitment
 * (CommitmentScheme::commit of one chunk).  `scalars` is a BN254 table: DPB_FR (Montgomery residues, arkworks'
 * in-memory form) or an integer table DPB_FR_I32 / DPB_FR_I64, whose negative entries add the negated point.
 * out_affine_xy: 64 bytes. */
int dpb_msm_g1(dpb_ctx* ctx, const dpb_g1_bases* bases, const dpb_mle* scalars, void* out_affine_xy);

/* PCS::batch_commit over already chunked polynomials (zkml/src/poly_commit/context.rs:72): one commitment per
 * table, out_affine_xy holds n_polys x 64 bytes in the tables' order.  Up to 16 commitments are in flight together
 * (on side streams of the context that start after everything queued on its stream and that its stream waits for):
 * one commitment's kernels are short chains of curve additions that leave most of the GPU idle. */
int dpb_pcs_batch_commit(dpb_ctx* ctx, const dpb_g1_bases* bases, dpb_mle* const* polys, uint32_t n_polys,
                         void* out_affine_xy);

#ifdef __cplusplus
}
#endif
#endif /* DPB_PCS_H */
