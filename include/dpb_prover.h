/*
 * dpb_prover — whole-protocol entry points above include/dpb.h: the host-side
 * transcript and the provers that drive the GPU rounds with it.  These are the
 * calls a binding at the level of zkml's layer provers would use (one FFI call
 * per sumcheck or per logup batch instead of one per round).
 *
 * Element layouts, status codes and threading rules are those of dpb.h.
 * "challenge element" = DPB_GL_EXT (16 B) or DPB_FR (32 B, Montgomery).
 */
#ifndef DPB_PROVER_H
#define DPB_PROVER_H

#include "dpb.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ---- transcript (dp_crypto::arkyper::transcript::blake3::Blake3Transcript) ---- */
typedef struct dpb_transcript dpb_transcript;
/* Blake3Transcript::new(label) (zkml/src/lib.rs:106-108).  family_dtype picks
 * the field the challenges are drawn from. */
int dpb_transcript_new(int family_dtype, const void* label, size_t label_len, dpb_transcript** out);
int dpb_transcript_clone(const dpb_transcript* t, dpb_transcript** out);
void dpb_transcript_free(dpb_transcript* t);
/* Transcript::append_scalars (zkml/src/lookup/logup_gkr/prover.rs:163-166) */
int dpb_transcript_append_scalars(dpb_transcript* t, const void* scalars, uint32_t n);
/* Transcript::append_and_sample (zkml/src/lookup/logup_gkr/prover.rs:171-173) */
int dpb_transcript_append_and_sample(dpb_transcript* t, const void* label, size_t label_len, void* out);
/* Transcript::challenge_scalar (zkml/src/lib.rs:176-184) */
int dpb_transcript_challenge_scalar(dpb_transcript* t, void* out);
/* 32-byte running state and the absorb counter, for comparing two transcripts. */
int dpb_transcript_state(const dpb_transcript* t, uint8_t out_state[32], uint32_t* out_round);

/* ---- expressions (dp_crypto::Expression) ---------------------------------- */
/* An expression as a postfix program: leaves push, operators pop. */
#define DPB_EXPR_WITIN 0     /* a = table id */
#define DPB_EXPR_CONSTANT 1  /* c0 = value */
#define DPB_EXPR_CHALLENGE 2 /* a = challenge id, b = power, c0 = scalar, c1 = offset */
#define DPB_EXPR_ADD 3
#define DPB_EXPR_SUB 4
#define DPB_EXPR_MUL 5
#define DPB_EXPR_NEG 6
typedef struct dpb_expr_node {
    uint32_t op;
    uint32_t a;
    uint32_t b;
    uint32_t pad;
    uint8_t c0[32];
    uint8_t c1[32];
} dpb_expr_node;
/* VirtualPolynomialsBuilder::to_virtual_polys (zkml/src/layers/einsum/prove.rs:177-182):
 * expands the expression under the challenge values into product terms.
 * Writes at most `cap` terms; *n_out is the number needed. */
int dpb_expr_to_terms(int family_dtype, const dpb_expr_node* nodes, uint32_t n_nodes,
                      const void* challenges, uint32_t n_challenges, dpb_term* out, uint32_t cap,
                      uint32_t* n_out);
/* eval_by_expr_with_instance with witness values and challenges
 * (zkml/src/lookup/logup_gkr/prover.rs:50-57). */
int dpb_expr_eval(int family_dtype, const dpb_expr_node* nodes, uint32_t n_nodes, const void* wit_evals,
                  uint32_t n_wit, const void* challenges, uint32_t n_challenges, void* out);

/* ---- closed-form evaluations between layers (host arithmetic, no device work) ---- */
/* compute_lookup_padding_evaluation (zkml/src/lookup/operation/mod.rs:289-340): the evaluation, at `point`
 * (over the PADDED shape, Shape::split_point order: the last dimension owns the first coordinates), of the
 * tensor that is zero inside the unpadded last two dimensions of `shape` and `padding_value` in their padding,
 * repeated over the unpadded leading indices -- what a lookup layer subtracts from its input claim.
 * padding_value, point and out are challenge elements of `family_dtype`.  DPB_EINVAL with the reference's
 * message when the point's length does not match the padded shape. */
int dpb_lookup_padding_evaluation(int family_dtype, const void* padding_value, const uint64_t* shape, uint32_t rank,
                                  const void* point, uint32_t n_point, void* out);
/* The inverse of a challenge element (host arithmetic; 0 maps to 0): what the host side of the split-eq rounds uses,
 * exported for callers that normalise by a challenge (e.g. 1 / 2 in the argmax linking's eq point,
 * zkml/src/layers/transformer/logits.rs:600-610). */
int dpb_scalar_inverse(int family_dtype, const void* a, void* out);
/* AxesMapping::compute_bias_evaluation and bias_evaluation_point (zkml/src/layers/einsum/axis.rs:583-720):
 * axis_in_bias[d] != 0 when output dimension d is an axis of the bias, bias_axis_position[d] its position in the
 * bias tensor (may be NULL: no bias point is produced).  out_eval = bias_eval times the less-than polynomial of
 * every output dimension the bias is broadcast along; out_bias_point (when given) = the point at which the
 * caller evaluates the bias tensor itself. */
int dpb_bias_evaluation(int family_dtype, const uint64_t* output_shape, uint32_t rank, const uint8_t* axis_in_bias,
                        const uint32_t* bias_axis_position, const void* point, uint32_t n_point, const void* bias_eval,
                        void* out_eval, void* out_bias_point, uint32_t bias_point_cap, uint32_t* n_bias_point);

/* ---- IOPProverState::prove -------------------------------------------------- */
/* Runs all num_vars rounds (zkml/src/layers/hadamard.rs:115-130).  Outputs, all
 * challenge elements: out_round_evals[num_vars * (degree+1)] (IOPProof),
 * out_point[num_vars] (collect_raw_challenges), out_final_evals[k]
 * (get_mle_flatten_final_evaluations).  *out_degree receives the degree. */
int dpb_prove_sumcheck(dpb_ctx* ctx, uint32_t num_vars, dpb_mle* const* mles, uint32_t k,
                       const dpb_term* terms, uint32_t n_terms, dpb_transcript* t, void* out_round_evals,
                       uint32_t round_evals_cap, void* out_point, void* out_final_evals, uint32_t* out_degree);

/* The same over the context's communicator: tables are this rank's shards (see
 * dpb_sumcheck_begin_sharded), num_vars counts all variables, every rank passes a
 * transcript in the same state and all ranks return the same proof. */
int dpb_prove_sumcheck_sharded(dpb_ctx* ctx, uint32_t num_vars, dpb_mle* const* mles, uint32_t k,
                               const dpb_term* terms, uint32_t n_terms, dpb_transcript* t, void* out_round_evals,
                               uint32_t round_evals_cap, void* out_point, void* out_final_evals,
                               uint32_t* out_degree);

/* hadamard::prove (zkml/src/layers/hadamard.rs:93-131): sum_x v1 v2 eq(point, x).
 * out_round_evals[n*4], out_point[n], out_claims[2] = (v1, v2) at the point. */
int dpb_hadamard_prove(dpb_ctx* ctx, dpb_mle* v1, dpb_mle* v2, const void* claim_point, uint32_t n,
                       dpb_transcript* t, void* out_round_evals, void* out_point, void* out_claims);

/* same_poly::Prover::prove (zkml/src/iop/same_poly.rs:84-114): merges n_claims
 * claims (points of n coordinates, row-major in `points`) on one table.
 * out_round_evals[n*3], out_point[n], out_eval[1]. */
int dpb_same_poly_prove(dpb_ctx* ctx, dpb_mle* poly, const void* points, uint32_t n_claims, uint32_t n,
                        dpb_transcript* t, void* out_round_evals, void* out_point, void* out_eval);

/* ---- claim batching of the opening proof ------------------------------------- */
/* One committed polynomial: its n_chunks (a power of two) chunk tables of equal
 * length, and the claims to batch for it.  A claim's point has
 * log2(chunk length) + log2(n_chunks) coordinates (ChunkedCommitment,
 * zkml/src/poly_commit/mod.rs:32-93). */
typedef struct dpb_committed_poly {
    dpb_mle* const* chunks;
    uint32_t n_chunks;
    uint32_t n_claims;
    const void* claim_points; /* n_claims points, row-major */
    const void* claim_evals;  /* n_claims elements */
} dpb_committed_poly;

/* CommitmentProver::claims_batching_sumcheck (zkml/src/poly_commit/prover.rs:140-255)
 * and, when out_rlc is not NULL, the step that follows it in
 * CommitmentProver::prove (prover.rs:113-122): point and evaluations go into the
 * transcript, one challenge per committed chunk is drawn, and the random linear
 * combination of the chunks is built (the polynomial the commitment scheme
 * opens; the scheme itself is outside this library).  `polys` in the order the
 * reference visits them: model commitments, then witness commitments.
 * out_round_evals[num_vars*3] (round_evals_cap elements of room),
 * out_point[num_vars], out_sumcheck_evals[total chunks] (evals_cap elements of
 * room), out_rlc_challenges[total chunks] (may be NULL with out_rlc);
 * *out_num_vars = the largest chunk's variables.  The caller frees *out_rlc. */
int dpb_claims_batching_prove(dpb_ctx* ctx, const dpb_committed_poly* polys, uint32_t n_polys, dpb_transcript* t,
                              void* out_round_evals, uint32_t round_evals_cap, void* out_point,
                              uint32_t* out_num_vars, void* out_sumcheck_evals, uint32_t evals_cap,
                              void* out_rlc_challenges, dpb_mle** out_rlc);

/* ---- batched logup-GKR ------------------------------------------------------- */
/* LogUpInput (zkml/src/lookup/logup_gkr/structs.rs:138-154) */
typedef struct dpb_logup_input {
    int kind; /* DPB_LOGUP_LOOKUP or DPB_LOGUP_TABLE */
    dpb_mle* const* columns;
    uint32_t n_columns;
    uint32_t columns_per_instance; /* lookups: columns per circuit */
    dpb_mle* multiplicities;       /* tables only */
    const void* constant_challenge;
    const void* column_separation_challenge;
} dpb_logup_input;
typedef struct dpb_logup_proof dpb_logup_proof;
/* new_batch_multiple_sizes_prove (zkml/src/lookup/logup_gkr/prover.rs:91-344) */
int dpb_logup_batch_prove(dpb_ctx* ctx, const dpb_logup_input* inputs, uint32_t n_inputs, dpb_transcript* t,
                          dpb_logup_proof** out);
/* The same batch with its INSTANCES spread over the ranks of ctx's communicator: every rank passes its own
 * instances, of the same kinds, sizes and column counts on every rank (DPB_EINVAL otherwise), and a transcript in the
 * same state.  Local instance i of rank g is instance i * G + g of the whole batch.  A rank builds only its own
 * fraction trees and runs its own part of each layer's sumcheck (dpb_sumcheck_begin_partial); the trees' outputs and
 * each layer's final evaluations are gathered over NCCL.  Every rank returns the proof of the whole batch, equal
 * byte for byte to dpb_logup_batch_prove of all instances in that order on one GPU.  Splitting a column of 2^m rows
 * into G instances of 2^m / G rows is how one large lookup is spread; the claims then speak about the slices. */
int dpb_logup_batch_prove_partial(dpb_ctx* ctx, const dpb_logup_input* inputs, uint32_t n_inputs, dpb_transcript* t,
                                  dpb_logup_proof** out);
/* Flat encoding of LogUpBatchProof (field order of
 * zkml/src/lookup/logup_gkr/structs.rs:561-578): u32 counts and canonical
 * scalars.  Writes at most cap bytes; *len is the size needed. */
int dpb_logup_proof_serialize(const dpb_logup_proof* p, void* buf, size_t cap, size_t* len);
void dpb_logup_proof_free(dpb_logup_proof* p);

/* ---- einsum layer ------------------------------------------------------------- */
/* One tensor of an einsum with what happens to each of its axes: DPB_AXIS_OUTER axes are bound to their point,
 * DPB_AXIS_STACKED axes are kept (one table per index) and their point gives the stacking coefficients,
 * DPB_AXIS_CONTRACTED axes are summed over by the sumcheck (no point).  `tensor` as for dpb_einsum_fix_axes. */
typedef struct dpb_einsum_operand {
    const int64_t* tensor;
    int32_t tensor_on_device;
    uint32_t rank;
    const uint64_t* shape;            /* unpadded extents */
    const uint8_t* axis_kind;         /* DPB_AXIS_* per axis */
    const void* const* axis_points;   /* per axis: challenge elements on the host, or NULL */
    const uint32_t* axis_point_len;
} dpb_einsum_operand;
typedef struct dpb_einsum_proof dpb_einsum_proof;
/* EinSum::prove_internal (zkml/src/layers/einsum/prove.rs:48-335) below the axis mapping and without biases (a
 * bias claim is an evaluation, dpb_bias_evaluation; it does not touch the transcript): n_rhs right tensors, one
 * output each; lhs_fixes[i] is the LEFT tensor with the fixes of output i (FixedAxesMapping::lhs_fixes,
 * einsum/axis.rs:1043-1075; the same tensor in every entry), rhs[i] the right tensor of output i.  Steps: axis
 * fixing of every operand, stacking coefficients prod evals(point)[..size] over the stacked axes (first stacked
 * axis slowest), gamma = append_and_sample("batching_challenge"), the sumcheck
 *   sum_i gamma^i sum_t coef[i][t] * lhs[i][t] * rhs[i][t]        (einsum/op_info.rs:159-195)
 * and the input claims (reconstruct_full_point, prove.rs:338-361).  With n_rhs > 1 the claims on the left tensor
 * are merged by the sumcheck  input * sum_i c^i eq_i  over `lhs_padded`, the left tensor padded to powers of two
 * per axis (prove.rs:260-288; c = append_and_sample("input_batching_challenge")); lhs_padded may be NULL when
 * n_rhs == 1. */
int dpb_einsum_prove(dpb_ctx* ctx, const dpb_einsum_operand* lhs_fixes, const dpb_einsum_operand* rhs, uint32_t n_rhs,
                     dpb_mle* lhs_padded, dpb_transcript* t, dpb_einsum_proof** out);
/* Flat encoding (u32 counts, canonical scalars): n_rhs, S, gamma, the n_rhs x S stacking coefficients, the sumcheck
 * (rounds, then per round its count and evaluations), the sumcheck point (count first), the final evaluations
 * (count first: the left tables of every output, then the right tables), per right tensor its claim (point count,
 * point, evaluation), the left tensor's claim in the same form, 1 or 0 for a merged left claim and, when 1, c and
 * the merging sumcheck.  Writes at most cap bytes; *len is the size needed. */
int dpb_einsum_proof_serialize(const dpb_einsum_proof* p, void* buf, size_t cap, size_t* len);
void dpb_einsum_proof_free(dpb_einsum_proof* p);

/* ---- lookup linking sumcheck ---------------------------------------------------- */
#define DPB_VARIANT_STANDARD 0 /* LookupVariant::Standard */
#define DPB_VARIANT_GLU 1      /* LookupVariant::GLU: one more witness table per slice, multiplied into the output */
#define DPB_VARIANT_SOFTMAX 2  /* LookupVariant::Softmax: one more challenge ("normalisation") and a third eq table,
                                * over (1/2, .., 1/2, the logup point's coordinates above the last dimension's), that
                                * sums the outputs along the last dimension */
#define DPB_VARIANT_NORMALISATION 3           /* LookupVariant::Normalisation { normalised_sum_value: None, .. } */
#define DPB_VARIANT_NORMALISATION_WITH_SUM 4  /* the same with normalised_sum_value: Some(..): the sums are tied too */
/* LookupInputConfig::prove_linking_sumcheck (zkml/src/lookup/operation/inputs/proving.rs:26-114)
 * with LookupVariant::build_full_sumcheck_expression (zkml/src/lookup/operation/variant.rs:55-262)
 * for the Standard, GLU and Softmax variants (the Normalisation variant is described below): ties the looked-up outputs of an
 * operation to the claim on its output tensor and to the logup point,
 *   sum_x sum_c b_c * ( eq(x, p_out) * (clamping_c(x) + selector_c(x) * value_c(x)) [* glu_c(x)]
 *                       + eq(x, p_logup) * sum_j s^j * witness_{c,j}(x) ).
 * shape[rank]: the operation's UNPADDED input shape; a slice c is one index of the leading
 * rank-2 dimensions, n = the variables of the last two padded dimensions.
 * mles: per slice its value chunk outputs then its zeroing chunk outputs (the output columns
 * of dpb_lookup_witness, in order), then for GLU one table per slice; every table 2^n entries.
 * table_min_output / table_max_output: Table::min_output_value / max_output_value.
 * last_claim_point: all the padded tensor's variables (Shape::split_point order: the last
 * dimension first); logup_point: n coordinates.  The transcript gives the challenge "sum";
 * the slices' coefficients b_c are the eq evaluations of the leading dimensions' coordinates
 * (Shape::compute_eq_point_and_batching_challenges, zkml/src/shape.rs:565-610).
 * Outputs: out_round_evals[n * (degree+1)] (capacity round_evals_cap elements),
 * out_point[n], out_evaluations[n_mles] (the witness tables at the point),
 * out_batching_challenges[1 + slices (+ 1 for Softmax, + 2 for Normalisation)] (capacity
 * chal_cap), *out_degree.
 * Normalisation (variant.rs:288-346): after the outputs, `mles` holds one input table per slice
 * and then one scaling table per slice; two more challenges ("normalisation", "input"); the
 * sums of squares of the outputs along the last dimension ride on the third eq table (and the
 * sums, with DPB_VARIANT_NORMALISATION_WITH_SUM); `weight` (may be NULL; only this variant takes
 * one) multiplies the output part (has_weight) and *out_weight_eval receives its evaluation. */
int dpb_lookup_linking_prove(dpb_ctx* ctx, int variant, const dpb_chunking_info* info, int64_t table_min_output,
                             int64_t table_max_output, const uint64_t* shape, uint32_t rank, dpb_mle* const* mles,
                             uint32_t n_mles, const void* last_claim_point, uint32_t n_claim_coords,
                             const void* logup_point, uint32_t n_logup_coords, dpb_transcript* t, void* out_round_evals,
                             uint32_t round_evals_cap, void* out_point, void* out_evaluations,
                             void* out_batching_challenges, uint32_t chal_cap, uint32_t* out_n_challenges,
                             uint32_t* out_degree, dpb_mle* weight, void* out_weight_eval);

#ifdef __cplusplus
}
#endif
#endif /* DPB_PROVER_H */
