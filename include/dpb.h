/*
 * dpb — C ABI of the B200 (sm_100a) sumcheck / multilinear-fold / logup-GKR
 * prover back end.
 *
 * The reference reaches this path through ordinary Rust calls into the
 * `dp-crypto` crate (Cargo.toml:42); there is no FFI in the reference.  Each
 * entry point below names the reference call (file:line, paths relative to the
 * reference repository) that a thin Rust shim inside `dp-crypto` would forward
 * to it.  The Fiat-Shamir transcript never crosses this boundary: the host
 * drives a sumcheck one challenge at a time.
 *
 * Conventions
 *  - Every function returns DPB_OK (0) or a negative status and never aborts,
 *    traps or throws.  dpb_last_error() gives a message for the calling thread.
 *  - Handles are owned by the caller and freed explicitly.  A dpb_ctx is used
 *    from one host thread at a time; kernels run on a stream private to it.
 *  - Host buffers are only read or written for the duration of the call.
 *  - Field elements cross the boundary in these layouts (all little-endian):
 *      DPB_GL_BASE  Goldilocks base element, canonical uint64          (8 B)
 *      DPB_GL_EXT   Goldilocks quadratic extension c0 + c1*X, X^2 = 7  (16 B)
 *      DPB_FR       BN254 Fr, 4 x uint64 Montgomery limbs (a*2^256 mod r),
 *                   the in-memory form of ark_ff's 4-limb Montgomery backend
 *                   (32 B)
 *    "challenge element" means DPB_GL_EXT for the Goldilocks family and
 *    DPB_FR for BN254.
 *  - Multilinear tables are indexed little-endian: bit i of the index is
 *    variable i (zkml/src/lib.rs:357-369).  Sumcheck round i binds variable i.
 */
#ifndef DPB_H
#define DPB_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define DPB_OK 0
#define DPB_EINVAL (-1)   /* bad argument, size or handle */
#define DPB_ENOMEM (-2)   /* device or host allocation failed */
#define DPB_ECUDA (-3)    /* CUDA runtime error */
#define DPB_ETIMEOUT (-4) /* a bounded device-side wait ran out */
#define DPB_ESTATE (-5)   /* call made in the wrong state */
#define DPB_ENCCL (-6)    /* NCCL error or library unavailable */

/* element layouts */
#define DPB_GL_BASE 0
#define DPB_GL_EXT 1
#define DPB_FR 2
/* Integer tables: the quantised tensors and lookup columns of the reference are small signed integers
 * (Element = i64, zkml/src/quantization/mod.rs:220-267; Tensor::to_field, zkml/src/layers/einsum/prove.rs:66-91).
 * A table of one of these layouts holds the integers themselves (8 or 4 bytes per entry) and stands for the
 * field elements they map to (negative x -> p - |x|) in the Goldilocks or in the BN254 family.  Every sumcheck
 * entry point, the folds, evaluate, the linear combination and the logup tree accept them; results are
 * bit-identical to those of the converted table, because the arithmetic is exact.  The product sumcheck over
 * DPB_FR_I32 tables runs its first round in integer arithmetic and its first fold through two precomputed rows. */
#define DPB_GL_I64 3
#define DPB_GL_I32 4
#define DPB_FR_I64 5
#define DPB_FR_I32 6

/* forms accepted by dpb_mle_from_host for DPB_FR tables */
#define DPB_FORM_NATIVE 0    /* already in the layout of `dtype` */
#define DPB_FORM_CANONICAL 1 /* DPB_FR only: 32-byte canonical integers */
#define DPB_FORM_I64 2       /* signed 64-bit integers, negative x -> p - |x|
                                (zkml/src/quantization/mod.rs:220-267) */

typedef struct dpb_ctx dpb_ctx;
typedef struct dpb_mle dpb_mle;
typedef struct dpb_sc dpb_sc;
typedef struct dpb_logup dpb_logup;

/* One product term  coeff * prod_j mle[idx[j]]  of a virtual polynomial, the
 * monomial form `VirtualPolynomialsBuilder::to_virtual_polys` produces
 * (zkml/src/layers/einsum/prove.rs:171-182).  `coeff` is a challenge element
 * stored in the first 16 (Goldilocks) or 32 (BN254) bytes. */
#define DPB_MAX_FACTORS 8
typedef struct dpb_term {
    uint8_t coeff[32];
    uint32_t n_factors;
    uint16_t idx[DPB_MAX_FACTORS];
} dpb_term;

/* ---- context ----------------------------------------------------------- */
/* Creates a context on CUDA device `device`.  Fails with DPB_ECUDA when no
 * usable GPU is present: there is no CPU fallback.
 * Device memory: tables and scratch are cut out of arenas of 8 GiB that the context takes from the device's
 * default stream-ordered pool and keeps (requests of 2 GiB and more get a block of their own; the last such blocks,
 * up to 16 and 96 GiB, are kept for a request of the same size).  Unused arenas and kept blocks go back to the pool when an
 * allocation fails, on dpb_trim and at dpb_shutdown.  The environment variable DPB_ARENA=0 sends every request to
 * the pool instead. */
int dpb_init(int device, dpb_ctx** out);
/* Gives the device memory the context keeps for reuse (freed blocks, the last sumcheck's block) back to the pool and
 * the pool's unused memory back to the device; waits for the context's stream.  For a process that moves on to a
 * job of different sizes, or shares the GPU's memory with another library. */
int dpb_trim(dpb_ctx* ctx);
void dpb_shutdown(dpb_ctx* ctx);
const char* dpb_last_error(void);
/* Blocks until all work queued on the context's stream has finished. */
int dpb_sync(dpb_ctx* ctx);
/* The context's CUDA stream (a cudaStream_t), for callers that time with
 * CUDA events or order their own copies against it. */
void* dpb_stream(dpb_ctx* ctx);

/* ---- multi-GPU (no counterpart in the reference, which has no collective) -- */
/* One process per GPU.  A sumcheck over n variables is sharded on its top
 * log2(G) variables: rank g holds entries [g*2^(n-c), (g+1)*2^(n-c)) of every
 * table, c = log2 G.  Rounds 0..n-c-1 fold locally; each rank's partial round
 * evaluations travel through one small NCCL all-gather and are added mod p on
 * every host, so all ranks drive identical transcripts.  When c variables are
 * left the one-entry shards are gathered and every rank finishes the same tail.
 * Waits on collectives are bounded (DPB_ETIMEOUT). */
#define DPB_COMM_ID_BYTES 128
/* ncclGetUniqueId; call on one rank and distribute the bytes to the others. */
int dpb_comm_unique_id(void* out_id);
/* ncclCommInitRank on the context's device; collective over all ranks.  nranks a power of two. */
int dpb_comm_init(dpb_ctx* ctx, const void* id, int rank, int nranks);
/* This rank's shard of the eq table of `point` (m coordinates), for sharded sumchecks with an eq factor (the
 * hadamard, same_poly and linking shapes): entries [rank * 2^(m-c), (rank+1) * 2^(m-c)) of dpb_eq_table's result,
 * c = log2(ranks), computed as the eq table of the low m - c coordinates times the eq value of the rank's bits at
 * the top c coordinates -- no rank ever holds the whole table.  Without a communicator it is dpb_eq_table. */
int dpb_eq_table_shard(dpb_ctx* ctx, int family_dtype, const void* point, uint32_t m, dpb_mle** out);
/* 1 when the ranks of this context's communicator exchange the per-round sums
 * through a shared host segment (all on one host), 0 when they use
 * ncclAllGather.  The environment variable DPB_NO_SHARED_EXCHANGE, set on every
 * rank before dpb_comm_init, forces the NCCL path. */
int dpb_comm_shared_exchange(const dpb_ctx* ctx);
int dpb_comm_rank(const dpb_ctx* ctx);
int dpb_comm_size(const dpb_ctx* ctx);
int dpb_comm_free(dpb_ctx* ctx);

/* ---- per-kernel timing (no counterpart in the reference) ---------------- */
/* When enabled, every sumcheck round brackets its kernel launches with CUDA
 * events on the context's stream and adds the elapsed device time to a log
 * keyed by (kernel, round).  alg_bytes_per_launch is the minimum traffic of
 * that round: tables read once, folded tables written once. */
typedef struct dpb_profile_entry {
    char kernel[48];
    uint32_t round;
    uint32_t launches;
    double total_ms;
    uint64_t alg_bytes_per_launch;
} dpb_profile_entry;
/* on != 0 clears the log and starts recording; 0 stops. */
int dpb_profile_enable(dpb_ctx* ctx, int on);
/* Copies at most cap entries; *n is the number available. */
int dpb_profile_read(dpb_ctx* ctx, dpb_profile_entry* out, uint32_t cap, uint32_t* n);

/* Host-side phase timers (no counterpart in the reference beyond its timed_instrument spans,
 * zkml/src/layers/activation.rs:620): when enabled, the whole-protocol entry points add the wall time of their
 * phases (tree builds, expression expansion, eq tables, sumcheck begin / rounds / finish, ...) to a process-wide log.
 * dpb_trace_read writes one line "phase<TAB>milliseconds<TAB>calls" per phase into `out` (NUL-terminated) when
 * `cap` suffices; *needed is the size required.  on != 0 clears the log. */
int dpb_trace_enable(int on);
int dpb_trace_read(char* out, size_t cap, size_t* needed);

/* Issue-rate probe: runs chains of one arithmetic primitive of the round
 * kernels on register operands on every SM and reports how many of them the
 * device completes per second -- the ceiling a kernel bound by the integer
 * pipes (every BN254 round) is measured against.  kind: 0 = 32x32->64
 * multiply-add with 64-bit addend, 1 = BN254 Montgomery product, 2 = BN254
 * product by a per-launch constant (the fold's challenge), 3 = Goldilocks
 * lazy multiply-accumulate, 4 = Goldilocks product with reduction.  iters =
 * chain length per thread (1..2^20).  No reference counterpart. */
int dpb_issue_rate_probe(dpb_ctx* ctx, int kind, uint32_t iters, double* ops_per_second, double* elapsed_ms);

/* The last rounds of a sumcheck (a few hundred pairs or fewer) run in one
 * resident kernel that exchanges round sums and challenges with the host
 * through mapped memory instead of one launch per round.  enable = 0 turns
 * that off (every round is a launch); wait_ms bounds how long the kernel
 * waits for the next challenge before it returns (default 1000; 0 keeps the
 * current value).  A kernel that returned this way is started again by the
 * sumcheck's next call, so a host that was held up only loses time; a caller
 * that synchronises the whole device between two rounds waits for that limit.
 * No reference counterpart: the reference's rounds are CPU loops. */
int dpb_resident_rounds(dpb_ctx* ctx, int enable, uint32_t wait_ms);

/* Kernels the sumcheck entry points (begin / round / finish) have launched on
 * this context so far.  No reference counterpart. */
uint64_t dpb_sumcheck_launches(const dpb_ctx* ctx);

/* ---- multilinear tables (dp_crypto::poly::dense::DensePolynomial) ------ */
/* Uploads `len` (a power of two) evaluations from host memory.
 * Replaces DensePolynomial::new / new_from_smart_slice
 * (zkml/src/lookup/logup_gkr/circuit.rs:262-269) and Tensor::to_field_mle
 * (zkml/src/layers/hadamard.rs:104-105) for DPB_FORM_I64. */
int dpb_mle_from_host(dpb_ctx* ctx, int dtype, const void* evals, uint64_t len, int form,
                      dpb_mle** out);
/* Wraps device memory the caller already owns (no copy, not freed). */
int dpb_mle_from_device(dpb_ctx* ctx, int dtype, void* dev_ptr, uint64_t len, dpb_mle** out);
/* Allocates an uninitialised device table. */
int dpb_mle_alloc(dpb_ctx* ctx, int dtype, uint64_t len, dpb_mle** out);
int dpb_mle_free(dpb_mle* mle);
/* Copies the table back (DensePolynomial::evals). `form` as above; DPB_FORM_I64 is invalid. */
int dpb_mle_to_host(const dpb_mle* mle, void* out, uint64_t len, int form);
uint64_t dpb_mle_len(const dpb_mle* mle);
int dpb_mle_dtype(const dpb_mle* mle);
void* dpb_mle_device_ptr(const dpb_mle* mle);
/* A borrowed view of `len` elements starting at `offset` (DensePolynomial::as_view_chunks,
 * and the low/high half split of zkml/src/lookup/logup_gkr/circuit.rs:260-261). */
int dpb_mle_view(const dpb_mle* mle, uint64_t offset, uint64_t len, dpb_mle** out);
/* A borrowed view that a sumcheck over MORE variables treats as zero-padded:
 * the table keeps its entries at indices below its length and reads as zero
 * above, i.e. it is a function of the FIRST variables times (1 - x_j) for every
 * added variable j (DensePolynomial::as_view + zero_pad_num_vars,
 * zkml/src/poly_commit/prover.rs:216-226; the verifier's formula for the padded
 * eq tables, zkml/src/poly_commit/verifier.rs:300-311, pins the convention).
 * Without this flag a smaller table is a function of the LAST variables. */
int dpb_mle_zero_padded(const dpb_mle* mle, dpb_mle** out);
/* out = sum_j coeffs[j] * mles[j] over challenge elements; shorter tables count
 * as zero-padded; the result has the length of the longest
 * (DensePolynomial::linear_combination, zkml/src/poly_commit/prover.rs:122). */
int dpb_linear_combination(dpb_ctx* ctx, dpb_mle* const* mles, const void* coeffs, uint32_t n, dpb_mle** out);

/* eq(x, point) for all x in {0,1}^m, little-endian index
 * (dp_crypto::poly::eq::evals; call sites zkml/src/lookup/logup_gkr/prover.rs:247-249,
 * zkml/src/layers/hadamard.rs:103).  `point` holds m challenge elements on the host. */
int dpb_eq_table(dpb_ctx* ctx, int family_dtype, const void* point, uint32_t m, dpb_mle** out);
/* n eq tables in one call: table t is over num_vars[t] variables and its point
 * is the next num_vars[t] elements of `points`.  All tables live in one block
 * owned by *out_owner (free it last); out_tables[t] are views.  For callers that
 * build one eq table per claim (zkml/src/poly_commit/prover.rs:172,201;
 * zkml/src/iop/same_poly.rs:90). */
int dpb_eq_tables(dpb_ctx* ctx, int family_dtype, const void* points, const uint32_t* num_vars, uint32_t n,
                  dpb_mle** out_owner, dpb_mle** out_tables);
/* The second eq table of a rotary-position layer: the entries of `eq` (challenge
 * elements) moved and negated the way the rotation pairs its inputs
 * (RopeLayout::permuted_eq_poly, zkml/src/layers/transformer/positional/rope.rs:238-258;
 * call site rope.rs:559).  layout 0, adjacent pairs: out[i] = eq[i+1] for even i,
 * -eq[i-1] for odd i.  layout 1, rotate half over rows of row_size entries:
 * out[i] = eq[i + row_size/2] in the first half of a row, -eq[i - row_size/2] in
 * the second (row_size is ignored for layout 0). */
int dpb_rope_permuted_eq(dpb_ctx* ctx, const dpb_mle* eq, int layout, uint64_t row_size, dpb_mle** out);

/* Binds the top k variables (variable n-k+j := point[j]) -> table of len/2^k.
 * DensePolynomial::fix_high_variables{,_parallel}
 * (zkml/src/layers/transformer/positional/rope.rs:556, zkml/src/iop/prover.rs:448). */
int dpb_fix_high(dpb_ctx* ctx, const dpb_mle* mle, const void* point, uint32_t k, dpb_mle** out);
/* Binds the bottom k variables (variable j := point[j]).
 * DensePolynomial::fix_low_variables{,_in_place_parallel}
 * (zkml/src/layers/transformer/embeddings.rs:432, zkml/src/layers/pooling.rs:933). */
int dpb_fix_low(dpb_ctx* ctx, const dpb_mle* mle, const void* point, uint32_t k, dpb_mle** out);
/* Full evaluation at an n-variable point (DensePolynomial::evaluate,
 * zkml/src/iop/mod.rs:196-207).  Result: one challenge element on the host. */
int dpb_mle_evaluate(dpb_ctx* ctx, const dpb_mle* mle, const void* point, uint32_t n, void* out);
/* n tables at ONE point of num_vars coordinates, in one pass over their entries: table t of 2^m_t <= 2^num_vars
 * entries counts as zero-padded (dpb_mle_zero_padded's convention: a function of the FIRST m_t variables times
 * (1 - x_j) for every further one), so out[t] = sum_x table_t[x] * eq(point[..m_t], x) * prod_{j >= m_t} (1 - point[j]).
 * What the claim batching hands on as the committed chunks' evaluations (zkml/src/poly_commit/prover.rs:246-251).
 * out: n challenge elements on the host. */
int dpb_mle_evaluate_many(dpb_ctx* ctx, dpb_mle* const* mles, uint32_t n, const void* point, uint32_t num_vars,
                          void* out);

/* ---- einsum axis fixing --------------------------------------------------- */
#define DPB_AXIS_CONTRACTED 0 /* summed over by the sumcheck: kept */
#define DPB_AXIS_OUTER 1      /* bound to a point: contracted against eq(point)[..size] */
#define DPB_AXIS_STACKED 2    /* kept; one output table per index */
/* AxesMapping::fix_axes -> FixedAxesMapping::mles_from_tensor
 * (zkml/src/layers/einsum/axis.rs:478-500, 1142-1234): `tensor` is the UNPADDED
 * row-major tensor of signed 64-bit quantised values (the reference's Element,
 * widened with the rule of zkml/src/quantization/mod.rs:220-267), in host memory
 * or, with tensor_on_device != 0, in device memory.  Every OUTER axis a is bound
 * to axis_points[a] (axis_point_len[a] challenge elements on the host, with
 * 2^len >= shape[a]); STACKED and CONTRACTED axes are kept in row-major order.
 * Produces one table per stacked index (S = product of the stacked sizes), each
 * holding the contracted axes' entries zero-padded to the next power of two.
 * out_mles receives S borrowed views (free each with dpb_mle_free) into
 * *out_owner, which owns the memory (free it last).  *n_out = S. */
int dpb_einsum_fix_axes(dpb_ctx* ctx, int family_dtype, const int64_t* tensor, int tensor_on_device,
                        const uint64_t* shape, const uint8_t* axis_kind, const void* const* axis_points,
                        const uint32_t* axis_point_len, uint32_t rank, dpb_mle** out_owner, dpb_mle** out_mles,
                        uint32_t out_cap, uint32_t* n_out);

/* ---- sumcheck (dp_crypto::structs::IOPProverState) --------------------- */
/* Starts a sumcheck over `num_vars` variables of  sum_t coeff_t * prod_j mle[idx_tj].
 * Tables are borrowed and never modified.  A table with fewer than num_vars
 * variables is a function of the LAST variables only (constant in the early
 * rounds), the convention the batched logup prover relies on
 * (zkml/src/lookup/logup_gkr/prover.rs:217-249).
 * Replaces IOPProverState::prove's set-up; call sites
 * zkml/src/layers/einsum/prove.rs:184, zkml/src/lookup/logup_gkr/prover.rs:275,
 * zkml/src/layers/hadamard.rs:115, zkml/src/iop/same_poly.rs:105. */
int dpb_sumcheck_begin(dpb_ctx* ctx, uint32_t num_vars, dpb_mle* const* mles, uint32_t k,
                       const dpb_term* terms, uint32_t n_terms, dpb_sc** out);
/* The same over a communicator (dpb_comm_init): num_vars counts ALL variables,
 * every table handle holds this rank's shard of 2^(num_vars - log2 G) entries
 * (the slice selected by the top log2 G index bits = the rank).  Every rank must
 * make the same sequence of calls with the same challenges; rounds and finish
 * return identical values on all ranks.  Without a communicator this is
 * dpb_sumcheck_begin. */
int dpb_sumcheck_begin_sharded(dpb_ctx* ctx, uint32_t num_vars, dpb_mle* const* mles, uint32_t k,
                               const dpb_term* terms, uint32_t n_terms, dpb_sc** out);
/* A sumcheck whose TERMS are spread over the ranks of the context's communicator (the instances of a batch, the
 * heads of a stacked product): every rank passes whole tables and its own part of the term list, of the same
 * degree on every rank; each round's sums are added over the ranks (same exchange as the sharded form), all ranks
 * feed the same transcript, and dpb_sumcheck_finish returns the final evaluations of THIS rank's tables.  The
 * messages equal those of one sumcheck over the union of the term lists.  With one rank: dpb_sumcheck_begin. */
int dpb_sumcheck_begin_partial(dpb_ctx* ctx, uint32_t num_vars, dpb_mle* const* mles, uint32_t k,
                               const dpb_term* terms, uint32_t n_terms, dpb_sc** out);
/* Degree of the round polynomial (max factors per term). */
uint32_t dpb_sumcheck_degree(const dpb_sc* sc);
/* One prover round.  `prev_challenge` is NULL on the first round, otherwise the
 * challenge the host sampled after the previous round (one challenge element).
 * Writes the round polynomial's evaluations at 0..=degree (degree+1 challenge
 * elements) to `out_evals`. */
int dpb_sumcheck_round(dpb_sc* sc, const void* prev_challenge, void* out_evals, uint32_t* n_evals);
/* Binds the last variable and returns every table's evaluation at the full
 * point, in registration order (IOPProverState::get_mle_flatten_final_evaluations,
 * zkml/src/lookup/logup_gkr/prover.rs:281). */
int dpb_sumcheck_finish(dpb_sc* sc, const void* last_challenge, void* out_final_evals);
void dpb_sumcheck_free(dpb_sc* sc);

/* First sumcheck round of a product of k tables without any allocation.
 * (No counterpart in the reference: its prover is CPU code and never had to
 * care who owns device memory.)
 *
 * Meant for callers that must not allocate on the device when they call in:
 * code running inside a region an outer runtime records for later replay, a
 * host that gave all device memory to its own pool, or a worker with a fixed
 * device-memory budget.  It needs no dpb_ctx.  The caller passes k (2..4)
 * device pointers to tables of `len` entries of layout `dtype`, all 16-byte
 * aligned, and a device buffer for k+1 challenge elements; on return the
 * kernel has been queued on `cuda_stream` (a cudaStream_t, on the current
 * device) and will write there the round polynomial's evaluations at 0..=k,
 * the same values dpb_sumcheck_begin + dpb_sumcheck_round return for the
 * term  table_0 * ... * table_{k-1}.  The caller synchronises.
 *
 * Limits and rules:
 *  - len is a power of two, 2 <= len <= 2^30; larger tables are rejected with
 *    DPB_EINVAL, as are k outside 2..4 and unaligned pointers.
 *  - The per-block partial sums live in a fixed scratch array inside the
 *    library's device image, about 160 KiB on every GPU that loads the
 *    library, kept until the process exits.  The first call on a device looks
 *    up that array's device address; make that first call outside any stream
 *    capture.
 *  - All calls on a device share the scratch array.  Each call zeroes the part
 *    that must start at zero, but two calls whose kernels can overlap on the
 *    GPU (different streams, no ordering between them) race on it: order them.
 *  - `cuda_stream` must belong to the device that is current when the call is
 *    made (the scratch array is per device); a stream of another device is
 *    rejected with DPB_EINVAL.
 *  - It calls no cudaMalloc / cudaFree and no allocating library routine. */
int dpb_product_round_noalloc(void* cuda_stream, int dtype, const void* const* tables_dev, uint32_t k,
                              uint64_t len, void* out_evals_dev);

/* ---- logup-GKR fraction tree ------------------------------------------- */
#define DPB_LOGUP_LOOKUP 0
#define DPB_LOGUP_TABLE 1
/* Builds every level of the fraction tree of one instance on the device
 * (LogUpCircuit::new, zkml/src/lookup/logup_gkr/circuit.rs:512-516;
 * LogUpLayer::next_layer, :88-184).  `columns` are n_cols tables of 2^m
 * entries; `mult` (tables only) the multiplicities.  constant_chal / sep_chal
 * are challenge elements on the host. */
int dpb_logup_build(dpb_ctx* ctx, int kind, dpb_mle* const* columns, uint32_t n_cols,
                    const dpb_mle* mult, const void* constant_chal, const void* sep_chal,
                    dpb_logup** out);
/* Number of levels above the input (m-1 ... down to the 2-element level). */
uint32_t dpb_logup_num_levels(const dpb_logup* lu);
/* Borrowed views [num_lo, num_hi, den_lo, den_hi] of tree level `level`
 * (1 = first computed level, arrays of 2^(m-1); num_levels = top, arrays of 2),
 * the MLEs LogUpLayer::layer_proving_info hands to the sumcheck
 * (zkml/src/lookup/logup_gkr/circuit.rs:255-271). Views must be freed with dpb_mle_free. */
int dpb_logup_level(const dpb_logup* lu, uint32_t level, dpb_mle* out_views[4]);
/* [num[0], num[1], den[0], den[1]] of the top level (LogUpCircuit::outputs, :558-560). */
int dpb_logup_outputs(const dpb_logup* lu, void* out4);
/* The same for n trees of one context and field with a single wait: out receives 4 elements per tree. */
int dpb_logup_outputs_batch(const dpb_logup* const* lus, uint32_t n, void* out);
void dpb_logup_free(dpb_logup* lu);

/* ---- lookup witness generation (zkml/src/lookup/operation, zkml/src/lookup/context.rs) ---- */
#define DPB_SIGN_POSITIVE 0 /* TableSign::Positive: inputs >= 0 (shift check, zero check) */
#define DPB_SIGN_NEGATIVE 1 /* TableSign::Negative: inputs <= 0 (exp) */
#define DPB_SIGN_MIXED 2    /* TableSign::Mixed: both signs (ReLU, GeLU, SiLU, requantise, signed zero check) */

/* The numbers ChunkingInfo holds (zkml/src/lookup/operation/decomposer.rs:12-42). */
typedef struct dpb_chunking_info {
    uint32_t right_shift;
    uint32_t value_chunk_bits; /* the value table's bit size */
    uint32_t n_value_chunks;
    uint32_t n_shifted_chunks;
    uint32_t n_zeroing_chunks;
    int32_t table_sign;
    int64_t offset;
    int64_t value_chunk_offset;
    int64_t shifted_chunk_multiplier;
    int64_t top_zeroing_chunk_offset;
} dpb_chunking_info;

/* ChunkingInfo::new(right_shift, table, max_bit_size, number_of_value_chunks)
 * (decomposer.rs:182-249); the table enters through its bit size and input sign.  Host only.
 * DPB_EINVAL for right_shift = 0 (the reference's error), for more than 4 chunks of a kind and
 * for a bit size outside 1..30. */
int dpb_chunking_info_new(uint32_t right_shift, uint32_t table_bits, int table_sign, uint32_t max_bit_size,
                          uint32_t n_value_chunks, dpb_chunking_info* out);

/* How often each row of one table was looked up (the per-table element counts of
 * LookupWitnessGen, zkml/src/lookup/context.rs:160-200), as 2^table_bits 64-bit counters on
 * the device, row i being the table's input min_input + i (Table::min_input_value,
 * zkml/src/lookup/table/mod.rs:135-142).  Counters start at zero and add up over every
 * dpb_lookup_witness call they are handed to, which is how lookups of several layers into
 * one table are merged (LookupWitnessGen::consume). */
typedef struct dpb_lookup_counts dpb_lookup_counts;
int dpb_lookup_counts_new(dpb_ctx* ctx, uint32_t table_bits, dpb_lookup_counts** out);
int dpb_lookup_counts_to_host(const dpb_lookup_counts* counts, uint64_t* out, uint64_t len);
void dpb_lookup_counts_free(dpb_lookup_counts* counts);
/* Adds one to counter rows[i] for every i < n: lookups that need no decomposition, such as the
 * 16-bit range-check chunks of the logits layer, which go straight into the shift-check table
 * (Logits::build_lookup_input, zkml/src/layers/transformer/logits.rs:300-345).  `rows` are row
 * indices (input - min_input), in host memory or (rows_on_device != 0) device memory.  A row
 * outside the table is not counted and the call returns DPB_EINVAL. */
int dpb_lookup_counts_add_rows(dpb_ctx* ctx, dpb_lookup_counts* counts, const int64_t* rows, int rows_on_device,
                               uint64_t n);

/* The table's multiplicity polynomial (context.rs:313-371): row i holds its count as a field
 * element.  The rows of the reference's tables are distinct (the input column is a range), so
 * the division by a row's number of copies (context.rs:349-357) never applies. */
int dpb_lookup_multiplicities(dpb_ctx* ctx, const dpb_lookup_counts* counts, int family_dtype, dpb_mle** out);

/* LookupOp::generate_witness (zkml/src/lookup/operation/mod.rs:103-160) followed by
 * LookupOpWitness::{input_mle_evals, output_mle_evals, get_counts} (mod.rs:193-282).
 * `tensor`: the operation's UNPADDED input, signed 64-bit, row-major, on the host or (with
 * tensor_on_device) on the device.  Every slice over the last two dimensions is padded to
 * powers of two with padding_value, every entry becomes x * fixed_point_multiplier +
 * 2^(right_shift-1) and is decomposed as `info` says.  `value_table_outputs`: the value
 * table's output column over its inputs min..=max (2^value_chunk_bits entries), or NULL for a
 * one-column table (requantise), whose output is its input; num_value_columns as
 * Table::num_columns.
 * Results, P = padded slice size, per slice in the reference's order:
 *   input columns:  shifted chunks (least significant first), value chunks when the value
 *                   table has two columns, zeroing chunks;
 *   output columns: value chunk outputs, zeroing chunk outputs (zero check: 1 at 0 else 0;
 *                   the top chunk of a Mixed operation: signum).
 * Columns are tables of DPB_GL_BASE or DPB_FR elements (negative x -> p - |x|): borrowed
 * views into *out_owner, as with dpb_einsum_fix_axes.  The four count handles may be NULL
 * (that table's lookups are not counted); shift, zero and signed-zero counts have 2^16 rows.
 * DPB_EINVAL with the reference's message when a top zeroing chunk falls outside the signed
 * zero-check table (an input beyond max_bit_size).  * family_dtype may also be an integer layout (DPB_FR_I64 / DPB_GL_I64): the columns then hold the chunks as
 * 64-bit integers (8 bytes per entry), which every sumcheck entry point, the logup tree and dpb_msm_g1 accept.
 */
int dpb_lookup_witness(dpb_ctx* ctx, int family_dtype, const dpb_chunking_info* info, int64_t fixed_point_multiplier,
                       int64_t padding_value, const int64_t* tensor, int tensor_on_device, const uint64_t* shape,
                       uint32_t rank, const int64_t* value_table_outputs, int outputs_on_device,
                       uint32_t num_value_columns, dpb_lookup_counts* shift_counts, dpb_lookup_counts* value_counts,
                       dpb_lookup_counts* zero_counts, dpb_lookup_counts* signed_zero_counts, dpb_mle** out_owner,
                       dpb_mle** out_input_columns, uint32_t in_cap, uint32_t* n_in, dpb_mle** out_output_columns,
                       uint32_t out_cap, uint32_t* n_out);

#ifdef __cplusplus
}
#endif
#endif /* DPB_H */
