/*
 * verinf_b200 — C ABI of the B200 (sm_100a) kernels for VerInf's prover
 * field-arithmetic hot path.
 *
 * Conventions
 *  - Every pointer named *_dev or typed as data (uint64_t*, uint8_t*) is a DEVICE
 *    pointer into memory the caller owns; the library allocates no outputs.
 *  - Field elements are uint64_t in canonical form [0, p), p = 2^64 - 2^32 + 1.
 *  - `stream` is a cudaStream_t passed as void* (NULL = legacy default stream).
 *  - Every function returns 0 on success; non-zero means nothing useful was
 *    written and vi_last_error() holds a message.  The library never exits the
 *    process and never traps the device.
 *  - The only memory the library owns are immutable per-device twiddle tables,
 *    allocated (cudaMalloc + synchronous upload) the first time a transform
 *    length is used on a device.
 *
 * Each declaration cites the reference interface it replaces (paths relative to
 * the reference project root).  A ctypes binding of these symbols is what the
 * drop-in modules verinf_b200/cuda_primitives.py and kquant_cuda.py use.
 */
#ifndef VERINF_B200_H
#define VERINF_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Text of the last error raised on the calling thread. */
const char* vi_last_error(void);

/* ---- elementwise field ops ------------------------------------------------
 * replace gl_mul/gl_add/gl_sub/gl_neg/gl_pow/gl_inv_batched/gl_axpy_inplace
 * (prover/cuda_primitives.py:208-303, prover/kernels/gl_extras.cuh:22-40).
 * op: 0 = mul, 1 = add, 2 = sub.  out may alias a or b. */
int vi_gl_binary(int op, const uint64_t* a, const uint64_t* b, uint64_t* out, int64_t n, void* stream);
/* out[i] = a[i] op b[i % nb]: the broadcast form callers build today with
 * .expand().contiguous() (prover/core.py:738-739, layergkr/gpu.py:189). */
int vi_gl_binary_bcast(int op, const uint64_t* a, const uint64_t* b, int64_t nb, uint64_t* out, int64_t n, void* stream);
int vi_gl_neg(const uint64_t* a, uint64_t* out, int64_t n, void* stream);
int vi_gl_pow(const uint64_t* base, uint64_t exp, uint64_t* out, int64_t n, void* stream);
int vi_gl_axpy(uint64_t* y, uint64_t alpha, const uint64_t* x, int64_t n, void* stream);

/* ---- NTT --------------------------------------------------------------------
 * replaces ntt_forward/ntt_inverse(_batched) (prover/cuda_primitives.py:347-409,
 * prover/kernels/ntt.cuh:310-770).  In place over m contiguous rows of length n
 * (power of two, 2 <= n <= 2^30), natural order in and out; the inverse scales by
 * n^-1.  Transforms longer than 1024 need scratch (any size >= n*8 bytes works;
 * vi_ntt_scratch_bytes gives the recommended size: the rows of a 1 GiB chunk).  Above
 * 2^24 the transform runs as three tile passes, one row at a time, and needs 2*n*8 bytes
 * (the reference's dispatch takes any power of two, prover/kernels/ntt.cuh:746-770). */
int64_t vi_ntt_scratch_bytes(int64_t m, int64_t n);
int vi_ntt_batched(uint64_t* rows, int64_t m, int64_t n, int inverse,
                   void* scratch, int64_t scratch_bytes, void* stream);

/* The library owns only immutable per-device tables (twiddles, four-step factors, coset
 * scalings), built on the first use of a length and kept for the life of the process, as the
 * reference keeps its twiddle contexts (prover/cuda_primitives.py:319-331).  vi_release_tables
 * frees them all; call it with no library kernel in flight. */
int vi_release_tables(void);

/* ---- Reed-Solomon row encode ---------------------------------------------------
 * replaces encode_messages + _coset_encode_codewords (prover/core.py:721-802) and
 * layergkr's encode_batch_ntt (layergkr/gpu.py:141-203): message row = values of a
 * degree-<K polynomial at the K-th roots of unity (slots [ell,K) are the pad);
 * polys[r] = its coefficients; codes[r][j] = its value at 7*w_N^j.
 *   msg      (m, ell) row-major
 *   pad_mode 0: pad slots are zero (layergkr); 1: pad slot k of row r is
 *            u64le(BLAKE3(seed || (row_off+r)_le8 || k_le8)[0:8]) % p  (row_prg)
 *   seed_dev 32 bytes on the device (pad_mode 1)
 *   polys    (m, K) or NULL;  codes (m, N) or NULL
 *   scratch  >= (K + N)*8 bytes (K*8 when codes is NULL); see vi_encode_scratch_bytes */
int64_t vi_encode_scratch_bytes(int64_t m, int64_t k, int64_t n);
int vi_encode_rows(const uint64_t* msg, int64_t m, int64_t ell, int64_t k, int64_t n,
                   int pad_mode, const uint8_t* seed_dev, int64_t row_off,
                   uint64_t* polys, uint64_t* codes,
                   void* scratch, int64_t scratch_bytes, void* stream);

/* ---- ZK pad PRG ---------------------------------------------------------------
 * replaces row_prg / row_prg_indexed (prover/cuda_primitives.py:877-974).
 * out (n_rows, slack).  rows_dev == NULL means rows row_off .. row_off+n_rows-1. */
int vi_row_prg(const uint8_t* seed_dev, int64_t row_off, const uint64_t* rows_dev,
               int64_t n_rows, int64_t slack, uint64_t* out, void* stream);

/* ---- challenge PRF --------------------------------------------------------------
 * replaces challenge_vec / challenge_at (prover/cuda_primitives.py:549-591,
 * prover/kernels/gl_spmv.cuh:51-66): out[i] = int(BLAKE3(seed || label ||
 * cid_le8)[:16], LE) % p with cid = cids_dev ? cids_dev[i] : i.  label_len <= 8. */
int vi_challenge(const uint8_t* seed_dev, const uint8_t* label_dev, int label_len,
                 const uint64_t* cids_dev, int64_t n, uint64_t* out, void* stream);

/* ---- BLAKE3 column hash ---------------------------------------------------------
 * replaces hash_columns_streamed (prover/cuda_primitives.py:796-808,
 * prover/kernels/blake3_columns.cuh:47-174): digest j = BLAKE3-256 of the bytes
 * le8(mat[0,j]) || le8(mat[1,j]) || ... of column j of the row-major (m, ncols)
 * matrix.  digests (ncols, 32).  scratch holds per-segment subtree chaining values;
 * vi_hash_columns_scratch_bytes gives the size (0 when a single segment is used). */
int64_t vi_hash_columns_scratch_bytes(int64_t m, int64_t ncols);
int vi_hash_columns(const uint64_t* mat, int64_t m, int64_t ncols, uint8_t* digests,
                    void* scratch, int64_t scratch_bytes, void* stream);

/* Same digests as vi_hash_columns for callers that cannot allocate device memory (no
 * counterpart in the reference).  The chaining-value state lives in a fixed 8 MiB device
 * array inside the library instead of caller scratch, so the call performs no cudaMalloc /
 * cudaFree and takes only inputs and outputs.  Inputs needing more state than
 * vi_hash_columns_noalloc_max_state_bytes() (= vi_hash_stream_state_bytes(ncols, m) for
 * m > 128; e.g. 65536 columns x up to 1024 rows) are rejected with an error.  The first
 * call on a device looks up the array's device address (cudaGetSymbolAddress); make that
 * first call before any stream capture, and do not use the entry point on a device after a
 * cudaDeviceReset (the looked-up address is kept).  All calls on a device share the array: calls
 * that overlap on the GPU race and must be serialised by the caller.  Every input is hashed with
 * one thread per column; vi_hash_columns splits matrices of fewer than 131072 columns into
 * concurrent row segments, so narrow inputs take longer here (same digests). */
int64_t vi_hash_columns_noalloc_max_state_bytes(void);
int vi_hash_columns_noalloc(const uint64_t* mat, int64_t m, int64_t ncols, uint8_t* digests, void* stream);

/* Streaming form: replaces hash_columns_stream_init/update/finalize and the state
 * machine behind MerkleColumnAccumulator (prover/cuda_primitives.py:813-853,976-987,
 * 1297-1385; prover/kernels/blake3_columns.cuh:184-328).  The state is a caller-owned
 * buffer of vi_hash_stream_state_bytes(ncols, total_rows) bytes; no initialisation
 * is needed.  Feed the rows in order: every call but the last must bring a multiple
 * of 128 rows; rows_done is the number of rows fed before this call.  The call that
 * reaches total_rows writes the digests. */
int64_t vi_hash_stream_state_bytes(int64_t ncols, int64_t total_rows);
int vi_hash_stream_update(void* state, int64_t ncols, int64_t total_rows, int64_t rows_done,
                          const uint64_t* rows, int64_t n_rows, uint8_t* digests, void* stream);

/* Sharded column hash (no counterpart in the reference, which is single-GPU): a rank that
 * holds a row range made of whole 128-row chunks hashes each aligned block of 2^level chunks
 * to one non-root sub-tree chaining value per column (vi_hash_subtree; first_chunk is the
 * block's global chunk index, a multiple of 2^level; only the stream's last chunk may be
 * short), the (ncols, 32) results of all ranks are gathered in row order, and
 * vi_hash_merge_subtrees folds them into the same digests vi_hash_columns gives on the whole
 * matrix.  levels is a HOST array with the level of each gathered block, left to right.
 * state: vi_hash_subtree_state_bytes(ncols, level) bytes of scratch. */
int64_t vi_hash_subtree_state_bytes(int64_t ncols, int level);
int vi_hash_subtree(const uint64_t* rows, int64_t n_rows, int64_t ncols, int64_t first_chunk, int level,
                    void* state, uint8_t* cv_out, void* stream);
int vi_hash_merge_subtrees(const uint8_t* cvs, const int32_t* levels, int nblocks, int64_t ncols,
                           uint8_t* digests, void* stream);

/* ---- Merkle tree ----------------------------------------------------------------
 * replaces merkle_build_blake3 / merkle_one_level (prover/cuda_primitives.py:990-1004,
 * 1388-1401; prover/kernels/merkle.cuh:18-37): parent = BLAKE3-256(left || right) as a
 * 64-byte message; an odd level pairs its last node with itself.
 * upper receives levels 1.. (level i has ceil(n_{i-1}/2) nodes) back to back:
 * vi_merkle_upper_nodes(n) nodes of 32 bytes; the root is the last one. */
int64_t vi_merkle_upper_nodes(int64_t n_leaves);
int vi_merkle_build(const uint8_t* leaves, int64_t n_leaves, uint8_t* upper, void* stream);
int vi_merkle_level(const uint8_t* nodes, int64_t n_nodes, uint8_t* parents, void* stream);

/* ---- Evaluation-domain fold of row products -----------------------------------------
 * The q_lin and p_0 folds multiply rows of coefficient polynomials pairwise and sum the
 * products over the rows (prover/core.py:1892-1911 `_compute_q_lin_inner_chunk`, fused
 * branch; prover/core.py:2166-2181 `compute_p_0_streaming`).  The reference builds zero-padded
 * copies, runs ntt_forward_batched on both, gl_mul, a transposed copy and gl_matvec.
 * vi_ntt_forward_padded: dst (m, n) = forward NTT of each src row (k_in <= n values) extended
 *   with zeros; out of place, no padded copy; scratch as vi_ntt_scratch_bytes(m, n).
 * vi_product_colsum: out[j] (+)= sum_{i<T} w[i] * EA[ia[i]*n + j] * EB[ib[i]*n + j] for j < n;
 *   ia / ib (device int64, may be null = identity) select rows of the transformed matrices, so
 *   a row used by several constraints is transformed once; w (device, may be null = ones);
 *   accumulate != 0 adds into out.  scratch: vi_product_colsum_scratch_bytes(T, n). */
int vi_ntt_forward_padded(const uint64_t* src, int64_t m, int64_t k_in, uint64_t* dst, int64_t n,
                          void* scratch, int64_t scratch_bytes, void* stream);
int64_t vi_product_colsum_scratch_bytes(int64_t T, int64_t n);
int vi_product_colsum(const uint64_t* EA, const uint64_t* EB, int64_t n,
                      const int64_t* ia_dev, const int64_t* ib_dev, const uint64_t* w_dev, int64_t T,
                      uint64_t* out, int accumulate, void* scratch, int64_t scratch_bytes, void* stream);

/* ---- Column openings ----------------------------------------------------------------
 * vi_open_columns replaces `codes.index_select(1, Q_set)` + per-column clone/cat
 * (prover/core.py:1304-1320): out[t*out_stride + row0 + r] = mat[r*n + cols[t]] for r < m,
 * t < T, so a matrix that arrives in row chunks fills one (T, total_rows) buffer, each
 * opened column contiguous.  cols is a device array; an index outside [0, n) yields zeros.
 * vi_merkle_paths replaces merkle_path over a host copy of the tree (prover/core.py:294-317):
 * for each queried leaf idx[t] and level l < depth (= vi_merkle_depth(n_leaves)),
 * siblings[(t*depth + l)*32 ..] is the sibling node (the node itself where an odd level has
 * no sibling) and sides[t*depth + l] is 1 when the path node is a left child, else 0.
 * leaves/upper are the buffers of vi_merkle_build (16-byte aligned); idx is a device
 * array, an index outside [0, n_leaves) yields the path of leaf 0. */
int vi_open_columns(const uint64_t* mat, int64_t m, int64_t n, const int64_t* cols_dev, int64_t T,
                    uint64_t* out, int64_t out_stride, int64_t row0, void* stream);
int vi_merkle_depth(int64_t n_leaves);
int vi_merkle_paths(const uint8_t* leaves, int64_t n_leaves, const uint8_t* upper,
                    const int64_t* idx_dev, int64_t T, uint8_t* siblings, uint8_t* sides, void* stream);

/* ---- K-quant lift -----------------------------------------------------------------
 * replaces kquant_to_field (prover/kquant_cuda.py:60-177): raw GGUF super-blocks ->
 * field integers round_half_even(double(v) * S), negative values as p - |v|, in stored
 * order.  qtype 4 = Q4_K (144 B), 5 = Q5_K (176 B), 6 = Q6_K (210 B); out n_blocks*256. */
int vi_kquant_to_field(const uint8_t* raw, int64_t n_blocks, int qtype, double S,
                       uint64_t* out, void* stream);

/* Fused lift + encode (no counterpart in the reference; equals kquant_to_field ->
 * optional transpose as prover/loader.py:433-436 -> row packing of
 * prover/core.py:389-458 -> encode_messages): the quantised (d_out, d_in) matrix is
 * lifted inside the encode's first pass, so lifted weights never reach HBM.
 * Message slot c of row r is flat element f = (first_row + r)*ell + c of the lifted
 * matrix, transposed (f = k_in*d_out + n_out) when transpose != 0; slots past the end
 * of the matrix are zero.  Other arguments as vi_encode_rows.  If the scratch has d_out*d_in/4 + 64
 * bytes beyond one row's (K+N)*8, its tail is used for pre-multiplied sub-block scales (faster gather). */
int vi_kquant_encode_rows(const uint8_t* raw, int qtype, double S, int64_t d_out, int64_t d_in,
                          int transpose, int64_t first_row, int64_t m,
                          int64_t ell, int64_t k, int64_t n,
                          int pad_mode, const uint8_t* seed_dev, int64_t row_off,
                          uint64_t* polys, uint64_t* codes,
                          void* scratch, int64_t scratch_bytes, void* stream);

/* ---- sumcheck ---------------------------------------------------------------------
 * replaces the per-round work of prove_terms_gpu / fold_t / gl_sum
 * (layergkr/gpu.py:326-410; CPU twin layergkr/sumcheck.py:153-226).
 * A problem is n_tables multilinear tables of `size` entries (power of two; entry i of
 * table k at tables[k*stride + i]) and n_terms products: term t = coefs[t] *
 * prod_{j < nfac[t]} table[fac[t*4 + j]]  (at most 8 tables, 8 terms, 4 factors).
 * coefs, nfac and fac are small HOST arrays (n_terms, n_terms, n_terms*4 entries).
 *   vi_sumcheck_claim   sum over the hypercube of all terms -> out[0]
 *   vi_sumcheck_round   flags bit 0 (fold): first folds every table with challenge r
 *                       (f'[i] = f[i] + r*(f[half+i] - f[i]), size -> size/2, in place),
 *                       then writes the round samples g(0..deg) of the (folded) tables
 *                       to out[0..deg].  `size` is the table length BEFORE the fold.
 *                       With size/2 == 1 after folding no samples exist; the final
 *                       values are tables[k*stride].
 *                       flags bit 1 (skip x = 1): out[1] is not computed (written as 0); the
 *                       caller derives it from g(0) + g(1) = g_prev(r), the value of the
 *                       previous round polynomial at its challenge (the sum of the terms over
 *                       the hypercube for the first round).  One product fewer per table pair.
 * partials: scratch of vi_sumcheck_scratch_bytes() bytes.  out: device, >= 8 u64. */
int64_t vi_sumcheck_scratch_bytes(void);
int vi_sumcheck_claim(const uint64_t* tables, int64_t stride, int n_tables, int64_t size,
                      int n_terms, const uint64_t* coefs, const int32_t* nfac, const int32_t* fac,
                      uint64_t* out, void* partials, void* stream);
/* All rounds for challenges known up front (HOST array coins[n_rounds], size = 2^n_rounds): queues
 * every fold+evaluate launch without a host round trip; samples (device, n_rounds x 8 u64) receives
 * g(0..deg) of round i at samples[8*i ..], EXCEPT g(1) of rounds i >= 1, which is left 0 and
 * follows from g_i(0) + g_i(1) = g_{i-1}(coins[i-1]) (round 0 is complete, so its g(0) + g(1) is
 * also the claim).  Equivalent to n_rounds + 1 calls of vi_sumcheck_round with flags 0, 3, 3, ..., 1. */
int vi_sumcheck_run(uint64_t* tables, int64_t stride, int n_tables, int64_t size,
                    int n_terms, const uint64_t* coefs, const int32_t* nfac, const int32_t* fac,
                    const uint64_t* coins, int n_rounds, uint64_t* samples, void* partials, void* stream);
int vi_sumcheck_round(uint64_t* tables, int64_t stride, int n_tables, int64_t size,
                      int n_terms, const uint64_t* coefs, const int32_t* nfac, const int32_t* fac,
                      int flags, uint64_t r, uint64_t* out, void* partials, void* stream);
/* Fills the g(1) that vi_sumcheck_run leaves out, on the device: for i = 1 .. n_rounds-1,
 * samples[8*i + 1] = g_{i-1}(coins[i-1]) - samples[8*i], with g_{i-1} interpolated from its deg + 1
 * samples at the nodes 0..deg (what the reference's verifier recomputes, layergkr/sumcheck.py:235-262).
 * coins: HOST array of n_rounds canonical challenges; n_rounds <= 64, 1 <= deg <= 7.  Row 0 must be
 * complete.  One launch of one CTA; lets the caller copy finished round polynomials in one transfer. */
int vi_sumcheck_complete(uint64_t* samples, int n_rounds, int deg, const uint64_t* coins, void* stream);

/* ---- remaining exports of the reference module (not on the hot path) -------------
 * poly_eval (prover/kernels/gl_extras.cuh:93-108), gl_matmul / gl_matvec
 * (prover/kernels/gl_matmul.cuh:28-59), gl_spmv / gl_spmv_challenged
 * (prover/kernels/gl_spmv.cuh:25-90), lookup multiplicities
 * (prover/kernels/gl_extras.cuh:118-149). */
int vi_poly_eval(const uint64_t* coeffs, int64_t m, int64_t d, const uint64_t* points, int64_t k,
                 uint64_t* out, void* stream);
int vi_gl_matmul(const uint64_t* A, const uint64_t* B, uint64_t* C, int64_t m, int64_t k, int64_t n, void* stream);
/* The same product on the integer tensor cores (no counterpart in the reference): operands are
 * split into byte planes in the scratch (vi_gl_matmul_tc_scratch_bytes(m, k, n) = 8 bytes per
 * padded operand element, 16-byte aligned), the 64 plane products run as u8 x u8 -> s32
 * mma.sync tiles and are recombined mod p.  Bit-identical to vi_gl_matmul. */
int64_t vi_gl_matmul_tc_scratch_bytes(int64_t m, int64_t k, int64_t n);
int vi_gl_matmul_tc(const uint64_t* A, const uint64_t* B, uint64_t* C, int64_t m, int64_t k, int64_t n,
                    void* scratch, int64_t scratch_bytes, void* stream);
/* The same product on the 5th-generation tensor cores (tcgen05.mma kind::i8, M128 x N256 x K32) with
 * the 15 plane-sum accumulators of a 128 x 32 output tile in tensor memory and the byte planes
 * brought in by TMA (no counterpart in the reference; replaces prover/kernels/gl_matmul.cuh:28-59
 * for large products).  scratch: vi_gl_matmul_umma_scratch_bytes(m, k, n) bytes, 256-byte aligned.
 * status_dev: optional device int32, cleared on the stream before the launch; the kernel sets it
 * non-zero if one of its bounded waits expired (it then frees its tensor memory and returns; C is
 * incomplete).  Read it after synchronising the stream.  Bit-identical to vi_gl_matmul. */
int64_t vi_gl_matmul_umma_scratch_bytes(int64_t m, int64_t k, int64_t n);
int vi_gl_matmul_umma(const uint64_t* A, const uint64_t* B, uint64_t* C, int64_t m, int64_t k, int64_t n,
                      void* scratch, int64_t scratch_bytes, int32_t* status_dev, void* stream);
int vi_gl_matvec(const uint64_t* M, const uint64_t* v, uint64_t* w, int64_t m, int64_t n, void* stream);
int vi_gl_spmv(const uint64_t* values, const uint64_t* col_idx, const uint64_t* row_ptr,
               const uint64_t* x, const uint8_t* seed_dev, const uint8_t* label_dev, int label_len,
               uint64_t* y, int64_t n_rows, void* stream);   /* x == NULL: challenged form */
int vi_lookup_multiplicities(const uint64_t* x, int64_t n_x, const uint64_t* table, int64_t n_table,
                             uint64_t* mult, void* stream);   /* table == NULL: range table [0, n_table) */

/* q_lin band interpreters (prover/cuda_primitives.py:605-790).  kind 0 = descriptor
 * band (u = desc_dev, tblA, tblB, chal_buf), 1 = causal_id (p0=base,p1=m,p2=h,p3=coef),
 * 2 = causal_c2 (p0=base,p1=h,p2=coef), 3 = embed (p0=base,p1=d,p2=rows_per_w,p3=ell,
 * aux0 = token ids int64, aux_n = count), 4 = rope_x (p0=base,p1=H,p2=d_h, aux0 = cos,
 * aux1 = sin). */
int vi_interp_band(int kind, uint64_t* out, int64_t out_off, int64_t flat_lo, int64_t n_slots,
                   uint64_t p0, uint64_t p1, uint64_t p2, uint64_t p3,
                   const uint64_t* desc_dev, const void* aux0, const void* aux1, const uint64_t* chal_buf,
                   int64_t aux_n, const uint8_t* seed_dev, const uint8_t* label_dev, int label_len,
                   void* stream);

/* ---- per-kernel timing ------------------------------------------------------------
 * CUDA events recorded around every launch on the launching stream while enabled (the
 * reference's nearest equivalent is its LIGERO_EPHASE event sums, prover/core.py:1139-1165).
 * vi_profile_enable(1) clears the counters; vi_profile_read waits for the recorded events
 * and returns total device milliseconds and launch count of one kernel tag. */
void vi_profile_enable(int on);
int vi_profile_num_tags(void);
const char* vi_profile_tag_name(int tag);
int vi_profile_read(int tag, double* total_ms, int64_t* launches);

#ifdef __cplusplus
}
#endif
#endif /* VERINF_B200_H */
