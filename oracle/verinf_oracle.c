/*
 * CPU oracle for the VerInf prover field-arithmetic hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * reference's algorithms, used as the checker in tests, in the smoke test and
 * as the timed CPU baseline of the benchmark.  Nothing in the shipped CUDA
 * path calls into it.
 *
 * Parity status: PINNED.  Every function below is checked (tests/test_oracle.py)
 * against fixtures under tests/golden/ that were produced by importing the
 * reference's own Python (prover/ref/goldilocks_ref.py, prover/protocol.py,
 * layergkr/rs.py, layergkr/sumcheck.py, layergkr/transcript.py) together with
 * the `blake3` and `gguf` packages the reference depends on; the generating
 * script is tests/golden/make_golden.py.
 *
 * Each function cites the reference file:line it follows (paths are relative
 * to the reference project root).
 *
 * Build: gcc -O2 -fopenmp -ffp-contract=off -fPIC -shared (see oracle/Makefile).
 */
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#include <math.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define GL_P 0xFFFFFFFF00000001ULL
typedef unsigned __int128 u128;

/* ------------------------------------------------------------------ */
/* Field: prover/ref/goldilocks_ref.py:25-49, prover/protocol.py:27-33 */
/* ------------------------------------------------------------------ */
static inline uint64_t f_add(uint64_t a, uint64_t b) { return (uint64_t)(((u128)a + b) % GL_P); }
static inline uint64_t f_sub(uint64_t a, uint64_t b) { return (uint64_t)(((u128)a + GL_P - (b % GL_P)) % GL_P); }
static inline uint64_t f_mul(uint64_t a, uint64_t b) { return (uint64_t)(((u128)a * b) % GL_P); }
static uint64_t f_pow(uint64_t b, uint64_t e) {
    uint64_t r = 1; b %= GL_P;
    while (e) { if (e & 1) r = f_mul(r, b); b = f_mul(b, b); e >>= 1; }
    return r;
}
static inline uint64_t f_inv(uint64_t a) { return f_pow(a, GL_P - 2); }

uint64_t or_gl_add(uint64_t a, uint64_t b) { return f_add(a, b); }
uint64_t or_gl_sub(uint64_t a, uint64_t b) { return f_sub(a, b); }
uint64_t or_gl_mul(uint64_t a, uint64_t b) { return f_mul(a, b); }
uint64_t or_gl_pow(uint64_t a, uint64_t e) { return f_pow(a, e); }
uint64_t or_gl_inv(uint64_t a) { return f_inv(a); }

/* primitive n-th root of unity: goldilocks_ref.py:45-49 (7^((p-1)/n)) */
/* C = A.B mod p, row-major (m,k).(k,n); definition of gl_matmul
 * (prover/cuda_primitives.py:1086-1106, prover/kernels/gl_matmul.cuh) */
void or_gl_matmul(const uint64_t* A, const uint64_t* B, uint64_t* C, int64_t m, int64_t k, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < m; ++i)
        for (int64_t j = 0; j < n; ++j) {
            uint64_t acc = 0;
            for (int64_t l = 0; l < k; ++l) acc = f_add(acc, f_mul(A[i * k + l], B[l * n + j]));
            C[i * n + j] = acc;
        }
}

uint64_t or_root_of_unity(uint64_t n) { return f_pow(7, (GL_P - 1) / n); }

/* ------------------------------------------------------------------ */
/* NTT: iterative decimation-in-time, prover/ref/goldilocks_ref.py:52-90 */
/* natural order in and out; inverse uses w^-1 and scales by n^-1.      */
/* ------------------------------------------------------------------ */
void or_ntt(uint64_t* a, int64_t n, int invert) {
    int64_t j = 0;
    for (int64_t i = 1; i < n; ++i) {
        int64_t bit = n >> 1;
        while (j & bit) { j ^= bit; bit >>= 1; }
        j ^= bit;
        if (i < j) { uint64_t t = a[i]; a[i] = a[j]; a[j] = t; }
    }
    uint64_t omega = or_root_of_unity((uint64_t)n);
    for (int64_t len = 2; len <= n; len <<= 1) {
        uint64_t w_len = f_pow(omega, (uint64_t)(n / len));
        if (invert) w_len = f_inv(w_len);
        int64_t half = len / 2;
        for (int64_t i = 0; i < n; i += len) {
            uint64_t w = 1;
            for (int64_t k = 0; k < half; ++k) {
                uint64_t u = a[i + k];
                uint64_t v = f_mul(a[i + k + half], w);
                a[i + k] = f_add(u, v);
                a[i + k + half] = f_sub(u, v);
                w = f_mul(w, w_len);
            }
        }
    }
    if (invert) {
        uint64_t n_inv = f_inv((uint64_t)n % GL_P);
        for (int64_t i = 0; i < n; ++i) a[i] = f_mul(a[i], n_inv);
    }
}

/* Faster transform with a precomputed twiddle table (same arithmetic, same
 * result); used for the large timed baseline and large-size oracles.
 * tw holds w^k (or w^-k) for k < n/2. */
static void ntt_table(uint64_t* a, int64_t n, const uint64_t* tw, int invert) {
    int64_t j = 0;
    for (int64_t i = 1; i < n; ++i) {
        int64_t bit = n >> 1;
        while (j & bit) { j ^= bit; bit >>= 1; }
        j ^= bit;
        if (i < j) { uint64_t t = a[i]; a[i] = a[j]; a[j] = t; }
    }
    for (int64_t len = 2; len <= n; len <<= 1) {
        int64_t half = len / 2, step = n / len;
        for (int64_t i = 0; i < n; i += len)
            for (int64_t k = 0; k < half; ++k) {
                uint64_t u = a[i + k];
                uint64_t v = f_mul(a[i + k + half], tw[k * step]);
                a[i + k] = f_add(u, v);
                a[i + k + half] = f_sub(u, v);
            }
    }
    if (invert) {
        uint64_t n_inv = f_inv((uint64_t)n % GL_P);
        for (int64_t i = 0; i < n; ++i) a[i] = f_mul(a[i], n_inv);
    }
}
static uint64_t* make_tw(int64_t n, int invert) {
    int64_t h = n / 2 > 0 ? n / 2 : 1;
    uint64_t* tw = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)h);
    uint64_t w = or_root_of_unity((uint64_t)n);
    if (invert) w = f_inv(w);
    uint64_t c = 1;
    for (int64_t k = 0; k < h; ++k) { tw[k] = c; c = f_mul(c, w); }
    return tw;
}

/* Batched in-place NTT over m rows: prover/cuda_primitives.py:388-409. */
void or_ntt_batched(uint64_t* rows, int64_t m, int64_t n, int invert) {
    uint64_t* tw = make_tw(n, invert);
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < m; ++r) ntt_table(rows + r * n, n, tw, invert);
    free(tw);
}

/* Evaluation-domain fold of row products: out[j] = sum_i w[i] * NTT_n(A_i|0)[j] * NTT_n(B_i|0)[j],
 * rows selected by ia/ib (NULL = identity), w NULL = ones.  Follows the fused branch of
 * _compute_q_lin_inner_chunk (prover/core.py:1892-1911) and the per-chunk weighted_eval of
 * compute_p_0_streaming (prover/core.py:2166-2181). */
void or_fold_products_eval(const uint64_t* A, int64_t rows_a, const uint64_t* B, int64_t rows_b, int64_t k,
                           const int64_t* ia, const int64_t* ib, const uint64_t* w, int64_t T,
                           int64_t n, uint64_t* out) {
    uint64_t* ea = (uint64_t*)calloc((size_t)(rows_a * n), 8);
    uint64_t* eb = (uint64_t*)calloc((size_t)(rows_b * n), 8);
    for (int64_t r = 0; r < rows_a; ++r) memcpy(ea + r * n, A + r * k, (size_t)k * 8);
    for (int64_t r = 0; r < rows_b; ++r) memcpy(eb + r * n, B + r * k, (size_t)k * 8);
    or_ntt_batched(ea, rows_a, n, 0);
    or_ntt_batched(eb, rows_b, n, 0);
    #pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < n; ++j) {
        uint64_t acc = 0;
        for (int64_t i = 0; i < T; ++i) {
            uint64_t a = ea[(ia ? ia[i] : i) * n + j], b = eb[(ib ? ib[i] : i) * n + j];
            uint64_t t = f_mul(a, b);
            if (w) t = f_mul(t, w[i]);
            acc = f_add(acc, t);
        }
        out[j] = acc;
    }
    free(ea); free(eb);
}

/* ------------------------------------------------------------------ */
/* RS encode: prover/core.py:721-743,746-802 (encode_messages /        */
/* _coset_encode_codewords) and layergkr/gpu.py:141-203.               */
/* padded: (m, K) message values at the K-th roots of unity (pad       */
/* already filled).  polys (m,K) <- iNTT_K; codes (m,N) <- NTT_N of    */
/* 7^l * poly[l] zero-extended.  Either output may be NULL.            */
/* ------------------------------------------------------------------ */
void or_encode_rows(const uint64_t* padded, int64_t m, int64_t K, int64_t N,
                    uint64_t* polys, uint64_t* codes) {
    uint64_t* twk = make_tw(K, 1);
    uint64_t* twn = make_tw(N, 0);
    uint64_t* gpow = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)K);
    uint64_t c = 1;
    for (int64_t l = 0; l < K; ++l) { gpow[l] = c; c = f_mul(c, 7); }
    #pragma omp parallel
    {
        uint64_t* poly = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)K);
        uint64_t* ext = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)N);
        #pragma omp for schedule(static)
        for (int64_t r = 0; r < m; ++r) {
            memcpy(poly, padded + r * K, sizeof(uint64_t) * (size_t)K);
            ntt_table(poly, K, twk, 1);
            if (polys) memcpy(polys + r * K, poly, sizeof(uint64_t) * (size_t)K);
            if (codes) {
                for (int64_t l = 0; l < K; ++l) ext[l] = f_mul(poly[l], gpow[l]);
                memset(ext + K, 0, sizeof(uint64_t) * (size_t)(N - K));
                ntt_table(ext, N, twn, 0);
                memcpy(codes + r * N, ext, sizeof(uint64_t) * (size_t)N);
            }
        }
        free(poly); free(ext);
    }
    free(twk); free(twn); free(gpow);
}

/* ------------------------------------------------------------------ */
/* BLAKE3 (published algorithm; the reference links the `blake3`       */
/* package 1.0.8 on the host and restates it in                        */
/* prover/kernels/blake3_compress.cuh:77-117, blake3_hash.cuh:124-202) */
/* ------------------------------------------------------------------ */
static const uint32_t B3_IV[8] = {0x6A09E667u, 0xBB67AE85u, 0x3C6EF372u, 0xA54FF53Au,
                                  0x510E527Fu, 0x9B05688Cu, 0x1F83D9ABu, 0x5BE0CD19u};
static const uint8_t B3_PERM[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};
enum { B3_CHUNK_START = 1, B3_CHUNK_END = 2, B3_PARENT = 4, B3_ROOT = 8 };

static inline uint32_t rotr32(uint32_t x, int n) { return (x >> n) | (x << (32 - n)); }
#define B3_G(a, b, c, d, mx, my) do { \
    v[a] = v[a] + v[b] + (mx); v[d] = rotr32(v[d] ^ v[a], 16); \
    v[c] = v[c] + v[d];        v[b] = rotr32(v[b] ^ v[c], 12); \
    v[a] = v[a] + v[b] + (my); v[d] = rotr32(v[d] ^ v[a], 8);  \
    v[c] = v[c] + v[d];        v[b] = rotr32(v[b] ^ v[c], 7); } while (0)

static void b3_compress(const uint32_t cv[8], const uint32_t msg[16], uint64_t counter,
                        uint32_t block_len, uint32_t flags, uint32_t out[8]) {
    uint32_t v[16], m[16], t[16];
    for (int i = 0; i < 8; ++i) v[i] = cv[i];
    for (int i = 0; i < 4; ++i) v[8 + i] = B3_IV[i];
    v[12] = (uint32_t)counter; v[13] = (uint32_t)(counter >> 32);
    v[14] = block_len; v[15] = flags;
    memcpy(m, msg, sizeof(m));
    for (int r = 0; r < 7; ++r) {
        B3_G(0, 4, 8, 12, m[0], m[1]);   B3_G(1, 5, 9, 13, m[2], m[3]);
        B3_G(2, 6, 10, 14, m[4], m[5]);  B3_G(3, 7, 11, 15, m[6], m[7]);
        B3_G(0, 5, 10, 15, m[8], m[9]);  B3_G(1, 6, 11, 12, m[10], m[11]);
        B3_G(2, 7, 8, 13, m[12], m[13]); B3_G(3, 4, 9, 14, m[14], m[15]);
        for (int i = 0; i < 16; ++i) t[i] = m[B3_PERM[i]];
        memcpy(m, t, sizeof(m));
    }
    for (int i = 0; i < 8; ++i) out[i] = v[i] ^ v[i + 8];
}

static void b3_load_block(const uint8_t* p, size_t len, uint32_t msg[16]) {
    uint8_t buf[64];
    memset(buf, 0, 64);
    if (len) memcpy(buf, p, len);
    for (int i = 0; i < 16; ++i)
        msg[i] = (uint32_t)buf[4 * i] | ((uint32_t)buf[4 * i + 1] << 8) |
                 ((uint32_t)buf[4 * i + 2] << 16) | ((uint32_t)buf[4 * i + 3] << 24);
}

/* chaining value of one chunk (<= 1024 bytes); root_flag applies to its last block */
static void b3_chunk_cv(const uint8_t* p, size_t len, uint64_t counter, uint32_t root_flag,
                        uint32_t out[8]) {
    uint32_t cv[8], msg[16];
    memcpy(cv, B3_IV, sizeof(cv));
    size_t nblocks = len == 0 ? 1 : (len + 63) / 64;
    for (size_t b = 0; b < nblocks; ++b) {
        size_t off = b * 64, bl = len - off < 64 ? len - off : 64;
        if (len == 0) bl = 0;
        uint32_t flags = 0;
        if (b == 0) flags |= B3_CHUNK_START;
        if (b == nblocks - 1) flags |= B3_CHUNK_END | root_flag;
        b3_load_block(p + off, bl, msg);
        b3_compress(cv, msg, counter, (uint32_t)bl, flags, cv);
    }
    memcpy(out, cv, sizeof(cv));
}

static void b3_parent(const uint32_t l[8], const uint32_t r[8], uint32_t root_flag, uint32_t out[8]) {
    uint32_t msg[16];
    memcpy(msg, l, 32); memcpy(msg + 8, r, 32);
    b3_compress(B3_IV, msg, 0, 64, B3_PARENT | root_flag, out);
}

/* subtree over chunks [c0, c0+n) of the input; n >= 1 */
static void b3_subtree_off(const uint8_t* p, size_t len, uint64_t c0, uint64_t n, int is_root,
                           uint64_t ctr_off, uint32_t out[8]) {
    if (n == 1) {
        size_t off = (size_t)c0 * 1024, l = len - off < 1024 ? len - off : 1024;
        if (len == 0) l = 0;
        b3_chunk_cv(p + off, l, c0 + ctr_off, is_root ? B3_ROOT : 0, out);
        return;
    }
    uint64_t left = 1;
    while (left * 2 < n) left *= 2;
    uint32_t a[8], b[8];
    b3_subtree_off(p, len, c0, left, 0, ctr_off, a);
    b3_subtree_off(p, len, c0 + left, n - left, 0, ctr_off, b);
    b3_parent(a, b, is_root ? B3_ROOT : 0, out);
}
static void b3_subtree(const uint8_t* p, size_t len, uint64_t c0, uint64_t n, int is_root, uint32_t out[8]) {
    b3_subtree_off(p, len, c0, n, is_root, 0, out);
}

void or_blake3(const uint8_t* data, int64_t len, uint8_t out[32]) {
    uint64_t nchunks = len == 0 ? 1 : ((uint64_t)len + 1023) / 1024;
    uint32_t h[8];
    b3_subtree(data, (size_t)len, 0, nchunks, 1, h);
    for (int i = 0; i < 8; ++i) {
        out[4 * i] = (uint8_t)h[i]; out[4 * i + 1] = (uint8_t)(h[i] >> 8);
        out[4 * i + 2] = (uint8_t)(h[i] >> 16); out[4 * i + 3] = (uint8_t)(h[i] >> 24);
    }
}

/* ------------------------------------------------------------------ */
/* Column leaves: leaf j = BLAKE3 of le8(mat[0,j]) || le8(mat[1,j]) …  */
/* prover/protocol.py:100-104, prover/kernels/blake3_columns.cuh:47-174 */
/* ------------------------------------------------------------------ */
void or_hash_columns(const uint64_t* mat, int64_t m, int64_t ncols, uint8_t* digests) {
    #pragma omp parallel
    {
        uint8_t* col = (uint8_t*)malloc((size_t)(m > 0 ? m : 1) * 8);
        #pragma omp for schedule(static)
        for (int64_t j = 0; j < ncols; ++j) {
            for (int64_t i = 0; i < m; ++i) {
                uint64_t v = mat[i * ncols + j];
                for (int b = 0; b < 8; ++b) col[i * 8 + b] = (uint8_t)(v >> (8 * b));
            }
            or_blake3(col, m * 8, digests + j * 32);
        }
        free(col);
    }
}

/* ------------------------------------------------------------------ */
/* Merkle: parent = BLAKE3(left || right) as a 64-byte message; an odd  */
/* level pairs its last node with itself.                               */
/* prover/cuda_primitives.py:1388-1401, prover/kernels/merkle.cuh:18-37, */
/* layergkr/rs.py:135-144.                                              */
/* levels_out receives every level back to back (leaves first); returns */
/* the number of levels.  Total nodes written = or_merkle_total_nodes.  */
/* ------------------------------------------------------------------ */
int64_t or_merkle_total_nodes(int64_t n) {
    int64_t t = n;
    while (n > 1) { n = (n + 1) / 2; t += n; }
    return t;
}
int or_merkle_levels(const uint8_t* leaves, int64_t n, uint8_t* levels_out) {
    memcpy(levels_out, leaves, (size_t)n * 32);
    uint8_t* cur = levels_out;
    int nl = 1;
    while (n > 1) {
        int64_t nn = (n + 1) / 2;
        uint8_t* nxt = cur + n * 32;
        #pragma omp parallel for schedule(static)
        for (int64_t i = 0; i < nn; ++i) {
            uint8_t buf[64];
            memcpy(buf, cur + (2 * i) * 32, 32);
            memcpy(buf + 32, cur + ((2 * i + 1 < n) ? (2 * i + 1) : (2 * i)) * 32, 32);
            or_blake3(buf, 64, nxt + i * 32);
        }
        cur = nxt; n = nn; ++nl;
    }
    return nl;
}

/* ------------------------------------------------------------------ */
/* ZK pad PRG: out[r,k] = u64_le(BLAKE3(seed32 || (row_off+r)_le8 ||   */
/* k_le8)[0:8]) % P.  prover/cuda_primitives.py:877-903,1262-1265.     */
/* ------------------------------------------------------------------ */
void or_row_prg_indexed(const uint8_t seed[32], const uint64_t* rows, int64_t n_rows,
                        int64_t slack, uint64_t* out) {
    #pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < n_rows; ++r) {
        uint8_t in[48], d[32];
        memcpy(in, seed, 32);
        for (int b = 0; b < 8; ++b) in[32 + b] = (uint8_t)(rows[r] >> (8 * b));
        for (int64_t k = 0; k < slack; ++k) {
            for (int b = 0; b < 8; ++b) in[40 + b] = (uint8_t)((uint64_t)k >> (8 * b));
            or_blake3(in, 48, d);
            uint64_t raw = 0;
            for (int b = 0; b < 8; ++b) raw |= (uint64_t)d[b] << (8 * b);
            out[r * slack + k] = raw % GL_P;
        }
    }
}
void or_row_prg(const uint8_t seed[32], int64_t row_off, int64_t n_rows, int64_t slack, uint64_t* out) {
    uint64_t* rows = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)(n_rows > 0 ? n_rows : 1));
    for (int64_t r = 0; r < n_rows; ++r) rows[r] = (uint64_t)(row_off + r);
    or_row_prg_indexed(seed, rows, n_rows, slack, out);
    free(rows);
}

/* ------------------------------------------------------------------ */
/* Challenge PRF: int(BLAKE3(seed32 || label || cid_le8)[:16], LE) % P */
/* prover/protocol.py:126-133, prover/kernels/gl_spmv.cuh:51-66.       */
/* ------------------------------------------------------------------ */
uint64_t or_challenge(const uint8_t seed[32], const uint8_t* label, int label_len, uint64_t cid) {
    uint8_t in[64], d[32];
    memcpy(in, seed, 32);
    memcpy(in + 32, label, (size_t)label_len);
    for (int b = 0; b < 8; ++b) in[32 + label_len + b] = (uint8_t)(cid >> (8 * b));
    or_blake3(in, 40 + label_len, d);
    u128 v = 0;
    for (int b = 15; b >= 0; --b) v = (v << 8) | d[b];
    return (uint64_t)(v % GL_P);
}

/* ------------------------------------------------------------------ */
/* K-quant super-block -> field.  Arithmetic of gguf-py 0.19.0          */
/* gguf/quants.py (Q4_K / Q5_K / Q6_K dequantize_blocks: fp32 multiply   */
/* then fp32 subtract, separately rounded) followed by                  */
/* prover/loader.py:52-70 (round-half-even of double(v)*S, negative      */
/* values map to P-|v|); CUDA twin prover/kquant_cuda.py:42-111.        */
/* qtype: 4 = Q4_K (144 B), 5 = Q5_K (176 B), 6 = Q6_K (210 B).         */
/* ------------------------------------------------------------------ */
static float half_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h >> 15) << 31, exp = (h >> 10) & 0x1F, man = h & 0x3FF, bits;
    if (exp == 0) {
        if (man == 0) bits = sign;
        else {
            int e = -1;
            do { man <<= 1; ++e; } while (!(man & 0x400));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3FF) << 13);
        }
    } else if (exp == 31) bits = sign | 0x7F800000u | (man << 13);
    else bits = sign | ((exp + 112) << 23) | (man << 13);
    float f; memcpy(&f, &bits, 4); return f;
}
static inline uint64_t lift(float v, double S) {
    long long ll = llrint((double)v * S);      /* default rounding mode = half-to-even */
    return ll >= 0 ? (uint64_t)ll : GL_P - (uint64_t)(-ll);
}
static inline void scale_min_k4(const uint8_t* s, int j, uint32_t* sc, uint32_t* mn) {
    if (j < 4) { *sc = s[j] & 63; *mn = s[j + 4] & 63; }
    else { *sc = (s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4); *mn = (s[j + 4] >> 4) | ((s[j] >> 6) << 4); }
}
int or_kquant_to_field(const uint8_t* raw, int64_t n_blocks, int qtype, double S, uint64_t* out) {
    if (qtype != 4 && qtype != 5 && qtype != 6) return 1;
    #pragma omp parallel for schedule(static)
    for (int64_t b = 0; b < n_blocks; ++b) {
        uint64_t* o = out + b * 256;
        if (qtype == 4 || qtype == 5) {
            const uint8_t* p = raw + b * (qtype == 4 ? 144 : 176);
            uint16_t hd, hm; memcpy(&hd, p, 2); memcpy(&hm, p + 2, 2);
            float d = half_to_float(hd), dmin = half_to_float(hm);
            const uint8_t* qh = p + 16;
            const uint8_t* qs = p + (qtype == 4 ? 16 : 48);
            for (int e = 0; e < 256; ++e) {
                uint32_t sc, mn; scale_min_k4(p + 4, e >> 5, &sc, &mn);
                int q = (qs[(e >> 6) * 32 + (e & 31)] >> (4 * ((e >> 5) & 1))) & 0xF;
                if (qtype == 5) q |= ((qh[e & 31] >> (e >> 5)) & 1) << 4;
                float ds = d * (float)sc;
                float dm = dmin * (float)mn;
                float t = ds * (float)q;
                float v = t - dm;
                o[e] = lift(v, S);
            }
        } else {
            const uint8_t* p = raw + b * 210;
            const uint8_t* ql = p; const uint8_t* qh = p + 128;
            const int8_t* sc = (const int8_t*)(p + 192);
            uint16_t hd; memcpy(&hd, p + 208, 2);
            float d = half_to_float(hd);
            for (int e = 0; e < 256; ++e) {
                int lo = (ql[(e >> 7) * 64 + (e & 63)] >> (4 * ((e >> 6) & 1))) & 0xF;
                int hi = (qh[(e >> 7) * 32 + (e & 31)] >> (2 * ((e >> 5) & 3))) & 3;
                int q = (int)(int8_t)(lo | (hi << 4)) - 32;
                float ds = d * (float)sc[e >> 4];
                float v = ds * (float)q;
                o[e] = lift(v, S);
            }
        }
    }
    return 0;
}

/* signed integer -> field (prover/loader.py:52-58) */
void or_signed_to_field(const int64_t* v, int64_t n, uint64_t* out) {
    for (int64_t i = 0; i < n; ++i) out[i] = v[i] >= 0 ? (uint64_t)v[i] : GL_P - (uint64_t)(-v[i]);
}

/* ------------------------------------------------------------------ */
/* Sumcheck of a sum of products of multilinear tables.                 */
/* layergkr/sumcheck.py:153-226 (prove_terms, pure-Python branch) and   */
/* :51-54 (_fold).  MSB variable first; per round samples g(x) for       */
/* x = 0..deg, then every table is folded with the round challenge.     */
/* tables: n_tables contiguous arrays of `size` (a power of two);        */
/* term t = coefs[t] * prod_{j<term_nfac[t]} tables[term_fac[t*max_fac+j]] */
/* samples_out: n_rounds * (deg+1) values; finals_out: n_tables values.  */
/* No mask is applied (mu = 0): the mask only shifts the scalar samples. */
/* ------------------------------------------------------------------ */
int or_sumcheck(const uint64_t* tables, int n_tables, int64_t size,
                int n_terms, const uint64_t* coefs, const int* term_nfac,
                const int* term_fac, int max_fac,
                const uint64_t* challenges, uint64_t* claim_out,
                uint64_t* samples_out, uint64_t* finals_out) {
    if (size <= 0 || (size & (size - 1))) return 1;
    int n_rounds = 0; while (((int64_t)1 << n_rounds) < size) ++n_rounds;
    int deg = 0;
    for (int t = 0; t < n_terms; ++t) if (term_nfac[t] > deg) deg = term_nfac[t];
    uint64_t* cur = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)size * (size_t)n_tables);
    memcpy(cur, tables, sizeof(uint64_t) * (size_t)size * (size_t)n_tables);

    uint64_t claim = 0;
    #pragma omp parallel
    {
        uint64_t local = 0;
        #pragma omp for schedule(static) nowait
        for (int64_t i = 0; i < size; ++i)
            for (int t = 0; t < n_terms; ++t) {
                uint64_t prod = coefs[t] % GL_P;
                for (int j = 0; j < term_nfac[t]; ++j)
                    prod = f_mul(prod, cur[(int64_t)term_fac[t * max_fac + j] * size + i]);
                local = f_add(local, prod);
            }
        #pragma omp critical
        claim = f_add(claim, local);
    }
    *claim_out = claim;

    int64_t len = size;
    for (int rnd = 0; rnd < n_rounds; ++rnd) {
        int64_t half = len / 2;
        for (int x = 0; x <= deg; ++x) {
            uint64_t acc = 0;
            #pragma omp parallel
            {
                uint64_t local = 0;
                #pragma omp for schedule(static) nowait
                for (int64_t i = 0; i < half; ++i)
                    for (int t = 0; t < n_terms; ++t) {
                        uint64_t prod = coefs[t] % GL_P;
                        for (int j = 0; j < term_nfac[t]; ++j) {
                            const uint64_t* f = cur + (int64_t)term_fac[t * max_fac + j] * size;
                            uint64_t fx = f_add(f[i], f_mul((uint64_t)x, f_sub(f[half + i], f[i])));
                            prod = f_mul(prod, fx);
                        }
                        local = f_add(local, prod);
                    }
                #pragma omp critical
                acc = f_add(acc, local);
            }
            samples_out[rnd * (deg + 1) + x] = acc;
        }
        uint64_t r = challenges[rnd] % GL_P;
        for (int k = 0; k < n_tables; ++k) {
            uint64_t* f = cur + (int64_t)k * size;
            #pragma omp parallel for schedule(static)
            for (int64_t i = 0; i < half; ++i)
                f[i] = f_add(f[i], f_mul(r, f_sub(f[half + i], f[i])));
        }
        len = half;
    }
    if (finals_out) for (int k = 0; k < n_tables; ++k) finals_out[k] = cur[(int64_t)k * size];
    free(cur);
    return 0;
}

/* Full commit of a row batch: encode -> column leaves -> Merkle root.
 * Composition used by the timed CPU baseline (prover/core.py:746-802 followed by
 * prover/cuda_primitives.py:796-808 and :1388-1401). */
void or_commit_rows(const uint64_t* padded, int64_t m, int64_t K, int64_t N, uint8_t root[32]) {
    uint64_t* codes = (uint64_t*)malloc(sizeof(uint64_t) * (size_t)m * (size_t)N);
    uint8_t* dig = (uint8_t*)malloc((size_t)N * 32);
    uint8_t* lv = (uint8_t*)malloc((size_t)or_merkle_total_nodes(N) * 32);
    or_encode_rows(padded, m, K, N, NULL, codes);
    or_hash_columns(codes, m, N, dig);
    or_merkle_levels(dig, N, lv);
    memcpy(root, lv + (or_merkle_total_nodes(N) - 1) * 32, 32);
    free(codes); free(dig); free(lv);
}

/* ------------------------------------------------------------------ */
/* Sharded column hash (no counterpart in the reference; BLAKE3's tree  */
/* rule applied to a row range).  Non-root chaining value of the        */
/* complete sub-tree formed by the chunks of `mat` (n_rows rows =       */
/* 2^level chunks, only the last may be short), whose first chunk has   */
/* global index first_chunk.  out: (ncols, 32).                         */
/* ------------------------------------------------------------------ */
void or_hash_subtree(const uint64_t* mat, int64_t n_rows, int64_t ncols, int64_t first_chunk, uint8_t* out) {
    uint64_t nchunks = ((uint64_t)n_rows + 127) / 128;
    #pragma omp parallel
    {
        uint8_t* col = (uint8_t*)malloc((size_t)n_rows * 8);
        #pragma omp for schedule(static)
        for (int64_t j = 0; j < ncols; ++j) {
            for (int64_t i = 0; i < n_rows; ++i) {
                uint64_t v = mat[i * ncols + j];
                for (int b = 0; b < 8; ++b) col[i * 8 + b] = (uint8_t)(v >> (8 * b));
            }
            uint32_t h[8];
            b3_subtree_off(col, (size_t)n_rows * 8, 0, nchunks, 0, (uint64_t)first_chunk, h);
            for (int i = 0; i < 8; ++i)
                for (int b = 0; b < 4; ++b) out[j * 32 + 4 * i + b] = (uint8_t)(h[i] >> (8 * b));
        }
        free(col);
    }
}

/* Fold gathered sub-tree values (nblocks, ncols, 32), block sizes 2^levels[i] chunks, left to  */
/* right, into the column digests: equal-sized neighbours merge as parents, the last block is   */
/* not merged eagerly, the remaining ones fold right to left and the last merge is the root.    */
int or_hash_merge_subtrees(const uint8_t* cvs, const int32_t* levels, int nblocks, int64_t ncols, uint8_t* out) {
    if (nblocks < 2) return 1;
    #pragma omp parallel for schedule(static)
    for (int64_t j = 0; j < ncols; ++j) {
        uint32_t st[64][8]; int lv[64]; int sp = 0;
        for (int i = 0; i < nblocks; ++i) {
            const uint8_t* p = cvs + ((int64_t)i * ncols + j) * 32;
            for (int w = 0; w < 8; ++w)
                st[sp][w] = (uint32_t)p[4 * w] | ((uint32_t)p[4 * w + 1] << 8) | ((uint32_t)p[4 * w + 2] << 16) | ((uint32_t)p[4 * w + 3] << 24);
            lv[sp++] = levels[i];
            if (i == nblocks - 1) break;
            while (sp >= 2 && lv[sp - 1] == lv[sp - 2]) {
                uint32_t o[8]; b3_parent(st[sp - 2], st[sp - 1], 0, o);
                --sp; memcpy(st[sp - 1], o, 32); ++lv[sp - 1];
            }
        }
        while (sp >= 2) {
            uint32_t o[8]; b3_parent(st[sp - 2], st[sp - 1], sp == 2 ? B3_ROOT : 0, o);
            --sp; memcpy(st[sp - 1], o, 32);
        }
        for (int i = 0; i < 8; ++i)
            for (int b = 0; b < 4; ++b) out[j * 32 + 4 * i + b] = (uint8_t)(st[0][i] >> (8 * b));
    }
    return 0;
}

/* Thread count of the OpenMP loops above: sets it when n > 0 (an OMP_NUM_THREADS value inherited  */
/* from a launcher is read once, at load time, and would otherwise stick) and returns the count in */
/* effect.                                                                                         */
int or_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
    return omp_get_max_threads();
#else
    (void)n;
    return 1;
#endif
}
