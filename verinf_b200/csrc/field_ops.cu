// Elementwise Goldilocks ops and the non-hot-path exports of the reference module
// (poly_eval, dense/sparse mat-vec, lookup multiplicities, q_lin band interpreters).
//
// Replaces k_gl_mul/add/sub/pow (prover/cuda_primitives.py:208-223), k_neg / k_axpy_inplace
// (prover/kernels/gl_extras.cuh) and k_matmul / k_matvec (prover/kernels/gl_matmul.cuh); the
// matmul, thin-matmul, matvec and product-column-sum kernels here are new (unreduced 160-bit
// accumulation).
//
// Ported from the reference, not redesigned (none of them is on the hot path; they exist so that
// every name the reference's callers import works): k_poly_eval and k_lookup follow
// prover/kernels/gl_extras.cuh:93-149 with 64-bit indices, k_spmv merges the two kernels of
// prover/kernels/gl_spmv.cuh:25-100, and k_band merges the five descriptor interpreters
// k_interp_band / k_band_causal_id / k_band_causal_c2 / k_band_embed / k_band_rope_x of
// prover/cuda_primitives.py:605-734 behind a `kind` switch, keeping their arithmetic and names.
#include "../../include/verinf_b200.h"
#include "blake3.cuh"
#include "common.cuh"
#include "gl.cuh"

namespace {

using vgl::add;
using vgl::mul;
using vgl::sub;

constexpr int BLOCK = 256;
inline unsigned grid_for(int64_t n, int per_thread = 1) {
    int64_t g = (n + (int64_t)BLOCK * per_thread - 1) / ((int64_t)BLOCK * per_thread);
    int64_t cap = 148 * 16;   // grid-stride loops: a few waves over the 148 SMs
    return (unsigned)(g < cap ? (g > 0 ? g : 1) : cap);
}

template <int OP>
__device__ __forceinline__ uint64_t apply(uint64_t a, uint64_t b) {
    return OP == 0 ? mul(a, b) : OP == 1 ? add(a, b) : sub(a, b);
}

// operands may alias the output (no __restrict__)
template <int OP>
__global__ void __launch_bounds__(BLOCK) k_binary_alias(const uint64_t* a, const uint64_t* b, uint64_t* out, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * BLOCK;
    for (int64_t i = (int64_t)blockIdx.x * BLOCK + threadIdx.x; i < n; i += stride) out[i] = apply<OP>(a[i], b[i]);
}
template <int OP>
__global__ void __launch_bounds__(BLOCK) k_binary_bcast(const uint64_t* a, const uint64_t* __restrict__ b, int64_t nb,
                                                        uint64_t* out, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * BLOCK;
    for (int64_t i = (int64_t)blockIdx.x * BLOCK + threadIdx.x; i < n; i += stride) out[i] = apply<OP>(a[i], __ldg(b + i % nb));
}
__global__ void __launch_bounds__(BLOCK) k_neg(const uint64_t* a, uint64_t* out, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * BLOCK;
    for (int64_t i = (int64_t)blockIdx.x * BLOCK + threadIdx.x; i < n; i += stride) out[i] = vgl::neg(a[i]);
}
__global__ void __launch_bounds__(BLOCK) k_pow(const uint64_t* a, uint64_t e, uint64_t* out, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * BLOCK;
    for (int64_t i = (int64_t)blockIdx.x * BLOCK + threadIdx.x; i < n; i += stride) out[i] = vgl::pow(a[i], e);
}
__global__ void __launch_bounds__(BLOCK) k_axpy(uint64_t* y, uint64_t alpha, const uint64_t* x, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * BLOCK;
    for (int64_t i = (int64_t)blockIdx.x * BLOCK + threadIdx.x; i < n; i += stride) y[i] = add(y[i], mul(alpha, x[i]));
}

__global__ void k_poly_eval(const uint64_t* __restrict__ coeffs, int64_t m, int64_t d,
                            const uint64_t* __restrict__ points, int64_t k, uint64_t* __restrict__ out) {
    const int64_t p = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t r = (int64_t)blockIdx.y * blockDim.y + threadIdx.y;
    if (p >= k || r >= m) return;
    const uint64_t x = points[p];
    const uint64_t* row = coeffs + r * d;
    uint64_t acc = 0;
    for (int64_t i = d - 1; i >= 0; --i) acc = add(mul(acc, x), row[i]);
    out[r * k + p] = acc;
}

using vgl::mac160;
using vgl::reduce160;

// C = A.B mod p with lazily reduced accumulation.
// CTA tile 64 x 32 outputs, k in slices of 32, 256 threads, 4 x 2 outputs per thread.  The
// 128-bit products are summed unreduced in five 32-bit limbs per output (8 multiply-adds with
// carry on the FMA pipe + 5 carry propagations on the ALU pipe per product, no modular
// reduction); the fifth limb counts the carries out of 2^128, so any k < 2^32 fits, and the
// 160-bit sum is reduced mod p once at the end (2^128 = -2^32).  Tiles arrive through cp.async into a
// double buffer when they are whole and 16-byte aligned, else through guarded loads with zero
// fill.  Measured on B200 (1000 x 4096 x 11008): 41 ms = 1.09 T multiply-adds/s, the heavy half
// of the FMA pipe 93 % busy (32-bit multiply-adds issue at 4 clocks per warp there); summing
// 22-bit-limb products with wide multiply-adds instead (no carries) took 50 ms because a wide
// multiply-add with a 64-bit addend is not one instruction on this architecture, and the
// reduce-every-product kernel this replaces 68 ms.
#ifndef VI_MM_MINB
#define VI_MM_MINB 2      // resident CTAs per SM asked of the compiler (128 registers per thread)
#endif
constexpr int MM_TM = 64, MM_TN = 32, MM_TK = 32, MM_AS = 34;   // MM_AS: row stride of the A tile (u64)
constexpr int MM_SMEM = 2 * (MM_TM * MM_AS + MM_TK * MM_TN) * 8;

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__global__ void __launch_bounds__(256, VI_MM_MINB) k_matmul(const uint64_t* __restrict__ A, const uint64_t* __restrict__ B,
                                                   uint64_t* __restrict__ C, int64_t m, int64_t k, int64_t n) {
    extern __shared__ __align__(16) uint64_t mm_smem[];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int64_t row0 = (int64_t)blockIdx.y * MM_TM, col0 = (int64_t)blockIdx.x * MM_TN;
    const int64_t nslices = (k + MM_TK - 1) / MM_TK;
    const bool a_fast = (k % 2 == 0) && (((uintptr_t)A) % 16 == 0) && row0 + MM_TM <= m;
    const bool b_fast = (n % 2 == 0) && (((uintptr_t)B) % 16 == 0) && col0 + MM_TN <= n;

    auto load_slice = [&](int64_t s, int buf) {
        uint64_t* sa = mm_smem + buf * (MM_TM * MM_AS + MM_TK * MM_TN);
        uint64_t* sb = sa + MM_TM * MM_AS;
        const int64_t l0 = s * MM_TK;
        const bool whole_k = l0 + MM_TK <= k;
        if (a_fast && whole_k) {
            // 64 rows x 16 chunks of 16 bytes: 4 per thread
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                int e = tid + 256 * q, r = e >> 4, c = e & 15;
                cp_async16(sa + r * MM_AS + 2 * c, A + (row0 + r) * k + l0 + 2 * c);
            }
        } else {
#pragma unroll
            for (int q = 0; q < 8; ++q) {
                int e = tid + 256 * q, r = e >> 5, l = e & 31;
                sa[r * MM_AS + l] = (row0 + r < m && l0 + l < k) ? A[(row0 + r) * k + l0 + l] : 0;
            }
        }
        if (b_fast && whole_k) {
            // 32 rows x 16 chunks of 16 bytes: 2 per thread
#pragma unroll
            for (int q = 0; q < 2; ++q) {
                int e = tid + 256 * q, l = e >> 4, c = e & 15;
                cp_async16(sb + l * MM_TN + 2 * c, B + (l0 + l) * n + col0 + 2 * c);
            }
        } else {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                int e = tid + 256 * q, l = e >> 5, c = e & 31;
                sb[l * MM_TN + c] = (l0 + l < k && col0 + c < n) ? B[(l0 + l) * n + col0 + c] : 0;
            }
        }
        cp_async_commit();
    };

    uint32_t acc[4][2][5];
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
            for (int t = 0; t < 5; ++t) acc[q][c][t] = 0;

    if (nslices > 0) load_slice(0, 0);
    for (int64_t s = 0; s < nslices; ++s) {
        const int buf = (int)(s & 1);
        if (s + 1 < nslices) { load_slice(s + 1, buf ^ 1); cp_async_wait<1>(); }
        else cp_async_wait<0>();
        __syncthreads();
        const uint64_t* sa = mm_smem + buf * (MM_TM * MM_AS + MM_TK * MM_TN);
        const uint64_t* sb = sa + MM_TM * MM_AS;
#pragma unroll 1
        for (int l = 0; l < MM_TK; ++l) {
            const uint4 bb = *reinterpret_cast<const uint4*>(sb + l * MM_TN + 2 * tx);
            const uint64_t bv[2] = {vgl::pack(bb.x, bb.y), vgl::pack(bb.z, bb.w)};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const uint64_t av = sa[(ty * 4 + q) * MM_AS + l];
#pragma unroll
                for (int c = 0; c < 2; ++c) mac160(acc[q][c], av, bv[c]);
            }
        }
        __syncthreads();
    }
#pragma unroll
    for (int q = 0; q < 4; ++q)
#pragma unroll
        for (int c = 0; c < 2; ++c) {
            const int64_t r = row0 + ty * 4 + q, cc = col0 + 2 * tx + c;
            if (r < m && cc < n) C[r * n + cc] = reduce160(acc[q][c]);
        }
}

// Thin product: M <= 4 rows of A against a tall B (k x n), out[mi][j] = sum_i A[mi][i] B[i][j].
// This is the random linear combination of matrix rows (q_irs accumulation, prover/core.py:1351-1379;
// combine_t, layergkr/gpu.py:301-308), which must stream B once: a CTA owns 32 columns, its 8 row
// lanes take the rows i = lane, lane + 8, ... (every warp reads 256 contiguous bytes per row) with
// unreduced 160-bit sums, and the 8 partial sums meet in shared memory.
template <int M>
__global__ void __launch_bounds__(256) k_matmul_thin(const uint64_t* __restrict__ A, const uint64_t* __restrict__ B,
                                                     uint64_t* __restrict__ C, int64_t k, int64_t n) {
    __shared__ uint64_t red[8][M][32];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t j = (int64_t)blockIdx.x * 32 + tx;
    uint32_t acc[M][5];
#pragma unroll
    for (int mi = 0; mi < M; ++mi)
#pragma unroll
        for (int l = 0; l < 5; ++l) acc[mi][l] = 0;
    if (j < n) {
        for (int64_t i = ty; i < k; i += 8) {
            const uint64_t b = B[i * n + j];
#pragma unroll
            for (int mi = 0; mi < M; ++mi) mac160(acc[mi], __ldg(A + mi * k + i), b);
        }
    }
#pragma unroll
    for (int mi = 0; mi < M; ++mi) red[ty][mi][tx] = reduce160(acc[mi]);
    __syncthreads();
    if (ty < M && j < n) {
        uint64_t v = 0;
#pragma unroll
        for (int r = 0; r < 8; ++r) v = add(v, red[r][ty][tx]);
        C[(int64_t)ty * n + j] = v;
    }
}

// Weighted product column sum: part[s][j] = sum over the rows i of split s of
// w[i] * EA[ia[i]][j] * EB[ib[i]][j].  One thread per column (coalesced rows), products summed
// unreduced in five 32-bit limbs, one reduction per thread at the end; k_colsum_finish adds the
// row splits (and the previous value when accumulating).
__global__ void __launch_bounds__(256) k_product_colsum(const uint64_t* __restrict__ EA, const uint64_t* __restrict__ EB,
                                                        int64_t n, const int64_t* __restrict__ ia,
                                                        const int64_t* __restrict__ ib, const uint64_t* __restrict__ w,
                                                        int64_t T, int64_t rows_per_split, uint64_t* __restrict__ part) {
    const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    const int64_t i0 = (int64_t)blockIdx.y * rows_per_split;
    const int64_t i1 = i0 + rows_per_split < T ? i0 + rows_per_split : T;
    uint32_t x[5] = {0, 0, 0, 0, 0};
    for (int64_t i = i0; i < i1; ++i) {
        const int64_t ra = ia ? __ldg(ia + i) : i, rb = ib ? __ldg(ib + i) : i;
        uint64_t a = EA[ra * n + j];
        const uint64_t b = EB[rb * n + j];
        if (w) a = mul(a, __ldg(w + i));
        mac160(x, a, b);
    }
    part[(int64_t)blockIdx.y * n + j] = reduce160(x);
}

__global__ void __launch_bounds__(256) k_colsum_finish(const uint64_t* __restrict__ part, int splits, int64_t n,
                                                       uint64_t* __restrict__ out, int accumulate) {
    const int64_t j = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= n) return;
    uint64_t v = accumulate ? out[j] : 0;
    for (int s = 0; s < splits; ++s) v = add(v, part[(int64_t)s * n + j]);
    out[j] = v;
}

// w = M.v: one warp per row, lanes stride the row summing unreduced products, shuffle reduction.
__global__ void __launch_bounds__(256) k_matvec(const uint64_t* __restrict__ M, const uint64_t* __restrict__ v,
                                                uint64_t* __restrict__ w, int64_t m, int64_t n) {
    const int lane = threadIdx.x & 31;
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    if (row >= m) return;
    const uint64_t* r = M + row * n;
    uint32_t x[5] = {0, 0, 0, 0, 0};
    for (int64_t j = lane; j < n; j += 32) mac160(x, r[j], __ldg(v + j));
    uint64_t acc = reduce160(x);
#pragma unroll
    for (int o = 16; o; o >>= 1) acc = add(acc, __shfl_xor_sync(0xffffffffu, acc, o));
    if (lane == 0) w[row] = acc;
}

__global__ void __launch_bounds__(BLOCK) k_spmv(const uint64_t* __restrict__ values, const uint64_t* __restrict__ col_idx,
                                                const uint64_t* __restrict__ row_ptr, const uint64_t* __restrict__ x,
                                                const uint8_t* __restrict__ seed, const uint8_t* __restrict__ label,
                                                int label_len, uint64_t* __restrict__ y, int64_t n_rows) {
    const int64_t i = (int64_t)blockIdx.x * BLOCK + threadIdx.x;
    if (i >= n_rows) return;
    uint32_t s[8];
    uint64_t lab = 0;
    if (!x) { vb3::load_seed(seed, s); lab = vb3::load_label(label, label_len); }
    uint64_t acc = 0;
    for (uint64_t p = row_ptr[i]; p < row_ptr[i + 1]; ++p) {
        uint64_t xv = x ? x[col_idx[p]] : vb3::challenge(s, lab, label_len, col_idx[p]);
        acc = add(acc, mul(values[p], xv));
    }
    y[i] = acc;
}

__global__ void __launch_bounds__(BLOCK) k_lookup(const uint64_t* __restrict__ x, int64_t n_x,
                                                  const uint64_t* __restrict__ table, int64_t n_table,
                                                  unsigned long long* __restrict__ mult) {
    const int64_t i = (int64_t)blockIdx.x * BLOCK + threadIdx.x;
    if (i >= n_x) return;
    const uint64_t xi = x[i];
    if (!table) {
        if (xi < (uint64_t)n_table) atomicAdd(&mult[xi], 1ULL);
        return;
    }
    for (int64_t j = 0; j < n_table; ++j)
        if (__ldg(table + j) == xi) { atomicAdd(&mult[j], 1ULL); return; }
}

struct BandArgs {
    int kind;
    uint64_t* out;
    int64_t out_off, flat_lo, n_slots;
    uint64_t p0, p1, p2, p3;
    const uint64_t* desc;
    const void* aux0;
    const void* aux1;
    const uint64_t* chal_buf;
    int64_t aux_n;
    const uint8_t* seed;
    const uint8_t* label;
    int label_len;
};

__global__ void __launch_bounds__(BLOCK) k_band(BandArgs a) {
    const int64_t s = (int64_t)blockIdx.x * BLOCK + threadIdx.x;
    if (s >= a.n_slots) return;
    uint32_t sd[8];
    vb3::load_seed(a.seed, sd);
    const uint64_t lab = vb3::load_label(a.label, a.label_len);
    auto chal = [&](uint64_t cid) { return vb3::challenge(sd, lab, a.label_len, cid); };
    uint64_t* o = a.out + a.out_off + s;
    const uint64_t f = (uint64_t)a.flat_lo + (uint64_t)s;
    if (a.kind == 0) {
        const uint64_t* d = a.desc;
        const uint64_t* tblA = (const uint64_t*)a.aux0;
        const uint64_t* tblB = (const uint64_t*)a.aux1;
        uint64_t rem = f;
        int q = (int)d[0];
        uint64_t cid = d[5], ia = 0, ib = 0;
        for (int j = q - 1; j >= 1; --j) {
            uint64_t dig = rem % d[1 + j];
            rem /= d[1 + j];
            cid += dig * d[6 + j]; ia += dig * d[14 + j]; ib += dig * d[18 + j];
        }
        cid += rem * d[6]; ia += rem * d[14]; ib += rem * d[18];
        uint64_t mode = d[12];
        uint64_t coef = mode == 0 ? d[13] : mode == 1 ? tblA[ia] : sub(0, mul(tblA[ia], tblB[ib]));
        uint64_t fan = d[10], fs = d[11], acc = 0;
        for (uint64_t t = 0; t < fan; ++t) {
            uint64_t c = cid + t * fs;
            acc = add(acc, d[22] ? a.chal_buf[c - d[23]] : chal(c));
        }
        *o = add(*o, mul(coef, acc));
    } else if (a.kind == 1) {
        uint64_t base = a.p0, m = a.p1, h = a.p2, coef = a.p3;
        uint64_t b = f / m, j = f % m, iq = b / h, hh = b % h;
        if (j > iq) return;
        uint64_t cid = base + h * iq * (iq + 1) / 2 + hh * (iq + 1) + j;
        *o = add(*o, mul(coef, chal(cid)));
    } else if (a.kind == 2) {
        uint64_t base = a.p0, h = a.p1, coef = a.p2;
        uint64_t iq = f / h, hh = f % h;
        uint64_t rank0 = base + h * iq * (iq + 1) / 2 + hh * (iq + 1), acc = 0;
        for (uint64_t jo = 0; jo <= iq; ++jo) acc = add(acc, chal(rank0 + jo));
        *o = add(*o, mul(coef, acc));
    } else if (a.kind == 3) {
        uint64_t base = a.p0, d = a.p1, rows_per_w = a.p2, ell = a.p3;
        const int64_t* tok = (const int64_t*)a.aux0;
        uint64_t row_off = f / ell, within = f % ell, rel = within / d, jj = within % d;
        if (rel >= rows_per_w) return;
        int64_t v = (int64_t)(row_off * rows_per_w + rel);
        uint64_t acc = 0;
        for (int64_t i = 0; i < a.aux_n; ++i)
            if (tok[i] == v) acc = add(acc, chal(base + (uint64_t)i * d + jj));
        *o = add(*o, sub(0, acc));
    } else {
        uint64_t base = a.p0, H = a.p1, d_h = a.p2, half = d_h / 2;
        const uint64_t* cos_t = (const uint64_t*)a.aux0;
        const uint64_t* sin_t = (const uint64_t*)a.aux1;
        uint64_t sq = f / (H * d_h), hh = (f / d_h) % H, k = f % d_h, e = k / half, kp = k % half;
        uint64_t pair_t = sq * H * half + hh * half + kp, ci = sq * half + kp;
        uint64_t c = cos_t[ci], sn = sin_t[ci];
        uint64_t r1 = chal(base + 2 * pair_t), r2 = chal(base + 2 * pair_t + 1);
        uint64_t c1 = e == 0 ? sub(0, c) : sn;
        uint64_t c2 = e == 0 ? sub(0, sn) : sub(0, c);
        *o = add(*o, add(mul(c1, r1), mul(c2, r2)));
    }
}

}  // namespace

#define VI_LAUNCH_1D(kernel, n, ...)                                                        \
    do {                                                                                    \
        if ((n) > 0) kernel<<<grid_for(n), BLOCK, 0, (cudaStream_t)stream>>>(__VA_ARGS__);  \
        return vi::check_launch(#kernel);                                                   \
    } while (0)

extern "C" int vi_gl_binary(int op, const uint64_t* a, const uint64_t* b, uint64_t* out, int64_t n, void* stream) {
    VI_REQUIRE(op >= 0 && op <= 2, "gl_binary: op must be 0 (mul), 1 (add) or 2 (sub)");
    VI_REQUIRE(n >= 0, "gl_binary: negative size");
    if (n == 0) return VI_OK;
    VI_REQUIRE(a && b && out, "gl_binary: null pointer");
    if (op == 0) VI_LAUNCH_1D(k_binary_alias<0>, n, a, b, out, n);
    if (op == 1) VI_LAUNCH_1D(k_binary_alias<1>, n, a, b, out, n);
    VI_LAUNCH_1D(k_binary_alias<2>, n, a, b, out, n);
}

extern "C" int vi_gl_binary_bcast(int op, const uint64_t* a, const uint64_t* b, int64_t nb, uint64_t* out, int64_t n, void* stream) {
    VI_REQUIRE(op >= 0 && op <= 2, "gl_binary_bcast: op must be 0 (mul), 1 (add) or 2 (sub)");
    VI_REQUIRE(n >= 0 && nb > 0, "gl_binary_bcast: bad size");
    if (n == 0) return VI_OK;
    VI_REQUIRE(a && b && out, "gl_binary_bcast: null pointer");
    if (op == 0) VI_LAUNCH_1D(k_binary_bcast<0>, n, a, b, nb, out, n);
    if (op == 1) VI_LAUNCH_1D(k_binary_bcast<1>, n, a, b, nb, out, n);
    VI_LAUNCH_1D(k_binary_bcast<2>, n, a, b, nb, out, n);
}

extern "C" int vi_gl_neg(const uint64_t* a, uint64_t* out, int64_t n, void* stream) {
    VI_REQUIRE(n >= 0, "gl_neg: negative size");
    if (n == 0) return VI_OK;
    VI_REQUIRE(a && out, "gl_neg: null pointer");
    VI_LAUNCH_1D(k_neg, n, a, out, n);
}
extern "C" int vi_gl_pow(const uint64_t* base, uint64_t exp, uint64_t* out, int64_t n, void* stream) {
    VI_REQUIRE(n >= 0, "gl_pow: negative size");
    if (n == 0) return VI_OK;
    VI_REQUIRE(base && out, "gl_pow: null pointer");
    VI_LAUNCH_1D(k_pow, n, base, exp, out, n);
}
extern "C" int vi_gl_axpy(uint64_t* y, uint64_t alpha, const uint64_t* x, int64_t n, void* stream) {
    VI_REQUIRE(n >= 0, "gl_axpy: negative size");
    if (n == 0) return VI_OK;
    VI_REQUIRE(y && x, "gl_axpy: null pointer");
    VI_LAUNCH_1D(k_axpy, n, y, alpha, x, n);
}

extern "C" int vi_poly_eval(const uint64_t* coeffs, int64_t m, int64_t d, const uint64_t* points, int64_t k,
                            uint64_t* out, void* stream) {
    VI_REQUIRE(m >= 0 && d >= 0 && k >= 0, "poly_eval: negative size");
    if (m == 0 || k == 0) return VI_OK;
    dim3 block(64, 4), grid((unsigned)((k + 63) / 64), (unsigned)((m + 3) / 4));
    VI_REQUIRE(grid.y <= 65535, "poly_eval: too many rows for one launch");
    k_poly_eval<<<grid, block, 0, (cudaStream_t)stream>>>(coeffs, m, d, points, k, out);
    return vi::check_launch("k_poly_eval");
}

extern "C" int vi_gl_matmul(const uint64_t* A, const uint64_t* B, uint64_t* C, int64_t m, int64_t k, int64_t n, void* stream) {
    VI_REQUIRE(m >= 0 && k >= 0 && n >= 0, "gl_matmul: negative size");
    if (m == 0 || n == 0) return VI_OK;
    VI_REQUIRE(A && B && C || k == 0, "gl_matmul: null pointer");
    VI_REQUIRE(C != A && C != B, "gl_matmul: the output must not alias an input");
    VI_REQUIRE(k < (int64_t(1) << 32), "gl_matmul: inner dimension must be below 2^32");
    if (n == 1 && k > 0) {                     // a single column of B is a vector: matrix-vector product
        int64_t g = (m * 32 + 255) / 256;
        VI_REQUIRE(g <= 0x7FFFFFFFLL, "gl_matmul: too many rows");
        k_matvec<<<(unsigned)g, 256, 0, (cudaStream_t)stream>>>(A, B, C, m, k);
        return vi::check_launch("k_matvec");
    }
    if (m <= 4 && k > 0 && (n + 31) / 32 <= 0x7FFFFFFFLL) {     // linear combination of the rows of B
        const unsigned g = (unsigned)((n + 31) / 32);
        cudaStream_t st = (cudaStream_t)stream;
        if (m == 1) k_matmul_thin<1><<<g, 256, 0, st>>>(A, B, C, k, n);
        else if (m == 2) k_matmul_thin<2><<<g, 256, 0, st>>>(A, B, C, k, n);
        else if (m == 3) k_matmul_thin<3><<<g, 256, 0, st>>>(A, B, C, k, n);
        else k_matmul_thin<4><<<g, 256, 0, st>>>(A, B, C, k, n);
        return vi::check_launch("k_matmul_thin");
    }
    dim3 grid((unsigned)((n + MM_TN - 1) / MM_TN), (unsigned)((m + MM_TM - 1) / MM_TM));
    VI_REQUIRE(grid.y <= 65535, "gl_matmul: too many rows for one launch (m <= 4194240)");
    VI_CUDA(cudaFuncSetAttribute(k_matmul, cudaFuncAttributeMaxDynamicSharedMemorySize, MM_SMEM));
    k_matmul<<<grid, 256, MM_SMEM, (cudaStream_t)stream>>>(A, B, C, m, k, n);
    return vi::check_launch("k_matmul");
}

extern "C" int vi_gl_matvec(const uint64_t* M, const uint64_t* v, uint64_t* w, int64_t m, int64_t n, void* stream) {
    VI_REQUIRE(m >= 0 && n >= 0, "gl_matvec: negative size");
    if (m == 0) return VI_OK;
    int64_t grid = (m * 32 + 255) / 256;
    VI_REQUIRE(grid <= 0x7FFFFFFFLL, "gl_matvec: too many rows");
    k_matvec<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(M, v, w, m, n);
    return vi::check_launch("k_matvec");
}

extern "C" int vi_gl_spmv(const uint64_t* values, const uint64_t* col_idx, const uint64_t* row_ptr,
                          const uint64_t* x, const uint8_t* seed_dev, const uint8_t* label_dev, int label_len,
                          uint64_t* y, int64_t n_rows, void* stream) {
    VI_REQUIRE(n_rows >= 0, "gl_spmv: negative size");
    VI_REQUIRE(x || (seed_dev && label_len >= 0 && label_len <= 8), "gl_spmv: need x or (seed, label<=8)");
    if (n_rows == 0) return VI_OK;
    int64_t grid = (n_rows + BLOCK - 1) / BLOCK;
    k_spmv<<<(unsigned)grid, BLOCK, 0, (cudaStream_t)stream>>>(values, col_idx, row_ptr, x, seed_dev, label_dev,
                                                             label_len, y, n_rows);
    return vi::check_launch("k_spmv");
}

extern "C" int vi_lookup_multiplicities(const uint64_t* x, int64_t n_x, const uint64_t* table, int64_t n_table,
                                        uint64_t* mult, void* stream) {
    VI_REQUIRE(n_x >= 0 && n_table >= 0, "lookup: negative size");
    if (n_x == 0) return VI_OK;
    int64_t grid = (n_x + BLOCK - 1) / BLOCK;
    VI_REQUIRE(grid <= 0x7FFFFFFFLL, "lookup: too many elements");
    k_lookup<<<(unsigned)grid, BLOCK, 0, (cudaStream_t)stream>>>(x, n_x, table, n_table, (unsigned long long*)mult);
    return vi::check_launch("k_lookup");
}

extern "C" int vi_interp_band(int kind, uint64_t* out, int64_t out_off, int64_t flat_lo, int64_t n_slots,
                              uint64_t p0, uint64_t p1, uint64_t p2, uint64_t p3,
                              const uint64_t* desc_dev, const void* aux0, const void* aux1, const uint64_t* chal_buf,
                              int64_t aux_n, const uint8_t* seed_dev, const uint8_t* label_dev, int label_len,
                              void* stream) {
    VI_REQUIRE(kind >= 0 && kind <= 4, "interp_band: unknown kind %d", kind);
    VI_REQUIRE(n_slots >= 0, "interp_band: negative size");
    VI_REQUIRE(label_len >= 0 && label_len <= 8, "interp_band: label must be <= 8 bytes");
    if (n_slots == 0) return VI_OK;
    BandArgs a{kind, out, out_off, flat_lo, n_slots, p0, p1, p2, p3, desc_dev, aux0, aux1, chal_buf, aux_n,
               seed_dev, label_dev, label_len};
    int64_t grid = (n_slots + BLOCK - 1) / BLOCK;
    VI_REQUIRE(grid <= 0x7FFFFFFFLL, "interp_band: too many slots");
    k_band<<<(unsigned)grid, BLOCK, 0, (cudaStream_t)stream>>>(a);
    return vi::check_launch("k_band");
}

namespace {
int colsum_splits(int64_t T, int64_t n) {
    // enough CTAs for ~4 per SM, at least 8 rows per split
    int64_t col_blocks = (n + 255) / 256;
    int64_t want = (148 * 4 + col_blocks - 1) / col_blocks;
    int64_t max_by_rows = (T + 7) / 8;
    int64_t s = want < max_by_rows ? want : max_by_rows;
    if (s < 1) s = 1;
    if (s > 1024) s = 1024;
    return (int)s;
}
}  // namespace

extern "C" int64_t vi_product_colsum_scratch_bytes(int64_t T, int64_t n) {
    if (T <= 0 || n <= 0) return 0;
    return (int64_t)colsum_splits(T, n) * n * 8;
}

extern "C" int vi_product_colsum(const uint64_t* EA, const uint64_t* EB, int64_t n,
                                 const int64_t* ia_dev, const int64_t* ib_dev, const uint64_t* w_dev, int64_t T,
                                 uint64_t* out, int accumulate, void* scratch, int64_t scratch_bytes, void* stream) {
    VI_REQUIRE(T >= 0 && n >= 0, "product_colsum: negative size");
    if (n == 0) return VI_OK;
    VI_REQUIRE(out != nullptr, "product_colsum: null output");
    cudaStream_t st = (cudaStream_t)stream;
    if (T == 0) {
        if (!accumulate) VI_CUDA(cudaMemsetAsync(out, 0, (size_t)n * 8, st));
        return VI_OK;
    }
    VI_REQUIRE(EA && EB, "product_colsum: null input");
    VI_REQUIRE(T < (int64_t(1) << 32), "product_colsum: too many rows");
    const int splits = colsum_splits(T, n);
    if (scratch == nullptr || scratch_bytes < (int64_t)splits * n * 8)
        return vi::fail(VI_ERR_SCRATCH, "product_colsum: scratch of at least %lld bytes required (see vi_product_colsum_scratch_bytes)",
                        (long long)((int64_t)splits * n * 8));
    const int64_t per = (T + splits - 1) / splits;
    const int64_t gx = (n + 255) / 256;
    if (gx > 0x7FFFFFFFLL) return vi::fail(VI_ERR_LIMIT, "product_colsum: too many columns");
    dim3 grid((unsigned)gx, (unsigned)splits);
    k_product_colsum<<<grid, 256, 0, st>>>(EA, EB, n, ia_dev, ib_dev, w_dev, T, per, (uint64_t*)scratch);
    int rc = vi::check_launch("k_product_colsum");
    if (rc) return rc;
    k_colsum_finish<<<(unsigned)gx, 256, 0, st>>>((const uint64_t*)scratch, splits, n, out, accumulate);
    return vi::check_launch("k_colsum_finish");
}
