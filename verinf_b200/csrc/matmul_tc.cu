// Field matmul C = A.B mod p on the integer tensor cores.
//
// What it replaces in the reference: gl_matmul (prover/kernels/gl_matmul.cuh,
// prover/cuda_primitives.py:1086-1106), one thread per output with a reduced multiply and add
// per term.
//
// A 64-bit operand is eight bytes, so A.B = sum_{i,j} 2^(8(i+j)) A_i.B_j where A_i, B_j are the
// byte planes and every A_i.B_j is an exact u8 x u8 -> s32 matrix product.  The 64 plane pairs
// of an output tile share 15 accumulators (one per weight s = i + j): at most 8 pairs x 4096
// terms x 255^2 < 2^31 fit, so k is processed in chunks of 4096 and each chunk ends with
// sum_s T_s 2^(8s) mod p (shifts: 2 has order 192 in this field) added into C.
//
//  * k_split_rows / k_split_cols write the byte planes K-contiguous: Ap[i][row][k], Bp[j][col][k]
//    (the second through a shared-memory transpose), zero padded to tile multiples.
//  * k_matmul_planes: CTA tile 64 x 32 outputs, 8 warps of 16 x 16, k in slices of 64 bytes
//    through a 3-stage cp.async pipeline (one barrier per slice); fragments by ldmatrix, products by
//    mma.sync.m16n8k32.s32.u8.u8.s32 (256 per warp and slice).  Rows of a slice are padded to
//    80 bytes in shared memory so that ldmatrix is free of bank conflicts.
#include "../../include/verinf_b200.h"
#include "common.cuh"
#include "gl.cuh"
#include "plane_fold.cuh"

namespace {

constexpr int TC_TM = 64, TC_TN = 32, TC_KS = 64;      // CTA tile and k slice (bytes per plane row)
constexpr int TC_ROWB = 80;                             // shared-memory bytes per plane row of a slice
constexpr int TC_STAGES = 3;
constexpr int TC_A_BYTES = 8 * TC_TM * TC_ROWB, TC_B_BYTES = 8 * TC_TN * TC_ROWB;
constexpr int TC_STAGE_BYTES = TC_A_BYTES + TC_B_BYTES;
constexpr int TC_SMEM = TC_STAGES * TC_STAGE_BYTES;
constexpr int64_t TC_KCHUNK = 4096;                     // 8 * 4096 * 255^2 < 2^31

__host__ __device__ inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

// planes[i][r][c] = byte i of src[r][c] for r < rows_pad, c < k_pad (zero outside the matrix)
__global__ void __launch_bounds__(256) k_split_rows(const uint64_t* __restrict__ src, int64_t rows, int64_t k,
                                                    int64_t rows_pad, int64_t k_pad, uint8_t* __restrict__ planes) {
    const int64_t c = (int64_t)blockIdx.y * blockDim.x + threadIdx.x;
    const int64_t r = blockIdx.x;
    if (c >= k_pad) return;
    const uint64_t v = (r < rows && c < k) ? src[r * k + c] : 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) planes[((int64_t)i * rows_pad + r) * k_pad + c] = (uint8_t)(v >> (8 * i));
}

// planes[j][c][r] = byte j of src[r][c] (src is k x n row-major): 32 x 32 tiles through shared memory
__global__ void __launch_bounds__(256) k_split_cols(const uint64_t* __restrict__ src, int64_t k, int64_t n,
                                                    int64_t n_pad, int64_t k_pad, uint8_t* __restrict__ planes) {
    __shared__ uint64_t tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;          // 32 x 8
    const int64_t r0 = (int64_t)blockIdx.y * 32, c0 = (int64_t)blockIdx.x * 32;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int64_t r = r0 + ty + 8 * q, c = c0 + tx;
        tile[ty + 8 * q][tx] = (r < k && c < n) ? src[r * n + c] : 0;
    }
    __syncthreads();
    // thread (tx = k offset, ty + 8q = column offset): 32 consecutive bytes along k per warp and plane
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int cl = ty + 8 * q;
        const uint64_t v = tile[tx][cl];
        const int64_t c = c0 + cl, r = r0 + tx;
        if (c < n_pad && r < k_pad) {
#pragma unroll
            for (int j = 0; j < 8; ++j) planes[((int64_t)j * n_pad + c) * k_pad + r] = (uint8_t)(v >> (8 * j));
        }
    }
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    unsigned sa = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(sa), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_row) {
    unsigned a = (unsigned)__cvta_generic_to_shared(smem_row);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_u8(int32_t (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.u8.u8.s32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
                 "{%0, %1, %2, %3};"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}


template <int I, int J>
__device__ __forceinline__ void mma_pairs(int32_t (&acc)[15][2][4], const uint32_t (&a)[4], const uint32_t (&b)[8][4]) {
    if constexpr (J < 8) {
        mma_u8(acc[I + J][0], a, b[J][0], b[J][1]);
        mma_u8(acc[I + J][1], a, b[J][2], b[J][3]);
        mma_pairs<I, J + 1>(acc, a, b);
    }
}
template <int I>
__device__ __forceinline__ void mma_planes(int32_t (&acc)[15][2][4], const uint8_t* a_row, const uint32_t (&b)[8][4]) {
    if constexpr (I < 8) {
        uint32_t a[4];
        ldmatrix_x4(a, a_row + I * (TC_TM * TC_ROWB));
        mma_pairs<I, 0>(acc, a, b);
        mma_planes<I + 1>(acc, a_row, b);
    }
}

__global__ void __launch_bounds__(256, 1) k_matmul_planes(const uint8_t* __restrict__ Ap, const uint8_t* __restrict__ Bp,
                                                          uint64_t* __restrict__ C, int64_t m, int64_t n,
                                                          int64_t m_pad, int64_t n_pad, int64_t k_pad) {
    extern __shared__ __align__(16) uint8_t tc_smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int wm = warp & 3, wn = warp >> 2;                 // 4 x 2 warps of 16 x 16 outputs
    const int64_t row0 = (int64_t)blockIdx.y * TC_TM, col0 = (int64_t)blockIdx.x * TC_TN;
    const int64_t nslices = k_pad / TC_KS;

    auto load_slice = [&](int64_t s, int stage) {
        uint8_t* sa = tc_smem + stage * TC_STAGE_BYTES;
        uint8_t* sb = sa + TC_A_BYTES;
        const int64_t k0 = s * TC_KS;
        // A: 8 planes x 64 rows x 4 chunks of 16 bytes = 2048 chunks, 8 per thread
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const int e = tid + 256 * q, ch = e & 3, r = (e >> 2) & 63, pl = e >> 8;
            cp_async16(sa + (pl * TC_TM + r) * TC_ROWB + ch * 16, Ap + ((int64_t)pl * m_pad + row0 + r) * k_pad + k0 + ch * 16);
        }
        // B: 8 planes x 32 columns x 4 chunks = 1024 chunks, 4 per thread
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int e = tid + 256 * q, ch = e & 3, r = (e >> 2) & 31, pl = e >> 7;
            cp_async16(sb + (pl * TC_TN + r) * TC_ROWB + ch * 16, Bp + ((int64_t)pl * n_pad + col0 + r) * k_pad + k0 + ch * 16);
        }
        cp_async_commit();
    };

    // ldmatrix row addresses of this lane: matrices 0..3 = (rows 0-7, k 0-15), (rows 8-15, k 0-15),
    // (rows 0-7, k 16-31), (rows 8-15, k 16-31) for A; for B (two 8-column groups): (cols 0-7, k 0-15),
    // (cols 0-7, k 16-31), (cols 8-15, k 0-15), (cols 8-15, k 16-31)
    const int mat = lane >> 3, rin = lane & 7;
    const int a_off = (wm * 16 + (mat & 1) * 8 + rin) * TC_ROWB + (mat >> 1) * 16;
    const int b_off = (wn * 16 + (mat >> 1) * 8 + rin) * TC_ROWB + (mat & 1) * 16;

    const int g = lane >> 2, tig = lane & 3;
    for (int64_t c0k = 0; c0k < nslices; c0k += TC_KCHUNK / TC_KS) {
        const int64_t c1k = c0k + TC_KCHUNK / TC_KS < nslices ? c0k + TC_KCHUNK / TC_KS : nslices;
        int32_t acc[15][2][4];
#pragma unroll
        for (int s = 0; s < 15; ++s)
#pragma unroll
            for (int t = 0; t < 2; ++t)
#pragma unroll
                for (int q = 0; q < 4; ++q) acc[s][t][q] = 0;
        // prologue: slices c0k, c0k+1 in flight; one barrier per slice: after it every warp has finished
        // the previous slice, so its stage can take slice s+2 while slice s is multiplied
        load_slice(c0k, 0);
        if (c0k + 1 < c1k) load_slice(c0k + 1, 1); else cp_async_commit();
        for (int64_t s = c0k; s < c1k; ++s) {
            const int stage = (int)((s - c0k) % TC_STAGES);
            cp_async_wait<1>();
            __syncthreads();
            if (s + 2 < c1k) load_slice(s + 2, (int)((s - c0k + 2) % TC_STAGES)); else cp_async_commit();
            const uint8_t* sa = tc_smem + stage * TC_STAGE_BYTES;
            const uint8_t* sb = sa + TC_A_BYTES;
#pragma unroll
            for (int h = 0; h < TC_KS / 32; ++h) {
                uint32_t b[8][4];
#pragma unroll
                for (int j = 0; j < 8; ++j) ldmatrix_x4(b[j], sb + j * (TC_TN * TC_ROWB) + b_off + h * 32);
                mma_planes<0>(acc, sa + a_off + h * 32, b);
            }
        }
        cp_async_wait<0>();
        __syncthreads();          // the next chunk's prologue overwrites stages 0 and 1
        // fold this chunk: acc[s][t][q] is output (row g (+8 for q >= 2), column 8t + 2 tig + (q & 1))
#pragma unroll
        for (int t = 0; t < 2; ++t)
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint32_t ts[15];
#pragma unroll
                for (int s = 0; s < 15; ++s) ts[s] = (uint32_t)acc[s][t][q];
                const uint64_t v = vpf::combine15(ts);
                const int64_t r = row0 + wm * 16 + g + (q >> 1) * 8;
                const int64_t c = col0 + wn * 16 + t * 8 + tig * 2 + (q & 1);
                if (r < m && c < n) C[r * n + c] = c0k == 0 ? v : vgl::add(C[r * n + c], v);
            }
    }
}

}  // namespace

extern "C" int64_t vi_gl_matmul_tc_scratch_bytes(int64_t m, int64_t k, int64_t n) {
    if (m <= 0 || k <= 0 || n <= 0) return 0;
    const int64_t k_pad = round_up(k, TC_KS);
    return 8 * (round_up(m, TC_TM) + round_up(n, TC_TN)) * k_pad;
}

extern "C" int vi_gl_matmul_tc(const uint64_t* A, const uint64_t* B, uint64_t* C, int64_t m, int64_t k, int64_t n,
                               void* scratch, int64_t scratch_bytes, void* stream) {
    VI_REQUIRE(m >= 0 && k >= 0 && n >= 0, "gl_matmul_tc: negative size");
    if (m == 0 || n == 0) return VI_OK;
    cudaStream_t st = (cudaStream_t)stream;
    VI_REQUIRE(C != nullptr, "gl_matmul_tc: null output");
    if (k == 0) { VI_CUDA(cudaMemsetAsync(C, 0, (size_t)(m * n) * 8, st)); return VI_OK; }
    VI_REQUIRE(A && B, "gl_matmul_tc: null input");
    VI_REQUIRE(C != A && C != B, "gl_matmul_tc: the output must not alias an input");
    const int64_t need = vi_gl_matmul_tc_scratch_bytes(m, k, n);
    if (scratch == nullptr || scratch_bytes < need)
        return vi::fail(VI_ERR_SCRATCH, "gl_matmul_tc: scratch of at least %lld bytes required (see vi_gl_matmul_tc_scratch_bytes)",
                        (long long)need);
    VI_REQUIRE(((uintptr_t)scratch) % 16 == 0, "gl_matmul_tc: scratch must be 16-byte aligned");
    const int64_t m_pad = round_up(m, TC_TM), n_pad = round_up(n, TC_TN), k_pad = round_up(k, TC_KS);
    VI_REQUIRE(m_pad / TC_TM <= 65535 && k_pad / 32 <= 65535 && m_pad < (int64_t(1) << 31) && n_pad / 32 < (int64_t(1) << 31),
               "gl_matmul_tc: matrix too large for one launch");
    uint8_t* Ap = (uint8_t*)scratch;
    uint8_t* Bp = Ap + 8 * m_pad * k_pad;
    {
        dim3 grid((unsigned)m_pad, (unsigned)((k_pad + 255) / 256));
        k_split_rows<<<grid, 256, 0, st>>>(A, m, k, m_pad, k_pad, Ap);
        int rc = vi::check_launch("k_split_rows");
        if (rc) return rc;
    }
    {
        dim3 grid((unsigned)(n_pad / 32), (unsigned)(k_pad / 32));
        k_split_cols<<<grid, 256, 0, st>>>(B, k, n, n_pad, k_pad, Bp);
        int rc = vi::check_launch("k_split_cols");
        if (rc) return rc;
    }
    VI_CUDA(cudaFuncSetAttribute(k_matmul_planes, cudaFuncAttributeMaxDynamicSharedMemorySize, TC_SMEM));
    dim3 grid((unsigned)(n_pad / TC_TN), (unsigned)(m_pad / TC_TM));
    k_matmul_planes<<<grid, 256, TC_SMEM, st>>>(Ap, Bp, C, m, n, m_pad, n_pad, k_pad);
    return vi::check_launch("k_matmul_planes");
}
