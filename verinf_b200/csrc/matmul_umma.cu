// Field matmul C = A.B mod p on the 5th-generation tensor cores (tcgen05) with the accumulators in
// tensor memory.
//
// What it replaces in the reference: gl_matmul (prover/kernels/gl_matmul.cuh:28-59,
// prover/cuda_primitives.py:1086-1106), one thread per output with a reduced multiply and add per
// term.  Same byte-plane formulation as matmul_tc.cu: A.B = sum_{i,j} 2^(8(i+j)) A_i.B_j with
// exact u8 x u8 -> s32 plane products that share 15 accumulators (one per weight s = i + j), k in
// chunks of 4096 terms, each chunk closed by sum_s T_s 2^(8s) mod p.
//
// Blackwell mapping:
//  * CTA tile 128 rows x 32 columns.  The 15 accumulators are 15 x 32 = 480 of the 512 tensor-memory
//    columns (the register file held them in matmul_tc.cu and capped its tile at 16 x 16 per warp).
//  * The 8 B planes of the tile are stacked along N in shared memory (row j*32 + c = byte j of
//    column c), so ONE tcgen05.mma of shape M128 x N256 x K32 multiplies A plane i by all 8 B planes,
//    and its 256-column result window starts at column 32*i: accumulator i+j receives A_i.B_j.
//    8 instructions per 32 bytes of k instead of 64 plane products.
//  * Operands arrive by TMA (cp.async.bulk.tensor.2d, 64-byte swizzle, this GPU's own plane buffers,
//    no multicast) into a 2-stage ring of 80 KB; mbarriers carry full/empty; one thread issues the
//    copies, one thread issues the MMAs, tcgen05.commit releases a stage and finally publishes the
//    accumulators; 8 warps read them back with tcgen05.ld and fold the 15 sums.
//  * Every wait is bounded: on expiry the kernel records a code in `status`, lets copies in flight
//    land, frees its tensor memory and returns.
#include <cuda.h>

#include "../../include/verinf_b200.h"
#include "common.cuh"
#include "gl.cuh"
#include "plane_fold.cuh"

namespace {

constexpr int UM_TM = 128, UM_TN = 32, UM_KS = 64;        // CTA tile, k bytes per stage
constexpr int UM_STAGES = 2;
constexpr int UM_A_PLANE = UM_TM * UM_KS;                  // 8192 bytes
constexpr int UM_B_PLANE = UM_TN * UM_KS;                  // 2048 bytes
constexpr int UM_A_BYTES = 8 * UM_A_PLANE, UM_B_BYTES = 8 * UM_B_PLANE;
constexpr int UM_STAGE_BYTES = UM_A_BYTES + UM_B_BYTES;    // 81920
constexpr int UM_SMEM = UM_STAGES * UM_STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;
constexpr int64_t UM_KCHUNK = 4096;                        // 8 * 4096 * 255^2 < 2^31
constexpr int UM_THREADS = 256;
constexpr uint32_t UM_TMEM_COLS = 512;
constexpr unsigned long long UM_WAIT_NS = 2000000000ull;   // a wait gives up after two seconds

__host__ __device__ inline int64_t round_up(int64_t x, int64_t m) { return (x + m - 1) / m * m; }

// planes[i][r][c] = byte i of src[r][c] for r < rows_pad, c < k_pad (zero outside the matrix)
__global__ void __launch_bounds__(256) k_um_split_rows(const uint64_t* __restrict__ src, int64_t rows, int64_t k,
                                                       int64_t rows_pad, int64_t k_pad, uint8_t* __restrict__ planes) {
    const int64_t c = (int64_t)blockIdx.y * blockDim.x + threadIdx.x;
    const int64_t r = blockIdx.x;
    if (c >= k_pad) return;
    const uint64_t v = (r < rows && c < k) ? src[r * k + c] : 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) planes[((int64_t)i * rows_pad + r) * k_pad + c] = (uint8_t)(v >> (8 * i));
}
// planes[j][c][r] = byte j of src[r][c] (src is k x n row-major): 32 x 32 tiles through shared memory
__global__ void __launch_bounds__(256) k_um_split_cols(const uint64_t* __restrict__ src, int64_t k, int64_t n,
                                                       int64_t n_pad, int64_t k_pad, uint8_t* __restrict__ planes) {
    __shared__ uint64_t tile[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t r0 = (int64_t)blockIdx.y * 32, c0 = (int64_t)blockIdx.x * 32;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        const int64_t r = r0 + ty + 8 * q, c = c0 + tx;
        tile[ty + 8 * q][tx] = (r < k && c < n) ? src[r * n + c] : 0;
    }
    __syncthreads();
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

// ---- PTX wrappers -----------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
// bounded wait for the phase with the given parity to complete (non-blocking test, short sleeps);
// false = gave up after UM_WAIT_NS
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    const unsigned long long t0 = global_ns();
    for (uint32_t it = 0;; ++it) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred p;\n\t"
                     "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
                     "selp.u32 %0, 1, 0, p;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if (it > 64) __nanosleep(64);
        if ((it & 1023) == 1023 && global_ns() - t0 > UM_WAIT_NS) return false;
    }
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int32_t x, int32_t y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y) : "memory");
}
__device__ __forceinline__ void umma_i8(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\t"
                 "setp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                 ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate), "r"(0u) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld4(uint32_t taddr, uint32_t (&r)[4]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(taddr));
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major tile with 64-byte rows and the 64-byte swizzle: groups of
// 8 rows are 512 bytes apart (stride offset), the leading offset is the canonical 1, version 1 (sm_100).
__device__ __forceinline__ uint64_t smem_desc_sw64(uint32_t saddr) {
    return (uint64_t)((saddr >> 4) & 0x3FFF) | ((uint64_t)1 << 16) | ((uint64_t)(512 >> 4) << 32) | ((uint64_t)1 << 46) |
           ((uint64_t)4 << 61);
}
// Instruction descriptor: u8 x u8 -> s32, both operands K-major, M = 128, N as given.
__host__ __device__ constexpr uint32_t idesc_u8(int n) {
    return (2u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(UM_TM >> 4) << 24);
}


enum { UM_ERR_FULL = 1, UM_ERR_EMPTY = 2, UM_ERR_ACC = 3 };

__global__ void __launch_bounds__(UM_THREADS, 1)
k_matmul_umma(const __grid_constant__ CUtensorMap mapA, const __grid_constant__ CUtensorMap mapB,
              uint64_t* __restrict__ C, int64_t m, int64_t n, int64_t m_pad, int64_t n_pad, int64_t k_pad,
              int* __restrict__ status) {
    extern __shared__ uint8_t um_raw[];
    // stage buffers start on a 1024-byte boundary (the swizzle pattern repeats every 512 bytes)
    uint8_t* base = (uint8_t*)(((uintptr_t)um_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(base + UM_STAGES * UM_STAGE_BYTES);   // full[2], empty[2], acc, then tmem slot + abort
    volatile uint32_t* tmem_slot = (volatile uint32_t*)(bars + 8);
    volatile uint32_t* abort_flag = tmem_slot + 1;
    const uint32_t full0 = smem_u32(bars), empty0 = smem_u32(bars + UM_STAGES), accb = smem_u32(bars + 2 * UM_STAGES);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int64_t row0 = (int64_t)blockIdx.y * UM_TM, col0 = (int64_t)blockIdx.x * UM_TN;
    const int64_t nslices = k_pad / UM_KS;

    if (tid == 0) {
        for (int s = 0; s < UM_STAGES; ++s) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        mbar_init(accb, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {      // one warp allocates the tensor memory (all 512 columns; one CTA per SM by shared memory)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32((const void*)tmem_slot)),
                     "r"(UM_TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    const int64_t slices_per_chunk = UM_KCHUNK / UM_KS;
    uint32_t full_par[UM_STAGES] = {0, 0}, empty_par[UM_STAGES] = {0, 0};   // phase parities (used by the two role threads)
    uint32_t acc_par = 0;
    int64_t produced = 0, consumed = 0;                                     // slices issued by the role threads, across chunks

    for (int64_t c0k = 0; c0k < nslices; c0k += slices_per_chunk) {
        const int64_t c1k = c0k + slices_per_chunk < nslices ? c0k + slices_per_chunk : nslices;
        if (warp == 0 && lane == 0) {
            // ---- producer: TMA loads of A planes (8 x [128 rows x 64 B]) and B planes (8 x [32 x 64 B]) per slice
            for (int64_t s = c0k; s < c1k && !*abort_flag; ++s, ++produced) {
                const int st = (int)(produced % UM_STAGES);
                if (produced >= UM_STAGES) {          // wait until the MMAs that read this stage have completed
                    if (!mbar_wait(empty0 + 8 * st, empty_par[st])) { *abort_flag = UM_ERR_EMPTY; break; }
                    empty_par[st] ^= 1;
                }
                const uint32_t fb = full0 + 8 * st;
                mbar_expect_tx(fb, UM_STAGE_BYTES);
                const uint32_t sa = smem_u32(base + st * UM_STAGE_BYTES), sb = sa + UM_A_BYTES;
                const int32_t k0 = (int32_t)(s * UM_KS);
#pragma unroll
                for (int i = 0; i < 8; ++i) tma_load_2d(sa + i * UM_A_PLANE, &mapA, k0, (int32_t)(i * m_pad + row0), fb);
#pragma unroll
                for (int j = 0; j < 8; ++j) tma_load_2d(sb + j * UM_B_PLANE, &mapB, k0, (int32_t)(j * n_pad + col0), fb);
            }
        } else if (warp == 1 && lane == 0) {
            // ---- MMA issuer: per 32 bytes of k, A plane i times the 8 stacked B planes into columns 32*i ..
            for (int64_t s = c0k; s < c1k && !*abort_flag; ++s, ++consumed) {
                const int st = (int)(consumed % UM_STAGES);
                if (!mbar_wait(full0 + 8 * st, full_par[st])) { *abort_flag = UM_ERR_FULL; break; }
                full_par[st] ^= 1;
                tc_fence_after();
                const uint32_t sa = smem_u32(base + st * UM_STAGE_BYTES), sb = sa + UM_A_BYTES;
#pragma unroll
                for (int kk = 0; kk < UM_KS / 32; ++kk) {
                    const bool first = (s == c0k && kk == 0);     // first product of the chunk: accumulators start over
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const uint64_t ad = smem_desc_sw64(sa + i * UM_A_PLANE + kk * 32);
                        const uint32_t d = tmem + 32 * i;
                        if (!first) {
                            umma_i8(d, ad, smem_desc_sw64(sb + kk * 32), idesc_u8(256), 1);
                        } else if (i == 0) {
                            umma_i8(d, ad, smem_desc_sw64(sb + kk * 32), idesc_u8(256), 0);
                        } else {
                            // accumulators i .. i+6 already hold the products of planes < i; accumulator i+7 is new
                            umma_i8(d, ad, smem_desc_sw64(sb + kk * 32), idesc_u8(224), 1);
                            umma_i8(d + 224, ad, smem_desc_sw64(sb + 7 * UM_B_PLANE + kk * 32), idesc_u8(32), 0);
                        }
                    }
                }
                if (s + 1 < c1k) umma_commit(empty0 + 8 * st);      // stage free once these MMAs have read it
                else { umma_commit(empty0 + 8 * st); umma_commit(accb); }
            }
        }
        // ---- epilogue: all 8 warps; warp w reads lanes 32*(w%4).., columns 16*(w/4)..
        __syncwarp();
        bool ok = mbar_wait(accb, acc_par);
        acc_par ^= 1;
        if (!ok && *abort_flag == 0) *abort_flag = UM_ERR_ACC;
        tc_fence_after();
        if (ok && *abort_flag == 0) {
            const int64_t r = row0 + 32 * (warp & 3) + lane;
            const uint32_t tbase = tmem + ((uint32_t)(32 * (warp & 3)) << 16) + 16 * (warp >> 2);
#pragma unroll 1
            for (int g = 0; g < 4; ++g) {
                uint32_t t[15][4];
#pragma unroll
                for (int s = 0; s < 15; ++s) tmem_ld4(tbase + 32 * s + 4 * g, t[s]);
                tmem_ld_wait();
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    uint32_t ts[15];
#pragma unroll
                    for (int s = 0; s < 15; ++s) ts[s] = t[s][q];
                    const uint64_t v = vpf::combine15(ts);
                    const int64_t c = col0 + 16 * (warp >> 2) + 4 * g + q;
                    if (r < m && c < n) C[r * n + c] = c0k == 0 ? v : vgl::add(C[r * n + c], v);
                }
            }
        }
        tc_fence_before();
        __syncthreads();          // every warp has read the accumulators before the next chunk overwrites them
        tc_fence_after();
        if (*abort_flag) break;
    }
    if (*abort_flag) {
        if (tid == 0 && status) atomicExch(status, (int)*abort_flag);
        // copies in flight write into this CTA's shared memory: give them time to land before it is released
        for (int i = 0; i < 2000; ++i) __nanosleep(1000);
    }
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(UM_TMEM_COLS) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return (EncodeTiledFn) nullptr;
        return q == cudaDriverEntryPointSuccess ? (EncodeTiledFn)p : (EncodeTiledFn) nullptr;
    }();
    return fn;
}
// 2-D byte tensor (rows x k_pad, row pitch k_pad), box of box_rows x 64 bytes, 64-byte swizzle
int make_plane_map(CUtensorMap* map, uint8_t* ptr, int64_t rows, int64_t k_pad, uint32_t box_rows) {
    EncodeTiledFn enc = encode_tiled_fn();
    if (!enc) return vi::fail(VI_ERR_CUDA, "gl_matmul_umma: cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)k_pad, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)k_pad};
    const cuuint32_t box[2] = {(cuuint32_t)UM_KS, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return vi::fail(VI_ERR_CUDA, "gl_matmul_umma: cuTensorMapEncodeTiled failed (%d)", (int)r);
    return VI_OK;
}

}  // namespace

extern "C" int64_t vi_gl_matmul_umma_scratch_bytes(int64_t m, int64_t k, int64_t n) {
    if (m <= 0 || k <= 0 || n <= 0) return 0;
    const int64_t k_pad = round_up(k, UM_KS);
    return 8 * (round_up(m, UM_TM) + round_up(n, UM_TN)) * k_pad + 256;     // planes + the status word
}

extern "C" int vi_gl_matmul_umma(const uint64_t* A, const uint64_t* B, uint64_t* C, int64_t m, int64_t k, int64_t n,
                                 void* scratch, int64_t scratch_bytes, int32_t* status_dev, void* stream) {
    VI_REQUIRE(m >= 0 && k >= 0 && n >= 0, "gl_matmul_umma: negative size");
    if (m == 0 || n == 0) return VI_OK;
    cudaStream_t st = (cudaStream_t)stream;
    VI_REQUIRE(C != nullptr, "gl_matmul_umma: null output");
    if (k == 0) { VI_CUDA(cudaMemsetAsync(C, 0, (size_t)(m * n) * 8, st)); return VI_OK; }
    VI_REQUIRE(A && B, "gl_matmul_umma: null input");
    VI_REQUIRE(C != A && C != B, "gl_matmul_umma: the output must not alias an input");
    const int64_t need = vi_gl_matmul_umma_scratch_bytes(m, k, n);
    if (scratch == nullptr || scratch_bytes < need)
        return vi::fail(VI_ERR_SCRATCH, "gl_matmul_umma: scratch of at least %lld bytes required (see vi_gl_matmul_umma_scratch_bytes)",
                        (long long)need);
    VI_REQUIRE(((uintptr_t)scratch) % 256 == 0, "gl_matmul_umma: scratch must be 256-byte aligned");
    const int64_t m_pad = round_up(m, UM_TM), n_pad = round_up(n, UM_TN), k_pad = round_up(k, UM_KS);
    VI_REQUIRE(m_pad / UM_TM <= 65535 && 8 * m_pad < (int64_t(1) << 31) && 8 * n_pad < (int64_t(1) << 31) &&
               k_pad < (int64_t(1) << 31) && (k_pad + 255) / 256 <= 65535 && k_pad / 32 <= 65535,
               "gl_matmul_umma: matrix too large for one launch");
    uint8_t* Ap = (uint8_t*)scratch;
    uint8_t* Bp = Ap + 8 * m_pad * k_pad;
    {
        dim3 grid((unsigned)m_pad, (unsigned)((k_pad + 255) / 256));
        k_um_split_rows<<<grid, 256, 0, st>>>(A, m, k, m_pad, k_pad, Ap);
        int rc = vi::check_launch("k_um_split_rows");
        if (rc) return rc;
    }
    {
        dim3 grid((unsigned)(n_pad / 32), (unsigned)(k_pad / 32));
        k_um_split_cols<<<grid, 256, 0, st>>>(B, k, n, n_pad, k_pad, Bp);
        int rc = vi::check_launch("k_um_split_cols");
        if (rc) return rc;
    }
    CUtensorMap mapA, mapB;
    int rc = make_plane_map(&mapA, Ap, 8 * m_pad, k_pad, UM_TM);
    if (rc) return rc;
    rc = make_plane_map(&mapB, Bp, 8 * n_pad, k_pad, UM_TN);
    if (rc) return rc;
    if (status_dev) VI_CUDA(cudaMemsetAsync(status_dev, 0, sizeof(int32_t), st));
    VI_CUDA(cudaFuncSetAttribute(k_matmul_umma, cudaFuncAttributeMaxDynamicSharedMemorySize, UM_SMEM));
    dim3 grid((unsigned)(n_pad / UM_TN), (unsigned)(m_pad / UM_TM));
    k_matmul_umma<<<grid, UM_THREADS, UM_SMEM, st>>>(mapA, mapB, C, m, n, m_pad, n_pad, k_pad, status_dev);
    return vi::check_launch("k_matmul_umma");
}
