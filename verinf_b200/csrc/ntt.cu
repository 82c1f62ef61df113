// Goldilocks NTT and fused Reed-Solomon row encode for sm_100a.
//
// What it replaces in the reference: the batched NTT engine
// (prover/kernels/ntt.cuh:310-770, prover/cuda_primitives.py:347-409) and the
// encode pipeline built on it (prover/core.py:721-802, layergkr/gpu.py:141-203).
//
// Design (differs from the reference's bit-reverse + per-stage passes):
//  * A transform of length n is n = n1*n2 (four-step); each step is a *tile pass*:
//    a CTA owns a tile of C columns x L points, keeps it in shared memory and runs
//    a Stockham autosort DFT of length L with radix-16 register butterflies.
//  * Inside a radix-16 butterfly every twiddle is a power of two (w_16 = 2^156 in
//    this field), so the register stages use shifts only; one full 64x64->128
//    modular multiply per element per shared-memory stage remains.
//  * Natural order in, natural order out; no bit-reversal pass, no scale pass
//    (n^-1 is folded into the last stage), intermediates of a row chunk stay in a
//    caller-provided scratch buffer sized to remain L2-resident.
//  * The encode runs three passes per row chunk: iNTT step 1 (message + pad
//    loader), iNTT step 2 fused with the coset twist and step 1 of all rho coset
//    NTTs, and step 2 of the coset NTTs writing the interleaved codeword.
#include <cstdlib>
#include <map>
#include <mutex>
#include <tuple>
#include <vector>

#include "../../include/verinf_b200.h"
#include "blake3.cuh"
#include "common.cuh"
#include "dft_reg.cuh"
#include "gl.cuh"
#include "kquant.cuh"
#include "ntt_lanes.cuh"

// Lane-form variants of the tile passes (k_pass_q, k_encode_mid_q; arithmetic of gl_lanes.cuh) are
// compiled in only with -DVI_LANES=1.  They are bit-identical and execute 16-17 % fewer
// instructions, spread over both integer pipes, but hold 64 data registers per thread, run at 16
// warps per SM and came out 11-18 % slower than the 64-bit kernels on B200 (pass 1 / middle / pass 3 of
// a 4096 x 2^16 -> 2^18 encode: 2.31 / 12.1 / 6.68 ms against 2.04 / 10.25 / 5.99 ms), so the default
// build leaves them out.
#ifndef VI_LANES
#define VI_LANES 0
#endif

namespace {

using vgl::add;
using vgl::mul;
using vgl::sub;
using vdft::brev;
using vdft::dif;

// Stage schedule of a length-2^LOGL tile DFT: radix-16 stages plus one smaller
// stage (first or last).  A thread owns EPT elements of one column.
template <int LOGL, bool SMALL_LAST>
struct Sched {
    static constexpr int B = LOGL % 4;
    static constexpr int NS = LOGL == 0 ? 0 : (LOGL < 4 ? 1 : LOGL / 4 + (B ? 1 : 0));
    static constexpr int EPT = LOGL >= 4 ? 16 : (1 << LOGL);
    static constexpr int TPC = (1 << LOGL) / EPT;   // threads per column
    __host__ __device__ static constexpr int logr(int s) {
        if (LOGL < 4) return LOGL;
        if (B == 0) return 4;
        if (SMALL_LAST) return s == NS - 1 ? B : 4;
        return s == 0 ? B : 4;
    }
    __host__ __device__ static constexpr int logp(int s) {
        int p = 0;
        for (int i = 0; i < s; ++i) p += logr(i);
        return p;
    }
    // register j of the first stage holds input index first_pos(j, w)
    __host__ __device__ static constexpr int first_pos(int j, int w) {
        if (NS == 0) return 0;
        int r = 1 << logr(0);
        return (w + (j / r) * TPC) + (j % r) * ((1 << LOGL) / r);
    }
    // register j after the last stage holds output index last_k(j, w)
    __host__ __device__ static constexpr int last_k(int j, int w) {
        if (NS == 0) return 0;
        int lr = logr(NS - 1), r = 1 << lr;
        return (w + (j / r) * TPC) + brev(j % r, lr) * ((1 << LOGL) / r);
    }
};

template <bool INV>
__device__ __forceinline__ uint64_t tw_at(const uint64_t* __restrict__ tw, uint32_t e, uint32_t mask) {
    return INV ? __ldg(tw + ((0u - e) & mask)) : __ldg(tw + e);   // w^-e = w^(n-e)
}

// Stages S..NS-1 of the tile DFT.  v is preloaded for stage S; on return it holds
// the outputs of the last stage (see Sched::last_k).  sm is the tile [pos*CP + col].
// RHO0 > 0 (forward only): the transform is the coset t of a length RHO0*L transform, input
// pre-multiplied by w_{RHO0*L}^(t*l) except for the factor common to a thread's first butterfly,
// w_{RHO0*L}^(t*qp), which is folded into the stage-0 twiddle here: w_L^(qp*c) * w_{RHO0*L}^(t*qp)
// = tw0[qp*(RHO0*c + t)] with tw0 the table of w_{RHO0*L}.
template <int LOGL, bool INV, bool SMALL_LAST, int S, int RHO0 = 0>
__device__ __forceinline__ void run_stages(uint64_t (&v)[Sched<LOGL, SMALL_LAST>::EPT], uint64_t* sm,
                                           int CP, int col, int w, const uint64_t* __restrict__ twL,
                                           const uint64_t* __restrict__ tw0 = nullptr, int t = 0) {
    using SC = Sched<LOGL, SMALL_LAST>;
    if constexpr (S < SC::NS) {
        constexpr int LOGR = SC::logr(S), R = 1 << LOGR, G = SC::EPT / R, LOGP = SC::logp(S);
        constexpr int L = 1 << LOGL, PP = 1 << LOGP;
        constexpr bool LAST = (S == SC::NS - 1);
        if constexpr (S > 0) {
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int i = 0; i < R; ++i)
                    v[g * R + i] = sm[((w + g * SC::TPC) + i * (L / R)) * CP + col];
        }
#pragma unroll
        for (int g = 0; g < G; ++g) dif<LOGR, LOGR, INV>(&v[g * R]);
        if constexpr (!LAST) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                uint32_t qp = (uint32_t)(w + g * SC::TPC) >> LOGP;
                if constexpr (S == 0 && RHO0 > 0) {
                    static_assert(!INV && LOGP == 0, "coset twiddles: forward stage 0 only");
#pragma unroll
                    for (int c = 0; c < R; ++c)
                        v[g * R + brev(c, LOGR)] = mul(v[g * R + brev(c, LOGR)], __ldg(tw0 + qp * (uint32_t)(RHO0 * c + t)));
                } else {
#pragma unroll
                    for (int c = 1; c < R; ++c) {
                        uint32_t e = (qp * c) << LOGP;
                        v[g * R + brev(c, LOGR)] = mul(v[g * R + brev(c, LOGR)], tw_at<INV>(twL, e, L - 1));
                    }
                }
            }
            __syncthreads();
#pragma unroll
            for (int g = 0; g < G; ++g) {
                int x = w + g * SC::TPC;
                int kappa = x & (PP - 1), qp = x >> LOGP;
#pragma unroll
                for (int c = 0; c < R; ++c)
                    sm[(qp * PP * R + kappa + PP * c) * CP + col] = v[g * R + brev(c, LOGR)];
            }
            __syncthreads();
            run_stages<LOGL, INV, SMALL_LAST, S + 1, RHO0>(v, sm, CP, col, w, twL, tw0, t);
        }
    }
}

// ---------------------------------------------------------------------------
// Generic tile pass.
// ---------------------------------------------------------------------------
enum { SRC_PLAIN = 0, SRC_MSG = 1, SRC_KQ = 2 };

struct PassArgs {
    const uint64_t* in;
    uint64_t* out;
    int logC;
    int64_t ncols;           // columns per item
    int64_t tiles_per_item;
    int64_t in_item, out_item;        // element stride between items (64-bit)
    uint32_t in_idx, in_col;          // element strides inside a tile (32-bit offsets from the tile base)
    uint32_t out_k, out_col;
    const uint64_t* twL;     // w_L^e, e < L
    const uint64_t* fs;      // four-step factors, fs[k*ncols + col] = w_n^(+-col*k), or null
    const uint64_t* fs_hi;   // split factor form (LD = 3, transforms above 2^24): w_n^(+-e) = fs[e & 8191] * fs_hi[e >> 13]
    uint64_t scale;          // multiply outputs by this unless 1
    int out_via_smem;        // outputs are contiguous along k: transpose through smem
    // SRC_MSG loader: input element (item=row, pos, col) is slot j = pos*in_idx + col of the
    // padded message row: j < ell -> msg[row*ell + j]; else zero or the pad PRG.
    int src_kind;
    int64_t ell;
    int pad_mode;            // 0 zeros, 1 PRG
    const uint8_t* seed;     // device pointer, 32 bytes (pad_mode 1)
    int64_t row_off;
    // SRC_KQ loader: slot j < ell of row `item` is element f = (kq_first_row + item)*ell + j of the
    // lifted (d_out, d_in) K-quant matrix (transposed view when kq_transpose), zero past its end.
    const uint8_t* kq_raw;
    int kq_type;
    int kq_transpose;
    double kq_S;
    int64_t kq_dout, kq_din, kq_first_row;
    const float* kq_table;   // pre-multiplied sub-block scales (vkq::fill_table) or null
    const uint8_t* kq_qT;    // transposed staging (vkq::lift_staged): one byte per weight in traversal order,
    const void* kq_sT;       //   and the scales per (sub-block of k, n); null = decode from the super-blocks
    uint64_t kq_magic;       // floor(2^64 / kq_dout) + 1 when the matrix has fewer than 2^32 elements (then
                             // f / kq_dout = umul64hi(f, kq_magic) exactly), else 0: 64-bit division
    // lane-form passes (k_pass_q): the same tables as balanced 24-bit digits, and the scale likewise
    const vln::W3* twL3;
    const vln::W3* fs3;
    vln::W3 scale3;
};

// Minimum resident CTAs per SM asked of the compiler for the 256-thread tiles (register budget =
// 65536 / (256 * blocks)).  Measured on B200 at K = 2^16: k_pass 1/3/4/5/6/8 blocks -> commit
// 32.6 / 30.2 / 27.5 / 27.3 / 28.5 / 32.0 ms; k_encode_mid is best at 2 (128 registers).
#ifndef VI_PASS_MINB
#define VI_PASS_MINB 5
#endif
#ifndef VI_PASS_MINB_L8
#define VI_PASS_MINB_L8 4    // MODE 1 passes of 256-point tiles (encode pass 3 at K = 2^16: 3/4/5/6 blocks ->
#endif                       // 6.03 / 5.98 / 6.21 / 6.56 ms; 128-point tiles prefer 5)
#ifndef VI_MID_MINB
#define VI_MID_MINB 2
#endif
#ifndef VI_PASS0_MINB
#define VI_PASS0_MINB 4      // MODE 0 passes (strided loads straight into registers; encode pass 1 at
#endif                       // K = 2^16: 3/4/5/6/8 blocks -> 2.95 / 2.79 / 2.89 / 3.77 / 5.11 ms)
// Columns per tile: fixed by the tile length from 128 points up (so that all tile index arithmetic is
// compile-time), chosen by the host from the column count below that (tile_logC on the host).
__host__ __device__ constexpr int fixed_logC(int logl) { return logl < 7 ? -1 : logl == 7 ? 5 : logl <= 9 ? 4 : 13 - logl; }
// MODE 0: input contiguous along columns; 1: along the DFT index
// tiles of DFT length 2^4..2^8 always run 256 threads (4096 elements / 16 per thread)
__host__ __device__ constexpr int tile_max_threads(int logl) { return (logl >= 4 && logl <= 8) ? 256 : 512; }

// LD selects the loader of a MODE 0 pass at compile time, so that the plain loaders do not carry the
// registers, code and barrier of the others: 0 = plain rows or message rows without pad, 1 = message
// rows with the PRG pad, 2 = K-quant lift (pad decided at run time), 3 = plain rows with the four-step
// factor taken from two small tables (the first pass of a three-pass transform, whose full factor table
// would have n entries)
template <int LOGL, bool INV, int MODE, int LD = 0>
__global__ void __launch_bounds__(tile_max_threads(LOGL), (LOGL >= 4 && LOGL <= 8) ? (MODE == 0 ? VI_PASS0_MINB : (LOGL == 8 ? VI_PASS_MINB_L8 : VI_PASS_MINB)) : 1) k_pass(PassArgs a) {
    using SC = Sched<LOGL, false>;
    constexpr int L = 1 << LOGL, EPT = SC::EPT;
    extern __shared__ uint64_t sm[];
    const int logC = fixed_logC(LOGL) >= 0 ? fixed_logC(LOGL) : a.logC;
    const int tid = threadIdx.x, C = 1 << logC, CP = C + 1;
    const int col = tid & (C - 1), w = tid >> logC;
    const uint32_t tpi = (uint32_t)a.tiles_per_item;          // the grid has fewer than 2^31 tiles: 32-bit division
    const uint32_t item32 = blockIdx.x / tpi;
    const int64_t item = item32;
    const int64_t col0 = (int64_t)(blockIdx.x - item32 * tpi) * C;
    const int64_t colg = col0 + col;
    const bool valid = colg < a.ncols;
    const int ncols_tile = a.ncols - col0 < C ? (int)(a.ncols - col0) : C;   // valid columns of this tile
    const uint32_t ncols32 = (uint32_t)a.ncols;
    uint64_t v[EPT];
    if constexpr (MODE == 0) {
        if ((LD == 0 || LD == 3) && a.src_kind == SRC_PLAIN) {
            const uint64_t* src = a.in + item * a.in_item + colg * (int64_t)a.in_col;
#pragma unroll
            for (int j = 0; j < EPT; ++j)
                v[j] = valid ? src[(uint32_t)SC::first_pos(j, w) * a.in_idx] : 0;
        } else {
            const uint64_t* src = a.in + item * a.ell;
            uint32_t seed[8] = {0, 0, 0, 0, 0, 0, 0, 0};
            // pad PRG: the part of the first BLAKE3 round that does not depend on the slot is computed once
            // per CTA (one CTA = one row) into the tile buffer, which is free until the first stage exchange
            uint32_t* prg_prefix = reinterpret_cast<uint32_t*>(sm);
            const bool pad = LD == 1 || (LD == 2 && a.pad_mode == 1);
            if (pad) {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    seed[i] = (uint32_t)__ldg(a.seed + 4 * i) | ((uint32_t)__ldg(a.seed + 4 * i + 1) << 8) |
                              ((uint32_t)__ldg(a.seed + 4 * i + 2) << 16) | ((uint32_t)__ldg(a.seed + 4 * i + 3) << 24);
                if (tid == 0) {
                    uint32_t pv[16];
                    vb3::pad_prg_prefix(seed, (uint64_t)(a.row_off + item), pv);
#pragma unroll
                    for (int i = 0; i < 16; ++i) prg_prefix[i] = pv[i];
                }
                __syncthreads();
            }
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                int64_t slot = (int64_t)SC::first_pos(j, w) * a.in_idx + colg;
                uint64_t x = 0;
                if (valid) {
                    if (slot < a.ell) {
                        if constexpr (LD != 2) x = src[slot];
                        else {
                            int64_t f = (a.kq_first_row + item) * a.ell + slot;
                            if (f < a.kq_dout * a.kq_din) {
                                if (a.kq_qT) {            // staged transposed layout: f = k*d_out + n
                                    const uint32_t f32 = (uint32_t)f;
                                    const uint32_t kk = (uint32_t)__umul64hi((uint64_t)f32, a.kq_magic);
                                    x = vkq::lift_staged(a.kq_type, a.kq_qT, a.kq_sT, f32, kk,
                                                         f32 - kk * (uint32_t)a.kq_dout, (uint32_t)a.kq_dout, a.kq_S);
                                } else {
                                    int64_t widx = f;
                                    if (a.kq_transpose) {
                                        if (a.kq_magic) {
                                            const uint32_t f32 = (uint32_t)f;
                                            const uint32_t q = (uint32_t)__umul64hi((uint64_t)f32, a.kq_magic);
                                            const uint32_t r = f32 - q * (uint32_t)a.kq_dout;
                                            widx = (int64_t)((uint64_t)r * (uint64_t)a.kq_din + q);
                                        } else {
                                            widx = (f % a.kq_dout) * a.kq_din + f / a.kq_dout;
                                        }
                                    }
                                    x = a.kq_table ? vkq::lift_any_tab(a.kq_type, a.kq_raw, a.kq_table, widx, a.kq_S)
                                                   : vkq::lift_any(a.kq_type, a.kq_raw, widx, a.kq_S);
                                }
                            }
                        }
                    } else if (pad) x = vb3::pad_prg_from(prg_prefix, seed, (uint64_t)(a.row_off + item), (uint64_t)(slot - a.ell));
                }
                v[j] = x;
            }
        }
    } else {
        const int nthr = blockDim.x;
        const uint64_t* src = a.in + item * a.in_item + col0 * (int64_t)a.in_col;
        if (LOGL >= 4 && logC == 4) {
            // 16 columns: the block has L threads, thread tid loads index tid of every column
            const uint64_t* p = src + (uint32_t)tid * a.in_idx;
            if (ncols_tile == 16) {
#pragma unroll
                for (int cl = 0; cl < 16; ++cl) sm[tid * 17 + cl] = p[(uint32_t)cl * a.in_col];
            } else {
#pragma unroll
                for (int cl = 0; cl < 16; ++cl) sm[tid * 17 + cl] = cl < ncols_tile ? p[(uint32_t)cl * a.in_col] : 0;
            }
        } else {
            for (int e = tid; e < L * C; e += nthr) {
                int idx = e & (L - 1), cl = e >> LOGL;
                sm[idx * CP + cl] = cl < ncols_tile ? src[(uint32_t)cl * a.in_col + (uint32_t)idx * a.in_idx] : 0;
            }
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < EPT; ++j) v[j] = sm[SC::first_pos(j, w) * CP + col];
    }

    run_stages<LOGL, INV, false, 0>(v, sm, CP, col, w, a.twL);

#pragma unroll
    // Every MODE 0 pass is the first step of a four-step transform: four-step factor, no scaling, strided
    // store.  MODE 1 passes are last steps: no factor, n^-1 on inverse transforms, and a store through
    // shared memory only for the single-pass transform (rows contiguous along the output index).
    for (int j = 0; j < EPT; ++j) {
        uint32_t k = SC::last_k(j, w);
        if constexpr (MODE == 0 && LD == 3) {
            if (valid) {
                const uint64_t e = (uint64_t)k * (uint64_t)colg;       // < n
                v[j] = mul(mul(v[j], __ldg(a.fs + (e & 8191))), __ldg(a.fs_hi + (e >> 13)));
            }
        } else if constexpr (MODE == 0) {
            if (valid) v[j] = mul(v[j], __ldg(a.fs + col0 + (k * ncols32 + (uint32_t)col)));
        } else if constexpr (INV) {
            if (a.scale != 1) v[j] = mul(v[j], a.scale);
        }
    }
    if (MODE == 0 || !a.out_via_smem) {
        if (valid) {
            uint64_t* dst = a.out + item * a.out_item + colg * (int64_t)a.out_col;
#pragma unroll
            for (int j = 0; j < EPT; ++j) dst[(uint32_t)SC::last_k(j, w) * a.out_k] = v[j];
        }
    } else {
        __syncthreads();
#pragma unroll
        for (int j = 0; j < EPT; ++j) sm[SC::last_k(j, w) * CP + col] = v[j];
        __syncthreads();
        const int nthr = blockDim.x;
        uint64_t* dst = a.out + item * a.out_item + col0 * (int64_t)a.out_col;
        for (int e = tid; e < L * C; e += nthr) {
            int k = e & (L - 1), cl = e >> LOGL;
            if (cl < ncols_tile) dst[(uint32_t)cl * a.out_col + (uint32_t)k * a.out_k] = sm[k * CP + cl];
        }
    }
}

// Resident CTAs asked of the compiler for the lane-form passes (16-byte tile elements: 3 tiles of
// 4096 elements fit in shared memory; 64 data registers per thread).
#ifndef VI_PASSQ_MINB
#define VI_PASSQ_MINB 2
#endif
#ifndef VI_MIDQ_MINB
#define VI_MIDQ_MINB 2
#endif

// The tile pass of k_pass in lane form (gl_lanes.cuh), for the plain loaders (LD = 0): values are
// converted from the canonical 64-bit form as they are loaded and back as they are stored; the
// stages in between (butterflies, stage twiddles, four-step factor, n^-1) never leave lane form.
template <int LOGL, bool INV, int MODE>
__global__ void __launch_bounds__(tile_max_threads(LOGL), (LOGL >= 4 && LOGL <= 8) ? VI_PASSQ_MINB : 1) k_pass_q(PassArgs a) {
    using SC = Sched<LOGL, false>;
    using vln::Q;
    constexpr int L = 1 << LOGL, EPT = SC::EPT;
    extern __shared__ int4 smq[];
    const int logC = fixed_logC(LOGL) >= 0 ? fixed_logC(LOGL) : a.logC;
    const int tid = threadIdx.x, C = 1 << logC, CP = C + 1;
    const int col = tid & (C - 1), w = tid >> logC;
    const uint32_t tpi = (uint32_t)a.tiles_per_item;
    const uint32_t item32 = blockIdx.x / tpi;
    const int64_t item = item32;
    const int64_t col0 = (int64_t)(blockIdx.x - item32 * tpi) * C;
    const int64_t colg = col0 + col;
    const bool valid = colg < a.ncols;
    const int ncols_tile = a.ncols - col0 < C ? (int)(a.ncols - col0) : C;
    const uint32_t ncols32 = (uint32_t)a.ncols;
    Q v[EPT];
    if constexpr (MODE == 0) {
        if (a.src_kind == SRC_PLAIN) {
            const uint64_t* src = a.in + item * a.in_item + colg * (int64_t)a.in_col;
#pragma unroll
            for (int j = 0; j < EPT; ++j)
                v[j] = vln::from_u64(valid ? src[(uint32_t)SC::first_pos(j, w) * a.in_idx] : 0);
        } else {       // message rows, zero past ELL
            const uint64_t* src = a.in + item * a.ell;
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                const int64_t slot = (int64_t)SC::first_pos(j, w) * a.in_idx + colg;
                v[j] = vln::from_u64((valid && slot < a.ell) ? src[slot] : 0);
            }
        }
    } else {
        const int nthr = blockDim.x;
        const uint64_t* src = a.in + item * a.in_item + col0 * (int64_t)a.in_col;
        if (LOGL >= 4 && logC == 4) {
            // 16 columns: the block has L threads, thread tid loads index tid of every column
            const uint64_t* p = src + (uint32_t)tid * a.in_idx;
            if (ncols_tile == 16) {
#pragma unroll
                for (int cl = 0; cl < 16; ++cl) vlt::sts_q(smq, tid * 17 + cl, vln::from_u64(p[(uint32_t)cl * a.in_col]));
            } else {
#pragma unroll
                for (int cl = 0; cl < 16; ++cl)
                    vlt::sts_q(smq, tid * 17 + cl, vln::from_u64(cl < ncols_tile ? p[(uint32_t)cl * a.in_col] : 0));
            }
        } else {
            for (int e = tid; e < L * C; e += nthr) {
                const int idx = e & (L - 1), cl = e >> LOGL;
                vlt::sts_q(smq, idx * CP + cl,
                           vln::from_u64(cl < ncols_tile ? src[(uint32_t)cl * a.in_col + (uint32_t)idx * a.in_idx] : 0));
            }
        }
        __syncthreads();
#pragma unroll
        for (int j = 0; j < EPT; ++j) v[j] = vlt::lds_q(smq, SC::first_pos(j, w) * CP + col);
    }

    vlt::run_stages_q<SC, LOGL, INV, 0>(v, smq, CP, col, w, a.twL3);

    uint64_t o[EPT];
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        const uint32_t k = SC::last_k(j, w);
        if constexpr (MODE == 0) {
            // first step of a four-step transform: four-step factor (also for invalid columns: any entry)
            const vln::W3 f = vlt::ldg_w3(a.fs3 + (valid ? col0 + (k * ncols32 + (uint32_t)col) : 0));
            o[j] = vln::to_u64(vln::mul(v[j], f));
        } else if constexpr (INV) {
            o[j] = vln::to_u64(vln::mul(v[j], a.scale3));      // n^-1
        } else {
            o[j] = vln::to_u64(v[j]);
        }
    }
    if (MODE == 0 || !a.out_via_smem) {
        if (valid) {
            uint64_t* dst = a.out + item * a.out_item + colg * (int64_t)a.out_col;
#pragma unroll
            for (int j = 0; j < EPT; ++j) dst[(uint32_t)SC::last_k(j, w) * a.out_k] = o[j];
        }
    } else {
        uint64_t* sm = reinterpret_cast<uint64_t*>(smq);
        __syncthreads();
#pragma unroll
        for (int j = 0; j < EPT; ++j) sm[SC::last_k(j, w) * CP + col] = o[j];
        __syncthreads();
        const int nthr = blockDim.x;
        uint64_t* dst = a.out + item * a.out_item + col0 * (int64_t)a.out_col;
        for (int e = tid; e < L * C; e += nthr) {
            const int k = e & (L - 1), cl = e >> LOGL;
            if (cl < ncols_tile) dst[(uint32_t)cl * a.out_col + (uint32_t)k * a.out_k] = sm[k * CP + cl];
        }
    }
}

// Transposed staging pre-pass: CTA = 32 output rows n x one super-block column (256 values of k).
// Quants go through a shared-memory transpose so that both the reads (a super-block's bytes)
// and the writes (32 consecutive n for one k) are contiguous.
template <int QT>
__global__ void __launch_bounds__(256) k_kq_stage_T(const uint8_t* __restrict__ raw, int64_t d_out, int64_t d_in,
                                                    uint8_t* __restrict__ qT, void* __restrict__ sT) {
    __shared__ uint8_t tile[256][33];
    const int tid = threadIdx.x;
    const int64_t n0 = (int64_t)blockIdx.x * 32, kb = blockIdx.y, bpr = d_in >> 8;   // super-blocks per matrix row
    for (int nl = 0; nl < 32; ++nl) {
        const int64_t n = n0 + nl;
        if (n < d_out) tile[tid][nl] = (uint8_t)vkq::raw_quant<QT>(raw + (n * bpr + kb) * vkq::block_bytes(QT), tid);
    }
    __syncthreads();
    const int nl = tid & 31;
    if (n0 + nl < d_out) {
#pragma unroll 4
        for (int i = 0; i < 32; ++i) {
            const int kk = (tid >> 5) + 8 * i;
            qT[(kb * 256 + kk) * d_out + n0 + nl] = tile[kk][nl];
        }
        const uint8_t* p = raw + ((n0 + nl) * bpr + kb) * vkq::block_bytes(QT);
        constexpr int SUBS = QT == vkq::Q6_K ? 16 : 8;
        for (int sub = tid >> 5; sub < SUBS; sub += 8) {
            float t[16];
            vkq::fill_table<QT>(p, sub, t);
            if constexpr (QT == vkq::Q6_K)
                reinterpret_cast<float*>(sT)[(kb * 16 + sub) * d_out + n0 + nl] = t[sub];
            else
                reinterpret_cast<float2*>(sT)[(kb * 8 + sub) * d_out + n0 + nl] = make_float2(t[2 * sub], t[2 * sub + 1]);
        }
    }
}

// one thread per (super-block, sub-block): pre-multiplied scales for the fused K-quant loader
__global__ void __launch_bounds__(256) k_kq_table(const uint8_t* __restrict__ raw, int qtype, int64_t n_blocks,
                                                  float* __restrict__ table) {
    const int per = qtype == vkq::Q6_K ? 16 : 8;
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_blocks * per) return;
    const int64_t b = i / per;
    const int sub = (int)(i - b * per);
    const uint8_t* p = raw + b * vkq::block_bytes(qtype);
    float* t = table + b * (vkq::TABLE_BYTES_PER_BLOCK / 4);
    if (qtype == vkq::Q4_K) vkq::fill_table<vkq::Q4_K>(p, sub, t);
    else if (qtype == vkq::Q5_K) vkq::fill_table<vkq::Q5_K>(p, sub, t);
    else vkq::fill_table<vkq::Q6_K>(p, sub, t);
}

// ---------------------------------------------------------------------------
// Encode middle pass: iNTT step 2 -> coefficients (x K^-1) -> for each coset t:
// twist by (7*w_N^t)^l, NTT step 1, four-step factor, store for step 2.
// Coefficients stay in registers across the rho cosets.
// ---------------------------------------------------------------------------
struct MidArgs {
    const uint64_t* s1;    // (rows, K): [k1*L + j2]
    uint64_t* polys;       // (rows, K) natural order, or null
    uint64_t* s2;          // (rows, rho*K): [(m1*rho + t)*n1 + l2], or null
    int logC;
    int64_t n1;            // number of columns (= K / L)
    int64_t tiles_per_item;
    int rho;
    int64_t K;
    const uint64_t* twL;   // w_L^e
    const uint64_t* fsK;   // forward four-step factors, fsK[m1*n1 + l2] = w_K^(l2*m1)
    const uint64_t* twist; // (rho, K): (7*w_N^t)^l
    uint64_t k_inv;
    // shift-twist form (RHO template parameter 2 or 4):
    const uint64_t* cscale;  // K entries: K^-1 * 7^l
    const uint64_t* twRL;    // w_{rho*L}^e, e < rho*L (stage-0 twiddles of the coset transforms)
    const uint64_t* fsN;     // N entries: fsN[kk*n1 + l2] = w_N^(l2*kk), kk = rho*m1 + t
    // lane-form kernel (k_encode_mid_q): the same tables as balanced 24-bit digits
    const vln::W3 *twL3, *cscale3, *twRL3, *fsN3;
    vln::W3 k_inv3;
};

// x * 2^E mod p for a compile-time E in [0, 192) (2^96 = -1)
template <int E>
__device__ __forceinline__ uint64_t mul_pow2_any(uint64_t x) {
    if constexpr (E == 0) return x;
    else if constexpr (E < 96) return vgl::mul_pow2<E>(x);
    else return vgl::sub(0, vgl::mul_pow2<E - 96>(x));
}
// v[j] = c[j] * w_{16*RHO}^(T*j), j < 16: the part of the coset twist that varies inside a thread's
// first radix-16 butterfly; w_{16*RHO} is a power of two for RHO <= 4, so these are shifts.
// The coefficients are read from the thread's own column of a shared-memory array (c[J * stride]): holding
// them in registers across the cosets costs 32 registers and one resident CTA.
template <int RHO, int T, int J = 0>
__device__ __forceinline__ void coset_shift(const uint64_t* __restrict__ c, int stride, uint64_t (&v)[16]) {
    if constexpr (J < 16) {
        constexpr int E = (vdft::root_exp(RHO == 4 ? 6 : RHO == 2 ? 5 : 4) * T * J) % 192;
        v[J] = mul_pow2_any<E>(c[J * stride]);
        coset_shift<RHO, T, J + 1>(c, stride, v);
    }
}

// RHO = 0: any blow-up factor, twist read from the (rho, K) table (one full multiply per element
// and coset).  RHO = 2 or 4 (tile length >= 16): the twist (7 w_N^t)^l with l = l1*n1 + l2,
// l1 = w + j*(L/16), is split into  K^-1 7^l (folded into the coefficient scaling, once),
// w_N^(t*l2) (folded into the four-step factor table), w_{RHO L}^(t*w) (folded into the stage-0
// twiddle) and w_{16 RHO}^(t*j), a power of two applied as a shift: no twist multiply remains.
template <int LOGL, int RHO>
__global__ void __launch_bounds__(tile_max_threads(LOGL), (LOGL >= 4 && LOGL <= 8) ? VI_MID_MINB : 1) k_encode_mid(MidArgs a) {
    using SI = Sched<LOGL, false>;   // inverse: small stage first, radix-16 last
    using SF = Sched<LOGL, true>;    // forward: radix-16 first, small stage last
    constexpr int L = 1 << LOGL, EPT = SI::EPT;
    constexpr int LR = SI::NS ? SI::logr(SI::NS - 1) : 0;   // last inverse radix == first forward radix
    static_assert(RHO == 0 || (LOGL >= 4 && (RHO == 2 || RHO == 4)), "shift-twist form needs radix-16 first stages");
    extern __shared__ uint64_t sm[];
    const int logC = fixed_logC(LOGL) >= 0 ? fixed_logC(LOGL) : a.logC;
    const int tid = threadIdx.x, C = 1 << logC, CP = C + 1;
    const int col = tid & (C - 1), w = tid >> logC;
    const uint32_t tpi = (uint32_t)a.tiles_per_item;          // the grid has fewer than 2^31 tiles: 32-bit division
    const uint32_t item32 = blockIdx.x / tpi;
    const int64_t item = item32;
    const int64_t col0 = (int64_t)(blockIdx.x - item32 * tpi) * C;
    const int64_t colg = col0 + col;
    // From 128-point tiles up every tile is full: n1 >= L >= 128 > C columns, all powers of two.
    const bool valid = fixed_logC(LOGL) >= 0 ? true : colg < a.n1;
    const int ncols_tile = fixed_logC(LOGL) >= 0 ? C : (a.n1 - col0 < C ? (int)(a.n1 - col0) : C);
    const uint32_t n1 = (uint32_t)a.n1, rho = (uint32_t)a.rho;

    {
        const int nthr = blockDim.x;
        const uint64_t* src = a.s1 + item * a.K + col0 * L;
        if (LOGL >= 4 && logC == 4) {
            // 16 columns: the block has L threads, thread tid loads index tid of every column
            if (ncols_tile == 16) {
#pragma unroll
                for (int cl = 0; cl < 16; ++cl) sm[tid * 17 + cl] = src[cl * L + tid];
            } else {
#pragma unroll
                for (int cl = 0; cl < 16; ++cl) sm[tid * 17 + cl] = cl < ncols_tile ? src[cl * L + tid] : 0;
            }
        } else {
            for (int e = tid; e < L * C; e += nthr) {
                int idx = e & (L - 1), cl = e >> LOGL;
                sm[idx * CP + cl] = cl < ncols_tile ? src[(uint32_t)(cl * L + idx)] : 0;
            }
        }
        __syncthreads();
    }
    uint64_t c[EPT], v[EPT];
#pragma unroll
    for (int j = 0; j < EPT; ++j) c[j] = sm[SI::first_pos(j, w) * CP + col];
    run_stages<LOGL, true, false, 0>(c, sm, CP, col, w, a.twL);
    if constexpr (RHO == 0) {
#pragma unroll
        for (int j = 0; j < EPT; ++j) c[j] = mul(c[j], a.k_inv);
    }
    if (a.polys && valid) {
        uint64_t* dst = a.polys + item * a.K + colg;
#pragma unroll
        for (int j = 0; j < EPT; ++j) dst[(uint32_t)SI::last_k(j, w) * n1] = RHO == 0 ? c[j] : mul(c[j], a.k_inv);
    }
    if (!a.s2) return;
    uint64_t* dst2 = a.s2 + item * a.K * a.rho + colg;
    if constexpr (RHO == 0) {
        for (int t = 0; t < a.rho; ++t) {
            const uint64_t* tw_t = a.twist + (int64_t)t * a.K + colg;
            if (SF::NS > 1) __syncthreads();   // previous coset finished reading the tile
#pragma unroll
            for (int j = 0; j < EPT; ++j) {
                // forward register j needs coefficient index l1 = first_pos(j): it is held in c[brev(j)]
                uint32_t l1 = SF::first_pos(j, w);
                uint64_t tw = valid ? __ldg(tw_t + n1 * l1) : 0;
                v[j] = mul(c[(j / (1 << LR)) * (1 << LR) + brev(j % (1 << LR), LR)], tw);
            }
            run_stages<LOGL, false, true, 0>(v, sm, CP, col, w, a.twL);
            if (valid) {
#pragma unroll
                for (int j = 0; j < EPT; ++j) {
                    uint32_t m1 = SF::last_k(j, w);
                    uint64_t x = mul(v[j], __ldg(a.fsK + colg + m1 * n1));
                    dst2[(m1 * rho + (uint32_t)t) * n1] = x;
                }
            }
        }
    } else {
        // c2[j] = coefficient l1 = first_pos(j) (held in c[brev(j)]) times K^-1 7^l, l = l1*n1 + l2; kept in
        // shared memory behind the tile, element j of thread tid at c2[j * blockDim.x + tid]
        uint64_t* c2 = sm + (size_t)L * CP + tid;
        const int nthr = blockDim.x;
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            uint32_t l1 = SF::first_pos(j, w);
            uint64_t sc = valid ? __ldg(a.cscale + colg + n1 * l1) : 0;
            c2[j * nthr] = mul(c[brev(j, LR)], sc);
        }
#pragma unroll 1   // (fully unrolled: no spills, but 11.9 ms against 10.9 ms at K = 2^16)
        for (int t = 0; t < RHO; ++t) {
            if (SF::NS > 1) __syncthreads();   // previous coset finished reading the tile
            switch (t) {
                case 0: coset_shift<RHO, 0>(c2, nthr, v); break;
                case 1: coset_shift<RHO, 1>(c2, nthr, v); break;
                case 2: coset_shift<RHO, 2 % RHO>(c2, nthr, v); break;
                default: coset_shift<RHO, 3 % RHO>(c2, nthr, v); break;
            }
            run_stages<LOGL, false, true, 0, RHO>(v, sm, CP, col, w, a.twL, a.twRL, t);
            if (valid) {
#pragma unroll
                for (int j = 0; j < EPT; ++j) {
                    uint32_t m1 = SF::last_k(j, w);
                    uint32_t kk = m1 * RHO + (uint32_t)t;
                    uint64_t x = mul(v[j], __ldg(a.fsN + colg + kk * n1));
                    dst2[kk * n1] = x;
                }
            }
        }
    }
}

// v[j] = c[j] * w_{16*RHO}^(T*j) in lane form (lane rotations and at most one lane shift each)
template <int RHO, int T, int J = 0>
__device__ __forceinline__ void coset_shift_q(const uint64_t (&c)[16], vln::Q (&v)[16]) {
    if constexpr (J < 16) {
        constexpr int E = (vdft::root_exp(RHO == 4 ? 6 : RHO == 2 ? 5 : 4) * T * J) % 192;
        v[J] = vln::mul_pow2<E>(vln::from_u64(c[J]));
        coset_shift_q<RHO, T, J + 1>(c, v);
    }
}

// The shift-twist middle pass (k_encode_mid<LOGL, RHO>, RHO = 2 or 4) in lane form, for tile lengths
// from 128 points (every tile is full).  The scaled coefficients are kept between the cosets in
// canonical 64-bit form (32 registers instead of 64) and unpacked per coset.
template <int LOGL, int RHO>
__global__ void __launch_bounds__(tile_max_threads(LOGL), LOGL <= 8 ? VI_MIDQ_MINB : 1) k_encode_mid_q(MidArgs a) {
    using SI = Sched<LOGL, false>;   // inverse: small stage first, radix-16 last
    using SF = Sched<LOGL, true>;    // forward: radix-16 first, small stage last
    using vln::Q;
    constexpr int L = 1 << LOGL, EPT = SI::EPT;
    constexpr int LR = SI::logr(SI::NS - 1);   // last inverse radix == first forward radix
    static_assert(LOGL >= 7 && (RHO == 2 || RHO == 4) && EPT == 16, "lane-form middle pass: full 16-column tiles");
    extern __shared__ int4 smq[];
    constexpr int logC = fixed_logC(LOGL), C = 1 << logC, CP = C + 1;
    const int tid = threadIdx.x;
    const int col = tid & (C - 1), w = tid >> logC;
    const uint32_t tpi = (uint32_t)a.tiles_per_item;
    const uint32_t item32 = blockIdx.x / tpi;
    const int64_t item = item32;
    const int64_t col0 = (int64_t)(blockIdx.x - item32 * tpi) * C;
    const int64_t colg = col0 + col;
    const uint32_t n1 = (uint32_t)a.n1;
    {
        const int nthr = blockDim.x;
        const uint64_t* src = a.s1 + item * a.K + col0 * L;
        if (logC == 4) {
#pragma unroll
            for (int cl = 0; cl < 16; ++cl) vlt::sts_q(smq, tid * 17 + cl, vln::from_u64(src[cl * L + tid]));
        } else {
            for (int e = tid; e < L * C; e += nthr) {
                const int idx = e & (L - 1), cl = e >> LOGL;
                vlt::sts_q(smq, idx * CP + cl, vln::from_u64(src[(uint32_t)(cl * L + idx)]));
            }
        }
        __syncthreads();
    }
    Q v[EPT];
#pragma unroll
    for (int j = 0; j < EPT; ++j) v[j] = vlt::lds_q(smq, SI::first_pos(j, w) * CP + col);
    vlt::run_stages_q<SI, LOGL, true, 0>(v, smq, CP, col, w, a.twL3);
    if (a.polys) {
        uint64_t* dst = a.polys + item * a.K + colg;
#pragma unroll
        for (int j = 0; j < EPT; ++j) dst[(uint32_t)SI::last_k(j, w) * n1] = vln::to_u64(vln::mul(v[j], a.k_inv3));
    }
    if (!a.s2) return;
    uint64_t* dst2 = a.s2 + item * a.K * a.rho + colg;
    // c2[j] = coefficient l1 = first_pos(j) (held in v[brev(j)]) times K^-1 7^l, l = l1*n1 + l2
    uint64_t c2[EPT];
#pragma unroll
    for (int j = 0; j < EPT; ++j) {
        const uint32_t l1 = SF::first_pos(j, w);
        c2[j] = vln::to_u64(vln::mul(v[brev(j, LR)], vlt::ldg_w3(a.cscale3 + colg + n1 * l1)));
    }
#pragma unroll 1
    for (int t = 0; t < RHO; ++t) {
        __syncthreads();   // previous coset (or the inverse transform) finished reading the tile
        switch (t) {
            case 0: coset_shift_q<RHO, 0>(c2, v); break;
            case 1: coset_shift_q<RHO, 1>(c2, v); break;
            case 2: coset_shift_q<RHO, 2 % RHO>(c2, v); break;
            default: coset_shift_q<RHO, 3 % RHO>(c2, v); break;
        }
        vlt::run_stages_q<SF, LOGL, false, 0, RHO>(v, smq, CP, col, w, a.twL3, a.twRL3, t);
#pragma unroll
        for (int j = 0; j < EPT; ++j) {
            const uint32_t m1 = SF::last_k(j, w);
            const uint32_t kk = m1 * RHO + (uint32_t)t;
            dst2[kk * n1] = vln::to_u64(vln::mul(v[j], vlt::ldg_w3(a.fsN3 + colg + kk * n1)));
        }
    }
}

// ---------------------------------------------------------------------------
// Host side: twiddle cache, launch planning.
// ---------------------------------------------------------------------------
struct DevTables {
    std::map<int64_t, uint64_t*> tw;                          // n -> w_n^e, e < n
    std::map<std::pair<int64_t, int64_t>, uint64_t*> twist;   // (K, N) -> (rho, K)
    std::map<int64_t, uint64_t*> cscale;                      // K -> K^-1 * 7^l
    std::map<std::tuple<int64_t, int64_t, bool>, uint64_t*> fs;   // (n, ncols, inverse) -> four-step factors
    std::map<const uint64_t*, vln::W3*> w3;                   // table -> the same constants as balanced 24-bit digits
    std::map<std::pair<int64_t, bool>, std::pair<uint64_t*, uint64_t*>> split;   // (n, inverse) -> (w^e, e < 8192; w^(8192 e))
};
std::mutex g_mu;
std::map<int, DevTables> g_tables;

// Allocates a table and fills it from the host vector.  The copy is followed by a device-wide
// synchronisation: a pageable-memory cudaMemcpy is ordered against the legacy default stream only
// and may return before the DMA has finished, and the kernels that read the table run on the
// caller's (possibly non-blocking) stream.  First use of a length must therefore happen outside
// stream capture.  The buffer is freed again if the copy fails.
int upload_table(const std::vector<uint64_t>& h, uint64_t** out) {
    uint64_t* d = nullptr;
    VI_CUDA(cudaMalloc(&d, h.size() * 8));
    cudaError_t e = cudaMemcpy(d, h.data(), h.size() * 8, cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(d);
        return vi::fail(VI_ERR_CUDA, "twiddle table upload: %s", cudaGetErrorString(e));
    }
    *out = d;
    return VI_OK;
}

// The lane-form kernels read their constants as three balanced 24-bit digits (vln::W3, 16 bytes).
int upload_w3(const std::vector<uint64_t>& h, vln::W3** out) {
    std::vector<vln::W3> hw(h.size());
    for (size_t i = 0; i < h.size(); ++i) hw[i] = vln::make_w3(h[i]);
    vln::W3* d = nullptr;
    VI_CUDA(cudaMalloc(&d, hw.size() * sizeof(vln::W3)));
    cudaError_t e = cudaMemcpy(d, hw.data(), hw.size() * sizeof(vln::W3), cudaMemcpyHostToDevice);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(d);
        return vi::fail(VI_ERR_CUDA, "twiddle table upload: %s", cudaGetErrorString(e));
    }
    *out = d;
    return VI_OK;
}
// digits table of a u64 table returned by get_tw / get_fs (null if there is none)
const vln::W3* w3_of(const uint64_t* table) {
    int dev;
    if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
    std::lock_guard<std::mutex> lk(g_mu);
    auto& T = g_tables[dev];
    auto it = T.w3.find(table);
    return it == T.w3.end() ? nullptr : it->second;
}

int get_tw(int64_t n, const uint64_t** out) {
    int dev;
    VI_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_mu);
    auto& T = g_tables[dev];
    auto it = T.tw.find(n);
    if (it != T.tw.end()) { *out = it->second; return VI_OK; }
    std::vector<uint64_t> h((size_t)n);
    uint64_t wn = vgl::hpow(7, (vgl::P - 1) / (uint64_t)n), cur = 1;
    for (int64_t e = 0; e < n; ++e) { h[(size_t)e] = cur; cur = vgl::hmul(cur, wn); }
    uint64_t* d = nullptr;
    int rc_up = upload_table(h, &d);
    if (rc_up) return rc_up;
    vln::W3* d3 = nullptr;
#if VI_LANES
    rc_up = upload_w3(h, &d3);
    if (rc_up) { cudaFree(d); return rc_up; }
#endif
    T.tw[n] = d;
    if (d3) T.w3[d] = d3;
    *out = d;
    return VI_OK;
}

// four-step factor table for n = ncols*L: fs[k*ncols + c] = w_n^(c*k) (inverse: w_n^(-c*k)),
// laid out so that the 16 columns of a tile read 128 contiguous bytes per output index k
int get_fs(int64_t n, int64_t ncols, bool inv, const uint64_t** out) {
    int dev;
    VI_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_mu);
    auto& T = g_tables[dev];
    auto key = std::make_tuple(n, ncols, inv);
    auto it = T.fs.find(key);
    if (it != T.fs.end()) { *out = it->second; return VI_OK; }
    const int64_t L = n / ncols;
    std::vector<uint64_t> h((size_t)n);
    uint64_t wn = vgl::hpow(7, (vgl::P - 1) / (uint64_t)n);
    if (inv) wn = vgl::hpow(wn, vgl::P - 2);
    uint64_t step = 1;                     // w^k
    for (int64_t k = 0; k < L; ++k) {
        uint64_t cur = 1;
        for (int64_t c = 0; c < ncols; ++c) { h[(size_t)(k * ncols + c)] = cur; cur = vgl::hmul(cur, step); }
        step = vgl::hmul(step, wn);
    }
    uint64_t* d = nullptr;
    int rc_up = upload_table(h, &d);
    if (rc_up) return rc_up;
    vln::W3* d3 = nullptr;
#if VI_LANES
    rc_up = upload_w3(h, &d3);
    if (rc_up) { cudaFree(d); return rc_up; }
#endif
    T.fs[key] = d;
    if (d3) T.w3[d] = d3;
    *out = d;
    return VI_OK;
}

// w_n^(+-e) as a product of two table entries: lo[e & 8191] * hi[e >> 13] (n > 8192)
int get_split(int64_t n, bool inv, const uint64_t** lo, const uint64_t** hi) {
    int dev;
    VI_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_mu);
    auto& T = g_tables[dev];
    auto key = std::make_pair(n, inv);
    auto it = T.split.find(key);
    if (it != T.split.end()) { *lo = it->second.first; *hi = it->second.second; return VI_OK; }
    uint64_t wn = vgl::hpow(7, (vgl::P - 1) / (uint64_t)n);
    if (inv) wn = vgl::hpow(wn, vgl::P - 2);
    std::vector<uint64_t> hl(8192), hh((size_t)(n >> 13));
    uint64_t cur = 1;
    for (size_t e = 0; e < hl.size(); ++e) { hl[e] = cur; cur = vgl::hmul(cur, wn); }
    const uint64_t step = cur;       // w^8192
    cur = 1;
    for (size_t e = 0; e < hh.size(); ++e) { hh[e] = cur; cur = vgl::hmul(cur, step); }
    uint64_t *dl = nullptr, *dh = nullptr;
    int rc_up = upload_table(hl, &dl);
    if (rc_up) return rc_up;
    rc_up = upload_table(hh, &dh);
    if (rc_up) { cudaFree(dl); return rc_up; }
    T.split[key] = std::make_pair(dl, dh);
    *lo = dl; *hi = dh;
    return VI_OK;
}

int get_twist(int64_t K, int64_t N, const uint64_t** out) {
    int dev;
    VI_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_mu);
    auto& T = g_tables[dev];
    auto key = std::make_pair(K, N);
    auto it = T.twist.find(key);
    if (it != T.twist.end()) { *out = it->second; return VI_OK; }
    int64_t rho = N / K;
    std::vector<uint64_t> h((size_t)(rho * K));
    uint64_t wN = vgl::hpow(7, (vgl::P - 1) / (uint64_t)N);
    for (int64_t t = 0; t < rho; ++t) {
        uint64_t g = vgl::hmul(7, vgl::hpow(wN, (uint64_t)t)), cur = 1;
        for (int64_t l = 0; l < K; ++l) { h[(size_t)(t * K + l)] = cur; cur = vgl::hmul(cur, g); }
    }
    uint64_t* d = nullptr;
    int rc_up = upload_table(h, &d);
    if (rc_up) return rc_up;
    T.twist[key] = d;
    *out = d;
    return VI_OK;
}

// K^-1 * 7^l, l < K: coefficient scaling of the shift-twist form of the encode
int get_cscale(int64_t K, const uint64_t** out) {
    int dev;
    VI_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lk(g_mu);
    auto& T = g_tables[dev];
    auto it = T.cscale.find(K);
    if (it != T.cscale.end()) { *out = it->second; return VI_OK; }
    std::vector<uint64_t> h((size_t)K);
    uint64_t cur = vgl::hpow(vgl::hpow(2, (uint64_t)vi::ilog2(K)), vgl::P - 2);     // K^-1
    for (int64_t l = 0; l < K; ++l) { h[(size_t)l] = cur; cur = vgl::hmul(cur, 7); }
    uint64_t* d = nullptr;
    int rc_up = upload_table(h, &d);
    if (rc_up) return rc_up;
    vln::W3* d3 = nullptr;
#if VI_LANES
    rc_up = upload_w3(h, &d3);
    if (rc_up) { cudaFree(d); return rc_up; }
#endif
    T.cscale[K] = d;
    if (d3) T.w3[d] = d3;
    *out = d;
    return VI_OK;
}

constexpr int MAX_LOGL = 12;      // tile DFT length up to 4096 (2 columns per tile) -> two-pass transforms up to 2^24
constexpr int SINGLE_LOGL = 10;   // transforms up to this length run as one pass over 16-row tiles

// columns per tile for a DFT length 2^logL given ncols available
int pick_logC(int logL, int64_t ncols) {
    if (fixed_logC(logL) >= 0) return fixed_logC(logL);   // the kernels assume it
    int logC = 12 - logL;                              // 4096-element tiles
    int logTPC = logL >= 4 ? logL - 4 : 0;
    if (logC > 9 - logTPC) logC = 9 - logTPC;          // at most 512 threads
    int need = vi::ilog2(ncols);
    if (need < 4) need = 4;
    if (logC > need && logC > 4) logC = need;
    return logC;
}
int tile_threads(int logL, int logC) {
    int ept = logL >= 4 ? 16 : (1 << logL);
    return ((1 << logL) / ept) << logC;
}
size_t tile_smem(int logL, int logC) { return (size_t)(1 << logL) * ((1 << logC) + 1) * 8; }

template <int LOGL, bool INV, int MODE>
int launch_pass_q(const PassArgs& a, int64_t items, cudaStream_t st, int tag) {
    size_t smem = 2 * tile_smem(LOGL, a.logC);
    auto fn = k_pass_q<LOGL, INV, MODE>;
    if (smem > 48 * 1024) VI_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int64_t grid = items * a.tiles_per_item;
    if (grid <= 0) return VI_OK;
    if (grid > 0x7FFFFFFFLL) return vi::fail(VI_ERR_LIMIT, "tile grid too large (%lld)", (long long)grid);
    vi::ProfScope prof(tag, st);
    fn<<<(unsigned)grid, tile_threads(LOGL, a.logC), smem, st>>>(a);
    return vi::check_launch("k_pass_q");
}

template <int LOGL, bool INV, int MODE, int LD = 0>
int launch_pass_t(const PassArgs& a, int64_t items, cudaStream_t st, int tag) {
    if constexpr (VI_LANES && LD == 0 && LOGL >= 4 && LOGL <= 10) {
        if (a.twL3 != nullptr && (MODE == 1 || a.fs3 != nullptr) && (a.src_kind == SRC_PLAIN || a.src_kind == SRC_MSG))
            return launch_pass_q<LOGL, INV, MODE>(a, items, st, tag);
    }
    size_t smem = tile_smem(LOGL, a.logC);
    auto fn = k_pass<LOGL, INV, MODE, LD>;
    if (smem > 48 * 1024) VI_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int64_t grid = items * a.tiles_per_item;
    if (grid <= 0) return VI_OK;
    if (grid > 0x7FFFFFFFLL) return vi::fail(VI_ERR_LIMIT, "tile grid too large (%lld)", (long long)grid);
    vi::ProfScope prof(tag, st);
    fn<<<(unsigned)grid, tile_threads(LOGL, a.logC), smem, st>>>(a);
    return vi::check_launch("k_pass");
}

template <bool INV, int MODE>
int launch_pass_l(int logL, const PassArgs& a, int64_t items, cudaStream_t st, int tag) {
    if constexpr (INV && MODE == 0) {
        if (a.src_kind == SRC_KQ) {     // encode pass 1 lifting K-quant weights
            switch (logL) {
#define VI_CASE(x) case x: return launch_pass_t<x, true, 0, 2>(a, items, st, tag);
                VI_CASE(0) VI_CASE(1) VI_CASE(2) VI_CASE(3) VI_CASE(4) VI_CASE(5)
                VI_CASE(6) VI_CASE(7) VI_CASE(8) VI_CASE(9) VI_CASE(10) VI_CASE(11) VI_CASE(12)
#undef VI_CASE
            }
        }
        if (a.pad_mode == 1) {          // encode pass 1 with the PRG pad
            switch (logL) {
#define VI_CASE(x) case x: return launch_pass_t<x, true, 0, 1>(a, items, st, tag);
                VI_CASE(0) VI_CASE(1) VI_CASE(2) VI_CASE(3) VI_CASE(4) VI_CASE(5)
                VI_CASE(6) VI_CASE(7) VI_CASE(8) VI_CASE(9) VI_CASE(10) VI_CASE(11) VI_CASE(12)
#undef VI_CASE
            }
        }
    }
    if constexpr (MODE == 0) {
        if (a.fs_hi != nullptr) {       // first pass of a three-pass transform: split factor tables
            switch (logL) {
#define VI_CASE(x) case x: return launch_pass_t<x, INV, 0, 3>(a, items, st, tag);
                VI_CASE(1) VI_CASE(2) VI_CASE(3) VI_CASE(4) VI_CASE(5) VI_CASE(6)
                VI_CASE(7) VI_CASE(8) VI_CASE(9) VI_CASE(10) VI_CASE(11) VI_CASE(12)
#undef VI_CASE
            }
        }
    }
    switch (logL) {
#define VI_CASE(x) case x: return launch_pass_t<x, INV, MODE>(a, items, st, tag);
        VI_CASE(0) VI_CASE(1) VI_CASE(2) VI_CASE(3) VI_CASE(4) VI_CASE(5)
        VI_CASE(6) VI_CASE(7) VI_CASE(8) VI_CASE(9) VI_CASE(10) VI_CASE(11) VI_CASE(12)
#undef VI_CASE
    }
    return vi::fail(VI_ERR_LIMIT, "unsupported tile length 2^%d", logL);
}

int launch_pass(int logL, bool inv, int mode, PassArgs& a, int64_t items, cudaStream_t st, int tag) {
    a.tiles_per_item = (a.ncols + (1 << a.logC) - 1) >> a.logC;
    int rc = get_tw(int64_t(1) << logL, &a.twL);
    if (rc) return rc;
    a.twL3 = w3_of(a.twL);
    a.fs3 = (a.fs && !a.fs_hi) ? w3_of(a.fs) : nullptr;
    a.scale3 = vln::make_w3(a.scale);
    if (inv) return mode ? launch_pass_l<true, 1>(logL, a, items, st, tag) : launch_pass_l<true, 0>(logL, a, items, st, tag);
    return mode ? launch_pass_l<false, 1>(logL, a, items, st, tag) : launch_pass_l<false, 0>(logL, a, items, st, tag);
}

template <int LOGL, int RHO>
int launch_mid_t(const MidArgs& a, int64_t items, cudaStream_t st) {
    size_t smem = tile_smem(LOGL, a.logC);
    if (RHO != 0) smem += (size_t)16 * tile_threads(LOGL, a.logC) * 8;     // the scaled coefficients between the cosets
    auto fn = k_encode_mid<LOGL, RHO>;
    if (smem > 48 * 1024) VI_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int64_t grid = items * a.tiles_per_item;
    if (grid <= 0) return VI_OK;
    if (grid > 0x7FFFFFFFLL) return vi::fail(VI_ERR_LIMIT, "tile grid too large (%lld)", (long long)grid);
    vi::ProfScope prof(vi::PROF_ENC_MID, st);
    fn<<<(unsigned)grid, tile_threads(LOGL, a.logC), smem, st>>>(a);
    return vi::check_launch("k_encode_mid");
}
// blow-up factors and tile lengths for which the shift-twist kernels are built
bool mid_shift_form(int logL, int64_t rho) {
    return (rho == 2 || rho == 4) && logL >= 4 && logL <= 10;
}
template <int LOGL, int RHO>
int launch_mid_q(const MidArgs& a, int64_t items, cudaStream_t st) {
    size_t smem = 2 * tile_smem(LOGL, a.logC);
    auto fn = k_encode_mid_q<LOGL, RHO>;
    if (smem > 48 * 1024) VI_CUDA(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int64_t grid = items * a.tiles_per_item;
    if (grid <= 0) return VI_OK;
    if (grid > 0x7FFFFFFFLL) return vi::fail(VI_ERR_LIMIT, "tile grid too large (%lld)", (long long)grid);
    vi::ProfScope prof(vi::PROF_ENC_MID, st);
    fn<<<(unsigned)grid, tile_threads(LOGL, a.logC), smem, st>>>(a);
    return vi::check_launch("k_encode_mid_q");
}
int launch_mid(int logL, const MidArgs& a, int64_t items, cudaStream_t st) {
#if VI_LANES
    if (mid_shift_form(logL, a.rho) && logL >= 7 && a.twL3 && a.cscale3 && a.twRL3 && a.fsN3) {
        switch (logL * 8 + a.rho) {
#define VI_CASE(x) case x * 8 + 2: return launch_mid_q<x, 2>(a, items, st); case x * 8 + 4: return launch_mid_q<x, 4>(a, items, st);
            VI_CASE(7) VI_CASE(8) VI_CASE(9) VI_CASE(10)
#undef VI_CASE
        }
    }
#endif
    if (mid_shift_form(logL, a.rho)) {
        switch (logL * 8 + a.rho) {
#define VI_CASE(x) case x * 8 + 2: return launch_mid_t<x, 2>(a, items, st); case x * 8 + 4: return launch_mid_t<x, 4>(a, items, st);
            VI_CASE(4) VI_CASE(5) VI_CASE(6) VI_CASE(7) VI_CASE(8) VI_CASE(9) VI_CASE(10)
#undef VI_CASE
        }
    }
    switch (logL) {
#define VI_CASE(x) case x: return launch_mid_t<x, 0>(a, items, st);
        VI_CASE(0) VI_CASE(1) VI_CASE(2) VI_CASE(3) VI_CASE(4) VI_CASE(5)
        VI_CASE(6) VI_CASE(7) VI_CASE(8) VI_CASE(9) VI_CASE(10) VI_CASE(11) VI_CASE(12)
#undef VI_CASE
    }
    return vi::fail(VI_ERR_LIMIT, "unsupported tile length 2^%d", logL);
}

uint64_t inv_pow2(int log) {   // 2^-log mod p
    return vgl::hpow(vgl::hpow(2, (uint64_t)log), vgl::P - 2);
}

// Row-chunk size the *_scratch_bytes helpers recommend (intermediates of one chunk live in the
// scratch buffer).  Measured on B200 for 4096 rows x 2^16 -> 2^18: 40 MB chunks (L2-resident
// intermediates, ~15 rows) leave most SMs idle between the three dependent launches (57 ms per
// commit); 1 GB chunks (~400 rows, thousands of CTAs per launch) give 37 ms although the
// intermediates then round-trip through HBM, because every pass is integer-ALU bound, not
// HBM bound.  A caller that wants another chunk size passes a scratch buffer of that size.
int64_t chunk_bytes() { return int64_t(1024) << 20; }

}  // namespace

// Frees every twiddle / four-step / twist table this library allocated (all devices).  No kernel of
// the library may be in flight; the tables are rebuilt on the next use of a length.
extern "C" int vi_release_tables(void) {
    std::lock_guard<std::mutex> lk(g_mu);
    int cur = 0;
    VI_CUDA(cudaGetDevice(&cur));
    for (auto& kv : g_tables) {
        VI_CUDA(cudaSetDevice(kv.first));
        VI_CUDA(cudaDeviceSynchronize());
        for (auto& t : kv.second.tw) cudaFree(t.second);
        for (auto& t : kv.second.twist) cudaFree(t.second);
        for (auto& t : kv.second.fs) cudaFree(t.second);
        for (auto& t : kv.second.cscale) cudaFree(t.second);
        for (auto& t : kv.second.w3) cudaFree(t.second);
        for (auto& t : kv.second.split) { cudaFree(t.second.first); cudaFree(t.second.second); }
    }
    g_tables.clear();
    VI_CUDA(cudaSetDevice(cur));
    return VI_OK;
}

constexpr int THREE_PASS_MAX_LOG = 30;   // tile-relative offsets are 32-bit: n * 8 bytes per row up to 8 GiB

extern "C" int64_t vi_ntt_scratch_bytes(int64_t m, int64_t n) {
    if (n <= (int64_t(1) << SINGLE_LOGL) || m <= 0) return 0;
    if (n > (int64_t(1) << (2 * MAX_LOGL))) return 2 * n * 8;      // three passes, one row at a time, two buffers
    int64_t row = n * 8;
    int64_t rows = chunk_bytes() / row;
    if (rows < 1) rows = 1;
    if (rows > m) rows = m;
    return rows * row;
}

extern "C" int vi_ntt_batched(uint64_t* rows, int64_t m, int64_t n, int inverse,
                              void* scratch, int64_t scratch_bytes, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    VI_REQUIRE(m >= 0, "ntt: negative row count");
    VI_REQUIRE(vi::is_pow2(n) && n >= 2, "NTT length must be a power of 2 >= 2 (got %lld)", (long long)n);
    int logn = vi::ilog2(n);
    if (logn > THREE_PASS_MAX_LOG) return vi::fail(VI_ERR_LIMIT, "NTT length 2^%d exceeds the supported 2^%d", logn, THREE_PASS_MAX_LOG);
    if (m == 0) return VI_OK;
    VI_REQUIRE(rows != nullptr, "ntt: null data pointer");
    const bool inv = inverse != 0;
    const uint64_t scale = inv ? inv_pow2(logn) : 1;
    if (logn > 2 * MAX_LOGL) {
        // Three passes, row by row: n = n1 * na * nb.  Pass A: length-n1 transforms over the n2 = na*nb columns
        // (stride n2), four-step factor w_n^(j2*k1) from the split tables, into s1[k1][j2].  Then the length-n2
        // transform of every row k1 of s1 as the usual two passes (through s2), the last one writing
        // X[k1 + n1*(k2a + na*k2b)] and applying n^-1 on the inverse.
        const int log1 = (logn + 2) / 3, logm = logn - log1, loga = (logm + 1) / 2, logb = logm - loga;
        const int64_t n1 = int64_t(1) << log1, n2 = int64_t(1) << logm, na = int64_t(1) << loga, nb = int64_t(1) << logb;
        VI_REQUIRE(scratch != nullptr && scratch_bytes >= 2 * n * 8,
                   "ntt: scratch of at least %lld bytes required (see vi_ntt_scratch_bytes)", (long long)(2 * n * 8));
        uint64_t* s1 = (uint64_t*)scratch;
        uint64_t* s2 = s1 + n;
        const uint64_t *flo, *fhi, *fs2;
        int rc = get_split(n, inv, &flo, &fhi);
        if (rc) return rc;
        rc = get_fs(n2, nb, inv, &fs2);
        if (rc) return rc;
        for (int64_t r = 0; r < m; ++r) {
            PassArgs a{};
            a.in = rows + r * n; a.out = s1;
            a.logC = pick_logC(log1, n2);
            a.ncols = n2;
            a.in_item = 0; a.in_idx = (uint32_t)n2; a.in_col = 1;
            a.out_item = 0; a.out_k = (uint32_t)n2; a.out_col = 1;
            a.fs = flo; a.fs_hi = fhi; a.scale = 1; a.out_via_smem = 0; a.src_kind = SRC_PLAIN;
            rc = launch_pass(log1, inv, 0, a, 1, st, vi::PROF_NTT_PASS);
            if (rc) return rc;
            PassArgs b{};
            b.in = s1; b.out = s2;
            b.logC = pick_logC(loga, nb);
            b.ncols = nb;
            b.in_item = n2; b.in_idx = (uint32_t)nb; b.in_col = 1;
            b.out_item = n2; b.out_k = (uint32_t)nb; b.out_col = 1;
            b.fs = fs2; b.scale = 1; b.out_via_smem = 0; b.src_kind = SRC_PLAIN;
            rc = launch_pass(loga, inv, 0, b, n1, st, vi::PROF_NTT_PASS);
            if (rc) return rc;
            PassArgs c{};
            c.in = s2; c.out = rows + r * n;
            c.logC = pick_logC(logb, na);
            c.ncols = na;
            c.in_item = n2; c.in_idx = 1; c.in_col = (uint32_t)nb;
            c.out_item = 1; c.out_k = (uint32_t)(n1 * na); c.out_col = (uint32_t)n1;
            c.fs = nullptr; c.scale = scale; c.out_via_smem = 0; c.src_kind = SRC_PLAIN;
            rc = launch_pass(logb, inv, 1, c, n1, st, vi::PROF_NTT_PASS);
            if (rc) return rc;
        }
        return VI_OK;
    }
    if (logn <= SINGLE_LOGL) {
        PassArgs a{};
        a.in = rows; a.out = rows;
        a.logC = pick_logC(logn, m);
        a.ncols = m;
        a.in_item = 0; a.in_idx = 1; a.in_col = (uint32_t)n;
        a.out_item = 0; a.out_k = 1; a.out_col = (uint32_t)n;
        a.fs = nullptr; a.scale = scale; a.out_via_smem = 1; a.src_kind = SRC_PLAIN;
        return launch_pass(logn, inv, 1, a, 1, st, vi::PROF_NTT_PASS);
    }
    const int log1 = (logn + 1) / 2, log2 = logn - log1;
    const int64_t n1 = int64_t(1) << log1, n2 = int64_t(1) << log2;
    VI_REQUIRE(scratch != nullptr && scratch_bytes >= n * 8,
               "ntt: scratch of at least %lld bytes required (see vi_ntt_scratch_bytes)", (long long)(n * 8));
    int64_t chunk = scratch_bytes / (n * 8);
    const uint64_t* fsn;
    int rc = get_fs(n, n2, inv, &fsn);
    if (rc) return rc;
    for (int64_t r0 = 0; r0 < m; r0 += chunk) {
        int64_t cnt = m - r0 < chunk ? m - r0 : chunk;
        PassArgs a{};
        a.in = rows + r0 * n; a.out = (uint64_t*)scratch;
        a.logC = pick_logC(log1, n2);
        a.ncols = n2;
        a.in_item = n; a.in_idx = (uint32_t)n2; a.in_col = 1;
        a.out_item = n; a.out_k = (uint32_t)n2; a.out_col = 1;
        a.fs = fsn; a.scale = 1; a.out_via_smem = 0; a.src_kind = SRC_PLAIN;
        rc = launch_pass(log1, inv, 0, a, cnt, st, vi::PROF_NTT_PASS);
        if (rc) return rc;
        PassArgs b{};
        b.in = (const uint64_t*)scratch; b.out = rows + r0 * n;
        b.logC = pick_logC(log2, n1);
        b.ncols = n1;
        b.in_item = n; b.in_idx = 1; b.in_col = (uint32_t)n2;
        b.out_item = n; b.out_k = (uint32_t)n1; b.out_col = 1;
        b.fs = nullptr; b.scale = scale; b.out_via_smem = 0; b.src_kind = SRC_PLAIN;
        rc = launch_pass(log2, inv, 1, b, cnt, st, vi::PROF_NTT_PASS);
        if (rc) return rc;
    }
    return VI_OK;
}

// dst (m, n) = forward NTT of each src row (k_in values) extended with zeros to length n.
// Above the single-pass length the zero extension costs nothing: the first pass reads through
// the message loader, which returns zero past k_in; no padded copy of the input is written.
extern "C" int vi_ntt_forward_padded(const uint64_t* src, int64_t m, int64_t k_in, uint64_t* dst, int64_t n,
                                     void* scratch, int64_t scratch_bytes, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    VI_REQUIRE(m >= 0 && k_in >= 0, "ntt_forward_padded: negative size");
    VI_REQUIRE(vi::is_pow2(n) && n >= 2, "NTT length must be a power of 2 >= 2 (got %lld)", (long long)n);
    VI_REQUIRE(k_in <= n, "ntt_forward_padded: rows of %lld values do not fit length %lld", (long long)k_in, (long long)n);
    const int logn = vi::ilog2(n);
    if (logn > 2 * MAX_LOGL) return vi::fail(VI_ERR_LIMIT, "NTT length 2^%d exceeds the supported 2^%d", logn, 2 * MAX_LOGL);
    if (m == 0) return VI_OK;
    VI_REQUIRE(dst != nullptr && (src != nullptr || k_in == 0), "ntt_forward_padded: null pointer");
    VI_REQUIRE(dst != src, "ntt_forward_padded: output must not alias the input");
    if (logn <= SINGLE_LOGL) {
        if (k_in < n) VI_CUDA(cudaMemsetAsync(dst, 0, (size_t)(m * n) * 8, st));
        if (k_in > 0)
            VI_CUDA(cudaMemcpy2DAsync(dst, (size_t)n * 8, src, (size_t)k_in * 8, (size_t)k_in * 8, (size_t)m,
                                      cudaMemcpyDeviceToDevice, st));
        return vi_ntt_batched(dst, m, n, 0, nullptr, 0, stream);
    }
    const int log1 = (logn + 1) / 2, log2 = logn - log1;
    const int64_t n1 = int64_t(1) << log1, n2 = int64_t(1) << log2;
    VI_REQUIRE(scratch != nullptr && scratch_bytes >= n * 8,
               "ntt: scratch of at least %lld bytes required (see vi_ntt_scratch_bytes)", (long long)(n * 8));
    const int64_t chunk = scratch_bytes / (n * 8);
    const uint64_t* fsn;
    int rc = get_fs(n, n2, false, &fsn);
    if (rc) return rc;
    for (int64_t r0 = 0; r0 < m; r0 += chunk) {
        const int64_t cnt = m - r0 < chunk ? m - r0 : chunk;
        PassArgs a{};
        a.in = src + r0 * k_in; a.out = (uint64_t*)scratch;
        a.logC = pick_logC(log1, n2);
        a.ncols = n2;
        a.in_item = k_in; a.in_idx = (uint32_t)n2; a.in_col = 1;
        a.out_item = n; a.out_k = (uint32_t)n2; a.out_col = 1;
        a.fs = fsn; a.scale = 1; a.out_via_smem = 0;
        a.src_kind = SRC_MSG; a.ell = k_in; a.pad_mode = 0;
        rc = launch_pass(log1, false, 0, a, cnt, st, vi::PROF_NTT_PASS);
        if (rc) return rc;
        PassArgs b{};
        b.in = (const uint64_t*)scratch; b.out = dst + r0 * n;
        b.logC = pick_logC(log2, n1);
        b.ncols = n1;
        b.in_item = n; b.in_idx = 1; b.in_col = (uint32_t)n2;
        b.out_item = n; b.out_k = (uint32_t)n1; b.out_col = 1;
        b.fs = nullptr; b.scale = 1; b.out_via_smem = 0; b.src_kind = SRC_PLAIN;
        rc = launch_pass(log2, false, 1, b, cnt, st, vi::PROF_NTT_PASS);
        if (rc) return rc;
    }
    return VI_OK;
}

extern "C" int64_t vi_encode_scratch_bytes(int64_t m, int64_t k, int64_t n) {
    if (m <= 0) return 0;
    int64_t row = (k + n) * 8;
    int64_t rows = chunk_bytes() / row;
    if (rows < 1) rows = 1;
    if (rows > m) rows = m;
    return rows * row;
}

namespace {
struct KqSrc { const uint8_t* raw; int qtype; int transpose; double S; int64_t d_out, d_in, first_row; const float* table;
               const uint8_t* qT; const void* sT; };
}

static int encode_impl(const uint64_t* msg, const KqSrc* kq, int64_t m, int64_t ell, int64_t k, int64_t n,
                       int pad_mode, const uint8_t* seed_dev32, int64_t row_off,
                       uint64_t* polys, uint64_t* codes,
                       void* scratch, int64_t scratch_bytes, void* stream) {
    cudaStream_t st = (cudaStream_t)stream;
    VI_REQUIRE(m >= 0, "encode: negative row count");
    VI_REQUIRE(vi::is_pow2(k) && k >= 2, "encode: K must be a power of 2 >= 2 (got %lld)", (long long)k);
    VI_REQUIRE(vi::is_pow2(n) && n >= k, "encode: N must be a power of 2 >= K (got %lld)", (long long)n);
    VI_REQUIRE(ell >= 0 && ell <= k, "encode: need 0 <= ELL <= K");
    VI_REQUIRE(pad_mode == 0 || pad_mode == 1, "encode: pad_mode must be 0 (zeros) or 1 (PRG)");
    VI_REQUIRE(pad_mode == 0 || ell == k || seed_dev32 != nullptr, "encode: PRG pad needs a 32-byte seed");
    const int logk = vi::ilog2(k);
    if (logk > 2 * MAX_LOGL) return vi::fail(VI_ERR_LIMIT, "encode: K = 2^%d exceeds the supported 2^%d", logk, 2 * MAX_LOGL);
    const int64_t rho = n / k;
    VI_REQUIRE(rho * k < (int64_t(1) << 31), "encode: N too large");
    if (m == 0) return VI_OK;
    VI_REQUIRE(kq != nullptr || msg != nullptr || ell == 0, "encode: null message pointer");
    const int log1 = (logk + 1) / 2, log2 = logk - log1;
    const int64_t n1 = int64_t(1) << log1, n2 = int64_t(1) << log2;
    const int64_t per_row = (k + (codes ? n : 0)) * 8;
    VI_REQUIRE(scratch != nullptr && scratch_bytes >= per_row,
               "encode: scratch of at least %lld bytes required (see vi_encode_scratch_bytes)", (long long)per_row);
    int64_t chunk = scratch_bytes / per_row;
    // Whole waves: with tiles per row a multiple of 16 (K >= 2^12) a row count that is a multiple of 37 makes
    // every grid of the three passes a multiple of 148 SMs x 4 resident CTAs, so no launch ends in a
    // nearly empty wave.
    if (chunk > 37 && chunk < m) chunk -= chunk % 37;
    const uint64_t *fs_inv, *fs_fwd = nullptr, *twist = nullptr;
    int rc = get_fs(k, n2, true, &fs_inv);        // inverse step 1: columns j2 (n2 of them), index k1
    if (rc) return rc;
    const uint64_t *cscale = nullptr, *twRL = nullptr, *fsN = nullptr;
    const bool shift_form = codes && mid_shift_form(log2, rho);
    if (shift_form) {
        rc = get_cscale(k, &cscale); if (rc) return rc;
        rc = get_tw(rho * n2, &twRL); if (rc) return rc;
        rc = get_fs(n, n1, false, &fsN); if (rc) return rc;                  // w_N^(l2*(rho*m1 + t))
    } else if (codes) {
        rc = get_fs(k, n1, false, &fs_fwd); if (rc) return rc;               // forward step 1: columns l2 (n1), index m1
        rc = get_twist(k, n, &twist); if (rc) return rc;
    }
    uint64_t* s1 = (uint64_t*)scratch;
    for (int64_t r0 = 0; r0 < m; r0 += chunk) {
        int64_t cnt = m - r0 < chunk ? m - r0 : chunk;
        uint64_t* s2 = s1 + cnt * k;
        // pass 1: inverse step 1 over j1 (length n1) for column tiles of j2
        PassArgs a{};
        a.in = kq ? nullptr : msg + r0 * ell; a.out = s1;
        a.logC = pick_logC(log1, n2);
        a.ncols = n2;
        a.in_item = ell; a.in_idx = (uint32_t)n2; a.in_col = 1;
        a.out_item = k; a.out_k = (uint32_t)n2; a.out_col = 1;
        a.fs = fs_inv; a.scale = 1; a.out_via_smem = 0;
        a.src_kind = kq ? SRC_KQ : SRC_MSG; a.ell = ell;
        if (kq) {
            a.kq_raw = kq->raw; a.kq_type = kq->qtype; a.kq_transpose = kq->transpose; a.kq_S = kq->S;
            a.kq_dout = kq->d_out; a.kq_din = kq->d_in; a.kq_first_row = kq->first_row + r0;
            a.kq_table = kq->table;
            a.kq_qT = kq->qT; a.kq_sT = kq->sT;
            a.kq_magic = (kq->d_out >= 2 && kq->d_out * kq->d_in < (int64_t(1) << 32))
                             ? ~uint64_t(0) / (uint64_t)kq->d_out + 1 : 0;
        } a.pad_mode = (ell < k) ? pad_mode : 0; a.row_off = row_off + r0;
        a.seed = seed_dev32;
        rc = launch_pass(log1, true, 0, a, cnt, st, vi::PROF_ENC_PASS1);
        if (rc) return rc;
        // pass 2: inverse step 2 (length n2) + twist + forward step 1 for every coset
        MidArgs mid{};
        mid.s1 = s1; mid.polys = polys ? polys + r0 * k : nullptr; mid.s2 = codes ? s2 : nullptr;
        mid.logC = pick_logC(log2, n1);
        mid.n1 = n1; mid.tiles_per_item = (n1 + (1 << mid.logC) - 1) >> mid.logC;
        VI_REQUIRE(fixed_logC(log2) < 0 || n1 % (int64_t(1) << mid.logC) == 0, "encode: internal tile shape");
        mid.rho = (int)rho; mid.K = k; mid.fsK = fs_fwd; mid.twist = twist; mid.k_inv = inv_pow2(logk);
        mid.cscale = cscale; mid.twRL = twRL; mid.fsN = fsN;
        rc = get_tw(n2, &mid.twL);
        if (rc) return rc;
        mid.twL3 = w3_of(mid.twL);
        mid.cscale3 = cscale ? w3_of(cscale) : nullptr;
        mid.twRL3 = twRL ? w3_of(twRL) : nullptr;
        mid.fsN3 = fsN ? w3_of(fsN) : nullptr;
        mid.k_inv3 = vln::make_w3(mid.k_inv);
        rc = launch_mid(log2, mid, cnt, st);
        if (rc) return rc;
        if (!codes) continue;
        // pass 3: forward step 2 (length n1) for columns (m1, t), interleaved codeword out
        PassArgs b{};
        b.in = s2; b.out = codes + r0 * n;
        b.ncols = rho * n2;
        b.logC = pick_logC(log1, b.ncols);
        b.in_item = n; b.in_idx = 1; b.in_col = (uint32_t)n1;
        b.out_item = n; b.out_k = (uint32_t)(rho * n2); b.out_col = 1;
        b.fs = nullptr; b.scale = 1; b.out_via_smem = 0; b.src_kind = SRC_PLAIN;
        rc = launch_pass(log1, false, 1, b, cnt, st, vi::PROF_ENC_PASS3);
        if (rc) return rc;
    }
    return VI_OK;
}

extern "C" int vi_encode_rows(const uint64_t* msg, int64_t m, int64_t ell, int64_t k, int64_t n,
                              int pad_mode, const uint8_t* seed_dev32, int64_t row_off,
                              uint64_t* polys, uint64_t* codes,
                              void* scratch, int64_t scratch_bytes, void* stream) {
    return encode_impl(msg, nullptr, m, ell, k, n, pad_mode, seed_dev32, row_off, polys, codes,
                       scratch, scratch_bytes, stream);
}

extern "C" int vi_kquant_encode_rows(const uint8_t* raw, int qtype, double S, int64_t d_out, int64_t d_in,
                                     int transpose, int64_t first_row, int64_t m,
                                     int64_t ell, int64_t k, int64_t n,
                                     int pad_mode, const uint8_t* seed_dev32, int64_t row_off,
                                     uint64_t* polys, uint64_t* codes,
                                     void* scratch, int64_t scratch_bytes, void* stream) {
    VI_REQUIRE(qtype == 4 || qtype == 5 || qtype == 6, "kquant encode: qtype must be 4, 5 or 6");
    VI_REQUIRE(d_out > 0 && d_in > 0 && (d_out * d_in) % 256 == 0, "kquant encode: d_out*d_in must be a multiple of 256");
    VI_REQUIRE(first_row >= 0 && raw != nullptr, "kquant encode: bad source");
    KqSrc kq{raw, qtype, transpose != 0, S, d_out, d_in, first_row, nullptr, nullptr, nullptr};
    // When the scratch has room beyond one row chunk, its tail holds the pre-multiplied sub-block
    // scales of the whole matrix (64 bytes per super-block), rebuilt on every call.
    const int64_t n_blocks = d_out * d_in / 256;
    const int64_t table_bytes = n_blocks * vkq::TABLE_BYTES_PER_BLOCK;
    const int64_t per_row = (k + (codes ? n : 0)) * 8;
    // Transposed traversal of a matrix whose rows are whole super-blocks: stage the quants and the
    // scales in traversal order (1.25 bytes per weight at the scratch tail) when there is room.
    const int64_t n_w = d_out * d_in;
    const int64_t scale_bytes = (n_w >> vkq::staged_sub_shift(qtype)) * vkq::staged_scale_bytes(qtype);
    const int64_t staged_bytes = ((n_w + 63) & ~int64_t(63)) + scale_bytes;
    if (m > 0 && transpose && d_in % 256 == 0 && d_out >= 2 && n_w < (int64_t(1) << 32) && d_in / 256 <= 65535 &&
        scratch != nullptr && scratch_bytes >= per_row + staged_bytes + 64) {
        char* base = (char*)scratch + ((scratch_bytes - staged_bytes) & ~int64_t(63));
        uint8_t* qT = (uint8_t*)base;
        void* sT = base + ((n_w + 63) & ~int64_t(63));
        dim3 grid((unsigned)((d_out + 31) / 32), (unsigned)(d_in / 256));
        cudaStream_t st = (cudaStream_t)stream;
        if (qtype == 4) k_kq_stage_T<vkq::Q4_K><<<grid, 256, 0, st>>>(raw, d_out, d_in, qT, sT);
        else if (qtype == 5) k_kq_stage_T<vkq::Q5_K><<<grid, 256, 0, st>>>(raw, d_out, d_in, qT, sT);
        else k_kq_stage_T<vkq::Q6_K><<<grid, 256, 0, st>>>(raw, d_out, d_in, qT, sT);
        int rc = vi::check_launch("k_kq_stage_T");
        if (rc) return rc;
        kq.qT = qT; kq.sT = sT;
        scratch_bytes = base - (char*)scratch;
    } else if (m > 0 && scratch != nullptr && scratch_bytes >= per_row + table_bytes + 64) {
        char* tab = (char*)scratch + ((scratch_bytes - table_bytes) & ~int64_t(63));
        const int per = qtype == 6 ? 16 : 8;
        const int64_t threads = n_blocks * per;
        k_kq_table<<<(unsigned)((threads + 255) / 256), 256, 0, (cudaStream_t)stream>>>(raw, qtype, n_blocks, (float*)tab);
        int rc = vi::check_launch("k_kq_table");
        if (rc) return rc;
        kq.table = (const float*)tab;
        scratch_bytes = tab - (char*)scratch;
    }
    return encode_impl(nullptr, &kq, m, ell, k, n, pad_mode, seed_dev32, row_off, polys, codes,
                       scratch, scratch_bytes, stream);
}
