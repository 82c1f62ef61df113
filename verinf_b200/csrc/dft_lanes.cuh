// In-register radix-2^k DFT butterflies over Goldilocks in lane form (gl_lanes.cuh): the twiddles
// inside a radix-<=64 butterfly are powers of two, i.e. lane rotations plus at most one lane shift.
// Same index conventions as dft_reg.cuh: X[c] = v[bitrev(c)] after dif().
#pragma once
#include "dft_reg.cuh"
#include "gl_lanes.cuh"

namespace vdft {

template <int LOGLEN, int K, bool INV>
__device__ __forceinline__ void bfly(vln::Q& a, vln::Q& b) {
    constexpr int s0 = (root_exp(LOGLEN) * K) % 192;
    constexpr int s = INV ? (192 - s0) % 192 : s0;
    const vln::Q t = vln::add(a, b);
    b = vln::sub_mul_pow2<s>(a, b);
    a = t;
}

template <int LOGR, int LOGLEN, int I, bool INV>
__device__ __forceinline__ void dif_level(vln::Q* v) {
    constexpr int R = 1 << LOGR, LEN = 1 << LOGLEN, HALF = LEN / 2;
    if constexpr (I < R / 2) {
        constexpr int blk = I / HALF, k = I % HALF;
        bfly<LOGLEN, k, INV>(v[blk * LEN + k], v[blk * LEN + k + HALF]);
        dif_level<LOGR, LOGLEN, I + 1, INV>(v);
    }
}
template <int LOGR, int LOGLEN, bool INV>
__device__ __forceinline__ void dif(vln::Q* v) {
    if constexpr (LOGLEN >= 1) {
        dif_level<LOGR, LOGLEN, 0, INV>(v);
        dif<LOGR, LOGLEN - 1, INV>(v);
    }
}

}  // namespace vdft
