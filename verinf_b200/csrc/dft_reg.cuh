// In-register radix-2^k DFT butterflies over Goldilocks with power-of-two twiddles.
// Shared by the NTT kernels (ntt.cu) and the integer-pipe microbenchmark.
#pragma once
#include <cstdint>

#include "gl.cuh"

namespace vdft {

using vgl::add;
using vgl::sub;

// w_R = 2^root_exp(log2 R): the reference's root_of_unity(R) = 7^((p-1)/R) for R = 2..64.
__host__ __device__ constexpr int root_exp(int logr) {
    return logr == 1 ? 96 : logr == 2 ? 48 : logr == 3 ? 120 : logr == 4 ? 156 : logr == 5 ? 78 : 39;
}

template <int LOGLEN, int K, bool INV>
__device__ __forceinline__ void bfly(uint64_t& a, uint64_t& b) {
    constexpr int s0 = (root_exp(LOGLEN) * K) % 192;
    constexpr int s = INV ? (192 - s0) % 192 : s0;
    uint64_t t = add(a, b);
    uint64_t d = (s >= 96) ? sub(b, a) : sub(a, b);   // 2^96 = -1
    a = t;
    b = vgl::mul_pow2<s % 96>(d);
}

template <int LOGR, int LOGLEN, int I, bool INV>
__device__ __forceinline__ void dif_level(uint64_t* v) {
    constexpr int R = 1 << LOGR, LEN = 1 << LOGLEN, HALF = LEN / 2;
    if constexpr (I < R / 2) {
        constexpr int blk = I / HALF, k = I % HALF;
        bfly<LOGLEN, k, INV>(v[blk * LEN + k], v[blk * LEN + k + HALF]);
        dif_level<LOGR, LOGLEN, I + 1, INV>(v);
    }
}
// In-register decimation-in-frequency DFT of R = 2^LOGR values: X[c] = v[bitrev(c)].
template <int LOGR, int LOGLEN, bool INV>
__device__ __forceinline__ void dif(uint64_t* v) {
    if constexpr (LOGLEN >= 1) {
        dif_level<LOGR, LOGLEN, 0, INV>(v);
        dif<LOGR, LOGLEN - 1, INV>(v);
    }
}

__host__ __device__ constexpr int brev(int x, int bits) {
    int r = 0;
    for (int i = 0; i < bits; ++i) r |= ((x >> i) & 1) << (bits - 1 - i);
    return r;
}

}  // namespace vdft
