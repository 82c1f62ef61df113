// Goldilocks arithmetic on four carry-free 24-bit lanes ("lane form") for sm_100a.
//
// p = 2^64 - 2^32 + 1 divides 2^96 + 1, so with psi = 2^24 the field is a quotient of
// Z[psi]/(psi^4 + 1).  A value is held as four signed 32-bit lanes
//     x = x0 + x1*psi + x2*psi^2 + x3*psi^3   (mod p)
// with 24 significant bits per lane after a multiplication and up to 6 bits of headroom:
//   * add / sub are four independent 32-bit adds, no carry chain, so the compiler may issue
//     them on either integer pipe (the 64-bit canonical form needs 5-8 carry-chain
//     instructions on the ALU pipe alone);
//   * multiplying by psi^k is a lane rotation with sign changes, folded into the subtraction
//     of a butterfly; every 8th root of unity is +-psi^k (w_8 = 2^24 up to sign);
//   * multiplying by 2^r, 0 < r < 24, splits every lane at bit 24-r and re-normalises
//     (12 instructions, any r): w_16 and w_64 are powers of two, so radix-16 butterflies need
//     no full multiply;
//   * a full multiply by a table constant is 12 wide multiply-adds (FMA pipe) into four 64-bit
//     sums plus a 3-way digit split; the constant is stored as three balanced digits
//     pre-shifted by 8 bits so that the split points fall on register boundaries.
// Conversion from the canonical 64-bit form is 4 instructions, back to it ~30.
//
// Semantics are those of the reference's gl::add/sub/mul (prover/kernels/goldilocks.cuh:28-81):
// to_u64(op(from_u64(a), from_u64(b))) is the canonical result.
#pragma once
#include <cstdint>

#include "gl.cuh"

namespace vln {

struct Q { int32_t x[4]; };

// Lane magnitudes: from_u64 and mul give |x_i| < NORM; add/sub may be applied while lanes stay
// below LIMIT (the bound mul and to_u64 accept).
constexpr int32_t NORM = (1 << 25) + (1 << 8);
constexpr int32_t LIMIT = 1 << 30;

// Twiddle constant for mul(): w = d0 + d1*2^24 + d2*2^48 with balanced digits
// d0, d1 in [-2^23, 2^23), d2 in [0, 2^16]; stored as d_j * 2^8.
struct W3 { int32_t w0, w1, w2, pad; };

__host__ __device__ __forceinline__ W3 make_w3(uint64_t w) {
    int64_t d0 = (int64_t)(w & 0xFFFFFF), d1 = (int64_t)((w >> 24) & 0xFFFFFF), d2 = (int64_t)(w >> 48);
    if (d0 >= (1 << 23)) { d0 -= 1 << 24; d1 += 1; }
    if (d1 >= (1 << 23)) { d1 -= 1 << 24; d2 += 1; }
    W3 r;
    r.w0 = (int32_t)(d0 * 256); r.w1 = (int32_t)(d1 * 256); r.w2 = (int32_t)(d2 * 256); r.pad = 0;
    return r;
}

__device__ __forceinline__ Q from_u64(uint64_t u) {   // any 64-bit representative
    const uint32_t lo = (uint32_t)u, hi = (uint32_t)(u >> 32);
    Q r;
    r.x[0] = (int32_t)(lo & 0xFFFFFFu);
    r.x[1] = (int32_t)(__funnelshift_r(lo, hi, 24) & 0xFFFFFFu);
    r.x[2] = (int32_t)(hi >> 16);
    r.x[3] = 0;
    return r;
}

__device__ __forceinline__ Q add(const Q& a, const Q& b) {
    Q r;
#pragma unroll
    for (int i = 0; i < 4; ++i) r.x[i] = a.x[i] + b.x[i];
    return r;
}
__device__ __forceinline__ Q sub(const Q& a, const Q& b) {
    Q r;
#pragma unroll
    for (int i = 0; i < 4; ++i) r.x[i] = a.x[i] - b.x[i];
    return r;
}

// x * 2^R for a compile-time 0 < R < 24; output lanes are below 2^24 + |x|_max / 2^(24-R)
template <int R>
__device__ __forceinline__ Q shl_bits(const Q& x) {
    static_assert(R > 0 && R < 24, "lane shift out of range");
    int32_t l[4], h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        l[i] = x.x[i] & ((1 << (24 - R)) - 1);
        h[i] = x.x[i] >> (24 - R);            // arithmetic: x = h * 2^(24-R) + l with 0 <= l
    }
    Q r;
    r.x[0] = (l[0] << R) - h[3];
    r.x[1] = (l[1] << R) + h[0];
    r.x[2] = (l[2] << R) + h[1];
    r.x[3] = (l[3] << R) + h[2];
    return r;
}

// same value, lanes brought back below 2^24 + |x|_max / 2^24: carries move up one lane, the top
// lane's carry re-enters lane 0 negated (psi^4 = -1).  For values that skip a multiply between two
// butterfly stages.
__device__ __forceinline__ Q renorm(const Q& x) {
    int32_t l[4], h[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        l[i] = x.x[i] & 0xFFFFFF;
        h[i] = x.x[i] >> 24;
    }
    Q r;
    r.x[0] = l[0] - h[3];
    r.x[1] = l[1] + h[0];
    r.x[2] = l[2] + h[1];
    r.x[3] = l[3] + h[2];
    return r;
}

// (a - b) * 2^E for a compile-time E in [0, 192): the sign (2^96 = -1) and the lane rotation
// (psi^k) are folded into the subtraction, the remaining 2^r (r < 24) is one shl_bits.
template <int E>
__device__ __forceinline__ Q sub_mul_pow2(const Q& a, const Q& b) {
    static_assert(E >= 0 && E < 192, "exponent out of range");
    constexpr bool NEG = E >= 96;
    constexpr int K = (E % 96) / 24, R = (E % 96) % 24;
    Q d;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const bool flip = NEG != (i + K >= 4);          // psi^4 = -1
        d.x[(i + K) & 3] = flip ? b.x[i] - a.x[i] : a.x[i] - b.x[i];
    }
    if constexpr (R == 0) return d;
    else return shl_bits<R>(d);
}
// x * 2^E, same decomposition (costs a negation per flipped lane)
template <int E>
__device__ __forceinline__ Q mul_pow2(const Q& x) {
    Q z;
#pragma unroll
    for (int i = 0; i < 4; ++i) z.x[i] = 0;
    if constexpr (E == 0) return x;
    else return sub_mul_pow2<E>(x, z);
}

// x * w (|x_i| < LIMIT): lanes of the result are below NORM
__device__ __forceinline__ Q mul(const Q& x, const W3& w) {
    const int32_t n2 = -x.x[2], n3 = -x.x[3];
    const int64_t y0 = (int64_t)x.x[0] * w.w0 + (int64_t)n3 * w.w1 + (int64_t)n2 * w.w2;
    const int64_t y1 = (int64_t)x.x[1] * w.w0 + (int64_t)x.x[0] * w.w1 + (int64_t)n3 * w.w2;
    const int64_t y2 = (int64_t)x.x[2] * w.w0 + (int64_t)x.x[1] * w.w1 + (int64_t)x.x[0] * w.w2;
    const int64_t y3 = (int64_t)x.x[3] * w.w0 + (int64_t)x.x[2] * w.w1 + (int64_t)x.x[1] * w.w2;
    // y_k = 2^8 * (a_k + b_k 2^24 + c_k 2^48): a = bits 8..31, b = bits 32..55, c = bits 56.. (signed)
    int32_t a[4], b[4], c[4];
    const int64_t y[4] = {y0, y1, y2, y3};
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const uint32_t lo = (uint32_t)y[k];
        const int32_t hi = (int32_t)(y[k] >> 32);
        a[k] = (int32_t)(lo >> 8);
        b[k] = hi & 0xFFFFFF;
        c[k] = hi >> 24;
    }
    Q r;
    r.x[0] = a[0] - b[3] - c[2];
    r.x[1] = a[1] + b[0] - c[3];
    r.x[2] = a[2] + b[1] + c[0];
    r.x[3] = a[3] + b[2] + c[1];
    return r;
}

// Lanes of a multiple of p, each in [2^30, 2^31]: added before the conversion so that every
// lane is non-negative (computed by bias_lane() at compile time).
__host__ __device__ constexpr uint32_t bias_lane(int i) {
    // T0 = 1.5*2^30 * (1 + 2^24 + 2^48 + 2^72); subtract T0 mod p digit-wise (base 2^24)
    unsigned __int128 t0 = 0;
    for (int k = 3; k >= 0; --k) t0 = (t0 << 24) + (unsigned __int128)(3u << 29);
    const uint64_t r = (uint64_t)(t0 % (unsigned __int128)vgl::P);
    const uint32_t dig[4] = {(uint32_t)(r & 0xFFFFFF), (uint32_t)((r >> 24) & 0xFFFFFF), (uint32_t)(r >> 48), 0u};
    return (3u << 29) - dig[i];
}

// canonical 64-bit value of x (|x_i| < LIMIT)
__device__ __forceinline__ uint64_t to_u64(const Q& x) {
    const uint32_t u0 = (uint32_t)x.x[0] + bias_lane(0), u1 = (uint32_t)x.x[1] + bias_lane(1);
    const uint32_t u2 = (uint32_t)x.x[2] + bias_lane(2), u3 = (uint32_t)x.x[3] + bias_lane(3);
    const uint64_t A = (uint64_t)u1 * (1u << 24) + u0;      // < 2^57
    const uint64_t B = (uint64_t)u3 * (1u << 24) + u2;
    // U = A + B * 2^48 as four 32-bit words
    const uint32_t a0 = (uint32_t)A, a1 = (uint32_t)(A >> 32), b0 = (uint32_t)B, b1 = (uint32_t)(B >> 32);
    uint32_t t1, t2, t3;
    asm("add.cc.u32 %0, %3, %4;\n\t"
        "addc.cc.u32 %1, %5, 0;\n\t"
        "addc.u32 %2, %6, 0;"
        : "=r"(t1), "=r"(t2), "=r"(t3)
        : "r"(a1), "r"(b0 << 16), "r"(__funnelshift_r(b0, b1, 16)), "r"(b1 >> 16));
    return vgl::reduce128(vgl::pack(a0, t1), vgl::pack(t2, t3));
}

}  // namespace vln
