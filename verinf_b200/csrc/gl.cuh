// Goldilocks field (p = 2^64 - 2^32 + 1) device arithmetic for sm_100a.
//
// Semantics follow the reference's gl::add/sub/mul/reduce128/pow
// (prover/kernels/goldilocks.cuh:28-81): canonical inputs in [0, p) give the
// canonical result.  The 128-bit product is reduced with 2^64 = 2^32 - 1 and
// 2^96 = -1 (mod p).
#pragma once
#include <cstdint>

namespace vgl {

constexpr uint64_t P = 0xFFFFFFFF00000001ull;
constexpr uint64_t EPS = 0xFFFFFFFFull;   // 2^32 - 1 = 2^64 mod p

__host__ __device__ __forceinline__ uint64_t add(uint64_t a, uint64_t b) {
    uint64_t s = a + b;
    if (s < a) s += EPS;          // wrapped past 2^64: +2^64 = +EPS (mod p)
    if (s >= P) s -= P;
    return s;
}

__host__ __device__ __forceinline__ uint64_t sub(uint64_t a, uint64_t b) {
    uint64_t d = a - b;
    if (a < b) d -= EPS;          // borrowed 2^64: -2^64 = -EPS (mod p)
    return d;
}

__host__ __device__ __forceinline__ uint64_t neg(uint64_t a) { return a == 0 ? 0 : P - a; }

// (hi:lo) mod p, canonical.  hi = hh*2^32 + hl:  x = lo - hh + hl*(2^32-1).
__host__ __device__ __forceinline__ uint64_t reduce128(uint64_t lo, uint64_t hi) {
    uint64_t hh = hi >> 32, hl = hi & EPS;
    uint64_t t0 = lo - hh;
    if (lo < hh) t0 -= EPS;
    uint64_t t1 = (hl << 32) - hl;
    uint64_t r = t0 + t1;
    if (r < t0) r += EPS;
    if (r >= P) r -= P;
    return r;
}

__device__ __forceinline__ uint64_t mul(uint64_t a, uint64_t b) {
    return reduce128(a * b, __umul64hi(a, b));
}

__device__ __forceinline__ uint64_t pow(uint64_t base, uint64_t e) {
    uint64_t r = 1;
    while (e) {
        if (e & 1) r = mul(r, base);
        base = mul(base, base);
        e >>= 1;
    }
    return r;
}

// x * 2^S mod p for a compile-time 0 <= S < 96 (x canonical -> canonical).
// Every 2^k-th root of unity with k <= 6 is a power of two in this field
// (2 has order 192), so radix-<=64 butterflies multiply by shifts only.
template <int S>
__device__ __forceinline__ uint64_t mul_pow2(uint64_t x) {
    static_assert(S >= 0 && S < 96, "shift out of range");
    if constexpr (S == 0) {
        return x;
    } else if constexpr (S < 64) {
        uint64_t lo = x << S, hi = x >> (64 - S);
        return reduce128(lo, hi);
    } else if constexpr (S == 64) {
        return reduce128(0, x);
    } else {
        // x*2^S = (y_hi*2^64 + y_lo) * 2^64 with y = x << (S-64) (< 2^96);
        // 2^128 = -2^32, so the result is reduce128(0, y_lo) - y_hi*2^32.
        constexpr int T = S - 64;
        uint64_t ylo = x << T, yhi = x >> (64 - T);
        return sub(reduce128(0, ylo), yhi << 32);
    }
}

// host-side helpers used when building twiddle tables
inline uint64_t hmul(uint64_t a, uint64_t b) {
    unsigned __int128 v = (unsigned __int128)a * b;
    return reduce128((uint64_t)v, (uint64_t)(v >> 64));
}
inline uint64_t hpow(uint64_t b, uint64_t e) {
    uint64_t r = 1;
    while (e) { if (e & 1) r = hmul(r, b); b = hmul(b, b); e >>= 1; }
    return r;
}

}  // namespace vgl
