// Goldilocks field (p = 2^64 - 2^32 + 1) device arithmetic for sm_100a.
//
// Semantics follow the reference's gl::add/sub/mul/reduce128/pow
// (prover/kernels/goldilocks.cuh:28-81): canonical inputs in [0, p) give the
// canonical result.  The 128-bit product is reduced with 2^64 = 2^32 - 1 and
// 2^96 = -1 (mod p).
//
// The device versions are written on 32-bit limbs with explicit carry chains
// (add.cc / subc): on sm_100a the integer ALU pipe and the FMA pipe each issue half a warp
// per cycle and the NTT kernels are bound by them, so every op is the shortest sequence found
// (sub = 5 instructions, add = neg + sub = 7, reduce128 = 16) with its instructions spread
// over both pipes (VGL_FMA_CARRY below).
#pragma once
#include <cstdint>

namespace vgl {

constexpr uint64_t P = 0xFFFFFFFF00000001ull;
constexpr uint64_t EPS = 0xFFFFFFFFull;   // 2^32 - 1 = 2^64 mod p

__host__ __device__ __forceinline__ uint64_t pack(uint32_t lo, uint32_t hi) { return ((uint64_t)hi << 32) | lo; }

// The carry-chain instructions of the ALU pipe (add.cc / addc / sub.cc / subc) have twins on the FMA pipe:
// mad.lo.cc / madc.lo with a multiplier of 1, -1 or 0 taken from the constant bank (so that the assembler
// keeps them multiply-adds).  With VGL_FMA_CARRY the conditional corrections of sub, reduce128 and the
// power-of-two shifts (+-(2^32 - 1) after a borrow or carry) and the products h*(2^32 - 1) are issued that
// way: the kernels built on these primitives are bound by the ALU pipe while the FMA pipe is a quarter busy.
// Bits: 1 = the correction of sub, 2 = reduce128 (the tail of every full multiply), 4 = the power-of-two shifts.
#ifndef VGL_FMA_CARRY
#define VGL_FMA_CARRY 7
#endif
#ifdef __CUDACC__
static __constant__ uint32_t VGL_ONE = 1u, VGL_M1 = 0xFFFFFFFFu, VGL_ZERO = 0u;
#endif

// ---- portable versions (host, and the oracle of the PTX versions) -----------------
__host__ __device__ __forceinline__ uint64_t add_c(uint64_t a, uint64_t b) {
    uint64_t s = a + b;
    if (s < a) s += EPS;          // wrapped past 2^64: +2^64 = +EPS (mod p)
    if (s >= P) s -= P;
    return s;
}
__host__ __device__ __forceinline__ uint64_t sub_c(uint64_t a, uint64_t b) {
    uint64_t d = a - b;
    if (a < b) d -= EPS;          // borrowed 2^64: -2^64 = -EPS (mod p)
    return d;
}
// (hi:lo) mod p, canonical.  hi = hh*2^32 + hl:  x = lo - hh + hl*(2^32-1).
__host__ __device__ __forceinline__ uint64_t reduce128_c(uint64_t lo, uint64_t hi) {
    uint64_t hh = hi >> 32, hl = hi & EPS;
    uint64_t t0 = lo - hh;
    if (lo < hh) t0 -= EPS;
    uint64_t t1 = (hl << 32) - hl;
    uint64_t r = t0 + t1;
    if (r < t0) r += EPS;
    if (r >= P) r -= P;
    return r;
}

// a - b mod p for canonical a, b (also exact for b == p): 5 instructions
__host__ __device__ __forceinline__ uint64_t sub(uint64_t a, uint64_t b) {
#ifdef __CUDA_ARCH__
    uint32_t d0, d1, m;
#if VGL_FMA_CARRY & 1
    asm("sub.cc.u32 %0, %3, %5;\n\t"
        "subc.cc.u32 %1, %4, %6;\n\t"
        "subc.u32 %2, 0, 0;\n\t"              // m = borrow ? 0xffffffff : 0
        "mad.lo.cc.u32 %0, %2, %7, %0;\n\t"   // d -= borrow ? EPS : 0:  lo += m*(-1) = (borrow ? 1 : 0),
        "madc.lo.u32 %1, %2, %8, %1;"          //                         hi += m*1 + carry = -borrow + carry
        : "=&r"(d0), "=&r"(d1), "=&r"(m)
        : "r"((uint32_t)a), "r"((uint32_t)(a >> 32)), "r"((uint32_t)b), "r"((uint32_t)(b >> 32)), "r"(VGL_M1), "r"(VGL_ONE));
#else
    asm("sub.cc.u32 %0, %3, %5;\n\t"
        "subc.cc.u32 %1, %4, %6;\n\t"
        "subc.u32 %2, 0, 0;\n\t"          // m = borrow ? 0xffffffff : 0
        "sub.cc.u32 %0, %0, %2;\n\t"      // d -= borrow ? EPS : 0
        "subc.u32 %1, %1, 0;"
        : "=&r"(d0), "=&r"(d1), "=&r"(m)
        : "r"((uint32_t)a), "r"((uint32_t)(a >> 32)), "r"((uint32_t)b), "r"((uint32_t)(b >> 32)));
#endif
    (void)m;
    return pack(d0, d1);
#else
    return sub_c(a, b);
#endif
}

__host__ __device__ __forceinline__ uint64_t add(uint64_t a, uint64_t b) {
#ifdef __CUDA_ARCH__
    // a + b = a - (p - b); p - b is p for b == 0, which sub() accepts as a subtrahend: 7 instructions
    uint32_t n0, n1;
    asm("sub.cc.u32 %0, 1, %2;\n\t"
        "subc.u32 %1, 0xffffffff, %3;"
        : "=&r"(n0), "=&r"(n1) : "r"((uint32_t)b), "r"((uint32_t)(b >> 32)));
    return sub(a, pack(n0, n1));
#else
    return add_c(a, b);
#endif
}

// (hi:lo) mod p, canonical: 17 instructions on the device
__host__ __device__ __forceinline__ uint64_t reduce128(uint64_t lo, uint64_t hi) {
#if defined(__CUDA_ARCH__) && (VGL_FMA_CARRY & 2)
    uint32_t r0, r1;
    asm("{\n\t.reg .u32 m, c, e0, e1;\n\t.reg .b64 e;\n\t.reg .pred q;\n\t"
        "sub.cc.u32 %0, %2, %5;\n\t"           // t = lo - hh
        "subc.cc.u32 %1, %3, 0;\n\t"
        "subc.u32 m, 0, 0;\n\t"
        "mad.lo.cc.u32 %0, m, %6, %0;\n\t"     // t -= borrow ? EPS : 0   (FMA pipe, cannot borrow again)
        "madc.lo.u32 %1, m, %7, %1;\n\t"
        "mul.wide.u32 e, %4, %6;\n\t"          // e = hl*EPS               (FMA pipe)
        "mov.b64 {e0, e1}, e;\n\t"
        "add.cc.u32 %0, %0, e0;\n\t"           // r = t + e
        "addc.cc.u32 %1, %1, e1;\n\t"
        "addc.u32 c, 0, 0;\n\t"                // c = carry
        "mad.lo.cc.u32 %0, c, %6, %0;\n\t"     // r += carry ? EPS : 0:  lo -= c, its carry k = no borrow,
        "madc.lo.u32 %1, c, %8, %1;\n\t"       //                        hi += k            (cannot carry again)
        "setp.eq.u32 q, %1, 0xffffffff;\n\t"   // r >= p  <=>  hi == 2^32-1 and lo != 0; then r - p = lo - 1
        "setp.ne.and.u32 q, %0, 0, q;\n\t"
        "@q mov.u32 %1, 0;\n\t"
        "@q add.u32 %0, %0, 0xffffffff;\n\t}"
        : "=&r"(r0), "=&r"(r1)
        : "r"((uint32_t)lo), "r"((uint32_t)(lo >> 32)), "r"((uint32_t)hi), "r"((uint32_t)(hi >> 32)),
          "r"(VGL_M1), "r"(VGL_ONE), "r"(VGL_ZERO));
    return pack(r0, r1);
#elif defined(__CUDA_ARCH__)
    uint32_t r0, r1;
    asm("{\n\t.reg .u32 m, e0, e1;\n\t.reg .pred q;\n\t"
        "sub.cc.u32 %0, %2, %5;\n\t"       // t = lo - hh
        "subc.cc.u32 %1, %3, 0;\n\t"
        "subc.u32 m, 0, 0;\n\t"
        "sub.cc.u32 %0, %0, m;\n\t"        // t -= borrow ? EPS : 0   (cannot borrow again)
        "subc.u32 %1, %1, 0;\n\t"
        "sub.cc.u32 e0, 0, %4;\n\t"        // e = hl*EPS = (hl<<32) - hl
        "subc.u32 e1, %4, 0;\n\t"
        "add.cc.u32 %0, %0, e0;\n\t"       // r = t + e
        "addc.cc.u32 %1, %1, e1;\n\t"
        "addc.u32 m, 0, 0;\n\t"            // m = carry ? 0xffffffff : 0 (carry of an add chain must be
        "neg.s32 m, m;\n\t"                //     read with addc: subc after add.cc sees it inverted)
        "add.cc.u32 %0, %0, m;\n\t"        // r += carry ? EPS : 0     (cannot carry again)
        "addc.u32 %1, %1, 0;\n\t"
        "setp.eq.u32 q, %1, 0xffffffff;\n\t"   // r >= p  <=>  hi == 2^32-1 and lo != 0; then r - p = lo - 1
        "setp.ne.and.u32 q, %0, 0, q;\n\t"
        "@q mov.u32 %1, 0;\n\t"
        "@q add.u32 %0, %0, 0xffffffff;\n\t}"
        : "=&r"(r0), "=&r"(r1)
        : "r"((uint32_t)lo), "r"((uint32_t)(lo >> 32)), "r"((uint32_t)hi), "r"((uint32_t)(hi >> 32)));
    return pack(r0, r1);
#else
    return reduce128_c(lo, hi);
#endif
}

#ifdef __CUDA_ARCH__
// (l1:l0) + h*(2^32-1) mod p, canonical; (l1:l0) is any u64, h any u32: 12 instructions
__device__ __forceinline__ uint64_t add_mul_eps(uint32_t l0, uint32_t l1, uint32_t h) {
    uint32_t r0, r1;
#if VGL_FMA_CARRY & 4
    asm("{\n\t.reg .u32 c, e0, e1;\n\t.reg .b64 e;\n\t.reg .pred q;\n\t"
        "mul.wide.u32 e, %4, %5;\n\t"          // e = h*EPS (FMA pipe)
        "mov.b64 {e0, e1}, e;\n\t"
        "add.cc.u32 %0, %2, e0;\n\t"
        "addc.cc.u32 %1, %3, e1;\n\t"
        "addc.u32 c, 0, 0;\n\t"
        "mad.lo.cc.u32 %0, c, %5, %0;\n\t"     // += carry ? EPS : 0 (FMA pipe)
        "madc.lo.u32 %1, c, %6, %1;\n\t"
        "setp.eq.u32 q, %1, 0xffffffff;\n\t"
        "setp.ne.and.u32 q, %0, 0, q;\n\t"
        "@q mov.u32 %1, 0;\n\t"
        "@q add.u32 %0, %0, 0xffffffff;\n\t}"
        : "=&r"(r0), "=&r"(r1) : "r"(l0), "r"(l1), "r"(h), "r"(VGL_M1), "r"(VGL_ZERO));
    return pack(r0, r1);
#endif
    asm("{\n\t.reg .u32 m, e0, e1;\n\t.reg .pred q;\n\t"
        "sub.cc.u32 e0, 0, %4;\n\t"
        "subc.u32 e1, %4, 0;\n\t"
        "add.cc.u32 %0, %2, e0;\n\t"
        "addc.cc.u32 %1, %3, e1;\n\t"
        "addc.u32 m, 0, 0;\n\t"
        "neg.s32 m, m;\n\t"
        "add.cc.u32 %0, %0, m;\n\t"
        "addc.u32 %1, %1, 0;\n\t"
        "setp.eq.u32 q, %1, 0xffffffff;\n\t"
        "setp.ne.and.u32 q, %0, 0, q;\n\t"
        "@q mov.u32 %1, 0;\n\t"
        "@q add.u32 %0, %0, 0xffffffff;\n\t}"
        : "=&r"(r0), "=&r"(r1) : "r"(l0), "r"(l1), "r"(h));
    return pack(r0, r1);
}
#endif

// full 64x64 -> 128 product on 32-bit limbs (4 wide multiply-adds), then reduce
__device__ __forceinline__ uint64_t mul(uint64_t a, uint64_t b) {
    const uint32_t a0 = (uint32_t)a, a1 = (uint32_t)(a >> 32), b0 = (uint32_t)b, b1 = (uint32_t)(b >> 32);
    uint64_t t = (uint64_t)a0 * b0;                          // bits 0..63
    uint64_t u = (uint64_t)a0 * b1 + (t >> 32);              // no overflow: (2^32-1)^2 + 2^32-1 < 2^64
    uint64_t v = (uint64_t)a1 * b0 + (uint32_t)u;            // idem
    uint64_t w = (uint64_t)a1 * b1 + (u >> 32) + (v >> 32);  // bits 64..127
    return reduce128(pack((uint32_t)t, (uint32_t)v), w);
}

// (x4:x3:x2:x1:x0) += a * b as integers: 8 multiply-adds with carry + 5 carry propagations,
// no modular reduction.  x4 counts the carries out of 2^128, so 2^32 products fit.
__device__ __forceinline__ void mac160(uint32_t (&x)[5], uint64_t a, uint64_t b) {
    const uint32_t a0 = (uint32_t)a, a1 = (uint32_t)(a >> 32), b0 = (uint32_t)b, b1 = (uint32_t)(b >> 32);
    asm("mad.lo.cc.u32 %0, %5, %7, %0;\n\t"
        "madc.hi.cc.u32 %1, %5, %7, %1;\n\t"
        "madc.lo.cc.u32 %2, %6, %8, %2;\n\t"
        "madc.hi.cc.u32 %3, %6, %8, %3;\n\t"
        "addc.u32 %4, %4, 0;\n\t"
        "mad.lo.cc.u32 %1, %5, %8, %1;\n\t"
        "madc.hi.cc.u32 %2, %5, %8, %2;\n\t"
        "addc.cc.u32 %3, %3, 0;\n\t"
        "addc.u32 %4, %4, 0;\n\t"
        "mad.lo.cc.u32 %1, %6, %7, %1;\n\t"
        "madc.hi.cc.u32 %2, %6, %7, %2;\n\t"
        "addc.cc.u32 %3, %3, 0;\n\t"
        "addc.u32 %4, %4, 0;"
        : "+r"(x[0]), "+r"(x[1]), "+r"(x[2]), "+r"(x[3]), "+r"(x[4])
        : "r"(a0), "r"(a1), "r"(b0), "r"(b1));
}
// the 160-bit sum mod p: 2^128 = -2^32 (mod p), and x4 << 32 <= p - 1 is canonical
__device__ __forceinline__ uint64_t reduce160(const uint32_t (&x)[5]) {
    return sub(reduce128(pack(x[0], x[1]), pack(x[2], x[3])), (uint64_t)x[4] << 32);
}

__host__ __device__ __forceinline__ uint64_t neg(uint64_t a) { return a == 0 ? 0 : P - a; }

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
// With phi = 2^32 (phi^2 = phi - 1, phi^3 = -1) and (l2:l1:l0) = x << (S mod 32):
//   S <  32: (l1:l0) + l2*(2^32-1)
//   S <  64: the general 128-bit reduction of (l2:l1:l0:0)
//   S >= 64: l0*(2^32-1) - (l2:l1)
// (Issuing the limb shifts as wide multiplies on the FMA pipe, or building the 64-bit sums from
// mad.wide plus a 64-bit compare instead of carry chains, was measured slower on B200: radix-16
// butterfly throughput 2004 and 1250 G element-stages/s against 2091 for this form.)
template <int S>
__device__ __forceinline__ uint64_t mul_pow2(uint64_t x) {
    static_assert(S >= 0 && S < 96, "shift out of range");
#ifdef __CUDA_ARCH__
    if constexpr (S == 0) {
        return x;
    } else {
        constexpr int V = S % 32, U = S / 32;
        // (l2:l1:l0) = x << V as three 32-bit limbs
        uint32_t l0 = (uint32_t)x, l1 = (uint32_t)(x >> 32), l2 = 0;
        if constexpr (V != 0) {
            l2 = l1 >> (32 - V); l1 = (l1 << V) | (l0 >> (32 - V)); l0 <<= V;
        }
        if constexpr (U == 0) {
            // l0 + l1 phi + l2 phi^2 = (l1:l0) + l2*(2^32-1)
            return add_mul_eps(l0, l1, l2);
        } else if constexpr (U == 1) {
            // l0 phi + l1 phi^2 + l2 phi^3: the 128-bit value (hi = (l2:l1), lo = (l0:0))
            return reduce128(pack(0, l0), pack(l1, l2));
        } else {
            // l0 phi^2 + l1 phi^3 + l2 phi^4 = l0*(2^32-1) - (l2:l1); (l2:l1) < 2^63 is canonical
#if VGL_FMA_CARRY & 4
            uint64_t e;
            asm("mul.wide.u32 %0, %1, %2;" : "=l"(e) : "r"(l0), "r"(VGL_M1));     // FMA pipe
            return sub(e, pack(l1, l2));
#else
            uint32_t e0, e1;
            asm("sub.cc.u32 %0, 0, %2;\n\t"
                "subc.u32 %1, %2, 0;"
                : "=&r"(e0), "=&r"(e1) : "r"(l0));
            return sub(pack(e0, e1), pack(l1, l2));
#endif
        }
    }
#else
    return x;
#endif
}

// host-side helpers used when building twiddle tables
inline uint64_t hmul(uint64_t a, uint64_t b) {
    unsigned __int128 v = (unsigned __int128)a * b;
    return reduce128_c((uint64_t)v, (uint64_t)(v >> 64));
}
inline uint64_t hpow(uint64_t b, uint64_t e) {
    uint64_t r = 1;
    while (e) { if (e & 1) r = hmul(r, b); b = hmul(b, b); e >>= 1; }
    return r;
}

}  // namespace vgl
