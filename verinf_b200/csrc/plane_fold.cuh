// Fold of the 15 byte-plane sums of a field product: sum_s T_s 2^(8 s) mod p, T_s < 2^32.
//
// The sum is built as one plain 160-bit integer and reduced once: the four sums whose weights differ by
// 2^32 (s = r, r+4, r+8, r+12) sit in separate 32-bit limbs, so they form a 128-bit number N_r for free,
// and the total is N_0 + (N_1 << 8) + (N_2 << 16) + (N_3 << 24): three funnel-shifted 5-limb additions
// and one reduction (about 55 instructions) instead of 15 modular shifts and additions (about 375).
#pragma once
#include <cstdint>

#include "gl.cuh"

namespace vpf {

// x (5 limbs) += (n3:n2:n1:n0) << SH, 0 < SH < 32
template <int SH>
__device__ __forceinline__ void add_shifted(uint32_t (&x)[5], uint32_t n0, uint32_t n1, uint32_t n2, uint32_t n3) {
    const uint32_t o0 = n0 << SH, o1 = __funnelshift_l(n0, n1, SH), o2 = __funnelshift_l(n1, n2, SH),
                   o3 = __funnelshift_l(n2, n3, SH), o4 = n3 >> (32 - SH);
    asm("add.cc.u32 %0, %0, %5;\n\t"
        "addc.cc.u32 %1, %1, %6;\n\t"
        "addc.cc.u32 %2, %2, %7;\n\t"
        "addc.cc.u32 %3, %3, %8;\n\t"
        "addc.u32 %4, %4, %9;"
        : "+r"(x[0]), "+r"(x[1]), "+r"(x[2]), "+r"(x[3]), "+r"(x[4])
        : "r"(o0), "r"(o1), "r"(o2), "r"(o3), "r"(o4));
}

__device__ __forceinline__ uint64_t combine15(const uint32_t (&t)[15]) {
    uint32_t x[5] = {t[0], t[4], t[8], t[12], 0};          // N_0
    add_shifted<8>(x, t[1], t[5], t[9], t[13]);
    add_shifted<16>(x, t[2], t[6], t[10], t[14]);
    add_shifted<24>(x, t[3], t[7], t[11], 0u);
    return vgl::reduce160(x);                               // total < 2^147: the top limb stays below 2^19
}

}  // namespace vpf
