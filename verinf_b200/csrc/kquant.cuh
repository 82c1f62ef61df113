// K-quant (GGUF Q4_K / Q5_K / Q6_K super-block) element decode -> Goldilocks field.
//
// Arithmetic contract (prover/kquant_cuda.py:42-111, which mirrors gguf-py's
// dequantize_blocks): v = (d*sc)*q - (dmin*mn) for Q4_K/Q5_K, v = (d*sc)*q for Q6_K,
// every fp32 operation rounded separately (the intrinsics below are never fused into
// an FMA), then ll = round_half_even(double(v) * S) and field = ll >= 0 ? ll : p - |ll|.
#pragma once
#include <cuda_fp16.h>
#include <cstdint>

namespace vkq {

constexpr int Q4_K = 4, Q5_K = 5, Q6_K = 6;
__host__ __device__ constexpr int block_bytes(int qtype) { return qtype == 4 ? 144 : qtype == 5 ? 176 : 210; }

__device__ __forceinline__ float ld_half(const uint8_t* __restrict__ p) {
    unsigned short bits = (unsigned short)__ldg(p) | ((unsigned short)__ldg(p + 1) << 8);
    return __half2float(__ushort_as_half(bits));
}

__device__ __forceinline__ uint64_t to_field(float v, double S) {
    long long ll = __double2ll_rn(__dmul_rn((double)v, S));
    return ll >= 0 ? (uint64_t)ll : 0xFFFFFFFF00000001ull - (uint64_t)(-ll);
}

// 6-bit (scale, min) of sub-block s in [0,8) from the 12 packed bytes
__device__ __forceinline__ void scale_min(const uint8_t* __restrict__ s12, int s, uint32_t& sc, uint32_t& mn) {
    if (s < 4) {
        sc = __ldg(s12 + s) & 63;
        mn = __ldg(s12 + s + 4) & 63;
    } else {
        uint32_t hi = __ldg(s12 + s + 4);
        sc = (hi & 0xF) | ((__ldg(s12 + s - 4) >> 6) << 4);
        mn = (hi >> 4) | ((__ldg(s12 + s) >> 6) << 4);
    }
}

// element e (0..255) of the super-block at p
template <int QT>
__device__ __forceinline__ uint64_t lift(const uint8_t* __restrict__ p, int e, double S) {
    if constexpr (QT == Q6_K) {
        const float d = ld_half(p + 208);
        int lo = (__ldg(p + (e >> 7) * 64 + (e & 63)) >> (4 * ((e >> 6) & 1))) & 0xF;
        int hi = (__ldg(p + 128 + (e >> 7) * 32 + (e & 31)) >> (2 * ((e >> 5) & 3))) & 3;
        int q = (lo | (hi << 4)) - 32;
        int sc = (int)(signed char)__ldg(p + 192 + (e >> 4));
        float v = __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
        return to_field(v, S);
    } else {
        const float d = ld_half(p), dmin = ld_half(p + 2);
        uint32_t sc, mn;
        scale_min(p + 4, e >> 5, sc, mn);
        const uint8_t* qs = p + (QT == Q4_K ? 16 : 48);
        int q = (__ldg(qs + (e >> 6) * 32 + (e & 31)) >> (4 * ((e >> 5) & 1))) & 0xF;
        if constexpr (QT == Q5_K) q |= ((__ldg(p + 16 + (e & 31)) >> (e >> 5)) & 1) << 4;
        float v = __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)mn));
        return to_field(v, S);
    }
}

__device__ __forceinline__ uint64_t lift_any(int qtype, const uint8_t* __restrict__ raw, int64_t widx, double S) {
    const uint8_t* p = raw + (widx >> 8) * block_bytes(qtype);
    const int e = (int)(widx & 255);
    return qtype == Q4_K ? lift<Q4_K>(p, e, S) : qtype == Q5_K ? lift<Q5_K>(p, e, S) : lift<Q6_K>(p, e, S);
}

// ---- pre-multiplied sub-block scales ---------------------------------------------------------
// 64 bytes per super-block: Q4_K/Q5_K: 8 x (d*sc, dmin*mn) as float2; Q6_K: 16 x (d*sc) as float.
// The products are the same separately-rounded fp32 multiplies lift<>() performs, so decoding
// through the table is bit-identical; it replaces five scattered header byte loads per element
// by one 8-byte (4-byte) load, which matters when consecutive elements come from different
// super-blocks (the transposed gather of the fused lift + encode).
constexpr int TABLE_BYTES_PER_BLOCK = 64;

template <int QT>
__device__ __forceinline__ void fill_table(const uint8_t* __restrict__ p, int sub, float* __restrict__ t) {
    if constexpr (QT == Q6_K) {
        t[sub] = __fmul_rn(ld_half(p + 208), (float)(int)(signed char)__ldg(p + 192 + sub));   // sub in [0,16)
    } else {
        uint32_t sc, mn;
        scale_min(p + 4, sub, sc, mn);                                                          // sub in [0,8)
        t[2 * sub] = __fmul_rn(ld_half(p), (float)sc);
        t[2 * sub + 1] = __fmul_rn(ld_half(p + 2), (float)mn);
    }
}

template <int QT>
__device__ __forceinline__ uint64_t lift_tab(const uint8_t* __restrict__ p, const float* __restrict__ t, int e, double S) {
    if constexpr (QT == Q6_K) {
        int lo = (__ldg(p + (e >> 7) * 64 + (e & 63)) >> (4 * ((e >> 6) & 1))) & 0xF;
        int hi = (__ldg(p + 128 + (e >> 7) * 32 + (e & 31)) >> (2 * ((e >> 5) & 3))) & 3;
        return to_field(__fmul_rn(__ldg(t + (e >> 4)), (float)((lo | (hi << 4)) - 32)), S);
    } else {
        const float2 sm = __ldg(reinterpret_cast<const float2*>(t) + (e >> 5));
        const uint8_t* qs = p + (QT == Q4_K ? 16 : 48);
        int q = (__ldg(qs + (e >> 6) * 32 + (e & 31)) >> (4 * ((e >> 5) & 1))) & 0xF;
        if constexpr (QT == Q5_K) q |= ((__ldg(p + 16 + (e & 31)) >> (e >> 5)) & 1) << 4;
        return to_field(__fsub_rn(__fmul_rn(sm.x, (float)q), sm.y), S);
    }
}

// ---- transposed staging ------------------------------------------------------------------------
// For the transposed traversal (flat index f = k*d_out + n of the (d_in, d_out) view) consecutive
// elements come from different super-blocks, so every element would cost two 32-byte sector
// fetches for half a byte of payload.  A pre-pass therefore writes, in traversal order, one
// byte per weight (the raw quant: 0..15 / 0..31 / 0..63) and the pre-multiplied sub-block
// scales per (sub-block of k, n); the loader then reads 16 contiguous bytes and 16 contiguous
// scales per tile row.  1.25 bytes per weight instead of the 8 of a lifted matrix.
// Raw quant of element e of the super-block at p.
template <int QT>
__device__ __forceinline__ uint32_t raw_quant(const uint8_t* __restrict__ p, int e) {
    if constexpr (QT == Q6_K) {
        uint32_t lo = (__ldg(p + (e >> 7) * 64 + (e & 63)) >> (4 * ((e >> 6) & 1))) & 0xF;
        uint32_t hi = (__ldg(p + 128 + (e >> 7) * 32 + (e & 31)) >> (2 * ((e >> 5) & 3))) & 3;
        return lo | (hi << 4);
    } else {
        const uint8_t* qs = p + (QT == Q4_K ? 16 : 48);
        uint32_t q = (__ldg(qs + (e >> 6) * 32 + (e & 31)) >> (4 * ((e >> 5) & 1))) & 0xF;
        if constexpr (QT == Q5_K) q |= ((__ldg(p + 16 + (e & 31)) >> (e >> 5)) & 1) << 4;
        return q;
    }
}
// scales per sub-block of k in the staged layout: Q4_K/Q5_K float2 per 32 k, Q6_K float per 16 k
__host__ __device__ constexpr int staged_sub_shift(int qtype) { return qtype == Q6_K ? 4 : 5; }
__host__ __device__ constexpr int staged_scale_bytes(int qtype) { return qtype == Q6_K ? 4 : 8; }

// element (k, n) from the staged arrays; same separately rounded fp32 operations as lift<>()
__device__ __forceinline__ uint64_t lift_staged(int qtype, const uint8_t* __restrict__ qT, const void* __restrict__ sT,
                                                uint32_t f, uint32_t k, uint32_t n, uint32_t d_out, double S) {
    const uint32_t q = __ldg(qT + f);
    if (qtype == Q6_K) {
        const float sc = __ldg(reinterpret_cast<const float*>(sT) + (size_t)(k >> 4) * d_out + n);
        return to_field(__fmul_rn(sc, (float)((int)q - 32)), S);
    }
    const float2 sm = __ldg(reinterpret_cast<const float2*>(sT) + (size_t)(k >> 5) * d_out + n);
    return to_field(__fsub_rn(__fmul_rn(sm.x, (float)q), sm.y), S);
}

__device__ __forceinline__ uint64_t lift_any_tab(int qtype, const uint8_t* __restrict__ raw,
                                                 const float* __restrict__ table, int64_t widx, double S) {
    const int64_t b = widx >> 8;
    const uint8_t* p = raw + b * block_bytes(qtype);
    const float* t = table + b * (TABLE_BYTES_PER_BLOCK / 4);
    const int e = (int)(widx & 255);
    return qtype == Q4_K ? lift_tab<Q4_K>(p, t, e, S) : qtype == Q5_K ? lift_tab<Q5_K>(p, t, e, S)
                                                                       : lift_tab<Q6_K>(p, t, e, S);
}

}  // namespace vkq
