// BLAKE3 compression function for sm_100a (published algorithm).
//
// Replaces the reference's b3::compress (prover/kernels/blake3_compress.cuh:77-117).
// The seven rounds and the message permutation are unrolled at compile time, so
// the message words are addressed as registers and no permutation is executed.
#pragma once
#include <cstdint>

namespace vb3 {

constexpr uint32_t CHUNK_START = 1, CHUNK_END = 2, PARENT = 4, ROOT = 8;
constexpr uint32_t IV0 = 0x6A09E667u, IV1 = 0xBB67AE85u, IV2 = 0x3C6EF372u, IV3 = 0xA54FF53Au,
                   IV4 = 0x510E527Fu, IV5 = 0x9B05688Cu, IV6 = 0x1F83D9ABu, IV7 = 0x5BE0CD19u;

__host__ __device__ constexpr int perm1(int i) {
    constexpr int p[16] = {2, 6, 3, 10, 7, 0, 4, 13, 1, 11, 12, 5, 9, 14, 15, 8};
    return p[i];
}
// index of the original message word used at position i of round r
__host__ __device__ constexpr int sched(int r, int i) {
    int idx = i;
    for (int k = 0; k < r; ++k) idx = perm1(idx);
    return idx;
}
// (round r reads m_r[i] = m_{r-1}[perm1(i)], hence m_r[i] = m_0[perm1 applied r times to i])

__device__ __forceinline__ uint32_t rotr16(uint32_t x) { return __byte_perm(x, x, 0x1032); }
__device__ __forceinline__ uint32_t rotr8(uint32_t x) { return __byte_perm(x, x, 0x0321); }
__device__ __forceinline__ uint32_t rotr12(uint32_t x) { return __funnelshift_r(x, x, 12); }
__device__ __forceinline__ uint32_t rotr7(uint32_t x) { return __funnelshift_r(x, x, 7); }

// On sm_100a xor/rotate can only issue on the integer ALU pipe (half a warp per cycle), which
// is what bounds the hash kernels.  The six additions of G are therefore issued as
// multiply-adds by a constant-bank 1 (x*1 + y), which run on the FMA pipe in parallel:
// 8 ALU + 6 FMA instructions per G instead of 12 ALU.
static __constant__ uint32_t ONE = 1;
__device__ __forceinline__ uint32_t fadd(uint32_t x, uint32_t y) {
    uint32_t r;
    asm("mad.lo.u32 %0, %1, %2, %3;" : "=r"(r) : "r"(x), "r"(ONE), "r"(y));
    return r;
}

#define VB3_G(a, b, c, d, mx, my)                          \
    do {                                                   \
        a = fadd(mx, fadd(a, b)); d = rotr16(d ^ a);       \
        c = fadd(c, d);           b = rotr12(b ^ c);       \
        a = fadd(my, fadd(a, b)); d = rotr8(d ^ a);        \
        c = fadd(c, d);           b = rotr7(b ^ c);        \
    } while (0)

template <int R>
__device__ __forceinline__ void round_fn(uint32_t (&v)[16], const uint32_t (&m)[16]) {
    VB3_G(v[0], v[4], v[8], v[12], m[sched(R, 0)], m[sched(R, 1)]);
    VB3_G(v[1], v[5], v[9], v[13], m[sched(R, 2)], m[sched(R, 3)]);
    VB3_G(v[2], v[6], v[10], v[14], m[sched(R, 4)], m[sched(R, 5)]);
    VB3_G(v[3], v[7], v[11], v[15], m[sched(R, 6)], m[sched(R, 7)]);
    VB3_G(v[0], v[5], v[10], v[15], m[sched(R, 8)], m[sched(R, 9)]);
    VB3_G(v[1], v[6], v[11], v[12], m[sched(R, 10)], m[sched(R, 11)]);
    VB3_G(v[2], v[7], v[8], v[13], m[sched(R, 12)], m[sched(R, 13)]);
    VB3_G(v[3], v[4], v[9], v[14], m[sched(R, 14)], m[sched(R, 15)]);
}

// cv <- first 8 words of compress(cv, m, counter, block_len, flags)
__device__ __forceinline__ void compress(uint32_t (&cv)[8], const uint32_t (&m)[16],
                                         uint64_t counter, uint32_t block_len, uint32_t flags) {
    uint32_t v[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = cv[i];
    v[8] = IV0; v[9] = IV1; v[10] = IV2; v[11] = IV3;
    v[12] = (uint32_t)counter; v[13] = (uint32_t)(counter >> 32);
    v[14] = block_len; v[15] = flags;
    round_fn<0>(v, m); round_fn<1>(v, m); round_fn<2>(v, m); round_fn<3>(v, m);
    round_fn<4>(v, m); round_fn<5>(v, m); round_fn<6>(v, m);
#pragma unroll
    for (int i = 0; i < 8; ++i) cv[i] = v[i] ^ v[i + 8];
}

__device__ __forceinline__ void set_iv(uint32_t (&cv)[8]) {
    cv[0] = IV0; cv[1] = IV1; cv[2] = IV2; cv[3] = IV3;
    cv[4] = IV4; cv[5] = IV5; cv[6] = IV6; cv[7] = IV7;
}

// parent node: compress(IV, left || right, 0, 64, PARENT | extra)
__device__ __forceinline__ void parent(const uint32_t (&l)[8], const uint32_t (&r)[8],
                                       uint32_t extra_flags, uint32_t (&out)[8]) {
    uint32_t m[16];
#pragma unroll
    for (int i = 0; i < 8; ++i) { m[i] = l[i]; m[i + 8] = r[i]; }
    set_iv(out);
    compress(out, m, 0, 64, PARENT | extra_flags);
}

// BLAKE3 of a message of <= 64 bytes held in m (zero padded), as a whole hash.
__device__ __forceinline__ void hash_one_block(const uint32_t (&m)[16], uint32_t len, uint32_t (&out)[8]) {
    set_iv(out);
    compress(out, m, 0, len, CHUNK_START | CHUNK_END | ROOT);
}

// ZK pad value: u64_le(BLAKE3(seed32 || row_le8 || k_le8)[0:8]) % p
// (reference formula: prover/cuda_primitives.py:877-903).
__device__ __forceinline__ uint64_t pad_prg(const uint32_t (&seed)[8], uint64_t row, uint64_t k) {
    uint32_t m[16], h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) m[i] = seed[i];
    m[8] = (uint32_t)row; m[9] = (uint32_t)(row >> 32);
    m[10] = (uint32_t)k;  m[11] = (uint32_t)(k >> 32);
    m[12] = m[13] = m[14] = m[15] = 0;
    hash_one_block(m, 48, h);
    uint64_t raw = (uint64_t)h[0] | ((uint64_t)h[1] << 32);
    return raw >= 0xFFFFFFFF00000001ull ? raw - 0xFFFFFFFF00000001ull : raw;
}


// The pad PRG hashes seed32 || row_le8 || k_le8: of the 8 G functions of the first round only one
// (words 1, 6, 11, 12 with the message words holding k) depends on k.  pad_prg_prefix computes
// the state after the other seven once per (seed, row); pad_prg_from finishes an element from it.
__device__ __forceinline__ void pad_prg_prefix(const uint32_t (&seed)[8], uint64_t row, uint32_t (&v)[16]) {
    v[0] = IV0; v[1] = IV1; v[2] = IV2; v[3] = IV3; v[4] = IV4; v[5] = IV5; v[6] = IV6; v[7] = IV7;
    v[8] = IV0; v[9] = IV1; v[10] = IV2; v[11] = IV3;
    v[12] = 0; v[13] = 0; v[14] = 48; v[15] = CHUNK_START | CHUNK_END | ROOT;
    const uint32_t r0 = (uint32_t)row, r1 = (uint32_t)(row >> 32), z = 0;
    VB3_G(v[0], v[4], v[8], v[12], seed[0], seed[1]);
    VB3_G(v[1], v[5], v[9], v[13], seed[2], seed[3]);
    VB3_G(v[2], v[6], v[10], v[14], seed[4], seed[5]);
    VB3_G(v[3], v[7], v[11], v[15], seed[6], seed[7]);
    VB3_G(v[0], v[5], v[10], v[15], r0, r1);
    VB3_G(v[2], v[7], v[8], v[13], z, z);
    VB3_G(v[3], v[4], v[9], v[14], z, z);
}
__device__ __forceinline__ uint64_t pad_prg_from(const uint32_t* __restrict__ prefix, const uint32_t (&seed)[8],
                                                 uint64_t row, uint64_t k) {
    uint32_t v[16], m[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = prefix[i];
#pragma unroll
    for (int i = 0; i < 8; ++i) m[i] = seed[i];
    m[8] = (uint32_t)row; m[9] = (uint32_t)(row >> 32);
    m[10] = (uint32_t)k;  m[11] = (uint32_t)(k >> 32);
    m[12] = m[13] = m[14] = m[15] = 0;
    VB3_G(v[1], v[6], v[11], v[12], m[10], m[11]);
    round_fn<1>(v, m); round_fn<2>(v, m); round_fn<3>(v, m);
    round_fn<4>(v, m); round_fn<5>(v, m); round_fn<6>(v, m);
    uint64_t raw = (uint64_t)(v[0] ^ v[8]) | ((uint64_t)(v[1] ^ v[9]) << 32);
    return raw >= 0xFFFFFFFF00000001ull ? raw - 0xFFFFFFFF00000001ull : raw;
}

// (hi:lo) mod p, canonical (p = 2^64 - 2^32 + 1; same steps as vgl::reduce128)
__device__ __forceinline__ uint64_t reduce128_p(uint64_t lo, uint64_t hi) {
    const uint64_t EPS = 0xFFFFFFFFull, PP = 0xFFFFFFFF00000001ull;
    uint64_t hh = hi >> 32, hl = hi & EPS;
    uint64_t t0 = lo - hh;
    if (lo < hh) t0 -= EPS;
    uint64_t t1 = (hl << 32) - hl;
    uint64_t r = t0 + t1;
    if (r < t0) r += EPS;
    if (r >= PP) r -= PP;
    return r;
}

// Challenge PRF of the protocol: int(BLAKE3(seed32 || label || cid_le8)[:16], LE) % p
// (prover/protocol.py:126-133).  label is passed packed little-endian in a u64.
__device__ __forceinline__ void load_seed(const uint8_t* __restrict__ s, uint32_t (&w)[8]) {
#pragma unroll
    for (int i = 0; i < 8; ++i)
        w[i] = (uint32_t)__ldg(s + 4 * i) | ((uint32_t)__ldg(s + 4 * i + 1) << 8) |
               ((uint32_t)__ldg(s + 4 * i + 2) << 16) | ((uint32_t)__ldg(s + 4 * i + 3) << 24);
}

__device__ __forceinline__ uint64_t challenge(const uint32_t (&s)[8], uint64_t label, int label_len,
                                                  uint64_t cid) {
    // message = seed(32) || label(label_len <= 8) || cid_le8, zero padded to one block
    uint64_t lo, hi;
    if (label_len == 0) { lo = cid; hi = 0; }
    else if (label_len == 8) { lo = label; hi = cid; }
    else { lo = label | (cid << (8 * label_len)); hi = cid >> (64 - 8 * label_len); }
    uint32_t m[16], h[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) m[i] = s[i];
    m[8] = (uint32_t)lo; m[9] = (uint32_t)(lo >> 32);
    m[10] = (uint32_t)hi; m[11] = (uint32_t)(hi >> 32);
    m[12] = m[13] = m[14] = m[15] = 0;
    vb3::hash_one_block(m, (uint32_t)(40 + label_len), h);
    uint64_t d0 = (uint64_t)h[0] | ((uint64_t)h[1] << 32);
    uint64_t d1 = (uint64_t)h[2] | ((uint64_t)h[3] << 32);
    return reduce128_p(d0, d1);
}

__device__ __forceinline__ uint64_t load_label(const uint8_t* __restrict__ label, int label_len) {
    uint64_t v = 0;
    for (int i = 0; i < label_len; ++i) v |= (uint64_t)__ldg(label + i) << (8 * i);
    return v;
}

}  // namespace vb3
