// Integer-pipe and field-primitive microbenchmarks for sm_100a.
//
// The hot path is bound by integer issue rates that no vendor peak figure covers, so the
// denominators are measured: register-resident kernels, 8 independent chains per thread, one
// instruction kind (or one field primitive) per kernel, timed with CUDA events.  Under
// `ncu --metrics smsp__inst_executed.sum,sm__inst_executed_pipe_alu.sum,sm__inst_executed_pipe_fma.sum
// --clock-control none` the same binary gives instructions per primitive.
// Build and run: python bench.py --micro int_pipes   (binary: build/int_pipes)
#include <cstdint>
#include <cstdio>
#include <cuda_runtime.h>

#include "verinf_b200/csrc/dft_lanes.cuh"
#include "verinf_b200/csrc/dft_reg.cuh"
#include "verinf_b200/csrc/gl.cuh"
#include "verinf_b200/csrc/gl_lanes.cuh"

namespace {
constexpr int ITERS = 1024, CHAINS = 8, GRID = 148 * 8, BLOCK = 256;

template <int OP>
__global__ void __launch_bounds__(BLOCK) k_raw(uint32_t* out, uint32_t a0, uint32_t m) {
    uint32_t x[CHAINS], y[CHAINS];
    uint64_t z[CHAINS];
#pragma unroll
    for (int i = 0; i < CHAINS; ++i) { x[i] = a0 + threadIdx.x + i; y[i] = a0 * 3 + i; z[i] = ((uint64_t)x[i] << 32) | y[i]; }
    for (int it = 0; it < ITERS; ++it) {
#pragma unroll
        for (int i = 0; i < CHAINS; ++i) {
            if (OP == 0) asm volatile("add.u32 %0, %0, %1;" : "+r"(x[i]) : "r"(y[i]));
            if (OP == 1) asm volatile("mad.lo.u32 %0, %0, %1, %2;" : "+r"(x[i]) : "r"(m), "r"(y[i]));
            if (OP == 2) asm volatile("mad.wide.u32 %0, %1, %2, %0;" : "+l"(z[i]) : "r"(x[i]), "r"(m));
            if (OP == 3) asm volatile("shf.r.wrap.b32 %0, %0, %0, %1;" : "+r"(x[i]) : "r"(m));
            if (OP == 4) asm volatile("prmt.b32 %0, %0, %0, 0x1032;" : "+r"(x[i]));
            if (OP == 5) asm volatile("add.cc.u32 %0, %0, %2; addc.u32 %1, %1, %3;" : "+r"(x[i]), "+r"(y[i]) : "r"(m), "r"(a0));
            if (OP == 7) asm volatile("mad.wide.s32 %0, %1, %2, %0;" : "+l"(z[i]) : "r"(x[i]), "r"(m));
            if (OP == 8) {      // wide product, then a 64-bit add of an independent value (no fused accumulate)
                uint64_t t;
                asm volatile("mul.wide.s32 %0, %1, %2;" : "=l"(t) : "r"(x[i]), "r"(m));
                asm volatile("add.s64 %0, %0, %1;" : "+l"(z[i]) : "l"(t));
            }
            if (OP == 9) asm volatile("mad.lo.s32 %0, %1, %2, %0;" : "+r"(y[i]) : "r"(x[i]), "r"(m));
            if (OP == 6) {
                asm volatile("add.u32 %0, %0, %1;" : "+r"(x[i]) : "r"(m));
                asm volatile("mad.lo.u32 %0, %0, %1, %2;" : "+r"(y[i]) : "r"(m), "r"(a0));
            }
        }
    }
    uint32_t acc = 0;
#pragma unroll
    for (int i = 0; i < CHAINS; ++i) acc ^= x[i] ^ y[i] ^ (uint32_t)z[i] ^ (uint32_t)(z[i] >> 32);
    out[blockIdx.x * BLOCK + threadIdx.x] = acc;
}

template <int OP>
__global__ void __launch_bounds__(BLOCK) k_field(uint64_t* out, uint64_t seed) {
    using namespace vgl;
    uint64_t v[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = (seed * (threadIdx.x + 1 + i * 977) + i) % P;
    for (int it = 0; it < ITERS / 4; ++it) {
        if (OP == 0) vdft::dif<4, 4, false>(v);
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (OP == 1) v[i] = sub(v[i], v[(i + 1) & 15]);
            if (OP == 2) v[i] = add(v[i], v[(i + 1) & 15]);
            if (OP == 3) v[i] = mul(v[i], v[(i + 1) & 15]);
            if (OP == 4) v[i] = mul_pow2<12>(v[i]);
            if (OP == 5) v[i] = mul_pow2<48>(v[i]);
            if (OP == 6) v[i] = mul_pow2<72>(v[i]);
        }
    }
    uint64_t acc = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) acc ^= v[i];
    out[blockIdx.x * BLOCK + threadIdx.x] = acc;
}

// lane form (gl_lanes.cuh): 16 values of four 32-bit lanes per thread
template <int OP>
__global__ void __launch_bounds__(BLOCK) k_lanes(uint64_t* out, uint64_t seed) {
    using namespace vln;
    Q v[16];
    W3 w[4];
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = from_u64((seed * (threadIdx.x + 1 + i * 977) + i) % vgl::P);
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = make_w3((seed * (threadIdx.x + 77 + i * 13)) % vgl::P);
    for (int it = 0; it < ITERS / 4; ++it) {
        if (OP == 0) {                       // radix-16 DFT, then renormalise by one multiply every 4th round
            vdft::dif<4, 4, false>(v);
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = shl_bits<1>(v[i]);   // keeps the lanes bounded (counted below)
        }
#pragma unroll
        for (int i = 0; i < 16; ++i) {
            if (OP == 1) v[i] = mul(v[i], w[i & 3]);
            if (OP == 2) v[i] = shl_bits<12>(v[i]);
            if (OP == 3) v[i] = from_u64(to_u64(v[i]));
            if (OP == 4) v[i] = shl_bits<1>(v[i]);
        }
    }
    uint64_t acc = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i) acc ^= to_u64(v[i]);
    out[blockIdx.x * BLOCK + threadIdx.x] = acc;
}


// ---- self-check of the device field primitives against 128-bit integer arithmetic ----------
template <int S> __device__ bool chk_pow2(uint64_t x) {
    unsigned __int128 v = (unsigned __int128)x;
    for (int i = 0; i < S; ++i) { v <<= 1; if (v >= vgl::P) v -= vgl::P; }
    return vgl::mul_pow2<S>(x) == (uint64_t)v;
}
__device__ uint64_t edge_or_rand(uint64_t i, uint64_t salt) {
    const uint64_t P = vgl::P;
    const uint64_t edges[12] = {0, 1, 2, P - 1, P - 2, 0xFFFFFFFFull, 0x100000000ull, 0xFFFFFFFF00000000ull,
                                0x8000000000000000ull, 0xFFFFFFFEFFFFFFFFull, 0x00000000FFFFFFFEull, P - 0xFFFFFFFFull};
    if ((i & 7) == 0) return edges[(i >> 3) % 12];
    uint64_t z = (i + salt) * 0x9E3779B97F4A7C15ull; z ^= z >> 31; z *= 0xBF58476D1CE4E5B9ull; z ^= z >> 29;
    return z % P;
}
__global__ void k_selfcheck(unsigned long long* bad) {
    using namespace vgl;
    uint64_t i = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x;
    uint64_t a = edge_or_rand(i, 1), b = edge_or_rand(i / 3 + (i & 7) * 11, 7);
    unsigned __int128 A = a, B = b;
    int f = 0;
    if (add(a, b) != (uint64_t)((A + B) % P)) f |= 1;
    if (sub(a, b) != (uint64_t)((A + P - B) % P)) f |= 2;
    if (mul(a, b) != (uint64_t)((A * B) % P)) f |= 4;
    uint64_t hi = edge_or_rand(i * 5 + 3, 99) | (i & 1 ? 0xFFFFFFFF00000000ull : 0), lo = a | (i & 2 ? 0xFFFFFFFF00000000ull : 0);
    unsigned __int128 W = ((unsigned __int128)hi << 64) | lo;
    if (reduce128(lo, hi) != (uint64_t)(W % P)) f |= 8;
    if (sub(a, P) != a) f |= 16;
    if (!(chk_pow2<1>(a) && chk_pow2<12>(a) && chk_pow2<24>(a) && chk_pow2<31>(a) && chk_pow2<32>(a) && chk_pow2<36>(a) &&
          chk_pow2<48>(a) && chk_pow2<60>(a) && chk_pow2<63>(a) && chk_pow2<64>(a) && chk_pow2<72>(a) && chk_pow2<84>(a) &&
          chk_pow2<95>(a))) f |= 32;
    {   // lane form against the same 128-bit arithmetic
        using namespace vln;
        const Q qa = from_u64(a), qb = from_u64(b | (i & 4 ? 0xFFFFFFFF00000000ull : 0));   // any 64-bit input
        const uint64_t bb = (b | (i & 4 ? 0xFFFFFFFF00000000ull : 0)) % P;
        if (to_u64(qa) != a) f |= 64;
        if (to_u64(add(qa, qb)) != (uint64_t)((A + bb) % P)) f |= 128;
        if (to_u64(sub(qa, qb)) != (uint64_t)((A + P - bb) % P)) f |= 128;
        const Q pr = mul(qb, make_w3(a));
        if (to_u64(pr) != (uint64_t)((A * bb) % P)) f |= 256;
        for (int k = 0; k < 4; ++k) if (pr.x[k] >= NORM || pr.x[k] <= -NORM) f |= 512;
        // a radix-16 DFT of 16 values in both forms (lanes reach 16 * NORM), then a multiply from there
        uint64_t v[16]; Q q[16];
        for (int k = 0; k < 16; ++k) { v[k] = edge_or_rand(i * 16 + k, 5); q[k] = mul(from_u64(v[k]), make_w3(1)); }
        vdft::dif<4, 4, false>(v); vdft::dif<4, 4, false>(q);
        for (int k = 0; k < 16; ++k) {
            if (to_u64(q[k]) != v[k]) f |= 1024;
            if (to_u64(mul(q[k], make_w3(b))) != mul(v[k], b)) f |= 2048;
        }
        for (int k = 0; k < 16; ++k) { v[k] = edge_or_rand(i * 16 + k, 6); q[k] = mul(from_u64(v[k]), make_w3(1)); }
        vdft::dif<4, 4, true>(v); vdft::dif<4, 4, true>(q);
        for (int k = 0; k < 16; ++k) if (to_u64(q[k]) != v[k]) f |= 4096;
        if (to_u64(shl_bits<12>(pr)) != mul_pow2<12>(to_u64(pr)) || to_u64(shl_bits<23>(pr)) != mul_pow2<23>(to_u64(pr)) ||
            to_u64(vln::mul_pow2<39>(pr)) != vgl::mul_pow2<39>(to_u64(pr)) ||
            to_u64(vln::mul_pow2<156>(pr)) != vgl::sub(0, vgl::mul_pow2<60>(to_u64(pr)))) f |= 8192;
    }
    if (f) atomicOr(bad, (unsigned long long)f);
}

template <class F>
float time_ms(F launch) {
    cudaEvent_t a, b;
    cudaEventCreate(&a); cudaEventCreate(&b);
    launch(); cudaDeviceSynchronize();
    cudaEventRecord(a); launch(); cudaEventRecord(b); cudaEventSynchronize(b);
    float ms = 0; cudaEventElapsedTime(&ms, a, b);
    cudaEventDestroy(a); cudaEventDestroy(b);
    return ms;
}
}  // namespace

int main() {
    void* d = nullptr;
    if (cudaMalloc(&d, (size_t)GRID * BLOCK * 8) != cudaSuccess) { printf("no CUDA device\n"); return 1; }
    {
        unsigned long long* bad; cudaMalloc(&bad, 8); cudaMemset(bad, 0, 8);
        k_selfcheck<<<4096, 256>>>(bad);
        unsigned long long h = 0; cudaMemcpy(&h, bad, 8, cudaMemcpyDeviceToHost);
        printf("self-check of add/sub/mul/reduce128/mul_pow2 and the lane form vs 128-bit arithmetic: %s (flags %llu) %s\n",
               h ? "MISMATCH" : "ok", h, cudaGetErrorString(cudaGetLastError()));
        cudaFree(bad);
    }
    int khz = 0; cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, 0);
    const double threads = (double)GRID * BLOCK;
    auto raw = [&](const char* name, int per, float ms) {
        double ops = threads * ITERS * CHAINS * per;
        printf("%-28s %8.3f ms %9.1f Gop/s %7.1f ops/clk/SM\n", name, ms, ops / ms / 1e6, ops / (ms * 1e-3) / 148 / (khz * 1e3));
    };
    raw("add.u32", 1, time_ms([&] { k_raw<0><<<GRID, BLOCK>>>((uint32_t*)d, 12345, 77); }));
    raw("mad.lo.u32", 1, time_ms([&] { k_raw<1><<<GRID, BLOCK>>>((uint32_t*)d, 12345, 77); }));
    raw("mad.wide.u32", 1, time_ms([&] { k_raw<2><<<GRID, BLOCK>>>((uint32_t*)d, 12345, 77); }));
    raw("shf.r.wrap", 1, time_ms([&] { k_raw<3><<<GRID, BLOCK>>>((uint32_t*)d, 12345, 77); }));
    raw("prmt", 1, time_ms([&] { k_raw<4><<<GRID, BLOCK>>>((uint32_t*)d, 12345, 77); }));
    raw("add.cc + addc", 2, time_ms([&] { k_raw<5><<<GRID, BLOCK>>>((uint32_t*)d, 12345, 77); }));
    raw("add.u32 + mad.lo.u32", 2, time_ms([&] { k_raw<6><<<GRID, BLOCK>>>((uint32_t*)d, 12345, 77); }));
    raw("mad.wide.s32", 1, time_ms([&] { k_raw<7><<<GRID, BLOCK>>>((uint32_t*)d, 12345, 77); }));
    raw("mul.wide.s32 + add.s64", 1, time_ms([&] { k_raw<8><<<GRID, BLOCK>>>((uint32_t*)d, 12345, 77); }));
    raw("mad.lo.s32", 1, time_ms([&] { k_raw<9><<<GRID, BLOCK>>>((uint32_t*)d, 12345, 77); }));
    auto fld = [&](const char* name, int per, float ms) {
        double ops = threads * (ITERS / 4) * per;
        printf("%-28s %8.3f ms %9.1f Gop/s\n", name, ms, ops / ms / 1e6);
    };
    fld("radix-16 DFT element-stage", 64, time_ms([&] { k_field<0><<<GRID, BLOCK>>>((uint64_t*)d, 12345); }));
    fld("gl sub", 16, time_ms([&] { k_field<1><<<GRID, BLOCK>>>((uint64_t*)d, 12345); }));
    fld("gl add", 16, time_ms([&] { k_field<2><<<GRID, BLOCK>>>((uint64_t*)d, 12345); }));
    fld("gl mul", 16, time_ms([&] { k_field<3><<<GRID, BLOCK>>>((uint64_t*)d, 12345); }));
    fld("gl mul_pow2<12>", 16, time_ms([&] { k_field<4><<<GRID, BLOCK>>>((uint64_t*)d, 12345); }));
    fld("gl mul_pow2<48>", 16, time_ms([&] { k_field<5><<<GRID, BLOCK>>>((uint64_t*)d, 12345); }));
    fld("gl mul_pow2<72>", 16, time_ms([&] { k_field<6><<<GRID, BLOCK>>>((uint64_t*)d, 12345); }));
    fld("lanes radix-16 DFT (+shl_bits<1>) element-stage", 64, time_ms([&] { k_lanes<0><<<GRID, BLOCK>>>((uint64_t*)d, 12345); }));
    fld("lanes mul", 16, time_ms([&] { k_lanes<1><<<GRID, BLOCK>>>((uint64_t*)d, 12345); }));
    fld("lanes shl_bits<12>", 16, time_ms([&] { k_lanes<2><<<GRID, BLOCK>>>((uint64_t*)d, 12345); }));
    fld("lanes to_u64 + from_u64", 16, time_ms([&] { k_lanes<3><<<GRID, BLOCK>>>((uint64_t*)d, 12345); }));
    fld("lanes shl_bits<1>", 16, time_ms([&] { k_lanes<4><<<GRID, BLOCK>>>((uint64_t*)d, 12345); }));
    cudaFree(d);
    return 0;
}
