// Sumcheck round kernel: fold with the previous challenge and evaluate the next
// round polynomial in one pass over the tables.
//
// Replaces the per-round work of layergkr/gpu.py:326-410 (fold_t, gl_sum,
// prove_terms_gpu; CPU twin layergkr/sumcheck.py:153-226), which issues ~10
// elementwise launches and a host sync per sample point.  Here one launch reads each
// table once, writes the folded half once and produces all deg+1 samples; a second
// tiny launch adds the per-CTA partial sums.  The arithmetic per sample is the
// reference's: g(x) = sum_i sum_t c_t prod_j (f[i] + x (f[half+i] - f[i])), variable
// order most-significant first, so results are bit-identical (field sums commute).
// (Summing the last multiply of every product unreduced, as the matmul does with
// vgl::mac160, was measured slower here: 1.21 ms against 1.05 ms of device time for
// the 2^24 x 3 degree-3 instance.  The kernel is bound by the multiplier half of the
// FMA pipe, which an unreduced multiply-add loads as much as a reduced one.)
#include "../../include/verinf_b200.h"
#include "common.cuh"
#include "gl.cuh"

namespace {

using vgl::add;
using vgl::mul;
using vgl::sub;

constexpr int MAX_TABLES = 8, MAX_TERMS = 8, MAX_FAC = 4, MAX_SAMPLES = 8;
constexpr int BLOCK = 256;
constexpr int MAX_GRID = 148 * 8;

struct Problem {
    uint64_t* tab[MAX_TABLES];
    int n_tables, n_terms, deg;
    uint64_t coef[MAX_TERMS];
    int nfac[MAX_TERMS];
    int fac[MAX_TERMS][MAX_FAC];
    int simple;   // one term, coefficient 1, factors = tables 0..n_tables-1 in order
};

// Block-level sum of ns per-thread accumulators -> partials[block*MAX_SAMPLES + x]
__device__ __forceinline__ void block_reduce(uint64_t (&acc)[MAX_SAMPLES], int ns, uint64_t* partials) {
    __shared__ uint64_t red[BLOCK / 32][MAX_SAMPLES];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
    for (int x = 0; x < MAX_SAMPLES; ++x) {
        if (x < ns) {
            uint64_t v = acc[x];
#pragma unroll
            for (int o = 16; o; o >>= 1) v = add(v, __shfl_xor_sync(0xffffffffu, v, o));
            if (lane == 0) red[wid][x] = v;
        }
    }
    __syncthreads();
    if (threadIdx.x < ns) {
        uint64_t v = 0;
#pragma unroll
        for (int w = 0; w < BLOCK / 32; ++w) v = add(v, red[w][threadIdx.x]);
        partials[(int64_t)blockIdx.x * MAX_SAMPLES + threadIdx.x] = v;
    }
}

// block_reduce followed by the cross-CTA sum in the same launch: the CTA that draws the last ticket of
// a wrapping counter (left at zero again for the next launch) adds all partial sums and writes
// out[0..ns).  Used by the queued run, which clears the counter once per run; saves one launch per round.
__device__ __forceinline__ void block_reduce_finish(uint64_t (&acc)[MAX_SAMPLES], int ns, uint64_t* partials,
                                                    unsigned* counter, uint64_t* out) {
    __shared__ uint64_t red2[BLOCK / 32][MAX_SAMPLES];
    __shared__ int is_last;
    block_reduce(acc, ns, partials);
    __threadfence();                       // this CTA's partial sums are visible before its ticket is drawn
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicInc(counter, gridDim.x - 1) == gridDim.x - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    uint64_t tot[MAX_SAMPLES];
#pragma unroll
    for (int x = 0; x < MAX_SAMPLES; ++x) tot[x] = 0;
    for (int b = threadIdx.x; b < (int)gridDim.x; b += BLOCK)
#pragma unroll
        for (int x = 0; x < MAX_SAMPLES; ++x)
            if (x < ns) tot[x] = add(tot[x], __ldcg(partials + (int64_t)b * MAX_SAMPLES + x));
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
    for (int x = 0; x < MAX_SAMPLES; ++x) {
        if (x < ns) {
            uint64_t v = tot[x];
#pragma unroll
            for (int o = 16; o; o >>= 1) v = add(v, __shfl_xor_sync(0xffffffffu, v, o));
            if (lane == 0) red2[wid][x] = v;
        }
    }
    __syncthreads();
    if (threadIdx.x < ns) {
        uint64_t v = 0;
#pragma unroll
        for (int w = 0; w < BLOCK / 32; ++w) v = add(v, red2[w][threadIdx.x]);
        out[threadIdx.x] = v;
    }
}

// MODE 0: claim (sum of products at every index, one "sample")
// MODE 1: round samples on the tables as they are (pairs i, i+half)
// MODE 2: fold with r (size -> size/2, in place), then round samples of the folded tables
template <int MODE>
__global__ void __launch_bounds__(BLOCK) k_sumcheck(Problem pb, int64_t size, uint64_t r, int skip1, uint64_t* partials) {
    // pair values of this thread for every table, staged for the runtime term structure:
    // 2 * n_tables * BLOCK words of dynamic shared memory
    extern __shared__ uint64_t sc_smem[];
    uint64_t (*slo)[BLOCK] = reinterpret_cast<uint64_t (*)[BLOCK]>(sc_smem);
    uint64_t (*sd)[BLOCK] = reinterpret_cast<uint64_t (*)[BLOCK]>(sc_smem + (size_t)pb.n_tables * BLOCK);
    const int ns = MODE == 0 ? 1 : pb.deg + 1;
    // number of work items: claim = size; plain round = size/2 pairs; fold+round = size/4 pairs of pairs
    const int64_t items = MODE == 0 ? size : MODE == 1 ? size / 2 : size / 4;
    const int64_t q = items;   // distance between the two entries of a pair (after folding in MODE 2)
    uint64_t acc[MAX_SAMPLES];
#pragma unroll
    for (int x = 0; x < MAX_SAMPLES; ++x) acc[x] = 0;
    const int tid = threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * BLOCK;
    for (int64_t i = (int64_t)blockIdx.x * BLOCK + tid; i < items; i += stride) {
        // per table: lo = f(x=0), d = f(1) - f(0) of the (folded) pair
#pragma unroll
        for (int k = 0; k < MAX_TABLES; ++k) {
            if (k < pb.n_tables) {
                uint64_t* f = pb.tab[k];
                uint64_t lo, hi;
                if (MODE == 0) { lo = f[i]; hi = lo; }
                else if (MODE == 1) { lo = f[i]; hi = f[i + q]; }
                else {
                    uint64_t a0 = f[i], b0 = f[i + q], a1 = f[i + 2 * q], b1 = f[i + 3 * q];
                    lo = add(a0, mul(r, sub(a1, a0)));
                    hi = add(b0, mul(r, sub(b1, b0)));
                    f[i] = lo;
                    f[i + q] = hi;
                }
                slo[k][tid] = lo;
                sd[k][tid] = sub(hi, lo);
            }
        }
        if (pb.simple) {
            // product of all tables, evaluated at x = 0..deg by stepping each factor by d
            uint64_t cur[MAX_FAC];
#pragma unroll
            for (int k = 0; k < MAX_FAC; ++k) cur[k] = k < pb.n_tables ? slo[k][tid] : 1;
#pragma unroll
            for (int x = 0; x < MAX_SAMPLES; ++x) {
                if (x < ns) {
                    if (!(skip1 && x == 1)) {       // g(1) follows from g(0) + g(1) = previous claim
                        uint64_t prod = cur[0];
#pragma unroll
                        for (int k = 1; k < MAX_FAC; ++k)
                            if (k < pb.n_tables) prod = mul(prod, cur[k]);
                        acc[x] = add(acc[x], prod);
                    }
#pragma unroll
                    for (int k = 0; k < MAX_FAC; ++k)
                        if (k < pb.n_tables) cur[k] = add(cur[k], sd[k][tid]);
                }
            }
        } else {
            for (int t = 0; t < pb.n_terms; ++t) {
                uint64_t cur[MAX_FAC], dd[MAX_FAC];
#pragma unroll
                for (int j = 0; j < MAX_FAC; ++j) {
                    int k = j < pb.nfac[t] ? pb.fac[t][j] : 0;
                    cur[j] = slo[k][tid];
                    dd[j] = sd[k][tid];
                }
#pragma unroll
                for (int x = 0; x < MAX_SAMPLES; ++x) {
                    if (x < ns) {
                        if (!(skip1 && x == 1)) {
                            uint64_t prod = pb.coef[t];
#pragma unroll
                            for (int j = 0; j < MAX_FAC; ++j)
                                if (j < pb.nfac[t]) prod = mul(prod, cur[j]);
                            acc[x] = add(acc[x], prod);
                        }
#pragma unroll
                        for (int j = 0; j < MAX_FAC; ++j) cur[j] = add(cur[j], dd[j]);
                    }
                }
            }
        }
    }
    block_reduce(acc, ns, partials);
}

// The common case -- one term, coefficient 1, the product of all NT tables (NT <= 4) -- with the
// table count known at compile time: the pair values stay in registers (no shared-memory staging,
// no per-table runtime predicates), which lifts the occupancy limit of the general kernel.
template <int MODE, int NT>
__global__ void __launch_bounds__(BLOCK) k_sumcheck_simple(Problem pb, int64_t size, uint64_t r, int skip1,
                                                           uint64_t* partials, unsigned* counter = nullptr,
                                                           uint64_t* out = nullptr) {
    constexpr int NS = MODE == 0 ? 1 : NT + 1;
    const int64_t items = MODE == 0 ? size : MODE == 1 ? size / 2 : size / 4;
    const int64_t q = items;
    uint64_t acc[MAX_SAMPLES];
#pragma unroll
    for (int x = 0; x < MAX_SAMPLES; ++x) acc[x] = 0;
    const int64_t stride = (int64_t)gridDim.x * BLOCK;
    for (int64_t i = (int64_t)blockIdx.x * BLOCK + threadIdx.x; i < items; i += stride) {
        uint64_t cur[NT], d[NT];
#pragma unroll
        for (int k = 0; k < NT; ++k) {
            uint64_t* f = pb.tab[k];
            uint64_t lo, hi;
            if (MODE == 0) { lo = f[i]; hi = lo; }
            else if (MODE == 1) { lo = f[i]; hi = f[i + q]; }
            else {
                const uint64_t a0 = f[i], b0 = f[i + q], a1 = f[i + 2 * q], b1 = f[i + 3 * q];
                lo = add(a0, mul(r, sub(a1, a0)));
                hi = add(b0, mul(r, sub(b1, b0)));
                f[i] = lo;
                f[i + q] = hi;
            }
            cur[k] = lo;
            d[k] = sub(hi, lo);
        }
#pragma unroll
        for (int x = 0; x < NS; ++x) {
            if (!(skip1 && x == 1)) {
                uint64_t prod = cur[0];
#pragma unroll
                for (int k = 1; k < NT; ++k) prod = mul(prod, cur[k]);
                acc[x] = add(acc[x], prod);
            }
            if (x + 1 < NS) {
#pragma unroll
                for (int k = 0; k < NT; ++k) cur[k] = add(cur[k], d[k]);
            }
        }
    }
    if (counter) block_reduce_finish(acc, NS, partials, counter, out);
    else block_reduce(acc, NS, partials);
}

template <int MODE>
void launch_simple(const Problem& pb, int g, cudaStream_t st, int64_t size, uint64_t r, int skip1, uint64_t* partials,
                   unsigned* counter = nullptr, uint64_t* out = nullptr) {
    switch (pb.n_tables) {
        case 1: k_sumcheck_simple<MODE, 1><<<g, BLOCK, 0, st>>>(pb, size, r, skip1, partials, counter, out); break;
        case 2: k_sumcheck_simple<MODE, 2><<<g, BLOCK, 0, st>>>(pb, size, r, skip1, partials, counter, out); break;
        case 3: k_sumcheck_simple<MODE, 3><<<g, BLOCK, 0, st>>>(pb, size, r, skip1, partials, counter, out); break;
        default: k_sumcheck_simple<MODE, 4><<<g, BLOCK, 0, st>>>(pb, size, r, skip1, partials, counter, out); break;
    }
}

__global__ void __launch_bounds__(BLOCK) k_sumcheck_finish(const uint64_t* __restrict__ partials, int n_blocks,
                                                           int ns, uint64_t* __restrict__ out) {
    uint64_t acc[MAX_SAMPLES];
#pragma unroll
    for (int x = 0; x < MAX_SAMPLES; ++x) acc[x] = 0;
    for (int b = threadIdx.x; b < n_blocks; b += BLOCK)
#pragma unroll
        for (int x = 0; x < MAX_SAMPLES; ++x)
            if (x < ns) acc[x] = add(acc[x], partials[(int64_t)b * MAX_SAMPLES + x]);
    __shared__ uint64_t red[BLOCK / 32][MAX_SAMPLES];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
    for (int x = 0; x < MAX_SAMPLES; ++x) {
        if (x < ns) {
            uint64_t v = acc[x];
#pragma unroll
            for (int o = 16; o; o >>= 1) v = add(v, __shfl_xor_sync(0xffffffffu, v, o));
            if (lane == 0) red[wid][x] = v;
        }
    }
    __syncthreads();
    if (threadIdx.x < ns) {
        uint64_t v = 0;
#pragma unroll
        for (int w = 0; w < BLOCK / 32; ++w) v = add(v, red[w][threadIdx.x]);
        out[threadIdx.x] = v;
    }
}

// All remaining rounds of a queued run in ONE launch of one CTA, once the tables are small: below a
// few thousand entries a round is two launches of ~3.5 us of pure latency (the 2^24 instance spends
// 13 of its 24 rounds there), while one CTA folds and evaluates such a table in well under that.
// Rounds rnd0 .. n_rounds-1 are produced (round rnd0 without a fold when rnd0 == 0), then the last
// fold; samples and the skipped g(1) follow the conventions of vi_sumcheck_run.
constexpr int TAIL_BLOCK = 512;
constexpr int64_t TAIL_SIZE = 1 << 13;      // table length (before the pending fold) from which the tail kernel takes over
constexpr int TAIL_MAX_ROUNDS = 16;
struct TailCoins { uint64_t c[TAIL_MAX_ROUNDS]; };

template <int NT>
__global__ void __launch_bounds__(TAIL_BLOCK) k_sumcheck_tail(Problem pb, int64_t size, int rnd0, int n_rounds,
                                                              TailCoins coins, uint64_t* __restrict__ samples) {
    constexpr int NS = NT + 1;
    __shared__ uint64_t red[TAIL_BLOCK / 32][NS];
    const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
    for (int rnd = rnd0; rnd < n_rounds; ++rnd) {
        const bool fold = rnd > 0;
        const uint64_t r = fold ? coins.c[rnd - rnd0] : 0;          // coins.c[j] = challenge of round rnd0 + j - 1
        const int64_t items = fold ? size / 4 : size / 2, q = items;
        uint64_t acc[NS];
#pragma unroll
        for (int x = 0; x < NS; ++x) acc[x] = 0;
        for (int64_t i = tid; i < items; i += TAIL_BLOCK) {
            uint64_t cur[NT], d[NT];
#pragma unroll
            for (int k = 0; k < NT; ++k) {
                uint64_t* f = pb.tab[k];
                uint64_t lo, hi;
                if (!fold) { lo = f[i]; hi = f[i + q]; }
                else {
                    const uint64_t a0 = f[i], b0 = f[i + q], a1 = f[i + 2 * q], b1 = f[i + 3 * q];
                    lo = add(a0, mul(r, sub(a1, a0)));
                    hi = add(b0, mul(r, sub(b1, b0)));
                    f[i] = lo;
                    f[i + q] = hi;
                }
                cur[k] = lo;
                d[k] = sub(hi, lo);
            }
#pragma unroll
            for (int x = 0; x < NS; ++x) {
                if (!(fold && x == 1)) {                 // g(1) of a folded round follows from g(0) + g(1) = g_prev(r)
                    uint64_t prod = cur[0];
#pragma unroll
                    for (int k = 1; k < NT; ++k) prod = mul(prod, cur[k]);
                    acc[x] = add(acc[x], prod);
                }
                if (x + 1 < NS) {
#pragma unroll
                    for (int k = 0; k < NT; ++k) cur[k] = add(cur[k], d[k]);
                }
            }
        }
#pragma unroll
        for (int x = 0; x < NS; ++x) {
            uint64_t v = acc[x];
#pragma unroll
            for (int o = 16; o; o >>= 1) v = add(v, __shfl_xor_sync(0xffffffffu, v, o));
            if (lane == 0) red[wid][x] = v;
        }
        __syncthreads();
        if (tid < NS) {
            uint64_t v = 0;
#pragma unroll
            for (int w = 0; w < TAIL_BLOCK / 32; ++w) v = add(v, red[w][tid]);
            samples[(int64_t)rnd * 8 + tid] = v;
        }
        if (fold) size /= 2;
        __syncthreads();          // folded entries (global memory) and `red` are reused by the next round
    }
    // last fold: size 2 -> 1
    if (tid < NT) {
        uint64_t* f = pb.tab[tid];
        const uint64_t r = coins.c[n_rounds - rnd0];
        f[0] = add(f[0], mul(r, sub(f[1], f[0])));
    }
}

// last fold: size 2 -> 1, no samples
__global__ void k_final_fold(Problem pb, uint64_t r) {
    int k = threadIdx.x;
    if (k < pb.n_tables) {
        uint64_t* f = pb.tab[k];
        f[0] = add(f[0], mul(r, sub(f[1], f[0])));
    }
}

int make_problem(Problem& pb, uint64_t* tables, int64_t stride, int n_tables, int n_terms,
                 const uint64_t* coefs, const int32_t* nfac, const int32_t* fac) {
    VI_REQUIRE(n_tables >= 1 && n_tables <= MAX_TABLES, "sumcheck: 1..%d tables supported (got %d)", MAX_TABLES, n_tables);
    VI_REQUIRE(n_terms >= 1 && n_terms <= MAX_TERMS, "sumcheck: 1..%d terms supported (got %d)", MAX_TERMS, n_terms);
    VI_REQUIRE(tables && coefs && nfac && fac, "sumcheck: null pointer");
    pb.n_tables = n_tables; pb.n_terms = n_terms; pb.deg = 0;
    for (int k = 0; k < MAX_TABLES; ++k) pb.tab[k] = k < n_tables ? tables + (int64_t)k * stride : nullptr;
    for (int t = 0; t < MAX_TERMS; ++t) {
        pb.coef[t] = 0; pb.nfac[t] = 0;
        for (int j = 0; j < MAX_FAC; ++j) pb.fac[t][j] = 0;
    }
    for (int t = 0; t < n_terms; ++t) {
        VI_REQUIRE(nfac[t] >= 1 && nfac[t] <= MAX_FAC, "sumcheck: a term needs 1..%d factors", MAX_FAC);
        VI_REQUIRE(coefs[t] < vgl::P, "sumcheck: coefficient not canonical");
        pb.coef[t] = coefs[t]; pb.nfac[t] = nfac[t];
        if (nfac[t] > pb.deg) pb.deg = nfac[t];
        for (int j = 0; j < nfac[t]; ++j) {
            int k = fac[t * MAX_FAC + j];
            VI_REQUIRE(k >= 0 && k < n_tables, "sumcheck: factor index out of range");
            pb.fac[t][j] = k;
        }
    }
    pb.simple = (n_terms == 1 && coefs[0] == 1 && nfac[0] == n_tables && n_tables <= MAX_FAC);
    if (pb.simple)
        for (int j = 0; j < n_tables; ++j)
            if (fac[j] != j) pb.simple = 0;
    return VI_OK;
}

size_t general_smem(const Problem& pb) { return (size_t)2 * pb.n_tables * BLOCK * sizeof(uint64_t); }

int grid_for(int64_t items) {
    int64_t g = (items + BLOCK - 1) / BLOCK;
    if (g < 1) g = 1;
    return (int)(g < MAX_GRID ? g : MAX_GRID);
}

}  // namespace

// per-CTA partial sums, then the ticket counter of the fused cross-CTA sum
extern "C" int64_t vi_sumcheck_scratch_bytes(void) { return (int64_t)MAX_GRID * MAX_SAMPLES * 8 + 64; }

extern "C" int vi_sumcheck_claim(const uint64_t* tables, int64_t stride, int n_tables, int64_t size,
                                 int n_terms, const uint64_t* coefs, const int32_t* nfac, const int32_t* fac,
                                 uint64_t* out, void* partials, void* stream) {
    Problem pb;
    int rc = make_problem(pb, const_cast<uint64_t*>(tables), stride, n_tables, n_terms, coefs, nfac, fac);
    if (rc) return rc;
    VI_REQUIRE(vi::is_pow2(size), "sumcheck: table size must be a power of two");
    VI_REQUIRE(out && partials, "sumcheck: null output/scratch");
    cudaStream_t st = (cudaStream_t)stream;
    int g = grid_for(size);
    vi::ProfScope prof(vi::PROF_SUMCHECK, st);
    if (pb.simple) launch_simple<0>(pb, g, st, size, 0, 0, (uint64_t*)partials);
    else k_sumcheck<0><<<g, BLOCK, general_smem(pb), st>>>(pb, size, 0, 0, (uint64_t*)partials);
    k_sumcheck_finish<<<1, BLOCK, 0, st>>>((const uint64_t*)partials, g, 1, out);
    return vi::check_launch("k_sumcheck<claim>");
}

extern "C" int vi_sumcheck_round(uint64_t* tables, int64_t stride, int n_tables, int64_t size,
                                 int n_terms, const uint64_t* coefs, const int32_t* nfac, const int32_t* fac,
                                 int flags, uint64_t r, uint64_t* out, void* partials, void* stream) {
    const int fold = flags & 1, skip1 = (flags >> 1) & 1;
    VI_REQUIRE((flags & ~3) == 0, "sumcheck: unknown flag bits");
    Problem pb;
    int rc = make_problem(pb, tables, stride, n_tables, n_terms, coefs, nfac, fac);
    if (rc) return rc;
    VI_REQUIRE(vi::is_pow2(size) && size >= 2, "sumcheck: table size must be a power of two >= 2");
    VI_REQUIRE(pb.deg + 1 <= MAX_SAMPLES, "sumcheck: degree too large");
    VI_REQUIRE(r < vgl::P, "sumcheck: challenge not canonical");
    VI_REQUIRE(out && partials, "sumcheck: null output/scratch");
    cudaStream_t st = (cudaStream_t)stream;
    vi::ProfScope prof(vi::PROF_SUMCHECK, st);
    if (!fold) {
        int g = grid_for(size / 2);
        if (pb.simple) launch_simple<1>(pb, g, st, size, 0, skip1, (uint64_t*)partials);
        else k_sumcheck<1><<<g, BLOCK, general_smem(pb), st>>>(pb, size, 0, skip1, (uint64_t*)partials);
        k_sumcheck_finish<<<1, BLOCK, 0, st>>>((const uint64_t*)partials, g, pb.deg + 1, out);
        return vi::check_launch("k_sumcheck<round>");
    }
    if (size == 2) {
        k_final_fold<<<1, 32, 0, st>>>(pb, r);
        return vi::check_launch("k_final_fold");
    }
    int g = grid_for(size / 4);
    if (pb.simple) launch_simple<2>(pb, g, st, size, r, skip1, (uint64_t*)partials);
    else k_sumcheck<2><<<g, BLOCK, general_smem(pb), st>>>(pb, size, r, skip1, (uint64_t*)partials);
    k_sumcheck_finish<<<1, BLOCK, 0, st>>>((const uint64_t*)partials, g, pb.deg + 1, out);
    return vi::check_launch("k_sumcheck<fold+round>");
}

// g_i(1) of the rounds i >= 1 of a queued run, on the device: g_i(1) = g_{i-1}(c_{i-1}) - g_i(0), with the
// previous round polynomial evaluated from its deg + 1 samples at the nodes 0..deg by Lagrange weights.
// The weights depend on the challenges only, so all rounds compute theirs at once (one thread per (round,
// node)); the chain over the rounds, which needs the completed row before, is left to one warp.
constexpr int COMPLETE_MAX_ROUNDS = 64;
struct CompleteArgs {
    uint64_t coin[COMPLETE_MAX_ROUNDS];      // coin[i] = challenge of round i
    uint64_t inv_den[MAX_SAMPLES];           // 1 / prod_{j != k} (k - j)
};

__global__ void __launch_bounds__(COMPLETE_MAX_ROUNDS * MAX_SAMPLES)
k_sumcheck_complete(uint64_t* __restrict__ samples, int n_rounds, int deg, CompleteArgs a) {
    __shared__ uint64_t w[COMPLETE_MAX_ROUNDS][MAX_SAMPLES];
    const int tid = threadIdx.x, rnd = tid / MAX_SAMPLES, k = tid % MAX_SAMPLES;
    if (rnd + 1 < n_rounds && k <= deg) {           // weight of node k for the polynomial of round rnd at coin[rnd]
        const uint64_t r = a.coin[rnd];
        uint64_t v = a.inv_den[k];
        for (int j = 0; j <= deg; ++j)
            if (j != k) v = mul(v, sub(r, (uint64_t)j));
        w[rnd][k] = v;
    }
    __syncthreads();
    if (tid < 32) {
        for (int i = 1; i < n_rounds; ++i) {
            uint64_t v = tid <= deg ? mul(w[i - 1][tid], samples[(int64_t)(i - 1) * 8 + tid]) : 0;
#pragma unroll
            for (int o = 4; o; o >>= 1) v = add(v, __shfl_xor_sync(0xffffffffu, v, o));   // MAX_SAMPLES = 8 lanes
            if (tid == 0) samples[(int64_t)i * 8 + 1] = sub(v, samples[(int64_t)i * 8]);
            __syncwarp();
        }
    }
}

extern "C" int vi_sumcheck_complete(uint64_t* samples, int n_rounds, int deg, const uint64_t* coins, void* stream) {
    VI_REQUIRE(n_rounds >= 0 && n_rounds <= COMPLETE_MAX_ROUNDS, "sumcheck_complete: at most 64 rounds");
    VI_REQUIRE(deg >= 1 && deg < MAX_SAMPLES, "sumcheck_complete: degree out of range");
    if (n_rounds < 2) return VI_OK;
    VI_REQUIRE(samples && coins, "sumcheck_complete: null pointer");
    CompleteArgs a{};
    for (int i = 0; i + 1 < n_rounds; ++i) {
        VI_REQUIRE(coins[i] < vgl::P, "sumcheck_complete: challenge not canonical");
        a.coin[i] = coins[i];
    }
    for (int k = 0; k <= deg; ++k) {
        uint64_t den = 1;
        for (int j = 0; j <= deg; ++j)
            if (j != k) den = vgl::hmul(den, j < k ? (uint64_t)(k - j) : vgl::P - (uint64_t)(j - k));
        a.inv_den[k] = vgl::hpow(den, vgl::P - 2);
    }
    k_sumcheck_complete<<<1, COMPLETE_MAX_ROUNDS * MAX_SAMPLES, 0, (cudaStream_t)stream>>>(samples, n_rounds, deg, a);
    return vi::check_launch("k_sumcheck_complete");
}

extern "C" int vi_sumcheck_run(uint64_t* tables, int64_t stride, int n_tables, int64_t size,
                               int n_terms, const uint64_t* coefs, const int32_t* nfac, const int32_t* fac,
                               const uint64_t* coins, int n_rounds, uint64_t* samples, void* partials, void* stream) {
    VI_REQUIRE(vi::is_pow2(size) && (int64_t(1) << n_rounds) == size, "sumcheck_run: size must be 2^n_rounds");
    VI_REQUIRE(n_rounds == 0 || (coins && samples), "sumcheck_run: null pointer");
    int64_t cur = size;
    unsigned* counter = partials ? (unsigned*)((char*)partials + (int64_t)MAX_GRID * MAX_SAMPLES * 8) : nullptr;
    bool counter_clear = false;
    for (int rnd = 0; rnd < n_rounds; ++rnd) {
        if (cur > TAIL_SIZE) {
            // large rounds of the common case: the cross-CTA sum is fused into the round kernel
            Problem pb;
            int rc = make_problem(pb, tables, stride, n_tables, n_terms, coefs, nfac, fac);
            if (rc) return rc;
            if (pb.simple) {
                VI_REQUIRE(samples && partials, "sumcheck: null output/scratch");
                cudaStream_t st = (cudaStream_t)stream;
                if (!counter_clear) { VI_CUDA(cudaMemsetAsync(counter, 0, sizeof(unsigned), st)); counter_clear = true; }
                vi::ProfScope prof(vi::PROF_SUMCHECK, st);
                uint64_t* out = samples + (int64_t)rnd * 8;
                if (rnd == 0) launch_simple<1>(pb, grid_for(cur / 2), st, cur, 0, 0, (uint64_t*)partials, counter, out);
                else {
                    VI_REQUIRE(coins[rnd - 1] < vgl::P, "sumcheck: challenge not canonical");
                    launch_simple<2>(pb, grid_for(cur / 4), st, cur, coins[rnd - 1], 1, (uint64_t*)partials, counter, out);
                    cur /= 2;
                }
                rc = vi::check_launch("k_sumcheck<fused>");
                if (rc) return rc;
                continue;
            }
        }
        if (cur <= TAIL_SIZE && n_rounds - rnd + 1 <= TAIL_MAX_ROUNDS) {
            // small tables: one single-CTA launch does rounds rnd .. n_rounds-1 and the last fold
            Problem pb;
            int rc = make_problem(pb, tables, stride, n_tables, n_terms, coefs, nfac, fac);
            if (rc) return rc;
            if (pb.simple) {
                VI_REQUIRE(samples && partials, "sumcheck: null output/scratch");
                TailCoins tc{};
                for (int j = 0; j <= n_rounds - rnd; ++j) {           // c[j] = challenge of round rnd + j - 1
                    const int idx = rnd + j - 1;
                    tc.c[j] = idx >= 0 ? coins[idx] : 0;
                    VI_REQUIRE(tc.c[j] < vgl::P, "sumcheck: challenge not canonical");
                }
                cudaStream_t st = (cudaStream_t)stream;
                vi::ProfScope prof(vi::PROF_SUMCHECK, st);
                switch (pb.n_tables) {
                    case 1: k_sumcheck_tail<1><<<1, TAIL_BLOCK, 0, st>>>(pb, cur, rnd, n_rounds, tc, samples); break;
                    case 2: k_sumcheck_tail<2><<<1, TAIL_BLOCK, 0, st>>>(pb, cur, rnd, n_rounds, tc, samples); break;
                    case 3: k_sumcheck_tail<3><<<1, TAIL_BLOCK, 0, st>>>(pb, cur, rnd, n_rounds, tc, samples); break;
                    default: k_sumcheck_tail<4><<<1, TAIL_BLOCK, 0, st>>>(pb, cur, rnd, n_rounds, tc, samples); break;
                }
                return vi::check_launch("k_sumcheck_tail");
            }
        }
        // rounds after the first skip the sample at x = 1 (flag 2): see the header
        int rc = vi_sumcheck_round(tables, stride, n_tables, cur, n_terms, coefs, nfac, fac, rnd > 0 ? 3 : 0,
                                   rnd > 0 ? coins[rnd - 1] : 0, samples + (int64_t)rnd * 8, partials, stream);
        if (rc) return rc;
        if (rnd > 0) cur /= 2;
    }
    if (n_rounds)   // last fold: every table collapses to its value at the challenge point
        return vi_sumcheck_round(tables, stride, n_tables, cur, n_terms, coefs, nfac, fac, 1, coins[n_rounds - 1],
                                 samples, partials, stream);
    return VI_OK;
}
