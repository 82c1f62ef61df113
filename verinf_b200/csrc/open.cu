// Column openings on the device: the T queried columns of a codeword matrix and the
// Merkle authentication paths of their leaves.
//
// What it replaces in the reference: `codes.index_select(1, Q_set)` followed by one
// `.clone()` per column and a final `torch.cat` per column (prover/core.py:1304-1320),
// and `merkle_path` over the whole tree pulled to the host as Python `bytes` lists
// (prover/core.py:294-317, 3532-3547).  Here the tree stays on the device and only
// T * depth * 32 bytes of siblings leave it.
#include "../../include/verinf_b200.h"
#include "common.cuh"

namespace {

// out[t * out_stride + row0 + r] = mat[r * n + cols[t]]; threads run along r so the stores of
// a column are contiguous; every load is its own 32-byte sector by nature of the gather.
__global__ void __launch_bounds__(256) k_open_columns(const uint64_t* __restrict__ mat, int64_t m, int64_t n,
                                                      const int64_t* __restrict__ cols, int64_t T,
                                                      uint64_t* __restrict__ out, int64_t out_stride, int64_t row0) {
    const int64_t r = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= m) return;
    const uint64_t* src = mat + r * n;
    for (int64_t t = blockIdx.y; t < T; t += gridDim.y) {
        const int64_t c = cols[t];
        out[t * out_stride + row0 + r] = (c >= 0 && c < n) ? __ldg(src + c) : 0;
    }
}

// one thread per (query, level, 16-byte quarter of the node)
__global__ void __launch_bounds__(256) k_merkle_paths(const uint8_t* __restrict__ leaves, int64_t n,
                                                      const uint8_t* __restrict__ upper, int depth,
                                                      const int64_t* __restrict__ idx, int64_t T,
                                                      uint8_t* __restrict__ siblings, uint8_t* __restrict__ sides) {
    const int64_t g = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int q = (int)(g & 1);
    const int64_t pair = g >> 1;
    if (pair >= T * depth) return;
    const int64_t t = pair / depth;
    const int lvl = (int)(pair - t * depth);
    // walk down to this level: size and base of the level, index of the node on the path
    int64_t size = n, i = idx[t];
    if (i < 0 || i >= n) i = 0;                 // rejected on the host; never read out of range
    const uint8_t* base = leaves;
    const uint8_t* nxt = upper;
    for (int l = 0; l < lvl; ++l) {
        i >>= 1;
        size = (size + 1) >> 1;
        base = nxt;
        nxt += size * 32;
    }
    int64_t sib = i ^ 1;
    if (sib >= size) sib = i;                   // odd level: the last node is paired with itself
    const uint4* src = reinterpret_cast<const uint4*>(base + sib * 32);
    uint4* dst = reinterpret_cast<uint4*>(siblings + pair * 32);
    dst[q] = __ldg(src + q);
    if (q == 0) sides[pair] = (i & 1) == 0 ? 1 : 0;
}

}  // namespace

extern "C" int vi_open_columns(const uint64_t* mat, int64_t m, int64_t n, const int64_t* cols_dev, int64_t T,
                               uint64_t* out, int64_t out_stride, int64_t row0, void* stream) {
    VI_REQUIRE(m >= 0 && n >= 0 && T >= 0, "open_columns: negative size");
    VI_REQUIRE(row0 >= 0 && out_stride >= row0 + m, "open_columns: rows %lld..%lld do not fit the output stride %lld",
               (long long)row0, (long long)(row0 + m), (long long)out_stride);
    if (m == 0 || T == 0) return VI_OK;
    VI_REQUIRE(mat && cols_dev && out, "open_columns: null pointer");
    const int64_t gx = (m + 255) / 256;
    if (gx > 0x7FFFFFFFLL) return vi::fail(VI_ERR_LIMIT, "open_columns: too many rows");
    dim3 grid((unsigned)gx, (unsigned)(T < 65535 ? T : 65535));
    k_open_columns<<<grid, 256, 0, (cudaStream_t)stream>>>(mat, m, n, cols_dev, T, out, out_stride, row0);
    return vi::check_launch("k_open_columns");
}

extern "C" int vi_merkle_depth(int64_t n_leaves) {
    int d = 0;
    while (n_leaves > 1) { n_leaves = (n_leaves + 1) / 2; ++d; }
    return d;
}

extern "C" int vi_merkle_paths(const uint8_t* leaves, int64_t n_leaves, const uint8_t* upper,
                               const int64_t* idx_dev, int64_t T, uint8_t* siblings, uint8_t* sides, void* stream) {
    VI_REQUIRE(n_leaves >= 1 && T >= 0, "merkle_paths: bad size");
    const int depth = vi_merkle_depth(n_leaves);
    if (T == 0 || depth == 0) return VI_OK;
    VI_REQUIRE(leaves && upper && idx_dev && siblings && sides, "merkle_paths: null pointer");
    VI_REQUIRE(((uintptr_t)leaves | (uintptr_t)upper | (uintptr_t)siblings) % 16 == 0,
               "merkle_paths: node buffers must be 16-byte aligned");
    const int64_t threads = T * depth * 2;
    const int64_t grid = (threads + 255) / 256;
    if (grid > 0x7FFFFFFFLL) return vi::fail(VI_ERR_LIMIT, "merkle_paths: too many queries");
    k_merkle_paths<<<(unsigned)grid, 256, 0, (cudaStream_t)stream>>>(leaves, n_leaves, upper, depth, idx_dev, T,
                                                                     siblings, sides);
    return vi::check_launch("k_merkle_paths");
}
