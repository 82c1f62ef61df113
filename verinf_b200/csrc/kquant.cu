// Standalone K-quant -> field lift (API-compatible with the reference's
// kquant_to_field, prover/kquant_cuda.py:60-177).  One warp per super-block: lane l
// decodes elements l, l+32, ..., l+224, so the 8-byte outputs of a warp are 256-byte
// contiguous stores and the header bytes are warp-uniform (one L1 line per block).
#include "../../include/verinf_b200.h"
#include "common.cuh"
#include "kquant.cuh"

namespace {

template <int QT>
__global__ void __launch_bounds__(256) k_kquant(const uint8_t* __restrict__ raw, int64_t n_blocks, double S,
                                                uint64_t* __restrict__ out) {
    const int lane = threadIdx.x & 31;
    const int64_t warps = ((int64_t)gridDim.x * blockDim.x) >> 5;
    for (int64_t b = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; b < n_blocks; b += warps) {
        const uint8_t* p = raw + b * vkq::block_bytes(QT);
        uint64_t* o = out + b * 256;
#pragma unroll
        for (int j = 0; j < 8; ++j) o[j * 32 + lane] = vkq::lift<QT>(p, j * 32 + lane, S);
    }
}

}  // namespace

extern "C" int vi_kquant_to_field(const uint8_t* raw, int64_t n_blocks, int qtype, double S,
                                  uint64_t* out, void* stream) {
    VI_REQUIRE(qtype == 4 || qtype == 5 || qtype == 6, "kquant: qtype must be 4 (Q4_K), 5 (Q5_K) or 6 (Q6_K)");
    VI_REQUIRE(n_blocks >= 0, "kquant: negative block count");
    if (n_blocks == 0) return VI_OK;
    VI_REQUIRE(raw && out, "kquant: null pointer");
    int64_t g = (n_blocks + 7) / 8;
    unsigned grid = (unsigned)(g < 148 * 32 ? g : 148 * 32);
    cudaStream_t st = (cudaStream_t)stream;
    vi::ProfScope prof(vi::PROF_KQUANT, st);
    if (qtype == 4) k_kquant<4><<<grid, 256, 0, st>>>(raw, n_blocks, S, out);
    else if (qtype == 5) k_kquant<5><<<grid, 256, 0, st>>>(raw, n_blocks, S, out);
    else k_kquant<6><<<grid, 256, 0, st>>>(raw, n_blocks, S, out);
    return vi::check_launch("k_kquant");
}
