// Tile-pass DFT stages in lane form (gl_lanes.cuh), included by ntt.cu after Sched / PassArgs.
//
// Same stage schedule, index conventions and shared-memory tile [pos * CP + col] as run_stages in
// ntt.cu, with 16-byte elements: butterflies are carry-free lane adds that the two integer pipes
// share, twiddle constants come from W3 tables (three balanced 24-bit digits), and values are
// converted from / to the canonical 64-bit form only at the global-memory boundary of a pass.
// Lane bounds: a load or a multiply leaves |lane| < 2^25.01, a radix-16 stage adds at most 4 bits,
// every stage but the last ends in a multiply and the last one in to_u64 (which accepts 2^30).
#pragma once
#include "dft_lanes.cuh"
#include "gl_lanes.cuh"

namespace vlt {

using vln::Q;
using vln::W3;

__device__ __forceinline__ W3 ldg_w3(const W3* p) {
    const int4 t = __ldg(reinterpret_cast<const int4*>(p));
    W3 w;
    w.w0 = t.x; w.w1 = t.y; w.w2 = t.z; w.pad = 0;
    return w;
}
__device__ __forceinline__ Q lds_q(const int4* sm, int idx) {
    const int4 t = sm[idx];
    Q q;
    q.x[0] = t.x; q.x[1] = t.y; q.x[2] = t.z; q.x[3] = t.w;
    return q;
}
__device__ __forceinline__ void sts_q(int4* sm, int idx, const Q& q) {
    sm[idx] = make_int4(q.x[0], q.x[1], q.x[2], q.x[3]);
}

template <bool INV>
__device__ __forceinline__ W3 tw3_at(const W3* __restrict__ tw, uint32_t e, uint32_t mask) {
    return ldg_w3(tw + (INV ? ((0u - e) & mask) : e));     // w^-e = w^(n-e)
}

// Stages S..NS-1 of the tile DFT on lane-form registers; v is preloaded for stage S and holds the
// outputs of the last stage on return (Sched::last_k).  SC is the Sched<LOGL, SMALL_LAST> of ntt.cu.
// RHO0 > 0 (forward only): the transform is coset t of a length RHO0*L transform whose input was
// pre-multiplied by w_{RHO0*L}^(t*l) except for the factor common to a thread's first butterfly,
// w_{RHO0*L}^(t*qp); that factor is folded into the stage-0 twiddle: w_L^(qp*c) * w_{RHO0*L}^(t*qp)
// = tw0[qp*(RHO0*c + t)] with tw0 the table of w_{RHO0*L} (every output is multiplied, also c = 0).
template <class SC, int LOGL, bool INV, int S, int RHO0 = 0>
__device__ __forceinline__ void run_stages_q(Q (&v)[SC::EPT], int4* sm, int CP, int col, int w,
                                             const W3* __restrict__ twL, const W3* __restrict__ tw0 = nullptr,
                                             int t = 0) {
    if constexpr (S < SC::NS) {
        constexpr int LOGR = SC::logr(S), R = 1 << LOGR, G = SC::EPT / R, LOGP = SC::logp(S);
        constexpr int L = 1 << LOGL, PP = 1 << LOGP;
        constexpr bool LAST = (S == SC::NS - 1);
        if constexpr (S > 0) {
#pragma unroll
            for (int g = 0; g < G; ++g)
#pragma unroll
                for (int i = 0; i < R; ++i)
                    v[g * R + i] = lds_q(sm, ((w + g * SC::TPC) + i * (L / R)) * CP + col);
        }
#pragma unroll
        for (int g = 0; g < G; ++g) vdft::dif<LOGR, LOGR, INV>(&v[g * R]);
        if constexpr (!LAST) {
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const uint32_t qp = (uint32_t)(w + g * SC::TPC) >> LOGP;
                if constexpr (S == 0 && RHO0 > 0) {
                    static_assert(!INV && LOGP == 0, "coset twiddles: forward stage 0 only");
#pragma unroll
                    for (int c = 0; c < R; ++c)
                        v[g * R + vdft::brev(c, LOGR)] =
                            vln::mul(v[g * R + vdft::brev(c, LOGR)], ldg_w3(tw0 + qp * (uint32_t)(RHO0 * c + t)));
                } else {
                    v[g * R] = vln::renorm(v[g * R]);     // output 0 has no twiddle: only bring its lanes back
#pragma unroll
                    for (int c = 1; c < R; ++c) {
                        const uint32_t e = (qp * c) << LOGP;
                        v[g * R + vdft::brev(c, LOGR)] =
                            vln::mul(v[g * R + vdft::brev(c, LOGR)], tw3_at<INV>(twL, e, L - 1));
                    }
                }
            }
            __syncthreads();
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const int x = w + g * SC::TPC;
                const int kappa = x & (PP - 1), qp = x >> LOGP;
#pragma unroll
                for (int c = 0; c < R; ++c)
                    sts_q(sm, (qp * PP * R + kappa + PP * c) * CP + col, v[g * R + vdft::brev(c, LOGR)]);
            }
            __syncthreads();
            run_stages_q<SC, LOGL, INV, S + 1, RHO0>(v, sm, CP, col, w, twL, tw0, t);
        }
    }
}

}  // namespace vlt
