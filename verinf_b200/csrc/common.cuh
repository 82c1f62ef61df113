// Shared host-side helpers of the C-ABI library: status codes, last-error text,
// launch checking.  No entry point ever exits the process or traps the device;
// every failure becomes a non-zero status plus a message (vi_last_error()).
#pragma once
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#define VI_OK 0
#define VI_ERR_ARG 1      // invalid argument (shape, alignment, size)
#define VI_ERR_CUDA 2     // a CUDA runtime call failed
#define VI_ERR_SCRATCH 3  // caller-provided scratch too small
#define VI_ERR_LIMIT 4    // size beyond what this build supports

namespace vi {

int fail(int code, const char* fmt, ...);   // records the message, returns code
int check_launch(const char* what);          // cudaGetLastError -> status

// Optional per-kernel timing with CUDA events on the launching stream (off by default).
enum ProfTag { PROF_ENC_PASS1 = 0, PROF_ENC_MID, PROF_ENC_PASS3, PROF_NTT_PASS, PROF_HASH, PROF_MERKLE,
               PROF_PRG, PROF_KQUANT, PROF_SUMCHECK, PROF_NTAGS };
struct ProfScope {
    int tag; cudaStream_t st; void* rec;
    ProfScope(int tag, cudaStream_t st);
    ~ProfScope();
};

inline bool is_pow2(int64_t n) { return n > 0 && (n & (n - 1)) == 0; }
inline int ilog2(int64_t n) { int l = 0; while ((int64_t(1) << l) < n) ++l; return l; }

}  // namespace vi

#define VI_REQUIRE(cond, ...) do { if (!(cond)) return vi::fail(VI_ERR_ARG, __VA_ARGS__); } while (0)
#define VI_CUDA(call) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) \
    return vi::fail(VI_ERR_CUDA, "%s: %s", #call, cudaGetErrorString(e_)); } while (0)
