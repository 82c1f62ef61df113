// Error text, launch checking and the optional CUDA-event profiler of the library.
#include <mutex>
#include <vector>

#include "../../include/verinf_b200.h"
#include "common.cuh"

namespace vi {

static thread_local char g_err[512] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return fail(VI_ERR_CUDA, "%s launch: %s", what, cudaGetErrorString(e));
    return VI_OK;
}

// ---- profiler: start/stop events around each launch, resolved on read ----------
struct Rec { int tag; cudaEvent_t a, b; };
static std::mutex g_pmu;
static bool g_on = false;
static std::vector<Rec> g_pending;
static std::vector<cudaEvent_t> g_pool;
static double g_ms[PROF_NTAGS];
static int64_t g_count[PROF_NTAGS];

static cudaEvent_t get_event() {
    if (!g_pool.empty()) { cudaEvent_t e = g_pool.back(); g_pool.pop_back(); return e; }
    cudaEvent_t e = nullptr;
    cudaEventCreate(&e);
    return e;
}

ProfScope::ProfScope(int tag_, cudaStream_t st_) : tag(tag_), st(st_), rec(nullptr) {
    if (!g_on) return;
    std::lock_guard<std::mutex> lk(g_pmu);
    Rec* r = new Rec{tag, get_event(), get_event()};
    cudaEventRecord(r->a, st);
    rec = r;
}
ProfScope::~ProfScope() {
    if (!rec) return;
    std::lock_guard<std::mutex> lk(g_pmu);
    Rec* r = (Rec*)rec;
    cudaEventRecord(r->b, st);
    g_pending.push_back(*r);
    delete r;
}

static void resolve() {
    for (auto& r : g_pending) {
        float ms = 0.f;
        if (cudaEventSynchronize(r.b) == cudaSuccess && cudaEventElapsedTime(&ms, r.a, r.b) == cudaSuccess) {
            g_ms[r.tag] += ms;
            g_count[r.tag] += 1;
        }
        g_pool.push_back(r.a);
        g_pool.push_back(r.b);
    }
    g_pending.clear();
}

}  // namespace vi

extern "C" const char* vi_last_error(void) { return vi::g_err; }

extern "C" void vi_profile_enable(int on) {
    std::lock_guard<std::mutex> lk(vi::g_pmu);
    vi::resolve();
    vi::g_on = on != 0;
    for (int t = 0; t < vi::PROF_NTAGS; ++t) { vi::g_ms[t] = 0; vi::g_count[t] = 0; }
}

extern "C" int vi_profile_num_tags(void) { return vi::PROF_NTAGS; }

extern "C" const char* vi_profile_tag_name(int tag) {
    static const char* names[vi::PROF_NTAGS] = {"encode_pass1", "encode_mid", "encode_pass3", "ntt_pass",
                                                "hash_columns", "merkle_level", "row_prg", "kquant", "sumcheck"};
    return (tag >= 0 && tag < vi::PROF_NTAGS) ? names[tag] : "?";
}

extern "C" int vi_profile_read(int tag, double* total_ms, int64_t* launches) {
    if (tag < 0 || tag >= vi::PROF_NTAGS) return vi::fail(VI_ERR_ARG, "profile: bad tag %d", tag);
    std::lock_guard<std::mutex> lk(vi::g_pmu);
    vi::resolve();
    if (total_ms) *total_ms = vi::g_ms[tag];
    if (launches) *launches = vi::g_count[tag];
    return VI_OK;
}
