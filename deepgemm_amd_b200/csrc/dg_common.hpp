// Shared host-side helpers: error reporting, lazily loaded CUDA driver entry points, process state.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <cstring>
#include <string>
#include <vector>

#include "../../include/deepgemm_b200.h"

extern "C" char** environ;          // the process environment (unistd.h declares it only with _GNU_SOURCE)

namespace dg {

// ---- errors -------------------------------------------------------------------------------------
std::string& last_error();
int fail(int code, const char* fmt, ...) __attribute__((format(printf, 2, 3)));

// The reference reports a failed check as "Assertion error (file:line): cond"
// (csrc/utils/exception.hpp:13-41); the same text is kept so callers can match on it.
#define DG_REQUIRE(cond)                                                                              \
    do {                                                                                              \
        if (!(cond))                                                                                  \
            return ::dg::fail(DG_ERR_INVALID_ARGUMENT, "Assertion error (%s:%d): %s", __FILE__, __LINE__, #cond); \
    } while (0)

#define DG_CUDA_RT(call)                                                                              \
    do {                                                                                              \
        cudaError_t e_ = (call);                                                                      \
        if (e_ != cudaSuccess)                                                                        \
            return ::dg::fail(DG_ERR_CUDA, "CUDA runtime error (%s:%d): %s: %s", __FILE__, __LINE__, #call, cudaGetErrorString(e_)); \
    } while (0)

// ---- CUDA driver, loaded on first use so that the library loads on machines without a GPU ---------
struct Driver {
    CUresult (*cuInit)(unsigned int) = nullptr;
    CUresult (*cuGetErrorString)(CUresult, const char**) = nullptr;
    CUresult (*cuCtxGetCurrent)(CUcontext*) = nullptr;
    CUresult (*cuModuleLoadData)(CUmodule*, const void*) = nullptr;
    CUresult (*cuModuleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
    CUresult (*cuFuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
    CUresult (*cuLaunchKernelEx)(const CUlaunchConfig*, CUfunction, void**, void**) = nullptr;
    CUresult (*cuOccupancyMaxActiveClusters)(int*, CUfunction, const CUlaunchConfig*) = nullptr;
    CUresult (*cuTensorMapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                       const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                       CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
    bool ok = false;
    std::string why;
};
const Driver& driver();
std::string cu_error(CUresult r);

#define DG_CUDA_DRV(call)                                                                             \
    do {                                                                                              \
        CUresult r_ = (call);                                                                         \
        if (r_ != CUDA_SUCCESS)                                                                       \
            return ::dg::fail(DG_ERR_CUDA, "CUDA driver error (%s:%d): %s: %s", __FILE__, __LINE__, #call, ::dg::cu_error(r_).c_str()); \
    } while (0)

// ---- process-wide state (csrc/runtime/runtime.hpp:20-104, heuristics/runtime.hpp:10-67) ------------
struct State {
    std::mutex mu;
    std::string library_root;
    int num_sms_override = 0;
    int tc_util = 100;
    int pdl = 0;
    int mk_alignment = 128;
    int* status_host = nullptr;      // pinned, mapped: kernels write failure codes here
    int* status_device = nullptr;
    bool shut_down = false;          // dg_shutdown() was called: buffers released, every later call fails
};
State& state();
int device_num_sms();                // SM count of the current device, 0 if there is none
int ensure_status_word();            // allocates the host-mapped status word on first GPU use
void release_split_workspaces();     // frees the library-owned split-K panels of every device
#define DG_REQUIRE_ALIVE() \
    do { if (::dg::state().shut_down) return ::dg::fail(DG_ERR_INVALID_ARGUMENT, "the runtime has been shut down (dg_shutdown)"); } while (0)

// Settings read from the environment: DG_<name> first, then DJ_<name> as the reference's runtime does (README.md:166).
// A GEMM call consults some twenty of them, and twenty getenv scans cost more host time than a decode-sized kernel
// runs, so each thread keeps the DG_* / DJ_* entries of its last look at `environ`; env_refresh() (one pass over
// `environ`, called at the top of every entry point that reads settings) notices any change through a hash of those
// entries, so a variable set between two calls is seen by the second.
struct EnvSnapshot {
    bool valid = false;
    uint64_t signature = 0;
    std::vector<std::pair<std::string, std::string>> vars;       // name without its three-character prefix, value; DG_ entries first
};
inline EnvSnapshot& env_snapshot() {
    thread_local EnvSnapshot snap;
    return snap;
}
inline void env_refresh() {
    const auto ours = [](const char* s) { return s[0] == 'D' && (s[1] == 'G' || s[1] == 'J') && s[2] == '_'; };
    uint64_t h = 1469598103934665603ull;
    for (char** e = environ; e != nullptr && *e != nullptr; ++e) {
        if (!ours(*e)) continue;
        for (const char* c = *e; *c; ++c) { h ^= static_cast<unsigned char>(*c); h *= 1099511628211ull; }
        h ^= 0xFFu; h *= 1099511628211ull;
    }
    EnvSnapshot& snap = env_snapshot();
    if (snap.valid && snap.signature == h) return;
    snap.vars.clear();
    for (int pass = 0; pass < 2; ++pass)                 // DG_ entries first, so that they win over DJ_ ones
        for (char** e = environ; e != nullptr && *e != nullptr; ++e) {
            const char* s = *e;
            if (!ours(s) || (s[1] == 'G') != (pass == 0)) continue;
            const char* eq = std::strchr(s, '=');
            if (eq == nullptr) continue;
            snap.vars.emplace_back(std::string(s + 3, eq), std::string(eq + 1));
        }
    snap.signature = h;
    snap.valid = true;
}
inline const char* env_raw(const char* name) {
    EnvSnapshot& snap = env_snapshot();
    if (!snap.valid) env_refresh();
    for (const auto& kv : snap.vars)
        if (kv.first == name) return kv.second.c_str();
    return nullptr;
}
inline int env_int(const char* name, int dflt = 0) {
    const char* v = env_raw(name);
    return v ? std::atoi(v) : dflt;
}
inline std::string env_str(const char* name) {
    const char* v = env_raw(name);
    return v ? std::string(v) : std::string();
}

template <typename T> static inline T ceil_div(T a, T b) { return (a + b - 1) / b; }
template <typename T> static inline T align_up(T a, T b) { return ceil_div(a, b) * b; }

}  // namespace dg
