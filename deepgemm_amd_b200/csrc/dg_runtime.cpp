// Process state, error strings, lazily loaded driver entry points and the settings API
// (counterpart of csrc/apis/config.hpp:9-47 and csrc/runtime/runtime.hpp:20-104 of the reference).
#include "dg_common.hpp"

#include <dlfcn.h>

#include <atomic>

namespace dg {

std::string& last_error() {
    static thread_local std::string e;
    return e;
}

int fail(int code, const char* fmt, ...) {
    char buf[4096];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error() = buf;
    return code;
}

State& state() {
    static State s;
    return s;
}

const Driver& driver() {
    static Driver d;
    static std::once_flag once;
    std::call_once(once, []() {
        void* h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) h = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) {
            d.why = std::string("cannot load libcuda.so.1: ") + dlerror();
            return;
        }
        auto sym = [&](const char* name, auto& fn) {
            fn = reinterpret_cast<std::remove_reference_t<decltype(fn)>>(dlsym(h, name));
            if (fn == nullptr && d.why.empty()) d.why = std::string("libcuda lacks ") + name;
        };
        sym("cuInit", d.cuInit);
        sym("cuGetErrorString", d.cuGetErrorString);
        sym("cuCtxGetCurrent", d.cuCtxGetCurrent);
        sym("cuModuleLoadData", d.cuModuleLoadData);
        sym("cuModuleGetFunction", d.cuModuleGetFunction);
        sym("cuFuncSetAttribute", d.cuFuncSetAttribute);
        sym("cuLaunchKernelEx", d.cuLaunchKernelEx);
        sym("cuOccupancyMaxActiveClusters", d.cuOccupancyMaxActiveClusters);
        sym("cuTensorMapEncodeTiled", d.cuTensorMapEncodeTiled);
        d.ok = d.why.empty();
    });
    return d;
}

std::string cu_error(CUresult r) {
    const char* s = nullptr;
    if (driver().ok && driver().cuGetErrorString(r, &s) == CUDA_SUCCESS && s != nullptr) return s;
    return "CUresult " + std::to_string(static_cast<int>(r));
}

int device_num_sms() {
    // asked on every GEMM call (the count is part of the plan's key): the attribute of a device never changes
    constexpr int kMaxDevices = 64;
    static std::atomic<int> counts[kMaxDevices];
    int dev = 0, n = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) { cudaGetLastError(); return 0; }
    if (dev >= 0 && dev < kMaxDevices && (n = counts[dev].load(std::memory_order_relaxed)) > 0) return n;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) { cudaGetLastError(); return 0; }
    if (dev >= 0 && dev < kMaxDevices) counts[dev].store(n, std::memory_order_relaxed);
    return n;
}

int ensure_status_word() {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mu);
    if (s.status_host != nullptr) return DG_OK;
    int* h = nullptr;
    DG_CUDA_RT(cudaHostAlloc(reinterpret_cast<void**>(&h), 64, cudaHostAllocMapped | cudaHostAllocPortable));
    *h = 0;
    int* d = nullptr;
    DG_CUDA_RT(cudaHostGetDevicePointer(reinterpret_cast<void**>(&d), h, 0));
    s.status_host = h;
    s.status_device = d;
    return DG_OK;
}

}  // namespace dg

using namespace dg;

extern "C" {

const char* dg_last_error(void) { return last_error().c_str(); }

int dg_init(const char* library_root) {
    State& s = state();
    std::lock_guard<std::mutex> lock(s.mu);
    s.library_root = library_root ? library_root : "";
    return DG_OK;
}

// csrc/apis/runtime.hpp of the reference: the runtime's resources are released once, a second call is a no-op, and the
// runtime is not recreated afterwards (every later call fails)
int dg_shutdown(void) {
    State& s = state();
    {
        std::lock_guard<std::mutex> lock(s.mu);
        if (s.shut_down) return DG_OK;
        s.shut_down = true;
        if (s.status_host != nullptr) cudaFreeHost(s.status_host);
        s.status_host = s.status_device = nullptr;
    }
    release_split_workspaces();
    cudaGetLastError();
    return DG_OK;
}

int dg_is_shut_down(void) { return state().shut_down ? 1 : 0; }

int dg_set_num_sms(int num_sms) {
    DG_REQUIRE_ALIVE();
    DG_REQUIRE(num_sms > 0 && num_sms % 2 == 0);
    const int dev = device_num_sms();
    if (dev > 0) DG_REQUIRE(num_sms <= dev);
    state().num_sms_override = num_sms;
    return DG_OK;
}

int dg_get_num_sms(void) {
    if (state().num_sms_override > 0) return state().num_sms_override;
    const int dev = device_num_sms();
    return dev > 0 ? dev : 148;
}

int dg_set_tc_util(int percent) {
    DG_REQUIRE_ALIVE();
    DG_REQUIRE(percent > 0 && percent <= 100);
    state().tc_util = percent;
    return DG_OK;
}
int dg_get_tc_util(void) { return state().tc_util; }
int dg_set_pdl(int enabled) {
    DG_REQUIRE_ALIVE(); state().pdl = enabled != 0; return DG_OK; }
int dg_get_pdl(void) { return state().pdl; }

int dg_set_mk_alignment_for_contiguous_layout(int alignment) {
    DG_REQUIRE_ALIVE(); state().mk_alignment = alignment; return DG_OK; }
int dg_get_mk_alignment_for_contiguous_layout(void) { return state().mk_alignment; }
int dg_get_theoretical_mk_alignment_for_contiguous_layout(int) { return 256; }

int dg_get_tma_aligned_size(int x, int element_size) {
    if (element_size <= 0 || 16 % element_size != 0) {
        fail(DG_ERR_INVALID_ARGUMENT, "Assertion error (%s:%d): kNumTMAAlignmentBytes %% element_size == 0", __FILE__, __LINE__);
        return -1;
    }
    return align_up(x, 16 / element_size);
}

int dg_kernel_status(void) {
    return state().status_host ? *reinterpret_cast<volatile int*>(state().status_host) : 0;
}
int dg_reset_kernel_status(void) {
    if (state().status_host) *reinterpret_cast<volatile int*>(state().status_host) = 0;
    return DG_OK;
}

// Runs the expiry path of the kernels' bounded waits on purpose: a one-CTA kernel built from the same ptx.cuh as the
// GEMM, with the limit lowered to `timeout_us`, in which one thread waits on an mbarrier that nobody arrives at while a
// second thread waits on another such barrier and must leave as soon as the first has given up (the CTA-wide abort
// flag).  The kernel returns normally; the status word then holds the first thread's code (role 7, site 3) and
// `elapsed_ns`, if given, how long that thread waited.  Synchronises the stream.
int dg_selftest_bounded_wait(uint32_t timeout_us, void* stream, uint64_t* elapsed_ns) {
    DG_REQUIRE_ALIVE();
    DG_REQUIRE(timeout_us >= 100 && timeout_us <= 1000000);
    int rc = DG_OK;
    const std::string src =
        "#define DG_WAIT_TIMEOUT_NS " + std::to_string(static_cast<unsigned long long>(timeout_us) * 1000ull) + "ull\n"
        "#include <dg/ptx.cuh>\n"
        "extern \"C\" __global__ void __launch_bounds__(64, 1) dg_selftest_bounded_wait_kernel(int* status, unsigned long long* out) {\n"
        "    using namespace dg;\n"
        "    __shared__ __align__(8) unsigned long long bars[2];\n"
        "    __shared__ uint32_t flag;\n"
        "    if (threadIdx.x == 0) { flag = 0; mbar_init(smem_u32(&bars[0]), 1); mbar_init(smem_u32(&bars[1]), 1); fence_mbar_init(); }\n"
        "    __syncthreads();\n"
        "    const AbortCtx ctx{&flag, status};\n"
        "    if (threadIdx.x == 0) {\n"
        "        const uint64_t t0 = global_timer_ns();\n"
        "        const bool ok = mbar_wait(smem_u32(&bars[0]), 0, ctx, 7, 3);      // nobody arrives: runs out\n"
        "        out[0] = global_timer_ns() - t0;\n"
        "        out[1] = ok ? 1 : 0;\n"
        "    } else if (threadIdx.x == 32) {\n"
        "        // starts half a limit later, so that its own limit cannot run out before the first waiter's does\n"
        "        const uint64_t t_delay = global_timer_ns();\n"
        "        while (global_timer_ns() - t_delay < DG_WAIT_TIMEOUT_NS / 2) { }\n"
        "        const uint64_t t0 = global_timer_ns();\n"
        "        const bool ok = mbar_wait(smem_u32(&bars[1]), 0, ctx, 7, 4);      // leaves when the flag is raised\n"
        "        out[2] = global_timer_ns() - t0;\n"
        "        out[3] = ok ? 1 : 0;\n"
        "    }\n"
        "    __syncthreads();\n"
        "}\n";
    dg_kernel_t kernel = nullptr;
    if ((rc = dg_jit_compile("selftest_bounded_wait", "dg_selftest_bounded_wait_kernel", src.c_str(), "", &kernel)) != DG_OK) return rc;
    if ((rc = ensure_status_word()) != DG_OK) return rc;
    // words 2..5 of the host-mapped status block receive the kernel's four results
    unsigned long long* out_host = reinterpret_cast<unsigned long long*>(state().status_host + 2);
    unsigned long long* out_dev = reinterpret_cast<unsigned long long*>(state().status_device + 2);
    for (int i = 0; i < 4; ++i) out_host[i] = ~0ull;
    int* status_dev = state().status_device;
    void* kargs[2] = {&status_dev, &out_dev};
    if ((rc = dg_jit_launch(kernel, 1, 64, 1, 0, 0, stream, kargs)) != DG_OK) return rc;
    DG_CUDA_RT(cudaStreamSynchronize(static_cast<cudaStream_t>(stream)));
    const volatile unsigned long long* res = out_host;
    if (res[1] != 0 || res[3] != 0)
        return fail(DG_ERR_CUDA, "bounded-wait self-test: a wait on a barrier nobody arrives at reported success (%llu, %llu)", res[1], res[3]);
    if (elapsed_ns != nullptr) { elapsed_ns[0] = res[0]; elapsed_ns[1] = res[2]; }
    return DG_OK;
}

}  // extern "C"
