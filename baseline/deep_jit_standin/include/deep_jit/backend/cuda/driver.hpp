// Stand-in for third-party/deep_jit of the reference: CUDA driver entry points resolved at first use (libcuda is not
// linked: the module imports on a machine without a GPU, as tests/test_lazy_init.py of the reference requires).
// The set is the one the reference calls: csrc/jit_kernels/impls/runtime_utils.hpp:153, csrc/runtime/locality_domain.hpp:61-93,
// csrc/runtime/mlopart.hpp:31, plus what the stand-in's own loader and launcher need.
#pragma once

#include <cuda.h>
#include <dlfcn.h>

#include <sstream>
#include <stdexcept>
#include <string>

namespace deep_jit::cuda::driver {

inline void* library() {
    static void* handle = [] {
        void* h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
        if (h == nullptr) h = dlopen("libcuda.so", RTLD_NOW | RTLD_GLOBAL);
        return h;
    }();
    if (handle == nullptr) throw std::runtime_error("deep_jit stand-in: libcuda.so.1 cannot be loaded (no NVIDIA driver on this machine)");
    return handle;
}

template <typename Fn>
Fn resolve(const char* versioned, const char* plain) {
    void* sym = dlsym(library(), versioned);
    if (sym == nullptr) sym = dlsym(library(), plain);
    if (sym == nullptr) throw std::runtime_error(std::string("deep_jit stand-in: libcuda has no ") + plain);
    return reinterpret_cast<Fn>(sym);
}

// One lazily resolved forwarder per driver function.  cuda.h renames some entry points with macros (name -> name_v2):
// the symbol looked up is the expanded name, then the plain one.
#define DJ_STANDIN_STR_(x) #x
#define DJ_STANDIN_STR(x) DJ_STANDIN_STR_(x)
#define DJ_STANDIN_LAZY(name)                                                                              \
    template <typename... Args>                                                                            \
    inline CUresult lazy_##name(Args... args) {                                                            \
        static const auto fn = resolve<decltype(&::name)>(DJ_STANDIN_STR(name), #name);                    \
        return fn(args...);                                                                                \
    }

DJ_STANDIN_LAZY(cuTensorMapEncodeTiled)
DJ_STANDIN_LAZY(cuMemGetAllocationGranularity)
DJ_STANDIN_LAZY(cuMemAddressReserve)
DJ_STANDIN_LAZY(cuMemAddressFree)
DJ_STANDIN_LAZY(cuMemMap)
DJ_STANDIN_LAZY(cuMemUnmap)
DJ_STANDIN_LAZY(cuMemRelease)
DJ_STANDIN_LAZY(cuMemSetAccess)
DJ_STANDIN_LAZY(cuMemImportFromShareableHandle)
DJ_STANDIN_LAZY(cuModuleLoadData)
DJ_STANDIN_LAZY(cuModuleUnload)
DJ_STANDIN_LAZY(cuModuleGetFunctionCount)
DJ_STANDIN_LAZY(cuModuleEnumerateFunctions)
DJ_STANDIN_LAZY(cuFuncSetAttribute)
DJ_STANDIN_LAZY(cuFuncGetName)
DJ_STANDIN_LAZY(cuLaunchKernelEx)
DJ_STANDIN_LAZY(cuGetErrorString)
DJ_STANDIN_LAZY(cuCtxGetCurrent)
DJ_STANDIN_LAZY(cuDeviceGet)
DJ_STANDIN_LAZY(cuDeviceGetAttribute)
DJ_STANDIN_LAZY(cuDeviceGetUuid)
DJ_STANDIN_LAZY(cuCtxGetDevice)
#undef DJ_STANDIN_LAZY
#undef DJ_STANDIN_STR
#undef DJ_STANDIN_STR_

inline std::string error_string(CUresult result) {
    const char* text = nullptr;
    if (lazy_cuGetErrorString(result, &text) == CUDA_SUCCESS && text != nullptr) return text;
    return "CUresult " + std::to_string(static_cast<int>(result));
}

}  // namespace deep_jit::cuda::driver

#define DJ_CUDA_DRIVER_CHECK(call)                                                                          \
    do {                                                                                                    \
        const CUresult dj_result_ = (call);                                                                 \
        if (dj_result_ != CUDA_SUCCESS) {                                                                   \
            std::ostringstream dj_message_;                                                                 \
            dj_message_ << "CUDA driver error (" << __FILE__ << ":" << __LINE__ << "): " #call ": "       \
                        << deep_jit::cuda::driver::error_string(dj_result_);                                \
            throw std::runtime_error(dj_message_.str());                                                    \
        }                                                                                                   \
    } while (0)
