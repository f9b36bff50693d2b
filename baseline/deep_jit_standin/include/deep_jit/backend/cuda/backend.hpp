// Stand-in for the un-vendored DeepJIT submodule of the reference (third-party/deep_jit, URL only in .gitmodules:4-6,
// no pinned revision): the run-time compiler, cache, loader and launcher behind `deep_gemm::jit`.
//
// The interface is the one visible through the reference's call sites, nothing more:
//   deep_jit::Config(root, env_prefix, cache_tag, include_dirs, header_prefixes)            csrc/runtime/jit.hpp:16-21
//   deep_jit::Runtime<deep_jit::CUDA>(config); .default_compiler_options.nvcc_flags->emplace_back(...)   :23-28
//   jit->compile(tag, code[, CompilerOptions{.arch}]) -> kernel; jit->launch(kernel, LaunchOptions{...}, args...)
//                                                            csrc/jit_kernels/impls/sm100_fp8_fp4_gemm_1d1d.hpp:40,82-89
//   jit->device.get_num_sms() / get_arch_major() / get_arch(bool) / get_prop()             csrc/runtime/runtime.hpp:86,
//                                                            csrc/utils/layout.hpp:43, csrc/jit_kernels/impls/epilogue_class.hpp:99
//   jit->default_launch_options.enable_pdl                                                  csrc/apis/config.hpp:27-32
// and the behaviour the reference's README documents for it (README.md:164-191): nvcc found through
// DG_JIT_NVCC_COMPILER / CUDA_HOME / CUDA_PATH / PATH / /usr/local/cuda, C++20, cubins cached under DG_JIT_CACHE_DIR
// (":"-separated, first hit wins, misses compile into the first) else $HOME/.dj, DG_JIT_DEBUG /
// DG_JIT_PRINT_COMPILER_COMMAND / DG_JIT_PTXAS_VERBOSE / DG_JIT_WITH_LINEINFO.
//
// It lets the UNMODIFIED reference be built and run beside this repository's kernels for timing.  It is not part of
// the product library and shares no code with it.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>

#include <unistd.h>

#include <algorithm>
#include <array>
#include <cstdio>
#include <cstdlib>
#include <filesystem>
#include <fstream>
#include <functional>
#include <map>
#include <memory>
#include <mutex>
#include <optional>
#include <sstream>
#include <stdexcept>
#include <string>
#include <vector>

#if __has_include(<c10/cuda/CUDAStream.h>)
#include <c10/cuda/CUDAStream.h>
#define DJ_STANDIN_HAS_TORCH_STREAM 1
#endif

#include "../../utils/env.hpp"
#include "../../utils/lazy.hpp"
#include "driver.hpp"

namespace deep_jit {

struct CUDA {};          // backend tag

struct Config {
    std::filesystem::path library_root;
    std::string env_prefix;                              // "DG": DG_JIT_* first, DJ_JIT_* as fallback
    std::string cache_tag;                               // part of every cache key ("cutlass-<version>")
    std::vector<std::filesystem::path> include_dirs;     // -I for every compilation
    std::vector<std::string> header_prefixes;            // headers whose contents belong to the cache key ("deep_gemm/")

    Config(std::filesystem::path root, std::string prefix, std::string tag, std::vector<std::filesystem::path> includes,
           std::vector<std::string> prefixes)
        : library_root(std::move(root)), env_prefix(std::move(prefix)), cache_tag(std::move(tag)),
          include_dirs(std::move(includes)), header_prefixes(std::move(prefixes)) {}
};

namespace cuda {

struct CompilerOptions {
    std::optional<std::string> arch;                     // e.g. "100a"; the device's own architecture when unset
    std::optional<std::vector<std::string>> nvcc_flags;  // appended to the command line
};

struct LaunchOptions {
    std::optional<int> num_smem_bytes;
    std::optional<dim3> grid_dim;
    std::optional<dim3> block_dim;
    std::optional<dim3> cluster_dim;
    std::optional<bool> enable_pdl;
};

class Device {
public:
    const cudaDeviceProp& get_prop() {
        int device = 0;
        check(cudaGetDevice(&device), "cudaGetDevice");
        std::lock_guard<std::mutex> lock(mutex_);
        auto it = props_.find(device);
        if (it == props_.end()) {
            cudaDeviceProp prop;
            check(cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
            it = props_.emplace(device, prop).first;
        }
        return it->second;
    }
    int get_num_sms() { return get_prop().multiProcessorCount; }
    int get_arch_major() { return get_prop().major; }
    int get_arch_minor() { return get_prop().minor; }
    // Architecture string for nvcc: the family-wide target ("100f") or the device-specific one ("100a")
    std::string get_arch(const bool family = false) {
        return std::to_string(get_arch_major() * 10 + get_arch_minor()) + (family ? "f" : "a");
    }

private:
    static void check(cudaError_t e, const char* what) {
        if (e != cudaSuccess) throw std::runtime_error(std::string("deep_jit stand-in: ") + what + ": " + cudaGetErrorString(e));
    }
    std::mutex mutex_;
    std::map<int, cudaDeviceProp> props_;
};

}  // namespace cuda

// A compiled kernel: the cubin on disk, loaded into a context on first launch
struct Kernel {
    std::string tag;
    std::filesystem::path cubin_path;
    std::mutex mutex;
    std::map<CUcontext, std::pair<CUmodule, CUfunction>> loaded;
    std::map<CUcontext, int> smem_limit;
};
using KernelHandle = std::shared_ptr<Kernel>;

template <typename Backend>
class Runtime;

template <>
class Runtime<CUDA> {
public:
    cuda::Device device;
    cuda::CompilerOptions default_compiler_options;
    cuda::LaunchOptions default_launch_options;

    explicit Runtime(Config config) : config_(std::move(config)) {
        default_compiler_options.nvcc_flags = std::vector<std::string>();
        default_launch_options.enable_pdl = false;
    }

    KernelHandle compile(const std::string& tag, const std::string& code, const cuda::CompilerOptions& options = {}) {
        const std::string arch = options.arch.has_value() ? *options.arch : device.get_arch(false);
        std::vector<std::string> flags = {"-std=c++" + std::to_string(env<int>("JIT_CPP_STANDARD", 20)), "-cubin", "-O3",
                                          "--expt-relaxed-constexpr", "--expt-extended-lambda",
                                          "-gencode=arch=compute_" + arch + ",code=sm_" + arch};
        if (env<int>("JIT_WITH_LINEINFO", 0) || debug()) flags.emplace_back("-lineinfo");
        if (env<int>("JIT_PTXAS_VERBOSE", 0) || debug()) flags.emplace_back("--ptxas-options=-v");
        for (const auto& f : *default_compiler_options.nvcc_flags) flags.push_back(f);
        if (options.nvcc_flags.has_value())
            for (const auto& f : *options.nvcc_flags) flags.push_back(f);
        // The cache key covers the flags that shape the code, not where the headers happen to live (their contents are
        // part of the key through headers_digest), so a cache directory can move with the installation
        std::string keyed_flags;
        for (const auto& f : flags) keyed_flags += f + " ";
        for (const auto& dir : config_.include_dirs) flags.push_back("-I" + dir.string());
        std::string joined;
        for (const auto& f : flags) joined += f + " ";

        const std::string key = tag + "." + hex(fnv(code + "\n" + keyed_flags + "\n" + config_.cache_tag + "\n" + nvcc_version() + "\n" + headers_digest()));
        {
            std::lock_guard<std::mutex> lock(mutex_);
            const auto it = kernels_.find(key);
            if (it != kernels_.end()) return it->second;
        }
        const auto dirs = cache_dirs();
        std::filesystem::path cubin;
        for (const auto& dir : dirs) {
            const auto candidate = dir / ("kernel." + key) / "kernel.cubin";
            if (std::filesystem::exists(candidate)) { cubin = candidate; break; }
        }
        if (cubin.empty()) cubin = build(dirs.front(), key, code, joined);
        auto kernel = std::make_shared<Kernel>();
        kernel->tag = tag;
        kernel->cubin_path = cubin;
        std::lock_guard<std::mutex> lock(mutex_);
        return kernels_.emplace(key, kernel).first->second;
    }

    template <typename... Args>
    void launch(const KernelHandle& kernel, const cuda::LaunchOptions& options, const Args&... args) {
        if (!options.grid_dim.has_value() || !options.block_dim.has_value())
            throw std::runtime_error("deep_jit stand-in: a launch needs grid_dim and block_dim");
        const CUfunction function = load(kernel, options.num_smem_bytes.value_or(0));
        void* pointers[] = {const_cast<void*>(static_cast<const void*>(&args))..., nullptr};

        CUlaunchConfig config = {};
        config.gridDimX = options.grid_dim->x; config.gridDimY = options.grid_dim->y; config.gridDimZ = options.grid_dim->z;
        config.blockDimX = options.block_dim->x; config.blockDimY = options.block_dim->y; config.blockDimZ = options.block_dim->z;
        config.sharedMemBytes = static_cast<unsigned>(options.num_smem_bytes.value_or(0));
        config.hStream = current_stream();
        CUlaunchAttribute attributes[2];
        unsigned count = 0;
        if (options.cluster_dim.has_value() && options.cluster_dim->x * options.cluster_dim->y * options.cluster_dim->z > 1) {
            attributes[count].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
            attributes[count].value.clusterDim.x = options.cluster_dim->x;
            attributes[count].value.clusterDim.y = options.cluster_dim->y;
            attributes[count].value.clusterDim.z = options.cluster_dim->z;
            ++count;
        }
        const bool pdl = options.enable_pdl.has_value() ? *options.enable_pdl : default_launch_options.enable_pdl.value_or(false);
        if (pdl) {
            attributes[count].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
            attributes[count].value.programmaticStreamSerializationAllowed = 1;
            ++count;
        }
        config.attrs = attributes;
        config.numAttrs = count;
        DJ_CUDA_DRIVER_CHECK(cuda::driver::lazy_cuLaunchKernelEx(&config, function, pointers, static_cast<void**>(nullptr)));
    }

    const Config& config() const { return config_; }

private:
    template <typename T>
    T env(const std::string& name, const T& fallback) const { return get_env<T>(config_.env_prefix + "_" + name, fallback); }
    bool debug() const { return env<int>("JIT_DEBUG", 0) != 0; }

    static CUstream current_stream() {
#ifdef DJ_STANDIN_HAS_TORCH_STREAM
        return c10::cuda::getCurrentCUDAStream().stream();       // the caller's current PyTorch stream
#else
        return nullptr;
#endif
    }

    static uint64_t fnv(const std::string& text) {
        uint64_t h = 1469598103934665603ull;
        for (const unsigned char c : text) { h ^= c; h *= 1099511628211ull; }
        return h;
    }
    static std::string hex(uint64_t v) {
        char buffer[17];
        std::snprintf(buffer, sizeof(buffer), "%016llx", static_cast<unsigned long long>(v));
        return buffer;
    }

    std::string nvcc_path() const {
        const auto explicit_path = env<std::string>("JIT_NVCC_COMPILER", "");
        if (!explicit_path.empty()) return explicit_path;
        for (const char* variable : {"CUDA_HOME", "CUDA_PATH"}) {
            const char* root = std::getenv(variable);
            if (root != nullptr && std::filesystem::exists(std::filesystem::path(root) / "bin" / "nvcc"))
                return (std::filesystem::path(root) / "bin" / "nvcc").string();
        }
        if (const char* path = std::getenv("PATH")) {
            std::istringstream in(path);
            std::string dir;
            while (std::getline(in, dir, ':'))
                if (!dir.empty() && std::filesystem::exists(std::filesystem::path(dir) / "nvcc")) return (std::filesystem::path(dir) / "nvcc").string();
        }
        return "/usr/local/cuda/bin/nvcc";
    }

    static std::string run(const std::string& command, int* status) {
        std::string output;
        FILE* pipe = popen((command + " 2>&1").c_str(), "r");
        if (pipe == nullptr) { *status = -1; return "popen failed"; }
        std::array<char, 4096> buffer;
        while (std::fgets(buffer.data(), buffer.size(), pipe) != nullptr) output += buffer.data();
        *status = pclose(pipe);
        return output;
    }

    std::string nvcc_version() {
        std::lock_guard<std::mutex> lock(mutex_);
        if (nvcc_version_.empty()) {
            int status = 0;
            nvcc_version_ = run(nvcc_path() + " --version", &status);
            if (status != 0) nvcc_version_ = "unknown";
        }
        return nvcc_version_;
    }

    // Sizes and modification-independent contents hash of the library's own device headers (the files under the
    // include directories whose path starts with one of the header prefixes): editing a kernel header invalidates
    // the cached cubins
    std::string headers_digest() {
        std::lock_guard<std::mutex> lock(mutex_);
        if (!headers_digest_.empty()) return headers_digest_;
        uint64_t h = 1469598103934665603ull;
        for (const auto& dir : config_.include_dirs)
            for (const auto& prefix : config_.header_prefixes) {
                const auto root = dir / prefix;
                if (!std::filesystem::is_directory(root)) continue;
                std::vector<std::filesystem::path> files;
                for (const auto& entry : std::filesystem::recursive_directory_iterator(root))
                    if (entry.is_regular_file()) files.push_back(entry.path());
                std::sort(files.begin(), files.end());
                for (const auto& file : files) {
                    std::ifstream in(file, std::ios::binary);
                    std::stringstream contents;
                    contents << in.rdbuf();
                    h ^= fnv(std::filesystem::relative(file, dir).string() + "\n" + contents.str());
                    h *= 1099511628211ull;
                }
            }
        headers_digest_ = hex(h);
        return headers_digest_;
    }

    std::vector<std::filesystem::path> cache_dirs() const {
        std::vector<std::filesystem::path> dirs;
        const auto listed = env<std::string>("JIT_CACHE_DIR", "");
        std::istringstream in(listed);
        std::string dir;
        while (std::getline(in, dir, ':'))
            if (!dir.empty()) dirs.emplace_back(dir);
        if (dirs.empty()) {
            const char* home = std::getenv("HOME");
            dirs.emplace_back(std::filesystem::path(home != nullptr ? home : "/tmp") / ".dj");
        }
        return dirs;
    }

    std::filesystem::path build(const std::filesystem::path& cache_dir, const std::string& key, const std::string& code,
                                const std::string& flags) {
        const auto final_dir = cache_dir / ("kernel." + key);
        const auto temp_dir = cache_dir / ("tmp." + key + "." + std::to_string(static_cast<long long>(::getpid())));
        std::filesystem::create_directories(temp_dir);
        {
            std::ofstream out(temp_dir / "kernel.cu");
            out << code;
        }
        const std::string command = nvcc_path() + " " + flags + "-o " + (temp_dir / "kernel.cubin").string() + " " + (temp_dir / "kernel.cu").string();
        if (env<int>("JIT_PRINT_COMPILER_COMMAND", 0) || debug()) std::fprintf(stderr, "[deep_jit stand-in] %s\n", command.c_str());
        int status = 0;
        const std::string output = run(command, &status);
        if (debug() || env<int>("JIT_PTXAS_VERBOSE", 0)) std::fprintf(stderr, "%s", output.c_str());
        if (status != 0 || !std::filesystem::exists(temp_dir / "kernel.cubin")) {
            std::filesystem::remove_all(temp_dir);
            throw std::runtime_error("deep_jit stand-in: nvcc failed for kernel `" + key + "`:\n" + command + "\n" + output);
        }
        std::error_code ec;
        std::filesystem::rename(temp_dir, final_dir, ec);          // atomic publish; a concurrent builder may have won
        if (ec) std::filesystem::remove_all(temp_dir);
        return final_dir / "kernel.cubin";
    }

    CUfunction load(const KernelHandle& kernel, const int smem_bytes) {
        // torch has made a context current by the time tensors exist
        CUcontext context = nullptr;
        DJ_CUDA_DRIVER_CHECK(cuda::driver::lazy_cuCtxGetCurrent(&context));
        if (context == nullptr) {
            cudaFree(nullptr);                                     // creates / binds the primary context
            DJ_CUDA_DRIVER_CHECK(cuda::driver::lazy_cuCtxGetCurrent(&context));
        }
        std::lock_guard<std::mutex> lock(kernel->mutex);
        auto it = kernel->loaded.find(context);
        if (it == kernel->loaded.end()) {
            std::ifstream in(kernel->cubin_path, std::ios::binary);
            std::stringstream image;
            image << in.rdbuf();
            const std::string bytes = image.str();
            if (bytes.empty()) throw std::runtime_error("deep_jit stand-in: empty cubin " + kernel->cubin_path.string());
            CUmodule module = nullptr;
            DJ_CUDA_DRIVER_CHECK(cuda::driver::lazy_cuModuleLoadData(&module, static_cast<const void*>(bytes.data())));
            unsigned count = 0;
            DJ_CUDA_DRIVER_CHECK(cuda::driver::lazy_cuModuleGetFunctionCount(&count, module));
            if (count == 0) throw std::runtime_error("deep_jit stand-in: no kernel in " + kernel->cubin_path.string());
            std::vector<CUfunction> functions(count);
            DJ_CUDA_DRIVER_CHECK(cuda::driver::lazy_cuModuleEnumerateFunctions(functions.data(), count, module));
            // The generated translation unit instantiates exactly one __global__ template
            if (count != 1) throw std::runtime_error("deep_jit stand-in: expected one kernel in " + kernel->cubin_path.string() +
                                                     ", found " + std::to_string(count));
            it = kernel->loaded.emplace(context, std::make_pair(module, functions[0])).first;
        }
        const CUfunction function = it->second.second;
        if (smem_bytes > kernel->smem_limit[context]) {
            DJ_CUDA_DRIVER_CHECK(cuda::driver::lazy_cuFuncSetAttribute(function, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, smem_bytes));
            kernel->smem_limit[context] = smem_bytes;
        }
        return function;
    }

    Config config_;
    std::mutex mutex_;
    std::map<std::string, KernelHandle> kernels_;
    std::string nvcc_version_, headers_digest_;
};

}  // namespace deep_jit
