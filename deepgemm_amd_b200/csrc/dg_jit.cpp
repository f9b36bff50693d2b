// Thin JIT runtime: source string -> sm_100a cubin through nvcc, content-addressed disk cache with
// atomic publication, lazy module load per CUDA context, launch through cuLaunchKernelEx.
// Stands in for the reference's csrc/runtime/jit.hpp + third-party/deep_jit (behaviour described in
// README.md:164-191; call sites csrc/jit_kernels/impls/sm100_fp8_fp4_gemm_1d1d.hpp:40,82-89).
#include "dg_common.hpp"

#include <fcntl.h>
#include <sys/stat.h>
#include <sys/wait.h>
#include <unistd.h>

#include <cerrno>
#include <cstring>
#include <fstream>
#include <map>
#include <memory>
#include <sstream>
#include <vector>

struct dg_kernel {
    std::string name, entry, dir, cubin_path;
    std::mutex mu;
    std::map<CUcontext, CUfunction> loaded;     // one module per context
    std::map<CUcontext, uint32_t> smem_set;     // largest dynamic shared memory size configured so far
};

namespace dg {
namespace {

uint64_t fnv1a(const std::string& s, uint64_t h) {
    for (unsigned char c : s) { h ^= c; h *= 0x100000001b3ull; }
    return h;
}

std::string hex_key(const std::string& s) {
    char buf[40];
    snprintf(buf, sizeof(buf), "%016llx%016llx",
             static_cast<unsigned long long>(fnv1a(s, 0xcbf29ce484222325ull)),
             static_cast<unsigned long long>(fnv1a(s, 0x9ae16a3b2f90404full)));
    return buf;
}

bool is_dir(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0 && S_ISDIR(st.st_mode);
}
bool is_file(const std::string& p) {
    struct stat st;
    return stat(p.c_str(), &st) == 0 && S_ISREG(st.st_mode) && st.st_size > 0;
}
bool make_dirs(const std::string& p) {
    if (p.empty()) return false;
    if (is_dir(p)) return true;
    const auto slash = p.find_last_of('/');
    if (slash != std::string::npos && slash > 0 && !make_dirs(p.substr(0, slash))) return false;
    return mkdir(p.c_str(), 0755) == 0 || errno == EEXIST;
}

std::string read_file(const std::string& p) {
    std::ifstream f(p, std::ios::binary);
    std::stringstream ss;
    ss << f.rdbuf();
    return ss.str();
}

// Run a shell command, capturing stdout+stderr.
int run(const std::string& cmd, std::string* output) {
    FILE* pipe = popen((cmd + " 2>&1").c_str(), "r");
    if (pipe == nullptr) return -1;
    char buf[4096];
    size_t n;
    while ((n = fread(buf, 1, sizeof(buf), pipe)) > 0) output->append(buf, n);
    const int status = pclose(pipe);
    return WIFEXITED(status) ? WEXITSTATUS(status) : -1;
}

std::string nvcc_path() {
    std::string p = env_str("JIT_NVCC_COMPILER");
    if (!p.empty()) return p;
    if (const char* home = std::getenv("CUDA_HOME")) {
        p = std::string(home) + "/bin/nvcc";
        if (is_file(p)) return p;
    }
    if (is_file("/usr/local/cuda/bin/nvcc")) return "/usr/local/cuda/bin/nvcc";
    return "nvcc";
}

const std::string& nvcc_version() {
    static std::string v;
    static std::once_flag once;
    std::call_once(once, []() {
        std::string out;
        run(nvcc_path() + " --version", &out);
        const auto pos = out.find("release");
        v = pos == std::string::npos ? out : out.substr(pos);
    });
    return v;
}

// Directories searched for a cached kernel, in order; new kernels go to the first writable one.
std::vector<std::string> cache_dirs() {
    std::vector<std::string> dirs;
    const std::string env = env_str("JIT_CACHE_DIR");
    if (!env.empty()) dirs.push_back(env);
    if (!state().library_root.empty()) dirs.push_back(state().library_root + "/_jit_cache");
    if (const char* home = std::getenv("HOME")) dirs.push_back(std::string(home) + "/.deepgemm_b200");
    dirs.push_back("/tmp/.deepgemm_b200");
    return dirs;
}

// Digest of every device header a generated kernel can include: editing one invalidates the cache.
const std::string& device_headers_digest() {
    static std::string digest;
    static std::once_flag once;
    std::call_once(once, []() {
        std::string all;
        for (const char* f : {"gemm_fp8_fp4.cuh", "gemm_config.hpp", "ptx.cuh", "tile_scheduler.cuh", "quant_math.cuh"})
            all += read_file(state().library_root + "/csrc/device/dg/" + f) + "\n//--\n";
        digest = hex_key(all);
    });
    return digest;
}

std::mutex& registry_mu() { static std::mutex m; return m; }
std::map<std::string, std::unique_ptr<dg_kernel>>& registry() {
    static std::map<std::string, std::unique_ptr<dg_kernel>> r;
    return r;
}

}  // namespace
}  // namespace dg

using namespace dg;

extern "C" {

int dg_jit_compile(const char* name, const char* entry, const char* source, const char* extra_flags, dg_kernel_t* kernel) {
    env_refresh();
    DG_REQUIRE(name != nullptr && entry != nullptr && source != nullptr && kernel != nullptr);
    const std::string include_dir = state().library_root + "/csrc/device";
    std::string flags = "-std=c++17 -gencode arch=compute_100a,code=sm_100a -O3 --expt-relaxed-constexpr -cubin";
    if (env_int("JIT_WITH_LINEINFO", 1)) flags += " -lineinfo";
    if (env_int("JIT_PTXAS_VERBOSE")) flags += " -Xptxas -v";
    if (extra_flags != nullptr && extra_flags[0] != 0) flags += std::string(" ") + extra_flags;

    const std::string key = hex_key(std::string(source) + "\n//" + flags + "\n//" + nvcc_version() + "\n//" + entry +
                                    "\n//" + device_headers_digest());
    const std::string leaf = std::string("kernel.") + name + "." + key;

    {
        std::lock_guard<std::mutex> lock(registry_mu());
        auto it = registry().find(leaf);
        if (it != registry().end()) { *kernel = it->second.get(); return DG_OK; }
    }

    // Cache lookup
    std::string found_dir;
    for (const auto& d : cache_dirs())
        if (is_file(d + "/" + leaf + "/kernel.cubin")) { found_dir = d + "/" + leaf; break; }

    if (found_dir.empty()) {
        std::string root;
        for (const auto& d : cache_dirs())
            if (make_dirs(d) && access(d.c_str(), W_OK) == 0) { root = d; break; }
        if (root.empty()) return fail(DG_ERR_JIT, "no writable kernel cache directory");
        char tmpl[64];
        snprintf(tmpl, sizeof(tmpl), "/tmp.%d.XXXXXX", static_cast<int>(getpid()));
        std::string tmp = root + tmpl;
        if (mkdtemp(tmp.data()) == nullptr) return fail(DG_ERR_JIT, "mkdtemp failed in %s: %s", root.c_str(), strerror(errno));
        {
            std::ofstream f(tmp + "/kernel.cu");
            f << source;
        }
        const std::string cmd = nvcc_path() + " " + flags + " -I" + include_dir + " -o " + tmp + "/kernel.cubin " + tmp + "/kernel.cu";
        if (env_int("JIT_DEBUG") || env_int("JIT_PRINT_COMPILER_COMMAND")) fprintf(stderr, "[dg jit] %s\n", cmd.c_str());
        std::string log;
        const int rc = run(cmd, &log);
        if (env_int("JIT_PTXAS_VERBOSE") && !log.empty()) fprintf(stderr, "%s\n", log.c_str());
        if (rc != 0 || !is_file(tmp + "/kernel.cubin")) {
            const int keep = env_int("JIT_DEBUG");
            if (!keep) { unlink((tmp + "/kernel.cu").c_str()); unlink((tmp + "/kernel.cubin").c_str()); rmdir(tmp.c_str()); }
            return fail(DG_ERR_JIT, "nvcc failed (exit %d) for kernel %s:\n%s", rc, name, log.c_str());
        }
        { std::ofstream f(tmp + "/command.txt"); f << cmd << "\n" << log; }
        // Publish atomically; if another process won the race its directory is equivalent
        const std::string final_dir = root + "/" + leaf;
        if (rename(tmp.c_str(), final_dir.c_str()) != 0) {
            unlink((tmp + "/kernel.cu").c_str()); unlink((tmp + "/kernel.cubin").c_str());
            unlink((tmp + "/command.txt").c_str()); rmdir(tmp.c_str());
            if (!is_file(final_dir + "/kernel.cubin"))
                return fail(DG_ERR_JIT, "cannot publish kernel into %s: %s", final_dir.c_str(), strerror(errno));
        }
        found_dir = final_dir;
    }

    auto k = std::make_unique<dg_kernel>();
    k->name = name;
    k->entry = entry;
    k->dir = found_dir;
    k->cubin_path = found_dir + "/kernel.cubin";
    std::lock_guard<std::mutex> lock(registry_mu());
    auto& slot = registry()[leaf];
    if (!slot) slot = std::move(k);
    *kernel = slot.get();
    return DG_OK;
}

const char* dg_jit_kernel_path(dg_kernel_t kernel) { return kernel ? kernel->cubin_path.c_str() : ""; }

}  // extern "C"

namespace {

// The kernel's function in the current context, loaded on first use, with enough dynamic shared memory allowed
int loaded_function(dg_kernel_t kernel, uint32_t smem_bytes, CUfunction* out) {
    const dg::Driver& drv = dg::driver();
    if (!drv.ok) return dg::fail(DG_ERR_CUDA, "CUDA driver unavailable: %s", drv.why.c_str());

    // Make sure the primary context exists and is current on this thread
    CUcontext ctx = nullptr;
    DG_CUDA_DRV(drv.cuCtxGetCurrent(&ctx));
    if (ctx == nullptr) {
        DG_CUDA_RT(cudaFree(nullptr));
        DG_CUDA_DRV(drv.cuCtxGetCurrent(&ctx));
        if (ctx == nullptr) return dg::fail(DG_ERR_CUDA, "no current CUDA context");
    }

    CUfunction fn = nullptr;
    std::lock_guard<std::mutex> lock(kernel->mu);
    auto it = kernel->loaded.find(ctx);
    if (it == kernel->loaded.end()) {
        const std::string image = read_file(kernel->cubin_path);
        if (image.empty()) return dg::fail(DG_ERR_JIT, "cached kernel %s is empty or unreadable", kernel->cubin_path.c_str());
        CUmodule mod = nullptr;
        CUresult r = drv.cuModuleLoadData(&mod, image.data());
        if (r != CUDA_SUCCESS)
            return dg::fail(DG_ERR_JIT, "cuModuleLoadData failed for %s: %s", kernel->cubin_path.c_str(), dg::cu_error(r).c_str());
        r = drv.cuModuleGetFunction(&fn, mod, kernel->entry.c_str());
        if (r != CUDA_SUCCESS)
            return dg::fail(DG_ERR_JIT, "entry %s not found in %s: %s", kernel->entry.c_str(), kernel->cubin_path.c_str(), dg::cu_error(r).c_str());
        kernel->loaded[ctx] = fn;
    } else {
        fn = it->second;
    }
    uint32_t& configured = kernel->smem_set[ctx];
    if (smem_bytes > configured) {
        DG_CUDA_DRV(drv.cuFuncSetAttribute(fn, CU_FUNC_ATTRIBUTE_MAX_DYNAMIC_SHARED_SIZE_BYTES, static_cast<int>(smem_bytes)));
        configured = smem_bytes;
    }
    *out = fn;
    return DG_OK;
}

}  // namespace

extern "C" {

int dg_jit_max_active_clusters(dg_kernel_t kernel, uint32_t block_x, uint32_t cluster_x, uint32_t smem_bytes, int* num_clusters) {
    DG_REQUIRE(kernel != nullptr && block_x > 0 && cluster_x > 0 && num_clusters != nullptr);
    CUfunction fn = nullptr;
    const int rc = loaded_function(kernel, smem_bytes, &fn);
    if (rc != DG_OK) return rc;
    const dg::Driver& drv = dg::driver();
    CUlaunchConfig cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDimX = cluster_x; cfg.gridDimY = 1; cfg.gridDimZ = 1;
    cfg.blockDimX = block_x; cfg.blockDimY = 1; cfg.blockDimZ = 1;
    cfg.sharedMemBytes = smem_bytes;
    CUlaunchAttribute attr;
    attr.id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
    attr.value.clusterDim.x = cluster_x;
    attr.value.clusterDim.y = 1;
    attr.value.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    DG_CUDA_DRV(drv.cuOccupancyMaxActiveClusters(num_clusters, fn, &cfg));
    return DG_OK;
}

int dg_jit_launch(dg_kernel_t kernel, uint32_t grid_x, uint32_t block_x, uint32_t cluster_x,
                  uint32_t smem_bytes, int enable_pdl, void* stream, void** kernel_args) {
    DG_REQUIRE(kernel != nullptr && grid_x > 0 && block_x > 0 && cluster_x > 0 && grid_x % cluster_x == 0);
    CUfunction fn = nullptr;
    {
        const int rc = loaded_function(kernel, smem_bytes, &fn);
        if (rc != DG_OK) return rc;
    }
    const dg::Driver& drv = dg::driver();

    CUlaunchConfig cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDimX = grid_x; cfg.gridDimY = 1; cfg.gridDimZ = 1;
    cfg.blockDimX = block_x; cfg.blockDimY = 1; cfg.blockDimZ = 1;
    cfg.sharedMemBytes = smem_bytes;
    cfg.hStream = static_cast<CUstream>(stream);
    CUlaunchAttribute attrs[2];
    unsigned num_attrs = 0;
    if (cluster_x > 1) {
        attrs[num_attrs].id = CU_LAUNCH_ATTRIBUTE_CLUSTER_DIMENSION;
        attrs[num_attrs].value.clusterDim.x = cluster_x;
        attrs[num_attrs].value.clusterDim.y = 1;
        attrs[num_attrs].value.clusterDim.z = 1;
        ++num_attrs;
    }
    if (enable_pdl) {
        attrs[num_attrs].id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
        attrs[num_attrs].value.programmaticStreamSerializationAllowed = 1;
        ++num_attrs;
    }
    cfg.attrs = attrs;
    cfg.numAttrs = num_attrs;
    DG_CUDA_DRV(drv.cuLaunchKernelEx(&cfg, fn, kernel_args, nullptr));
    return DG_OK;
}

}  // extern "C"
