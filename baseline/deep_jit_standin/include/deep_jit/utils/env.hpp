// Stand-in for the un-vendored DeepJIT submodule of the reference (third-party/deep_jit): environment lookups.
// Written from the call sites in the reference tree only (e.g. csrc/jit_kernels/heuristics/common.hpp:44,
// csrc/runtime/runtime.hpp:47-51); it exists so that the UNMODIFIED reference can be built and timed beside this
// repository's kernels.  Not part of the product library.
#pragma once

#include <cstdlib>
#include <sstream>
#include <string>

namespace deep_jit {

// Value of an environment variable parsed as T, `default_value` when unset.  A name with the runtime's prefix
// ("DG_JIT_...") falls back to the global "DJ_JIT_..." spelling (README.md:166 of the reference).
template <typename T>
T get_env(const std::string& name, const T& default_value = T()) {
    const char* raw = std::getenv(name.c_str());
    if (raw == nullptr) {
        const auto pos = name.find("_JIT_");
        if (pos != std::string::npos) raw = std::getenv(("DJ" + name.substr(pos)).c_str());
    }
    if (raw == nullptr) return default_value;
    if constexpr (std::is_same_v<T, std::string>) {
        return std::string(raw);
    } else {
        std::istringstream in(raw);
        T value = default_value;
        in >> value;
        return value;
    }
}

}  // namespace deep_jit
