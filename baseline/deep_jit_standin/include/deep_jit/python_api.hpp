// Stand-in for third-party/deep_jit of the reference: what the JIT runtime registers on the extension module
// (csrc/python_api.cpp:28).  The reference's Python package imports nothing of it (deep_gemm/__init__.py:16-108), so
// the stand-in registers only two read-only helpers used by this repository's timing harness.
#pragma once

#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "backend/cuda/backend.hpp"

namespace deep_jit {

inline void register_python_api(pybind11::module_& m, LazyInit<Runtime<CUDA>>& jit) {
    m.def("_jit_standin", []() { return true; }, "True: the JIT runtime of this build is the stand-in, not DeepJIT");
    m.def("_jit_include_dirs", [&jit]() {
        std::vector<std::string> dirs;
        for (const auto& d : jit->config().include_dirs) dirs.push_back(d.string());
        return dirs;
    });
}

}  // namespace deep_jit
