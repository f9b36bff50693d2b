// Compiled host binding for the hot GEMM entry points: the argument checks of the reference's API layer
// (csrc/apis/gemm.hpp:78-133,181-250,269-318, csrc/utils/layout.hpp:19-140) and the filling of dg_gemm_args_t done in
// C++ on torch tensors, so that a call costs the host a few microseconds instead of an interpreter's worth of attribute
// lookups.  It is the counterpart of the reference's pybind11 module (csrc/python_api.cpp:24-47) for the calls a serving
// loop makes: dense, m-grouped contiguous and m-grouped masked GEMMs whose scales arrive already packed (int32 UE8M0,
// MN-major), without an epilogue object.  Each function takes the Python call's arguments as they are and returns
// false, untouched, when the call is not of that kind; deepgemm_amd_b200/api.py then runs it through its own path, as it
// does everything else (FP32 scales that need their transform kernel, epilogue objects, the einsum / k-grouped / BF16
// families, settings).  The checks and their messages are the ones api.py applies to the same call.
#include <torch/extension.h>

#include <c10/cuda/CUDAStream.h>

#include <optional>
#include <sstream>
#include <utility>
#include <vector>
#include <stdexcept>
#include <string>

#include "../../include/deepgemm_b200.h"

namespace py = pybind11;

namespace {

[[noreturn]] void fail(const char* cond, int line) {
    std::ostringstream s;
    s << "Assertion error (deepgemm_amd_b200/csrc/python_binding.cpp:" << line << "): " << cond;
    throw std::runtime_error(s.str());
}
#define DG_BIND_REQUIRE(cond, text) do { if (!(cond)) fail(text, __LINE__); } while (0)

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
inline int64_t align_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

constexpr auto kPackedFP4 = torch::kInt8;        // csrc/utils/math.hpp:11

struct Operand {
    int dtype;       // dg_dtype_t
    int major;       // dg_major_t
    int64_t mn, k;   // logical extents (a packed FP4 tensor holds two elements per byte along its contiguous dimension)
    int64_t ld;      // pitch of the non-contiguous dimension in storage elements
};

// csrc/utils/layout.hpp:19-33,66-83
Operand describe(const torch::Tensor& t, int expected_dim) {
    DG_BIND_REQUIRE(t.is_cuda(), "t.is_cuda()");
    DG_BIND_REQUIRE(t.dim() == expected_dim, "t.dim() == N");
    if (t.dim() == 3) DG_BIND_REQUIRE(t.stride(0) == t.size(-2) * t.size(-1), "t.stride(0) == t.size(-2) * t.size(-1)");
    DG_BIND_REQUIRE(t.stride(-2) == 1 || t.stride(-1) == 1, "t.stride(-2) == 1 or t.stride(-1) == 1");
    Operand o;
    o.major = t.stride(-1) == 1 ? DG_MAJOR_K : DG_MAJOR_MN;
    if (t.scalar_type() == torch::kFloat8_e4m3fn) {
        o.dtype = DG_FP8_E4M3;
    } else {
        DG_BIND_REQUIRE(t.scalar_type() == kPackedFP4, "ab.scalar_type() == kPackedFP4 and arch_major == 10");
        o.dtype = DG_FP4_E2M1_X2;
    }
    o.mn = t.size(-2);
    o.k = t.size(-1);
    if (o.dtype == DG_FP4_E2M1_X2) (o.major == DG_MAJOR_K ? o.k : o.mn) *= 2;
    o.ld = o.major == DG_MAJOR_K ? t.stride(-2) : t.stride(-1);
    return o;
}

// csrc/utils/layout.hpp:101-140 for a packed (int32) scale tensor, with the stride checks of the TMA path
void check_packed_sf(const torch::Tensor& sf, int64_t mn, int64_t k, int gran_k, std::optional<int64_t> num_groups) {
    DG_BIND_REQUIRE(sf.is_cuda(), "t.is_cuda()");
    DG_BIND_REQUIRE(sf.scalar_type() == torch::kInt, "sf.scalar_type() == type_check.value()");
    DG_BIND_REQUIRE(gran_k == 32 || gran_k == 128, "gran_k == 32 or gran_k == 128");
    DG_BIND_REQUIRE(sf.dim() == (num_groups.has_value() ? 3 : 2), "sf.dim() == static_cast<int>(num_groups.has_value()) + 2");
    if (num_groups.has_value()) DG_BIND_REQUIRE(sf.size(-3) == *num_groups, "sf.size(-3) == num_groups.value()");
    DG_BIND_REQUIRE(sf.size(-2) == mn, "sf.size(-2) == ceil_div(mn, gran_mn)");
    DG_BIND_REQUIRE(sf.size(-1) == ceil_div(k, static_cast<int64_t>(gran_k) * 4),
                    "sf.size(-1) == ceil_div(k, gran_k * (sf_dtype == torch::kFloat ? 1 : 4))");
    if (num_groups.has_value())
        DG_BIND_REQUIRE(sf.stride(-3) == sf.stride(-1) * sf.size(-1), "sf.stride(-3) == sf.stride(-1) * sf.size(-1)");
    DG_BIND_REQUIRE(sf.stride(-2) == 1 || mn == 1, "sf.stride(-2) == 1 or mn == 1");
    DG_BIND_REQUIRE(sf.stride(-1) >= align_up(mn, 4), "sf.stride(-1) >= compact_stride");
    DG_BIND_REQUIRE(sf.stride(-1) % 4 == 0, "sf.stride(-1) % 4 == 0");
}

void check_cd(const torch::Tensor& t) {
    DG_BIND_REQUIRE(t.is_cuda(), "t.is_cuda()");
    DG_BIND_REQUIRE(t.stride(-2) == 1 || t.stride(-1) == 1, "t.stride(-2) == 1 or t.stride(-1) == 1");
    DG_BIND_REQUIRE(t.stride(-1) == 1, "t.stride(-1) == 1");
}

void fill_common(dg_gemm_args_t& g, const torch::Tensor& a, const torch::Tensor& sfa, const torch::Tensor& b, const torch::Tensor& sfb,
                 const torch::Tensor& d, const Operand& oa, const Operand& ob, int gran_k_a, int gran_k_b) {
    g.a = a.data_ptr(); g.sfa = sfa.data_ptr(); g.b = b.data_ptr(); g.sfb = sfb.data_ptr(); g.d = d.data_ptr();
    g.a_dtype = oa.dtype; g.b_dtype = ob.dtype;
    g.major_a = oa.major; g.major_b = ob.major;
    g.lda = oa.ld; g.ldb = ob.ld; g.ldd = d.stride(-2);
    g.sfa_pitch = sfa.stride(-1); g.sfb_pitch = sfb.stride(-1);
    g.gran_k_a = gran_k_a; g.gran_k_b = gran_k_b;
    g.stream = c10::cuda::getCurrentCUDAStream().stream();
}

// The granularities along K when both scale tensors arrive packed (int32, one scale per row of MN) and the recipe is
// one this module serves; csrc/apis/layout.hpp:11-87 reduce to layout checks then.  false sends the call back to the
// interpreter path, which also words every recipe error.
bool packed_grans(const torch::Tensor& sfa, const torch::Tensor& sfb, const py::object& recipe, const py::object& recipe_a,
                  const py::object& recipe_b, bool disable_ue8m0_cast, int* gran_k_a, int* gran_k_b) {
    if (disable_ue8m0_cast || sfa.scalar_type() != torch::kInt || sfb.scalar_type() != torch::kInt) return false;
    const auto ints = [](const py::object& o, std::vector<int>* out) {
        try {
            for (const auto& item : py::reinterpret_borrow<py::sequence>(o)) out->push_back(py::cast<int>(item));
            return true;
        } catch (const std::exception&) {
            return false;
        }
    };
    const auto fine = [](int g) { return g == 32 || g == 128; };
    if (recipe_a.is_none() && recipe_b.is_none()) {
        if (recipe.is_none()) {
            *gran_k_a = *gran_k_b = 128;              // default recipe for packed scales: (1, 1, 128)
            return true;
        }
        std::vector<int> r;
        if (!ints(recipe, &r) || r.size() != 3 || r[0] != 1 || r[1] != 1 || !fine(r[2])) return false;
        *gran_k_a = *gran_k_b = r[2];
        return true;
    }
    if (!recipe.is_none() || recipe_a.is_none() || recipe_b.is_none()) return false;
    std::vector<int> ra, rb;
    if (!ints(recipe_a, &ra) || !ints(recipe_b, &rb) || ra.size() != 2 || rb.size() != 2 || ra[0] != 1 || rb[0] != 1 ||
        !fine(ra[1]) || !fine(rb[1]))
        return false;
    *gran_k_a = ra[1];
    *gran_k_b = rb[1];
    return true;
}

using TensorPair = std::pair<torch::Tensor, torch::Tensor>;

void check_rc(int rc) {
    if (rc != DG_OK) {
        const char* msg = dg_last_error();
        throw std::runtime_error(msg != nullptr && msg[0] != 0 ? msg : "deepgemm_b200 error " + std::to_string(rc));
    }
}

// fp8_fp4_gemm_nt with packed scales: D = [D +] alpha A B^T  (csrc/apis/gemm.hpp:78-133).  Takes the arguments of the
// Python function as they come; returns false, having done nothing, when the call is not one this module serves.
bool dense_nt(const TensorPair& a_pair, const TensorPair& b_pair, const torch::Tensor& d, const std::optional<torch::Tensor>& c,
              const py::object& recipe, const py::object& recipe_a, const py::object& recipe_b, bool disable_ue8m0_cast,
              std::optional<double> alpha, const py::object& epilogue) {
    const torch::Tensor &a = a_pair.first, &sfa = a_pair.second, &b = b_pair.first, &sfb = b_pair.second;
    int gran_k_a = 0, gran_k_b = 0;
    if (!epilogue.is_none() || (c.has_value() && c->unsafeGetTensorImpl() != d.unsafeGetTensorImpl()) ||
        !packed_grans(sfa, sfb, recipe, recipe_a, recipe_b, disable_ue8m0_cast, &gran_k_a, &gran_k_b))
        return false;
    const bool accumulate = c.has_value();
    const Operand oa = describe(a, 2), ob = describe(b, 2);
    if (oa.dtype == DG_FP4_E2M1_X2 && ob.dtype == DG_FP4_E2M1_X2)
        DG_BIND_REQUIRE(oa.major == DG_MAJOR_K && ob.major == DG_MAJOR_K, "major == cute::UMMA::Major::K");
    DG_BIND_REQUIRE(d.dim() == 2, "t.dim() == N");
    check_cd(d);
    const int64_t m = oa.mn, n = ob.mn, k = oa.k;
    DG_BIND_REQUIRE(m == d.size(0) && n == d.size(1) && k == ob.k, "m == m_ and n == n_ and k == k_");
    DG_BIND_REQUIRE(d.scalar_type() == torch::kBFloat16 || d.scalar_type() == torch::kFloat,
                    "d.scalar_type() == torch::kBFloat16 or d.scalar_type() == torch::kFloat");
    if (m == 0 || n == 0) return true;               // early_return, gemm.hpp:17-53
    if (k == 0) {
        if (!accumulate) d.zero_();
        return true;
    }
    check_packed_sf(sfa, m, k, gran_k_a, std::nullopt);
    check_packed_sf(sfb, n, k, gran_k_b, std::nullopt);
    dg_gemm_args_t g{};
    fill_common(g, a, sfa, b, sfb, d, oa, ob, gran_k_a, gran_k_b);
    g.m = static_cast<int32_t>(m); g.n = static_cast<int32_t>(n); g.k = static_cast<int32_t>(k); g.num_groups = 1;
    g.d_dtype = d.scalar_type() == torch::kBFloat16 ? DG_BF16 : DG_FP32;
    g.accumulate = accumulate ? 1 : 0;
    g.has_alpha = alpha.has_value() ? 1 : 0;
    g.alpha = alpha.has_value() ? static_cast<float>(*alpha) : 1.0f;
    check_rc(dg_fp8_fp4_gemm(&g));
    return true;
}

// m_grouped_fp8_fp4_gemm_nt_contiguous with packed scales (csrc/apis/gemm.hpp:181-250)
bool m_grouped_contiguous(const TensorPair& a_pair, const TensorPair& b_pair, const torch::Tensor& d, const torch::Tensor& grouped_layout,
                          const py::object& recipe, const py::object& recipe_a, const py::object& recipe_b, bool disable_ue8m0_cast,
                          bool use_psum_layout, bool ensure_zero_padding, std::optional<int64_t> expected_m_for_psum_layout,
                          const py::object& epilogue) {
    const torch::Tensor &a = a_pair.first, &sfa = a_pair.second, &b = b_pair.first, &sfb = b_pair.second;
    int gran_k_a = 0, gran_k_b = 0;
    if (!epilogue.is_none() || !packed_grans(sfa, sfb, recipe, recipe_a, recipe_b, disable_ue8m0_cast, &gran_k_a, &gran_k_b)) return false;
    const Operand oa = describe(a, 2);
    DG_BIND_REQUIRE(oa.major == DG_MAJOR_K, "major_a == cute::UMMA::Major::K");
    DG_BIND_REQUIRE(grouped_layout.is_contiguous(), "grouped_layout.is_contiguous()");
    DG_BIND_REQUIRE(b.dim() == 3, "t.dim() == N");
    const Operand ob = describe(b, 3);
    const int64_t m = oa.mn, n = ob.mn, k = oa.k, num_groups = b.size(0);
    DG_BIND_REQUIRE(d.dim() == 2, "t.dim() == N");
    DG_BIND_REQUIRE(m == d.size(0) && n == d.size(1) && k == ob.k, "m == m_ and n == n_ and k == k_");
    DG_BIND_REQUIRE(n > 0 && k > 0 && num_groups > 0, "n > 0 and k > 0 and num_groups > 0");
    DG_BIND_REQUIRE(d.scalar_type() == torch::kBFloat16, "d.scalar_type() == torch::kBFloat16");
    DG_BIND_REQUIRE(grouped_layout.is_cuda() && grouped_layout.scalar_type() == torch::kInt, "grouped_layout.scalar_type() == torch::kInt");
    if (use_psum_layout) {
        DG_BIND_REQUIRE(grouped_layout.dim() == 1 && grouped_layout.size(0) == num_groups, "num_groups == num_groups_");
    } else {
        DG_BIND_REQUIRE(grouped_layout.dim() == 1 && grouped_layout.size(0) == m, "m == m__");
        DG_BIND_REQUIRE(!expected_m_for_psum_layout.has_value(), "not expected_m_for_psum_layout.has_value()");
    }
    check_cd(d);
    if (m == 0) return true;
    check_packed_sf(sfa, m, k, gran_k_a, std::nullopt);
    check_packed_sf(sfb, n, k, gran_k_b, num_groups);
    dg_gemm_args_t g{};
    fill_common(g, a, sfa, b, sfb, d, oa, ob, gran_k_a, gran_k_b);
    g.m = static_cast<int32_t>(m); g.n = static_cast<int32_t>(n); g.k = static_cast<int32_t>(k); g.num_groups = static_cast<int32_t>(num_groups);
    g.d_dtype = DG_BF16;
    g.grouped_layout = grouped_layout.data_ptr<int32_t>();
    g.expected_m = static_cast<int32_t>(expected_m_for_psum_layout.value_or(0));
    g.use_psum_layout = use_psum_layout ? 1 : 0;
    g.ensure_zero_padding = use_psum_layout && ensure_zero_padding ? 1 : 0;
    check_rc(dg_m_grouped_fp8_fp4_gemm_contiguous(&g));
    return true;
}

// m_grouped_fp8_fp4_gemm_nt_masked with packed scales (csrc/apis/gemm.hpp:269-318)
bool m_grouped_masked(const TensorPair& a_pair, const TensorPair& b_pair, const torch::Tensor& d, const torch::Tensor& masked_m,
                      int64_t expected_m, const py::object& recipe, const py::object& recipe_a, const py::object& recipe_b,
                      bool disable_ue8m0_cast, const py::object& epilogue) {
    const torch::Tensor &a = a_pair.first, &sfa = a_pair.second, &b = b_pair.first, &sfb = b_pair.second;
    int gran_k_a = 0, gran_k_b = 0;
    if (!epilogue.is_none() || !packed_grans(sfa, sfb, recipe, recipe_a, recipe_b, disable_ue8m0_cast, &gran_k_a, &gran_k_b)) return false;
    DG_BIND_REQUIRE(a.dim() == 3 && b.dim() == 3 && d.dim() == 3, "t.dim() == N");
    const Operand oa = describe(a, 3), ob = describe(b, 3);
    DG_BIND_REQUIRE(oa.major == DG_MAJOR_K && ob.major == DG_MAJOR_K, "major_a == cute::UMMA::Major::K and major_b == cute::UMMA::Major::K");
    DG_BIND_REQUIRE(masked_m.is_contiguous(), "masked_m.is_contiguous()");
    const int64_t m = oa.mn, n = ob.mn, k = oa.k, groups = a.size(0);
    DG_BIND_REQUIRE(groups == b.size(0) && groups == d.size(0) && groups == masked_m.numel(),
                    "num_groups == num_groups_ and num_groups == num_groups__ and num_groups == num_groups___");
    DG_BIND_REQUIRE(m == d.size(1) && n == d.size(2) && k == ob.k, "m == m_ and n == n_ and k == k_");
    DG_BIND_REQUIRE(expected_m > 0 && m > 0 && n > 0 && k > 0 && groups > 0, "expected_m > 0 and m > 0 and n > 0 and k > 0 and num_groups > 0");
    DG_BIND_REQUIRE(d.scalar_type() == torch::kBFloat16, "d.scalar_type() == torch::kBFloat16");
    DG_BIND_REQUIRE(masked_m.is_cuda() && masked_m.scalar_type() == torch::kInt, "masked_m.scalar_type() == torch::kInt");
    DG_BIND_REQUIRE(d.stride(0) == d.size(-2) * d.size(-1), "t.stride(0) == t.size(-2) * t.size(-1)");
    check_cd(d);
    check_packed_sf(sfa, m, k, gran_k_a, groups);
    check_packed_sf(sfb, n, k, gran_k_b, groups);
    dg_gemm_args_t g{};
    fill_common(g, a, sfa, b, sfb, d, oa, ob, gran_k_a, gran_k_b);
    g.m = static_cast<int32_t>(m); g.n = static_cast<int32_t>(n); g.k = static_cast<int32_t>(k); g.num_groups = static_cast<int32_t>(groups);
    g.d_dtype = DG_BF16;
    g.grouped_layout = masked_m.data_ptr<int32_t>();
    g.expected_m = static_cast<int32_t>(expected_m);
    check_rc(dg_m_grouped_fp8_fp4_gemm_masked(&g));
    return true;
}

}  // namespace

PYBIND11_MODULE(_C, m) {
    m.doc() = "Compiled host binding of the block-scaled GEMM entry points (packed scales, no epilogue object)";
    m.def("dense_nt", &dense_nt);
    m.def("m_grouped_contiguous", &m_grouped_contiguous);
    m.def("m_grouped_masked", &m_grouped_masked);
}
