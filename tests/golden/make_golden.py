"""Generate the golden fixtures in this folder from the reference's own Python.

Run where the reference checkout is available:

    python tests/golden/make_golden.py /path/to/reference

It loads ``deep_gemm/utils/math.py`` and ``deep_gemm/testing/numeric.py`` by file path
(the package ``__init__`` needs the compiled extension, these two files do not), pulls
the pure-torch layout model out of ``tests/test_layout.py`` and the E2M1->E4M3 re-encoder
out of ``tests/utils.py`` by function name, runs them on seeded CPU inputs and stores
inputs and outputs as ``.npz``.  The fixtures are what pins the numpy oracle; the GPU
box never needs the reference checkout.
"""
from __future__ import annotations

import ast
import importlib.util
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _load(path, name):
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def _extract_function(path, func_name, namespace):
    tree = ast.parse(open(path).read())
    for node in tree.body:
        if isinstance(node, ast.FunctionDef) and node.name == func_name:
            code = compile(ast.Module(body=[node], type_ignores=[]), path, "exec")
            exec(code, namespace)
            return namespace[func_name]
    raise KeyError(func_name)


def bf16_bits(t: torch.Tensor) -> np.ndarray:
    return t.contiguous().view(torch.int16).numpy().view(np.uint16).copy()


def main(ref_root: str):
    math = _load(os.path.join(ref_root, "deep_gemm/utils/math.py"), "ref_math")
    numeric = _load(os.path.join(ref_root, "deep_gemm/testing/numeric.py"), "ref_numeric")

    def get_tma_aligned_size(x, element_size):  # csrc/utils/math.hpp:23-27 (the compiled helper)
        return math.align(x, 16 // element_size)

    ns = {"torch": torch, "align": math.align, "get_tma_aligned_size": get_tma_aligned_size}
    layout_model = _extract_function(os.path.join(ref_root, "tests/test_layout.py"),
                                     "get_mn_major_tma_aligned_packed_ue8m0_tensor_torch_impl", ns)
    ns2 = {"torch": torch, "Tuple": tuple}
    convert_to_fp8 = _extract_function(os.path.join(ref_root, "tests/utils.py"), "convert_to_fp8", ns2)

    out = {}
    torch.manual_seed(0)

    # ---- quantisers ------------------------------------------------------------------------
    x = torch.randn(37, 300, dtype=torch.bfloat16)
    x[0, :] = 0                      # all-zero row -> clamp(1e-4) path
    x[1, :5] = torch.tensor([1e-6, -1e-6, 3e-5, 448.0, -448.0], dtype=torch.bfloat16)
    x[2, 128:256] *= 1000.0          # large block
    x[3, :] *= 1e-3                  # small block
    out["quant_x_bits"] = bf16_bits(x)
    for gran_k in (32, 128):
        for ue in (False, True):
            q, sf = math.per_token_cast_to_fp8(x, use_ue8m0=ue, gran_k=gran_k)
            out[f"tok_fp8_g{gran_k}_ue{int(ue)}_q"] = q.view(torch.uint8).numpy()
            out[f"tok_fp8_g{gran_k}_ue{int(ue)}_sf"] = sf.numpy()
            out[f"tok_fp8_g{gran_k}_ue{int(ue)}_back"] = math.cast_back_from_fp8(q, sf, gran_k).numpy()
        q, psf = math.per_token_cast_to_fp8(x, use_ue8m0=True, gran_k=gran_k, use_packed_ue8m0=True)
        out[f"tok_fp8_g{gran_k}_packed_sf"] = psf.numpy()
        q4, sf4 = math.per_token_cast_to_fp4(x, use_ue8m0=True, gran_k=gran_k)
        out[f"tok_fp4_g{gran_k}_q"] = q4.numpy()
        out[f"tok_fp4_g{gran_k}_sf"] = sf4.numpy()
        out[f"tok_fp4_g{gran_k}_back"] = math.cast_back_from_fp4(q4, sf4, gran_k).numpy()
        q4n, sf4n = math.per_token_cast_to_fp4(x, use_ue8m0=False, gran_k=gran_k)
        out[f"tok_fp4_g{gran_k}_ue0_q"] = q4n.numpy()
        out[f"tok_fp4_g{gran_k}_ue0_sf"] = sf4n.numpy()
        _, psf4 = math.per_token_cast_to_fp4(x, use_ue8m0=True, gran_k=gran_k, use_packed_ue8m0=True)
        out[f"tok_fp4_g{gran_k}_packed_sf"] = psf4.numpy()
    xb = torch.randn(200, 300, dtype=torch.bfloat16)
    out["block_x_bits"] = bf16_bits(xb)
    for ue in (False, True):
        q, sf = math.per_block_cast_to_fp8(xb, use_ue8m0=ue)
        out[f"blk_fp8_ue{int(ue)}_q"] = q.view(torch.uint8).numpy()
        out[f"blk_fp8_ue{int(ue)}_sf"] = sf.numpy()

    # ceil_to_ue8m0 on edge values
    edge = torch.tensor([1e-4 / 448, 2.0 ** -20, 1.0, 1.0000001, 0.75, 3.0, 1e-38, 1e38, 6.0 / 448], dtype=torch.float)
    out["ceil_in"] = edge.numpy()
    out["ceil_out"] = math.ceil_to_ue8m0(edge).numpy()

    # every e4m3 code round trip + a dense sweep of the rounding grid
    sweep = torch.cat([torch.linspace(-500, 500, 20001), torch.logspace(-12, 3, 4001)]).float()
    out["e4m3_sweep_in"] = sweep.numpy()
    out["e4m3_sweep_out"] = sweep.to(torch.float8_e4m3fn).view(torch.uint8).numpy()
    codes = torch.arange(256, dtype=torch.int32).to(torch.uint8)
    out["e4m3_all_codes_value"] = codes.view(torch.float8_e4m3fn).float().numpy()

    # FP4 helpers
    q4, sf4 = math.per_token_cast_to_fp4(x[:36], use_ue8m0=True, gran_k=32)
    out["fp4_transposed"] = math.transpose_packed_fp4(q4).numpy()
    out["fp4_as_e4m3"] = convert_to_fp8((q4, sf4))[0].view(torch.uint8).numpy()

    # ---- packed SF layout model (values, shape and strides) --------------------------------
    cases = []
    for mn, k, groups, gran_k in ((40, 128, 1, 128), (41, 640, 1, 128), (41, 640, 2, 32), (129, 7296, 4, 128),
                                  (64, 1184, 1, 32), (130, 96, 3, 32)):
        xs = torch.randn(groups * mn, k, dtype=torch.bfloat16) * torch.logspace(-3, 3, groups * mn).unsqueeze(1).bfloat16()
        _, sf = math.per_token_cast_to_fp8(xs, use_ue8m0=True, gran_k=gran_k)
        sf = sf if groups == 1 else sf.view(groups, mn, -1)
        packed = layout_model(sf)
        tag = f"layout_mn{mn}_k{k}_g{groups}_gk{gran_k}"
        out[tag + "_sf"] = sf.numpy()
        out[tag + "_packed"] = packed.contiguous().numpy()
        out[tag + "_strides"] = np.array(packed.stride(), dtype=np.int64)
        # raw storage in memory order so the padding content is pinned too
        span = 1 + sum((s - 1) * st for s, st in zip(packed.shape, packed.stride()))
        out[tag + "_storage"] = torch.as_strided(packed, (span,), (1,)).numpy().copy()
        cases.append(tag)
    out["layout_cases"] = np.array(cases)

    # ---- dequantise-then-matmul and calc_diff ---------------------------------------------
    a = torch.randn(48, 384, dtype=torch.bfloat16)
    b = torch.randn(80, 384, dtype=torch.bfloat16)
    out["gemm_a_bits"], out["gemm_b_bits"] = bf16_bits(a), bf16_bits(b)
    qa, sfa = math.per_token_cast_to_fp8(a, use_ue8m0=True, gran_k=128)
    qb, sfb = math.per_block_cast_to_fp8(b, use_ue8m0=True)
    ref_unq = a.float() @ b.float().T
    da = math.cast_back_from_fp8(qa, sfa, 128)
    sfb_rows = sfb.index_select(0, torch.arange(80) // 128)
    db = math.cast_back_from_fp8(qb, sfb_rows, 128)
    ref_deq = da @ db.T
    out["gemm_fp8_ref_dequant"] = ref_deq.numpy()
    out["gemm_fp8_diff_unq_vs_deq"] = np.float64(numeric.calc_diff(ref_unq, ref_deq))
    qb4, sfb4 = math.per_token_cast_to_fp4(b, use_ue8m0=True, gran_k=32)
    db4 = math.cast_back_from_fp4(qb4, sfb4, 32)
    ref_deq4 = da @ db4.T
    out["gemm_fp4_ref_dequant"] = ref_deq4.numpy()
    out["gemm_fp4_diff_unq_vs_deq"] = np.float64(numeric.calc_diff(ref_unq, ref_deq4))
    out["calc_diff_zero"] = np.float64(numeric.calc_diff(torch.zeros(4), torch.zeros(4)))
    out["calc_diff_bf16"] = np.float64(numeric.calc_diff(ref_deq.bfloat16(), ref_deq))

    np.savez_compressed(os.path.join(HERE, "reference_python.npz"), **out)
    print(f"wrote {len(out)} arrays")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path of the reference's source tree>")
    main(sys.argv[1])
