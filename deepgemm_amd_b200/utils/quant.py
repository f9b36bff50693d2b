"""Torch helpers that produce the quantised operands the GEMMs consume: float8_e4m3 with one scale per
1 x gran_k (activations) or gran_k x gran_k (weights) block, and packed float4_e2m1 with one scale per
1 x gran_k.  Same numerical recipe as the reference's deep_gemm/utils/math.py:13-176 (scale = amax / qmax,
rounded up to a power of two for UE8M0, clamped to 1e-4), written for whole-tensor vectorised execution on
the GPU.  They are input preparation for callers and tests, not part of the GEMM kernels."""
from __future__ import annotations

from typing import Tuple

import torch

_E2M1_GRID = (0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0)


def ceil_div(x: int, y: int) -> int:
    return -(-x // y)


def align(x: int, y: int) -> int:
    return ceil_div(x, y) * y


def ceil_to_ue8m0(x: torch.Tensor) -> torch.Tensor:
    """Smallest power of two >= |x| (exponent clamped to [1, 254])."""
    bits = x.abs().float().view(torch.int32)
    exponent = (bits >> 23) & 0xFF
    exponent = exponent + ((bits & 0x7FFFFF) != 0).to(torch.int32)
    return (exponent.clamp_(1, 254) << 23).view(torch.float32)


def _block_view(x: torch.Tensor, gran_k: int) -> Tuple[torch.Tensor, int]:
    rows, cols = x.shape
    padded = align(cols, gran_k)
    if padded != cols:
        x = torch.nn.functional.pad(x, (0, padded - cols))
    return x.reshape(rows, padded // gran_k, gran_k), padded


def _scales(amax: torch.Tensor, qmax: float, use_ue8m0: bool) -> torch.Tensor:
    sf = amax.float().clamp_min(1e-4) / qmax
    return ceil_to_ue8m0(sf) if use_ue8m0 else sf


def pack_ue8m0_to_int(sf: torch.Tensor) -> torch.Tensor:
    """Four power-of-two FP32 scales along the last axis -> one int32 (byte j = exponent of scale j)."""
    assert sf.dtype == torch.float32 and sf.size(-1) % 4 == 0
    bits = sf.contiguous().view(torch.int32)
    assert bool(((bits & 0x807FFFFF) == 0).all()), "scales must be positive powers of two"
    return (bits >> 23).to(torch.uint8).view(torch.int32)


def _maybe_pack(sf: torch.Tensor, packed: bool) -> torch.Tensor:
    if not packed:
        return sf
    tail = (-sf.size(-1)) % 4
    if tail:
        sf = torch.nn.functional.pad(sf, (0, tail), value=1.0)
    return pack_ue8m0_to_int(sf)


def per_token_cast_to_fp8(x: torch.Tensor, use_ue8m0: bool, gran_k: int = 128, use_packed_ue8m0: bool = False):
    assert x.dim() == 2 and (use_ue8m0 or not use_packed_ue8m0)
    cols = x.size(1)
    blocks, padded = _block_view(x, gran_k)
    sf = _scales(blocks.abs().amax(dim=2), 448.0, use_ue8m0)
    q = (blocks * (1.0 / sf).unsqueeze(2)).to(torch.float8_e4m3fn).reshape(x.size(0), padded)[:, :cols].contiguous()
    return q, _maybe_pack(sf, use_packed_ue8m0)


def per_block_cast_to_fp8(x: torch.Tensor, use_ue8m0: bool, gran_k: int = 128):
    assert x.dim() == 2
    rows, cols = x.shape
    pr, pc = align(rows, gran_k), align(cols, gran_k)
    xp = torch.nn.functional.pad(x, (0, pc - cols, 0, pr - rows)) if (pr, pc) != (rows, cols) else x
    tiles = xp.reshape(pr // gran_k, gran_k, pc // gran_k, gran_k)
    sf = _scales(tiles.abs().amax(dim=(1, 3), keepdim=True), 448.0, use_ue8m0)
    q = (tiles * (1.0 / sf)).to(torch.float8_e4m3fn).reshape(pr, pc)[:rows, :cols].contiguous()
    return q, sf.reshape(pr // gran_k, pc // gran_k)


def per_channel_cast_to_fp8(x: torch.Tensor, use_ue8m0: bool, gran_k: int = 128):
    """e4m3 with one scale per column and `gran_k` rows (deep_gemm/utils/math.py:52-59): the quantisation of the
    [sum_k, M] / [sum_k, N] operands of the k-grouped GEMM, whose K runs down the rows.  Returns (q, sf [rows / gran_k, cols])."""
    assert x.dim() == 2 and x.size(0) % gran_k == 0
    rows, cols = x.shape
    slabs = x.reshape(rows // gran_k, gran_k, cols)
    sf = _scales(slabs.abs().amax(dim=1), 448.0, use_ue8m0)
    return (slabs * (1.0 / sf.unsqueeze(1))).to(torch.float8_e4m3fn).reshape(rows, cols), sf


def per_custom_dims_cast_to_fp8(x: torch.Tensor, dims: Tuple, use_ue8m0: bool):
    """e4m3 with one scale per index of the dimensions in `dims` (the maximum is taken over all the others;
    deep_gemm/utils/math.py:75-81).  Returns (q, sf squeezed to the kept dimensions)."""
    reduced = tuple(i for i in range(x.dim()) if i not in set(dims))
    sf = _scales(x.abs().amax(dim=reduced, keepdim=True), 448.0, use_ue8m0)
    return (x * (1.0 / sf)).to(torch.float8_e4m3fn), sf.squeeze()


def transpose_packed_fp4(a: torch.Tensor) -> torch.Tensor:
    """[rows, cols / 2] int8 holding two e2m1 codes per byte (low nibble first) -> the packed [cols, rows / 2] transpose
    (deep_gemm/utils/math.py:128-141)."""
    assert a.dtype == torch.int8 and a.dim() == 2 and a.size(0) % 2 == 0
    rows, half = a.shape
    nibbles = torch.stack((a & 0x0F, (a >> 4) & 0x0F), dim=-1).reshape(rows, 2 * half)      # one code per element
    pairs = nibbles.t().reshape(2 * half, rows // 2, 2)
    return (pairs[..., 0] | (pairs[..., 1] << 4)).to(torch.int8).contiguous()


def _e2m1_codes(x: torch.Tensor) -> torch.Tensor:
    """Nearest e2m1 code, ties to the even mantissa, sign in bit 3 (negative zero is not produced)."""
    mag = x.abs()
    grid = torch.tensor(_E2M1_GRID, dtype=torch.float32, device=x.device)
    mids = (grid[:-1] + grid[1:]) / 2                                   # .25 .75 1.25 1.75 2.5 3.5 5
    ties_up = torch.tensor([False, True, False, True, False, True, False], device=x.device)
    above = mag.unsqueeze(-1) > mids
    at = (mag.unsqueeze(-1) == mids) & ties_up
    code = (above | at).sum(dim=-1).to(torch.uint8)
    negative = ((x < 0) & (code != 0)).to(torch.uint8)
    return code | (negative << 3)


def per_token_cast_to_fp4(x: torch.Tensor, use_ue8m0: bool, gran_k: int = 128, use_packed_ue8m0: bool = False):
    assert x.dim() == 2 and x.size(1) % 2 == 0 and (use_ue8m0 or not use_packed_ue8m0)
    rows, cols = x.shape
    blocks, padded = _block_view(x, gran_k)
    sf = _scales(blocks.abs().amax(dim=2), 6.0, use_ue8m0)
    codes = _e2m1_codes((blocks * (1.0 / sf).unsqueeze(2)).float()).reshape(rows, padded)
    packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).view(torch.int8)[:, : cols // 2].contiguous()
    return packed, _maybe_pack(sf, use_packed_ue8m0)


def unpack_ue8m0_from_int(packed: torch.Tensor) -> torch.Tensor:
    return (packed.contiguous().view(torch.uint8).to(torch.int32) << 23).view(torch.float32)


def cast_back_from_fp8(q: torch.Tensor, sf: torch.Tensor, gran_k: int = 128, use_packed_ue8m0: bool = False):
    if use_packed_ue8m0:
        sf = unpack_ue8m0_from_int(sf)
    idx = torch.arange(q.size(1), device=q.device) // gran_k
    return q.float() * sf[:, idx]


def cast_back_from_fp4(packed: torch.Tensor, sf: torch.Tensor, gran_k: int = 128, use_packed_ue8m0: bool = False):
    if use_packed_ue8m0:
        sf = unpack_ue8m0_from_int(sf)
    b = packed.view(torch.uint8)
    codes = torch.stack((b & 0xF, b >> 4), dim=-1).flatten(-2).long()
    grid = torch.tensor(_E2M1_GRID, dtype=torch.float32, device=packed.device)
    vals = grid[codes & 7] * (1.0 - 2.0 * ((codes >> 3) & 1).float())
    idx = torch.arange(vals.size(1), device=packed.device) // gran_k
    return vals * sf[:, idx]
