"""Epilogue selectors of the reference's `deep_gemm.epilogue` submodule
(csrc/jit_kernels/impls/epilogue_class.hpp:19-127): Identity; Alpha (dense GEMM); FP8Quantization (dense and batched
GEMMs: D written as e4m3 with one UE8M0 scale per row and 32 columns into `sfd`); BF16StochasticRounding (any GEMM with
a BF16 D that is written directly).  They do not compose."""
from __future__ import annotations


class Epilogue:
    pass


class Identity(Epilogue):
    pass


class Alpha(Epilogue):
    def __init__(self, alpha: float):
        self.alpha = float(alpha)


class FP8Quantization(Epilogue):
    def __init__(self, sfd):
        self.sfd = sfd


class BF16StochasticRounding(Epilogue):
    pass
