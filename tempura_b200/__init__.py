"""tempura_b200 -- B200 (sm_100a) KV-cache handoff for disaggregated prefill -> decode.

The package holds the CUDA kernels and C ABI (``csrc/``, built into ``lib/libtkv.so``)
and a thin Python face over that ABI.  Importing the package does not load the
library; the first call does, and fails loudly if it was never built.
"""
from ._native import (DTYPE_E4M3, DTYPE_F16, DTYPE_F32, PLAN_ALLOW_SHARED_DST, PLAN_FORCE_BULK,
                      PLAN_FORCE_VECTOR, PLAN_INT_QUANTIZER, TkvError, lib)
from ._build import build as build_native

__all__ = ["DTYPE_E4M3", "DTYPE_F16", "DTYPE_F32", "PLAN_ALLOW_SHARED_DST", "PLAN_FORCE_BULK",
           "PLAN_FORCE_VECTOR", "PLAN_INT_QUANTIZER", "TkvError", "lib", "build_native"]
