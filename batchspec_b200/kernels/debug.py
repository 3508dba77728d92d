"""Switches for debugging and tuning the kernels, read once from the environment when the library is loaded.
None of them is a product option: the defaults are what measurement chose, and every value gives the same
results (only other kernels or other launch plans).

    BSPEC_PDL=0                 no programmatic dependent launch (every kernel waits for its predecessor to finish)
    BSPEC_GEMM_SPLITS=n         force the number of K slices of the small-M tcgen05 GEMM
    BSPEC_TC_GEMM=auto|all|none which bfloat16 products run on this package's tcgen05 kernel
    BSPEC_TC_GEMM_MAX_M=n       "auto": products of at most n rows
    BSPEC_GLU_FUSION=0          gate/up product and activation as two kernels
    BSPEC_QKV_ROPE_FUSION=0     q/k/v product, rotary encoding and cache append as three kernels
    BSPEC_TMA_ATTENTION=0       decode attention without TMA (cp.async kernel)
    BSPEC_TC_ATTENTION=0        prompt attention without the tcgen05 kernel
    BSPEC_BALANCED_ATTENTION=0  decode attention cut per request instead of in equal shares
"""
from __future__ import annotations

import os
from ctypes import c_int


def apply_environment(ops, lib) -> None:
    env = os.environ
    flag = lambda name: env.get(name, "1") != "0"
    if not flag("BSPEC_PDL"):
        lib.bspec_set_pdl.argtypes = [c_int]
        lib.bspec_set_pdl.restype = None
        lib.bspec_set_pdl(0)
    if env.get("BSPEC_GEMM_SPLITS"):
        lib.bspec_gemm_tc_force_splits.argtypes = [c_int]
        lib.bspec_gemm_tc_force_splits(int(env["BSPEC_GEMM_SPLITS"]))
    ops.TC_GEMM = env.get("BSPEC_TC_GEMM", ops.TC_GEMM)
    ops.TC_GEMM_MAX_M = int(env.get("BSPEC_TC_GEMM_MAX_M", ops.TC_GEMM_MAX_M))
    ops.GLU_FUSION = flag("BSPEC_GLU_FUSION")
    ops.FUSE_QKV_ROPE = flag("BSPEC_QKV_ROPE_FUSION")
    ops.USE_TMA_ATTENTION = flag("BSPEC_TMA_ATTENTION")
    ops.USE_TC_ATTENTION = flag("BSPEC_TC_ATTENTION")
    ops.BALANCED_ATTENTION = flag("BSPEC_BALANCED_ATTENTION")
