"""ctypes binding of ``_mm_kernels.so`` (the sm_100a CUDA kernel library).

The library has a plain C ABI: every entry point takes raw device pointers,
sizes and a ``cudaStream_t`` and returns 0 on success. Loading fails loudly
when a CUDA device is present but the library has not been built.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_int64, c_void_p
from pathlib import Path

_PKG = Path(__file__).resolve().parent.parent
_LIB = None

_P = c_void_p
_SIGS = {
    "mm_read_status": (c_int, [c_int]),
    "mm_sm_count": (c_int, []),
    "mm_status_ptr": (c_void_p, []),
    "mm_set_peer_wait_ms": (c_int, [c_int]),
    "mm_gemm_bf16": (c_int, [_P, c_int, c_int64, _P, c_int, c_int64, _P, c_int, c_int64,
                             c_int, c_int, c_int, _P]),
    "mm_gemm_pair_bf16": (c_int, [_P, c_int, c_int64, _P, c_int, c_int64, _P, c_int, c_int64,
                                  c_int, c_int, c_int, _P]),
    "mm_gemm_pair_dyn_bf16": (c_int, [_P, c_int, c_int64, _P, c_int, c_int64, _P, c_int, c_int64,
                                      c_int, c_int, c_int, _P, _P, _P]),
    "mm_zero_row_tail": (c_int, [_P, c_int64, _P, c_int, c_int, _P]),
    "mm_rmsnorm_fwd": (c_int, [_P, _P, _P, _P, c_int64, c_int, c_float, _P]),
    "mm_rmsnorm_bwd_parts": (c_int, [c_int64]),
    "mm_rmsnorm_bwd": (c_int, [_P, _P, _P, _P, _P, _P, _P, c_int64, c_int, c_int, c_int, _P]),
    "mm_rope": (c_int, [_P, _P, _P, c_int64, c_int, c_int, c_int, c_int64, c_int, c_int, c_int, _P]),
    "mm_swiglu_fwd": (c_int, [_P, _P, c_int64, c_int, _P]),
    "mm_swiglu_bwd": (c_int, [_P, _P, _P, c_int64, c_int, _P]),
    "mm_swiglu_fwd_rows": (c_int, [_P, _P, c_int64, c_int, _P, _P]),
    "mm_swiglu_bwd_rows": (c_int, [_P, _P, _P, c_int64, c_int, _P, _P]),
    "mm_cross_entropy": (c_int, [_P, _P, _P, _P, _P, c_int64, c_int, c_int64, c_int, c_float,
                                 c_int, _P]),
    "mm_ce_combine": (c_int, [_P, c_int, _P, _P, _P, c_int64, _P]),
    "mm_embedding_fwd": (c_int, [_P, _P, _P, c_int64, c_int, c_int, c_int, _P]),
    "mm_embedding_bwd": (c_int, [_P, _P, _P, c_int64, c_int, c_int, c_int, _P]),
    "mm_add_bf16": (c_int, [_P, _P, _P, c_int64, _P]),
    "mm_accumulate_f32_bf16": (c_int, [_P, _P, c_int64, _P]),
    "mm_adamw": (c_int, [_P, _P, _P, _P, _P, c_int64, c_float, c_float, c_float, c_float,
                         c_float, c_int, c_float, _P, _P]),
    "mm_sumsq_f32": (c_int, [_P, c_int64, _P, _P]),
    "mm_memcpy_d2d": (c_int, [_P, _P, c_int64, _P]),
    "mm_peer_copy": (c_int, [_P, _P, c_int64, _P]),
    "mm_zero": (c_int, [_P, c_int64, _P]),
    "mm_f32_to_bf16": (c_int, [_P, _P, c_int64, _P]),
    "mm_bf16_to_f32": (c_int, [_P, _P, c_int64, c_int, _P]),
    "mm_accumulate_f32": (c_int, [_P, _P, c_int64, _P]),
    "mm_fill_f32": (c_int, [_P, c_float, c_int64, _P]),
    "mm_sum_scale_f32": (c_int, [_P, c_int64, c_float, _P, _P]),
    "mm_scale_bf16": (c_int, [_P, _P, _P, c_int64, _P]),
    "mm_add_i64": (c_int, [_P, c_int64, _P, c_int64, _P]),
}


def lib_path() -> Path:
    """The kernel library this process uses: the checked build (index checks that record
    MM_ERR_BOUNDS instead of trapping) when MM_CHECKED=1, else the normal one."""
    import os
    alt = os.environ.get("MM_KERNEL_LIB")      # another build of the library inside the package directory (experiments)
    if alt:
        return _PKG / os.path.basename(alt)
    return _PKG / ("_mm_kernels_checked.so" if os.environ.get("MM_CHECKED", "0") == "1" else "_mm_kernels.so")


def load():
    """Returns the loaded kernel library, building nothing: raises if absent."""
    global _LIB
    if _LIB is not None:
        return _LIB
    path = lib_path()
    if not path.exists():
        raise RuntimeError(
            f"{path} is missing: run `python -m multimesh_jax_b200.csrc.build` "
            "(or __graft_entry__.build()) before using CUDA tensors")
    lib = ctypes.CDLL(str(path))
    for name, (res, args) in _SIGS.items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            continue
        fn.restype = res
        fn.argtypes = args
    _LIB = lib
    return lib


def register(name: str, restype, argtypes) -> None:
    """Lets other modules declare signatures of further entry points."""
    _SIGS[name] = (restype, argtypes)
    if _LIB is not None and hasattr(_LIB, name):
        fn = getattr(_LIB, name)
        fn.restype = restype
        fn.argtypes = argtypes


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"{what} failed with code {rc}")
