"""Loads the compiled CUDA library and declares its C entry points.

There is no fallback: if the library cannot be built or loaded, or the GPU is
not a compute-capability-10 part, every operation raises `ExtensionError`.
"""
from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_ulonglong, c_void_p

_lib = None
_checked_arch = False


class ExtensionError(RuntimeError):
    """The CUDA library of this package is missing, cannot be built, or cannot run here."""


class KernelError(RuntimeError):
    """An entry point refused its arguments or the launch failed."""


P, I, L, F = c_void_p, c_int, c_longlong, c_float

_SIGNATURES = {
    "gi_device_arch": ([], I),
    "gi_embedding": ([P, P, I, P, I, I, I, P], I),
    "gi_add_rmsnorm": ([P, P, P, I, P, I, P, I, I, F, I, P], I),
    "gi_residual_add": ([P, I, P, L, P], I),
    "gi_swiglu": ([P, P, I, I, I, P], I),
    "gi_cast": ([P, I, P, I, L, P], I),
    "gi_qk_norm_rope_append": ([P, P, P, P, I, P, P, I, F, P, P, I, P, P, P,
                                I, I, I, I, I, I, I, I, I, P, P], I),
    "gi_attention_generic": ([P, P, P, I, P, P, P, P, I, I, I, I, I, I, I, I, F, P, P], I),
    "gi_attention_prefill_bf16": ([P, P, P, P, P, I, P, I, I, I, I, I, I, I, F, P], I),
    "gi_attention_prefill_tcgen05": ([P, P, P, P, P, I, P, I, I, I, I, I, I, I, I, F, P, P], I),
    "gi_attention_decode_bf16": ([P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, P], I),
    "gi_set_pdl": ([I], None),
    "gi_attention_decode_tcgen05": ([P, P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, P, P], I),
    "gi_attention_decode_combine": ([P, P, P, I, I, I, P], I),
    "gi_sgemm_nt": ([P, P, P, I, I, I, L, L, P], I),
    "gi_gemv_bf16": ([P, P, P, I, I, I, I, P], I),
    "gi_gemm_skinny_bf16": ([P, P, P, I, I, I, I, I, I, P], I),
    "gi_gemv_swiglu_bf16": ([P, P, P, I, I, P], I),
    "gi_gemm_skinny_swiglu_bf16": ([P, P, P, I, I, I, I, I, P], I),
    "gi_gemm_tcgen05_swiglu_bf16": ([P, P, P, I, I, I, P, P], I),
    "gi_gemm_streamk_bf16": ([P, P, P, I, I, I, I, P, P, P, P], I),
    "gi_gemm_streamk_workspace_floats": ([], L),
    "gi_gemm_streamk_flags": ([], I),
    "gi_gemm_streamk_test_unanswered_flags": ([I], None),
    "gi_gemm_tcgen05_bf16": ([P, P, P, I, I, I, I, P, P], I),
    "gi_sample": ([P, L, I, I, P, P, P, c_ulonglong, P, P, P, P], I),
    "gi_sample_chunks": ([I], I),
    "gi_sample_uniform": ([c_ulonglong, L, I, I], F),
    "gi_sample_uniform_from_hash": ([c_ulonglong], F),
    "gi_random_normal": ([P, I, L, c_ulonglong, F, F, P], I),
    "gi_random_sum12": ([c_ulonglong, c_ulonglong], I),
}


def declare(lib, signatures=None) -> None:
    for name, (argtypes, restype) in (signatures or _SIGNATURES).items():
        try:
            fn = getattr(lib, name)
        except AttributeError:
            raise ExtensionError(f"the compiled library lacks {name}: it is stale; delete "
                                 "garlic_inference_b200/csrc/_build and run again") from None
        fn.argtypes = argtypes
        fn.restype = restype
    lib.gi_last_error.restype = ctypes.c_char_p
    lib.gi_last_error.argtypes = []


def lib():
    """The loaded library (built at the first call if needed)."""
    global _lib
    if _lib is None:
        from ..csrc.build import BuildError, library_path
        try:
            path = library_path()
        except BuildError as e:
            raise ExtensionError(f"cannot build the CUDA library of garlic_inference_b200: {e}") from None
        try:
            loaded = ctypes.CDLL(str(path))
        except OSError as e:
            raise ExtensionError(f"cannot load {path}: {e}") from None
        declare(loaded)
        _lib = loaded
    return _lib


def require_gpu():
    """The library, after checking once that the current device can run sm_100a code."""
    global _checked_arch
    l = lib()
    if not _checked_arch:
        import torch
        if not torch.cuda.is_available():
            raise ExtensionError("no CUDA device: garlic_inference_b200 runs on a B200 GPU only "
                                 "(there is no CPU path)")
        arch = l.gi_device_arch()
        if arch < 0:
            raise ExtensionError(f"cannot query the GPU: {l.gi_last_error().decode()}")
        if arch // 10 != 10:
            raise ExtensionError(f"the GPU has compute capability {arch // 10}.{arch % 10}; the kernels "
                                 "are built for sm_100a (B200) only")
        _checked_arch = True
    return l


class _Counters:
    """How many of this library's kernels were launched (library products are not counted)."""
    launches = 0


counters = _Counters()


def check(rc: int, l=None) -> None:
    """Every entry point's return code goes through here: one call, one kernel launched."""
    if rc != 0:
        l = l or lib()
        raise KernelError(l.gi_last_error().decode() or f"error code {rc}")
    counters.launches += 1
