"""y = x W^T for a weight stored [out, in], the way every projection here is.

Which product runs:
  * float32 weight: this package's own float32 FMA kernel (no tensor-core or
    reduced-precision mode); bfloat16 activations are widened first and the
    result narrowed again.
  * bfloat16 weight of 256 MB and more (the head), 1 to 64 rows, and of 90 MB
    and more (the feed-forward's) at 9 to 32 rows: this package's stream-K
    tcgen05 kernel, which cuts the weight evenly over the SMs.
  * bfloat16 weight, 1 to 8 rows: this package's tensor-core kernel for
    decode batches, which reads the weight once (or, when `GEMV_MAX_ROWS`
    says so, the plain bandwidth kernel for one row).
  * bfloat16 weight, more rows: the library product (cuBLAS through
    `torch.mm`), float32 accumulation, or this package's tcgen05 kernel when
    `LARGE_GEMM` says so.  Upstream uses the same library for all
    its products (src/src-cuda/mat-ops/gemm/gemm.cu:22-41).
`swiglu_product` is the gate/up product of a SwiGLU feed-forward with its activation: one
tcgen05 kernel for prompts, product and SwiGLU kernel otherwise.
"""
from __future__ import annotations

import os
from typing import Optional

import torch

from . import kernels
from .library import KernelError

# Which product takes bfloat16 weights with more than SKINNY_MAX_ROWS rows of x: "library" (cuBLAS through
# torch.mm) or "tcgen05" (this package's TMA/tcgen05 kernel).  Measured at 2,048 rows and Qwen3-8B sizes the
# library runs 1.43-1.55 PFLOP/s and the tcgen05 kernel 1.26-1.40 (pairs of CTAs), so the library is the default; set
# GARLIC_B200_GEMM=tcgen05 (or this variable) to run this package's kernel instead.
LARGE_GEMM = os.environ.get("GARLIC_B200_GEMM", "library")

# From how many rows of x on the gate/up product of a SwiGLU feed-forward runs as this package's tcgen05
# kernel with the activation in its epilogue (bfloat16).  Measured at 2,048 rows and Qwen3-8B sizes: 295 us
# against 276 us for the library product plus 33 us for the SwiGLU kernel.  0 switches it off.
FUSED_SWIGLU_MIN_ROWS = int(os.environ.get("GARLIC_B200_FUSED_SWIGLU_ROWS", "512"))

# Which kernel takes bfloat16 products of 1 to 16 rows whose weight has at least this many bytes: the stream-K
# tcgen05 kernel (W cut evenly over the SMs, 6.6 TB/s once it runs but about 10 us to start and to merge the
# cut tiles).  Measured at 8 rows: 189 against 216 us on the 1.24 GB head, 39.4 against 38.9 us on 201 MB,
# 27.8 against 22.8 us on 101 MB; so smaller weights stay with the skinny kernel.  0 switches it off.
STREAMK_MIN_BYTES = int(os.environ.get("GARLIC_B200_STREAMK_MIN_BYTES", str(256 << 20)))

STREAMK_MAX_ROWS = 64
# From 9 to 32 rows (where the skinny kernel no longer competes and the alternative is the library product) the
# stream-K kernel takes smaller weights too: it starts its stream of W behind the kernel before it, which a
# library kernel does not.  Measured inside a decode step with the feed-forward's two products (201 and 101 MB)
# on it / with the head only / with all products: 16 sequences 4.43 / 4.63 / 4.79 ms, 32 sequences 5.39 / 5.43 /
# 5.72 ms.  At 64 sequences the kernel alone is slower than the library on those two (40.6 against 38.5 and 29.8
# against 22.4 us) and the step with them 7.65 against 7.56 ms, so from 33 rows on it keeps the head only.
STREAMK_WIDE_MAX_ROWS = 32
STREAMK_MIN_BYTES_WIDE = int(os.environ.get("GARLIC_B200_STREAMK_MIN_BYTES_WIDE", str(90 << 20)))
# Up to how many rows of x the plain bandwidth kernel (a warp per row of W) takes a product: none by default.
# Alone it is as fast as the others at one row (175 us on the 1.24 GB head against 181 skinny and 183 stream-K),
# but it gains nothing from being launched early behind its predecessor: a whole step of one sequence takes
# 3.26 ms with the skinny and stream-K kernels, 3.29 ms with this kernel on the head only and 3.62 ms with it
# everywhere.  GARLIC_B200_GEMV_ROWS=1 (or this variable) switches it on; the microbenchmark times it beside the others.
GEMV_MAX_ROWS = int(os.environ.get("GARLIC_B200_GEMV_ROWS", "0"))
SKINNY_MAX_ROWS = 8        # up to here: the tensor-core kernel that streams W once (it takes 16; the library is faster from 9 on)


def _streamk_min_bytes(m: int) -> int:
    return STREAMK_MIN_BYTES_WIDE if SKINNY_MAX_ROWS < m <= STREAMK_WIDE_MAX_ROWS else STREAMK_MIN_BYTES


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None) -> torch.Tensor:
    if x.dim() != 2 or w.dim() != 2 or x.shape[1] != w.shape[1]:
        raise KernelError(f"linear: x {tuple(x.shape)} does not fit a weight {tuple(w.shape)} ([out, in])")
    out_dtype = out_dtype or x.dtype
    if w.dtype == torch.float32:
        y = kernels.sgemm_nt(kernels.cast(x, torch.float32), w)
        return kernels.cast(y, out_dtype)
    if w.dtype != torch.bfloat16:
        raise KernelError(f"linear: weight dtype {w.dtype}")
    if x.dtype != torch.bfloat16:
        raise KernelError(f"linear: a bfloat16 weight takes bfloat16 activations, not {x.dtype}")
    m, k = x.shape
    if m == 0:
        return torch.empty((0, w.shape[0]), dtype=out_dtype, device=x.device)
    aligned = k % 8 == 0 and w.data_ptr() % 16 == 0 and x.data_ptr() % 16 == 0
    if m <= GEMV_MAX_ROWS and aligned:
        return kernels.gemv_bf16(x, w, out_dtype)
    if m <= STREAMK_MAX_ROWS and aligned and 0 < _streamk_min_bytes(m) <= w.numel() * 2:
        return kernels.gemm_streamk_bf16(x, w, out_dtype)
    if m <= SKINNY_MAX_ROWS and aligned:
        return kernels.gemm_skinny_bf16(x, w, out_dtype)
    kernels.require_gpu()
    if LARGE_GEMM == "tcgen05" and k % 8 == 0 and w.data_ptr() % 16 == 0 and x.data_ptr() % 16 == 0:
        return kernels.gemm_tcgen05_bf16(x, w, out_dtype)
    if out_dtype == torch.float32:
        return torch.mm(x, w.t(), out_dtype=torch.float32)
    return torch.mm(x, w.t())


def swiglu_product(x: torch.Tensor, w_gate_up: torch.Tensor) -> torch.Tensor:
    """silu(x . Wg^T) * (x . Wu^T) for the packed weight [Wg; Wu]: prompts in bfloat16 run it as one tcgen05
    kernel (product and activation), decode batches of 1 to 8 as one skinny (or gemv) kernel, everything else as the
    product of `linear` and the SwiGLU kernel."""
    m, k = x.shape
    if (FUSED_SWIGLU_MIN_ROWS > 0 and m >= FUSED_SWIGLU_MIN_ROWS and x.dtype == torch.bfloat16
            and w_gate_up.dtype == torch.bfloat16 and k % 8 == 0 and w_gate_up.shape[0] % 2 == 0
            and x.data_ptr() % 16 == 0 and w_gate_up.data_ptr() % 16 == 0):
        return kernels.gemm_tcgen05_swiglu_bf16(x, w_gate_up)
    if (0 < m <= SKINNY_MAX_ROWS and x.dtype == torch.bfloat16 and w_gate_up.dtype == torch.bfloat16
            and k % 8 == 0 and w_gate_up.shape[0] % 2 == 0 and x.data_ptr() % 16 == 0 and w_gate_up.data_ptr() % 16 == 0
            and (m <= GEMV_MAX_ROWS or not (0 < STREAMK_MIN_BYTES <= w_gate_up.numel() * 2))):
        # decode batches: the activation in the product's last step
        if m <= GEMV_MAX_ROWS:
            return kernels.gemv_swiglu_bf16(x, w_gate_up)
        return kernels.gemm_skinny_swiglu_bf16(x, w_gate_up)
    return kernels.swiglu(linear(x, w_gate_up))
