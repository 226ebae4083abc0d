"""Matrix products ``y = x · Wᵀ`` for the parts, with the choice of kernel in one place.

``W`` is stored ``[out, in]`` as in the checkpoint (K-major, which is what every
kernel here wants), ``x`` is ``[tokens, in]``.  The reference dispatches on the
weight format (``matmul_dispatch``, src/model.cu:797-825); here the choice is by
compute dtype and by the number of rows:

* float32: the CUDA-core FMA kernel, always (true 32-bit arithmetic);
* bfloat16, few rows (decode): the weight-streaming kernel;
* bfloat16, many rows (prefill): the tcgen05 tensor-core kernel;
* any shape a fast kernel refuses (alignment, size) goes to the CUDA-core kernel,
  which takes every shape.
"""
from __future__ import annotations

from typing import Optional

import torch

from ..csrc import ops

# Rows up to which the weight-streaming kernel is used instead of the tensor-core one.
SKINNY_MAX_ROWS = 32

_force_plain = False


def force_plain_kernels(on: bool) -> None:
    """Route every product to the CUDA-core kernel (used by tests as the yardstick)."""
    global _force_plain
    _force_plain = bool(on)


def plain_forced() -> bool:
    return _force_plain


def skinny_max_rows() -> int:
    return SKINNY_MAX_ROWS


def linear(x: torch.Tensor, w: torch.Tensor, out_dtype: Optional[torch.dtype] = None,
           out: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
    M, K = x.shape
    N = w.shape[0]
    if out is None:
        out = torch.empty((M, N), dtype=out_dtype or x.dtype, device=x.device)
    if M == 0:
        return out
    if x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and not _force_plain:
        if M <= SKINNY_MAX_ROWS and ops.gemv_supported(x, w, out):
            ops.gemv_bf16(x, w, out, accumulate)
            return out
        if ops.gemm_tc_supported(x, w, out):
            ops.gemm_tc(x, w, out, accumulate)
            return out
    ops.gemm_simt(x, w, out, accumulate)
    return out
