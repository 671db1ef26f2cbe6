"""Matrix products y = x W^T with 32-bit sums and a 32-bit result.

Few rows (a decode step) go to the hand-written weight-streaming kernels: bfloat16
with up to 64 rows to the tensor-core one, float32 (and odd inner sizes) with up to
16 rows to the plain one.  More rows go to the library product, as in the reference,
whose dispatcher sends up to 16 rows to its own kernels and the rest to cuBLAS
(ggml-cuda/ggml-cuda.cu:1812-1866).  In the 32-bit engine the library product
runs in plain float32: the reduced-precision (TF32) mode is switched off and
checked at every call.
"""
from __future__ import annotations

import torch

from ..kernels import ops


def require_true_fp32() -> None:
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")


def linear(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """x [M, K] (the weight's dtype) times weight [N, K] transposed -> float32 [M, N]."""
    M, K = x.shape
    if weight.dtype == torch.bfloat16 and M <= ops.STREAM_M and K % 8 == 0:
        return ops.gemm_stream(x, weight)
    if M <= ops.SMALL_M:
        return ops.gemm_small(x, weight)
    if weight.dtype == torch.bfloat16:
        return torch.mm(x, weight.t(), out_dtype=torch.float32)
    if torch.backends.cuda.matmul.allow_tf32 or torch.get_float32_matmul_precision() != "highest":
        raise RuntimeError("the 32-bit engine needs plain float32 matrix products; a reduced-precision "
                           "mode was switched on after the engine was made")
    return torch.mm(x, weight.t())
