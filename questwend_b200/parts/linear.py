"""Matrix products y = x W^T with 32-bit sums and a 32-bit result.

Few rows (a decode step) go to the hand-written weight-streaming kernels: bfloat16
with up to 8 rows (up to 16 where ``_few_rows`` says so: at the Qwen3-8B and 0.6B sizes every
product) to the tensor-core one (``gemm_ring``: W streamed by TMA through a ring in shared
memory, mma.sync), which also folds the residual sum or the gated SiLU into its epilogue, or
leaves a product that is added onto the residual stream as partial sums for the norm that
follows (``linear_onto``); float32 (and odd inner sizes) with few rows to the plain one.  More rows go to the library product, as in the reference,
whose dispatcher sends up to 16 rows to its own kernels and the rest to cuBLAS
(ggml-cuda/ggml-cuda.cu:1812-1866); the residual sum rides in the library call
(beta = 1).  The exception is the gate/up projection of many bfloat16 rows: the
tcgen05 kernel (TMA-fed, accumulators in tensor memory) with the gated SiLU in its
epilogue beats the library product followed by a separate kernel.  That kernel's
plain and residual-add epilogues are measured against the library in the
microbenchmark and lose to it (by 4-11 % at 2,048 rows, by 2x at 256 rows, where
it has too few tiles for 148 SMs), so the engine does not use them.
In the 32-bit engine the library product runs in plain float32: the
reduced-precision (TF32) mode is switched off and checked at every call.
"""
from __future__ import annotations

import os

import torch

from ..kernels import ops


def kernel_modules(dtype: torch.dtype) -> tuple:
    """The kernel modules that ``linear`` may launch for this engine dtype."""
    few_rows = "gemm_ring" if FEW_ROWS_KERNEL == "ring" else "gemm_stream"
    return ("gemm_small", few_rows, "gemm_tc") if dtype == torch.bfloat16 else ("gemm_small",)


def require_true_fp32() -> None:
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")


STREAM_MAX_ROWS = 8         # up to here the own weight-streaming product is always the fastest.  With 9 to 16 rows (its
                            # two-tile form) it is where the rows of x cost it nothing or little: rows of up to 2,048 or 4,096
                            # values (the ring product then keeps its pieces of x in registers: at 16 rows q/k/v 12.7 us
                            # against the library's 12.1, o 9.6 against 9.3, gate/up with the SiLU 37.1 against 34.7 + 3 for
                            # the separate SiLU kernel, the head 198 against 208), matrices of up to 16 M weights (the
STREAM_WIDE_MAX_WEIGHT = 1 << 24   # 0.6B model's) and long rows (below)

LONG_ROWS = 8192            # with 9 to 16 rows of at least this many values the ring product is within a few per cent of the
                            # library again (Qwen3-8B down projection, 12,288: 21.1 against 21.3 us at 12 rows, 23.0 against
                            # 21.3 at 16).  What is left to the library with 9 to 16 rows, all at the 32B sizes: rows between
                            # 4,096 and 8,192 values of matrices above 16 M weights (q/k/v and gate/up, rows of 5,120: 26.5
                            # and 107 us against 21.1 and 91) and matrices whose tiles fill the SMs' rounds badly (o and down)

FEW_ROWS_KERNEL = os.environ.get("QWB200_FEW_ROWS", "ring")     # "ring" (gemm_ring, the default) or "stream" (gemm_stream, the
                                                                # kernel before it, kept for comparison)


def _few_rows(M: int, weight: torch.Tensor) -> bool:
    """Whether M rows of this bfloat16 weight go to the own few-rows product (else to the library).  The choice follows
    from the shape alone, so the same trace gives the same bits in every process."""
    if M <= STREAM_MAX_ROWS:
        return True
    if M > ops.STREAM_M:
        return False
    N, K = weight.shape
    if FEW_ROWS_KERNEL != "ring":
        return weight.numel() <= STREAM_WIDE_MAX_WEIGHT
    if weight.numel() <= STREAM_WIDE_MAX_WEIGHT:
        return True
    if ops.ring_split_plan(N, K, weight.device) is not None:
        return False            # whole tiles would fill the SMs' rounds badly, and with the split form a step of 16 rows at
                                # the Qwen3-32B sizes is 3 % slower than with the library (1,132 against 1,165 tokens/s)
    return -(-K // ops.RING_STAGE_K) in ops.RING_KEEPS_X_STAGES or K >= LONG_ROWS


def _stream(x, weight, add_to, kind):
    if FEW_ROWS_KERNEL == "ring":
        if kind == "swiglu":
            return ops.gemm_ring_swiglu(x, weight)
        return ops.gemm_ring(x, weight, residual=add_to)
    if kind == "swiglu":
        return ops.gemm_stream_swiglu(x, weight)
    return ops.gemm_stream(x, weight, residual=add_to)


TC_SWIGLU_MIN_ROWS = 512    # from here on the tcgen05 gate/up product with the SiLU in its epilogue beats library + kernel,
TC_SWIGLU_MIN_INNER = 2048  # for rows of x this long (with 1,024 a tile's set-up outweighs its 16 steps: 16.9 against 12.6 us)


def _check_true_fp32() -> None:
    if torch.backends.cuda.matmul.allow_tf32 or torch.get_float32_matmul_precision() != "highest":
        raise RuntimeError("the 32-bit engine needs plain float32 matrix products; a reduced-precision "
                           "mode was switched on after the engine was made")


def linear(x: torch.Tensor, weight: torch.Tensor, add_to: torch.Tensor | None = None) -> torch.Tensor:
    """x [M, K] (the weight's dtype) times weight [N, K] transposed -> float32 [M, N].
    With ``add_to`` (float32 [M, N]) the product is added onto it in place and it is returned."""
    M, K = x.shape
    bf16 = weight.dtype == torch.bfloat16
    if bf16 and M <= ops.STREAM_M and K % 8 == 0:
        if _few_rows(M, weight):
            return _stream(x, weight, add_to, "add" if add_to is not None else "plain")
    elif M <= (STREAM_MAX_ROWS if bf16 else ops.SMALL_M):     # float32; bfloat16 rows whose length is no multiple of 8
        return ops.gemm_small(x, weight, residual=add_to)
    if bf16:
        if add_to is not None:
            return torch.addmm(add_to, x, weight.t(), out_dtype=torch.float32, out=add_to)
        return torch.mm(x, weight.t(), out_dtype=torch.float32)
    _check_true_fp32()
    if add_to is not None:
        return torch.addmm(add_to, x, weight.t(), out=add_to)
    return torch.mm(x, weight.t())


def linear_onto(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor):
    """The product x W^T that is to be added onto ``residual`` (float32 [M, N]).  Returns None when it was added in place
    (in the product's epilogue), or the product still to be added, as a ``SplitSum``: few bfloat16 rows times a matrix
    whose whole tiles would leave the SMs' last round mostly empty go to the ring product's split form, and the norm that
    follows adds its planes (``settle`` for any other consumer)."""
    M, K = x.shape
    if (FEW_ROWS_KERNEL == "ring" and weight.dtype == torch.bfloat16 and M <= ops.STREAM_M and K % 8 == 0
            and _few_rows(M, weight)):
        plan = ops.ring_split_plan(weight.shape[0], K, x.device)
        if plan is not None:
            return ops.gemm_ring_split(x, weight, plan)
    linear(x, weight, add_to=residual)
    return None


def settle(h: torch.Tensor, delta, norm=None):
    """What a block hands its norm: ``delta`` as it is if the norm can add it, else added onto ``h`` (returns None)."""
    if isinstance(delta, ops.SplitSum) and not getattr(norm, "adds_split_sums", False):
        delta.add_onto(h)
        return None
    return delta


def linear_swiglu(x: torch.Tensor, weight_gate_up: torch.Tensor, out_dtype: torch.dtype, interleave: int = 0) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for the stacked weight [2F, K] -> [M, F] in ``out_dtype``.  ``interleave`` 0: gate rows
    first; ``ops.GATE_UP_GROUP``: gate and up rows interleaved in groups of that many features, which lets the products
    with a fused epilogue find a feature's gate and up in one thread."""
    if interleave == ops.GATE_UP_GROUP and x.dtype == torch.bfloat16 and out_dtype == torch.bfloat16:
        if x.shape[0] <= ops.STREAM_M and x.shape[1] % 8 == 0:
            if _few_rows(x.shape[0], weight_gate_up):
                return _stream(x, weight_gate_up, None, "swiglu")
        if x.shape[0] >= TC_SWIGLU_MIN_ROWS and x.shape[1] >= TC_SWIGLU_MIN_INNER and x.shape[1] % 8 == 0:
            return ops.gemm_tc(x, weight_gate_up, epilogue="swiglu", tile_n=256)
    return ops.silu_mul(linear(x, weight_gate_up), out_dtype, interleave)
