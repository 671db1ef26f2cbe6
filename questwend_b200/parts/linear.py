"""Matrix products y = x W^T with 32-bit sums and a 32-bit result.

Few rows (a decode step) go to the hand-written weight-streaming kernels: bfloat16
with up to 8 rows (up to 16 for matrices of at most 16 M weights) to the tensor-core
one (mma.sync), which also folds the residual sum or the gated SiLU into its
epilogue; float32 (and odd inner sizes) with few rows to the plain one.  More rows go to the library product, as in the reference,
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
    return ("gemm_small", "gemm_stream", "gemm_ring", "gemm_tc") if dtype == torch.bfloat16 else ("gemm_small",)


def require_true_fp32() -> None:
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    torch.set_float32_matmul_precision("highest")


STREAM_MAX_ROWS = 8         # up to here the own weight-streaming product is always the fastest.  With 9 to 16 rows (its
STREAM_WIDE_MAX_WEIGHT = 1 << 24   # two-tile form) it still is for matrices of up to 16 M weights (the 0.6B model's, an
                            # 8B model's o projection); beyond, the library is: at 16 rows the down projection of Qwen3-8B
                            # (50 M weights) takes 30.7 us against 21.2 us


def _stream_rows(M: int, weight: torch.Tensor) -> bool:
    return M <= STREAM_MAX_ROWS or (M <= ops.STREAM_M and weight.numel() <= STREAM_WIDE_MAX_WEIGHT)


# Which few-rows product is fastest depends on the matrix: at 8 rows the own kernel needs 19 us for Qwen3-8B's down
# projection where the library needs 31, and 62 us for Qwen3-32B's where the library needs 45.  So for matrices large
# enough to matter, the first step that meets a shape (rows up to 8, or 9 to 16; plain, residual-add or SwiGLU) times
# the candidates once, each on a cold L2 as inside a step, and the choice is kept for the process -- if QWB200_TUNE=1 asks
# for it (``bench.py`` does, for the largest model).  By default the choice follows from the shape alone, so that the same
# trace gives the same bits in every process; ``tuned_choices()`` tells what a tuned process chose.
TUNE_MIN_WEIGHT_BYTES = 8 << 20     # smaller matrices stay in L2 anyway and every choice is at its launch floor
TUNE = os.environ.get("QWB200_TUNE", "0") == "1"      # off unless asked for: a timed choice can differ from run to run, and
                                                      # with it the order of a sum and a logit's last bits
LIBRARY_MUST_WIN_BY = 0.90          # the own kernel starts under the tail of the kernel before it, the library's does not
CHANGE_MUST_WIN_BY = 0.92           # what the usual choice must lose by before another is taken
_CHOICES: dict = {}                 # (device, N, K, rows, kind) -> ("stream", (u, w) or None) | ("library", None)


def tuned_choices() -> dict:
    """What the measuring has chosen so far in this process: {(N, K, rows up to, kind): "stream u x w" or "library"}."""
    return {k[1:]: ("library" if how == "library" else f"stream {cfg[0]}x{cfg[1]}" if cfg else "stream")
            for k, (how, cfg) in _CHOICES.items()}


def _library(x, weight, add_to, kind, interleave):
    if kind == "swiglu":
        return ops.silu_mul(torch.mm(x, weight.t(), out_dtype=torch.float32), torch.bfloat16, interleave)
    if add_to is not None:
        return torch.addmm(add_to, x, weight.t(), out_dtype=torch.float32, out=add_to)
    return torch.mm(x, weight.t(), out_dtype=torch.float32)


FEW_ROWS_KERNEL = os.environ.get("QWB200_FEW_ROWS", "ring")     # "ring" or "stream": which few-rows kernel the engine uses


def _stream(x, weight, add_to, kind, config):
    if config is None and FEW_ROWS_KERNEL == "ring":
        if kind == "swiglu":
            return ops.gemm_ring_swiglu(x, weight)
        return ops.gemm_ring(x, weight, residual=add_to)
    if kind == "swiglu":
        return ops.gemm_stream_swiglu(x, weight, config=config)
    return ops.gemm_stream(x, weight, residual=add_to, config=config)


def _measure(weight: torch.Tensor, rows: int, kind: str, default, static) -> tuple:
    N, K = weight.shape
    x = torch.randn(rows, K, device=weight.device).to(torch.bfloat16)
    res = torch.zeros(rows, N, device=weight.device) if kind == "add" else None
    flush = torch.empty(192 << 20, dtype=torch.uint8, device=weight.device)      # larger than L2
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)

    def time_of(fn) -> float:
        times = []
        for i in range(7):
            flush.zero_()
            start.record()
            fn()
            end.record()
            end.synchronize()
            if i >= 2:
                times.append(start.elapsed_time(end))
        return sorted(times)[len(times) // 2]

    timed = {("stream", cfg): time_of(lambda: _stream(x, weight, res, kind, cfg)) for cfg in ops.STREAM_CONFIGS}
    # the library's kernel starts only when the kernel before it has ended, the own one under its tail: count that
    timed[("library", None)] = time_of(lambda: _library(x, weight, res, kind, ops.GATE_UP_GROUP)) / LIBRARY_MUST_WIN_BY
    usual = ("stream", default) if static[0] == "stream" else ("library", None)
    best = min(timed, key=timed.get)
    # only a clear win changes the usual choice: timings of single kernels are not quite what a step sees
    return best if timed[best] < CHANGE_MUST_WIN_BY * timed[usual] else (static[0], default if static[0] == "stream" else None)


def _few_rows_choice(M: int, weight: torch.Tensor, kind: str) -> tuple:
    """("stream", config or None) or ("library", None) for M <= 16 rows of this weight."""
    static = ("stream", None) if _stream_rows(M, weight) else ("library", None)
    if not TUNE or weight.numel() * weight.element_size() < TUNE_MIN_WEIGHT_BYTES:
        return static
    rows = STREAM_MAX_ROWS if M <= STREAM_MAX_ROWS else ops.STREAM_M
    key = (weight.device.index, weight.shape[0], weight.shape[1], rows, kind)
    choice = _CHOICES.get(key)
    if choice is None:
        if torch.cuda.is_current_stream_capturing():
            return static                                # no measuring inside a capture (plain steps come before it)
        N, K = weight.shape
        default = (8, 8) if K >= 8192 else ((2, 16) if N <= 4096 else (2, 8))      # the kernel's own choice by shape
        choice = _CHOICES[key] = _measure(weight, rows, kind, default, static)
    return choice

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
        how, config = _few_rows_choice(M, weight, "plain" if add_to is None else "add")
        if how == "stream":
            return _stream(x, weight, add_to, "add" if add_to is not None else "plain", config)
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


def linear_swiglu(x: torch.Tensor, weight_gate_up: torch.Tensor, out_dtype: torch.dtype, interleave: int = 0) -> torch.Tensor:
    """silu(x Wg^T) * (x Wu^T) for the stacked weight [2F, K] -> [M, F] in ``out_dtype``.  ``interleave`` 0: gate rows
    first; ``ops.GATE_UP_GROUP``: gate and up rows interleaved in groups of that many features, which lets the products
    with a fused epilogue find a feature's gate and up in one thread."""
    if interleave == ops.GATE_UP_GROUP and x.dtype == torch.bfloat16 and out_dtype == torch.bfloat16:
        if x.shape[0] <= ops.STREAM_M and x.shape[1] % 8 == 0:
            how, config = _few_rows_choice(x.shape[0], weight_gate_up, "swiglu")
            if how == "stream":
                return _stream(x, weight_gate_up, None, "swiglu", config)
        if x.shape[0] >= TC_SWIGLU_MIN_ROWS and x.shape[1] >= TC_SWIGLU_MIN_INNER and x.shape[1] % 8 == 0:
            return ops.gemm_tc(x, weight_gate_up, epilogue="swiglu", tile_n=256)
    return ops.silu_mul(linear(x, weight_gate_up), out_dtype, interleave)
