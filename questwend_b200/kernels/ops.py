"""Python entry points of the hand-written kernels.

Each function checks its tensors (device, dtype, layout), calls the C launcher
on the current CUDA stream and raises ``KernelError`` with the launcher's
message if it refuses the sizes.  Tensors must live on a CUDA device: there is
no CPU path.
"""
from __future__ import annotations

import ctypes
import math

import torch

from .build import load_module

DT_F32, DT_BF16 = 0, 1
PAGE_SIZE = 64          # tokens per cache page


class KernelError(RuntimeError):
    pass


def _dt(t: torch.dtype) -> int:
    if t == torch.float32:
        return DT_F32
    if t == torch.bfloat16:
        return DT_BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {t}")


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _stream() -> ctypes.c_void_p:
    """The current stream of the current device (also inside a graph capture, which runs on a stream of its own)."""
    if _raw_stream is not None:                      # the handle itself: a tenth of the cost of making a Stream object
        return ctypes.c_void_p(_raw_stream(torch.cuda.current_device()))
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _ptr(t: torch.Tensor | None) -> ctypes.c_void_p:
    return ctypes.c_void_p(0 if t is None else t.data_ptr())


def _need(t: torch.Tensor, name: str, dtype=None, ndim=None):
    if not t.is_cuda:
        raise KernelError(f"{name}: must be a CUDA tensor (this library has no CPU path)")
    if not t.is_contiguous():
        raise KernelError(f"{name}: must be contiguous")
    if dtype is not None and t.dtype != dtype:
        raise KernelError(f"{name}: must be {dtype}, got {t.dtype}")
    if ndim is not None and t.dim() != ndim:
        raise KernelError(f"{name}: must have {ndim} dimensions, got {t.dim()}")


LAUNCHES = [0]          # kernels of this library launched so far (through these entry points)


_FUNCTIONS: dict = {}    # (module, name) -> (library, its function), looked up once


def _lookup(module: str, fn: str):
    entry = _FUNCTIONS.get((module, fn))
    if entry is None:
        lib = load_module(module)
        entry = _FUNCTIONS[module, fn] = (lib, getattr(lib, fn))
    return entry


def _call(module: str, fn: str, *args, kernels: int = 1):
    entry = _lookup(module, fn)
    rc = entry[1](*args)
    LAUNCHES[0] += kernels
    if rc != 0:
        raise KernelError(entry[0].qwb_last_error().decode("utf-8", "replace") or f"{fn} failed with code {rc}")


_i = ctypes.c_int
_f = ctypes.c_float


# ----------------------------------------------------------------------------- elementwise
def embed_gather(ids: torch.Tensor, table: torch.Tensor, bad_token: torch.Tensor | None = None) -> torch.Tensor:
    """Rows of ``table`` [V, D] for int32 ``ids`` [T], as float32 [T, D]."""
    _need(ids, "ids", torch.int32, 1)
    _need(table, "table", ndim=2)
    T, (V, D) = ids.numel(), table.shape
    out = torch.empty((T, D), dtype=torch.float32, device=table.device)
    _call("elementwise", "qwb_embed_gather", _ptr(ids), _ptr(table), _i(_dt(table.dtype)), _ptr(out),
          _i(T), _i(D), _i(V), _ptr(bad_token), _stream())
    return out


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, out_dtype: torch.dtype,
            delta: torch.Tensor | None = None, write_sum: bool = False,
            rows: torch.Tensor | None = None) -> torch.Tensor:
    """RMS norm of the rows of float32 ``x`` [T, D] (plus ``delta``), times ``weight``.

    With ``write_sum`` the sum x + delta replaces x.  With ``rows`` (int32) only
    those rows are normed and the output has one row per entry.  ``delta`` may be a ``SplitSum``
    (a product left as sums over pieces of k): its planes are added in their order.
    """
    _need(x, "x", torch.float32, 2)
    _need(weight, "weight", torch.float32, 1)
    T, D = x.shape
    if weight.numel() != D:
        raise KernelError(f"rmsnorm: weight has {weight.numel()} entries for rows of {D}")
    n_rows = T
    if rows is not None:
        _need(rows, "rows", torch.int32, 1)
        n_rows = rows.numel()
    out = torch.empty((n_rows, D), dtype=out_dtype, device=x.device)
    if isinstance(delta, SplitSum):
        if tuple(delta.planes.shape[1:]) != (T, D):
            raise KernelError(f"rmsnorm: planes {tuple(delta.planes.shape)} do not match x {tuple(x.shape)}")
        _call("elementwise", "qwb_rmsnorm_planes", _ptr(x), _ptr(delta.planes), _ptr(delta.plane_count),
              _i(delta.planes.shape[0]), _i(T), _ptr(x if write_sum else None), _ptr(weight), _ptr(out), _i(_dt(out_dtype)),
              _ptr(rows), _i(n_rows), _i(D), _f(eps), _stream())
        return out
    if delta is not None:
        _need(delta, "delta", torch.float32, 2)
        if delta.shape != x.shape:
            raise KernelError(f"rmsnorm: delta {tuple(delta.shape)} does not match x {tuple(x.shape)}")
    _call("elementwise", "qwb_rmsnorm", _ptr(x), _ptr(delta), _ptr(x if (write_sum and delta is not None) else None),
          _ptr(weight), _ptr(out), _i(_dt(out_dtype)), _ptr(rows), _i(n_rows), _i(D), _f(eps), _stream())
    return out


GATE_UP_GROUP = 8       # the fused products want gate and up rows interleaved in groups of this many features


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor, group: int = GATE_UP_GROUP) -> torch.Tensor:
    """[F, K] gate and up rows as one [2F, K] matrix: for every ``group`` features their gate rows, then their up rows.
    A reordering of rows; the products are the same numbers."""
    F, K = gate.shape
    if up.shape != gate.shape or F % group:
        raise KernelError(f"interleave_gate_up: shapes {tuple(gate.shape)}, {tuple(up.shape)} with groups of {group}")
    return torch.cat([gate.reshape(F // group, group, K), up.reshape(F // group, group, K)], dim=1).reshape(2 * F, K).contiguous()


def silu_mul(gate_up: torch.Tensor, out_dtype: torch.dtype, interleave: int = 0) -> torch.Tensor:
    """silu(gate) * up from a float32 [T, 2F] matrix: gate columns first (``interleave`` 0), or for every
    ``interleave`` features their gates and then their ups."""
    _need(gate_up, "gate_up", torch.float32, 2)
    T, F2 = gate_up.shape
    if F2 % 2:
        raise KernelError(f"silu_mul: {F2} columns cannot be split into gate and up")
    out = torch.empty((T, F2 // 2), dtype=out_dtype, device=gate_up.device)
    _call("elementwise", "qwb_silu_mul", _ptr(gate_up), _ptr(out), _i(_dt(out_dtype)), _i(T), _i(F2 // 2), _i(interleave),
          _stream())
    return out


def add_inplace(out: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
    _need(out, "out", torch.float32)
    _need(delta, "delta", torch.float32)
    if out.shape != delta.shape:
        raise KernelError(f"add_inplace: shapes {tuple(out.shape)} and {tuple(delta.shape)} differ")
    _call("elementwise", "qwb_add_inplace", _ptr(out), _ptr(delta), ctypes.c_longlong(out.numel()), _stream())
    return out


# ----------------------------------------------------------------------------- rope + cache write
def rope_table(positions: torch.Tensor, inv_freq: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
    """cos and sin of positions[t] * inv_freq[i] as float32 [T, half]; the angles are formed in float64."""
    _need(positions, "positions", torch.int32, 1)
    _need(inv_freq, "inv_freq", torch.float64, 1)
    T, half = positions.numel(), inv_freq.numel()
    cos = torch.empty((T, half), dtype=torch.float32, device=positions.device)
    sin = torch.empty_like(cos)
    _call("rope_kv", "qwb_rope_table", _ptr(positions), _ptr(inv_freq), _ptr(cos), _ptr(sin), _i(T), _i(half), _stream())
    return cos, sin


def qk_norm_rope_store(qkv: torch.Tensor, q_weight, k_weight, cos, sin, tok_seq, tok_pos, page_table,
                       k_pool, v_pool, n_heads: int, n_kv_heads: int, head_dim: int, rotary_dim: int,
                       eps: float, store_kv: bool = True) -> torch.Tensor:
    """Per-head norm, rotation and cache write.  ``qkv`` float32 [T, (Hq + 2 Hkv) * hd];
    returns the rotated queries [T, Hq, hd] in the cache's dtype."""
    _need(qkv, "qkv", torch.float32, 2)
    T = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim:
        raise KernelError(f"qk_norm_rope_store: qkv has {qkv.shape[1]} columns, expected "
                          f"{(n_heads + 2 * n_kv_heads) * head_dim}")
    _need(k_pool, "k_pool", ndim=4)
    _need(v_pool, "v_pool", k_pool.dtype, 4)
    if tuple(k_pool.shape[1:]) != (n_kv_heads, k_pool.shape[2], head_dim) or v_pool.shape != k_pool.shape:
        raise KernelError(f"qk_norm_rope_store: cache pool {tuple(k_pool.shape)} does not fit "
                          f"{n_kv_heads} heads of {head_dim}")
    for name, t in (("q_weight", q_weight), ("k_weight", k_weight)):
        if t is not None:
            _need(t, name, torch.float32, 1)
            if t.numel() != head_dim:
                raise KernelError(f"qk_norm_rope_store: {name} has {t.numel()} entries for heads of {head_dim}")
    if rotary_dim:
        _need(cos, "cos", torch.float32, 2)
        _need(sin, "sin", torch.float32, 2)
        if tuple(cos.shape) != (T, rotary_dim // 2) or sin.shape != cos.shape:
            raise KernelError(f"qk_norm_rope_store: cos/sin {tuple(cos.shape)} do not fit {T} tokens and "
                              f"rotary size {rotary_dim}")
    _need(tok_seq, "tok_seq", torch.int32, 1)
    _need(tok_pos, "tok_pos", torch.int32, 1)
    _need(page_table, "page_table", torch.int32, 2)
    q_out = torch.empty((T, n_heads, head_dim), dtype=k_pool.dtype, device=qkv.device)
    _call("rope_kv", "qwb_qk_norm_rope_store", _ptr(qkv), _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin),
          _ptr(tok_seq), _ptr(tok_pos), _ptr(page_table), _ptr(q_out), _ptr(k_pool), _ptr(v_pool),
          _i(_dt(k_pool.dtype)), _i(T), _i(n_heads), _i(n_kv_heads), _i(head_dim), _i(rotary_dim), _f(eps),
          _i(k_pool.shape[2]), _i(page_table.shape[1]), _i(1 if store_kv else 0), _stream())
    return q_out


# ----------------------------------------------------------------------------- attention
def mma_attention_fits(dtype: torch.dtype, head_dim: int, page_size: int) -> bool:
    """Whether the tensor-core attention kernels take this case (else the plain ones do)."""
    return dtype == torch.bfloat16 and head_dim in (64, 128) and page_size == 64


def tc_attention_fits(dtype: torch.dtype, head_dim: int, page_size: int, group: int) -> bool:
    """Whether the tcgen05 prefill attention kernel takes this case."""
    return mma_attention_fits(dtype, head_dim, page_size) and 1 <= group <= 64


def attn_prefill(q, k_pool, v_pool, page_table, cu_seqlens, pos0, max_new: int, scale: float,
                 window: int = 0, impl: str = "auto") -> torch.Tensor:
    """Causal attention of new tokens over the cache.  q [T, Hq, hd]; returns [T, Hq * hd].
    impl: "auto" (the fastest that fits), "tc" (tcgen05), "mma" (mma.sync), or "plain"."""
    _need(q, "q", k_pool.dtype, 3)
    _need(k_pool, "k_pool", ndim=4)
    _need(v_pool, "v_pool", k_pool.dtype, 4)
    _need(page_table, "page_table", torch.int32, 2)
    _need(cu_seqlens, "cu_seqlens", torch.int32, 1)
    _need(pos0, "pos0", torch.int32, 1)
    T, Hq, hd = q.shape
    B = pos0.numel()
    if cu_seqlens.numel() != B + 1 or page_table.shape[0] < B:
        raise KernelError("attn_prefill: cu_seqlens / page_table do not fit the batch")
    out = torch.empty((T, Hq * hd), dtype=q.dtype, device=q.device)
    group = Hq // max(1, k_pool.shape[1])
    # the tcgen05 kernel works on tiles of 128 rows: it pays from a few dozen new tokens per sequence on
    use_tc = impl == "tc" or (impl == "auto" and max_new * group >= 64 and
                              tc_attention_fits(q.dtype, hd, k_pool.shape[2], group))
    if use_tc:
        if q.dtype != torch.bfloat16:
            raise KernelError("attn_prefill: the tensor-core kernel takes bfloat16 only")
        _call("attention_tc", "qwb_attn_tc_prefill", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table),
              _ptr(cu_seqlens), _ptr(pos0), _ptr(out), _i(B), _i(T), _i(max_new), _i(k_pool.shape[0]), _i(Hq),
              _i(k_pool.shape[1]), _i(hd), _i(k_pool.shape[2]), _i(page_table.shape[1]), _f(scale), _i(window),
              _ptr(gemm_tc_error_word(q.device)), _stream())
        return out
    use_mma = impl == "mma" or (impl == "auto" and mma_attention_fits(q.dtype, hd, k_pool.shape[2]))
    if use_mma:
        if q.dtype != torch.bfloat16:
            raise KernelError("attn_prefill: the tensor-core kernel takes bfloat16 only")
        _call("attention_mma", "qwb_attn_mma_prefill", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table),
              _ptr(cu_seqlens), _ptr(pos0), _ptr(out), _i(B), _i(max_new), _i(Hq), _i(k_pool.shape[1]), _i(hd),
              _i(k_pool.shape[2]), _i(page_table.shape[1]), _f(scale), _i(window), _stream())
        return out
    _call("attention", "qwb_attn_prefill", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _ptr(cu_seqlens),
          _ptr(pos0), _ptr(out), _i(_dt(q.dtype)), _i(B), _i(max_new), _i(Hq), _i(k_pool.shape[1]), _i(hd),
          _i(k_pool.shape[2]), _i(page_table.shape[1]), _f(scale), _i(window), _stream())
    return out


def attn_decode_scratch_floats(B: int, Hq: int, hd: int, max_runs: int) -> int:
    return B * Hq * max_runs * (hd + 2)


MMA_RUNS_TARGET = 16        # the tensor-core decode kernel cuts a sequence into about this many runs of keys ...
MMA_RUN_PAGES_MAX = 8       # ... of at most this many pages each (more runs beyond that)


def mma_decode_runs(max_len: int, runs_target: int = MMA_RUNS_TARGET, run_pages_max: int = MMA_RUN_PAGES_MAX) -> int:
    """The most runs that the tensor-core decode kernel cuts a sequence of up to ``max_len`` keys into."""
    return int(load_module("attention_mma").qwb_attn_mma_decode_runs(_i(max_len), _i(runs_target), _i(run_pages_max)))


def attn_decode(q, k_pool, v_pool, page_table, seq_len, scale: float, max_len: int, window: int = 0,
                split_tokens: int = 256, scratch: torch.Tensor | None = None, impl: str = "auto",
                runs_target: int = MMA_RUNS_TARGET, run_pages_max: int = MMA_RUN_PAGES_MAX) -> torch.Tensor:
    """Attention of one new token per sequence over the cache.  q [B, Hq, hd]; ``seq_len`` counts
    the new token; ``max_len`` bounds every entry of ``seq_len``.  Returns [B, Hq * hd].

    The keys are cut into runs whose partial results are merged.  The plain kernel cuts into runs of
    ``split_tokens`` keys.  The tensor-core kernel cuts a sequence of p pages into runs of
    clamp(ceil(p / runs_target), 1, run_pages_max) pages (``runs_target`` 1: runs of exactly ``run_pages_max``
    pages): by the sequence's own length, never by what else is in the batch."""
    _need(q, "q", k_pool.dtype, 3)
    _need(k_pool, "k_pool", ndim=4)
    _need(v_pool, "v_pool", k_pool.dtype, 4)
    _need(page_table, "page_table", torch.int32, 2)
    _need(seq_len, "seq_len", torch.int32, 1)
    B, Hq, hd = q.shape
    use_mma = impl == "mma" or (impl == "auto" and mma_attention_fits(q.dtype, hd, k_pool.shape[2]))
    if use_mma and q.dtype != torch.bfloat16:
        raise KernelError("attn_decode: the tensor-core kernel takes bfloat16 only")
    if use_mma:
        max_runs = max(1, mma_decode_runs(max_len, runs_target, run_pages_max))
    else:
        max_runs = max(1, math.ceil(max_len / split_tokens))
    need = attn_decode_scratch_floats(B, Hq, hd, max_runs) if max_runs > 1 else 0
    if need and (scratch is None or scratch.numel() < need):
        scratch = torch.empty(need, dtype=torch.float32, device=q.device)
    if scratch is not None:
        _need(scratch, "scratch", torch.float32)
    out = torch.empty((B, Hq * hd), dtype=q.dtype, device=q.device)
    if use_mma:
        _call("attention_mma", "qwb_attn_mma_decode", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table),
              _ptr(seq_len), _ptr(scratch), _ptr(out), _i(B), _i(Hq), _i(k_pool.shape[1]), _i(hd), _i(k_pool.shape[2]),
              _i(page_table.shape[1]), _f(scale), _i(window), _i(runs_target), _i(run_pages_max), _i(max_len), _stream(),
              kernels=2 if max_runs > 1 else 1)
        return out
    _call("attention", "qwb_attn_decode", _ptr(q), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _ptr(seq_len),
          _ptr(scratch), _ptr(out), _i(_dt(q.dtype)), _i(B), _i(Hq), _i(k_pool.shape[1]), _i(hd),
          _i(k_pool.shape[2]), _i(page_table.shape[1]), _f(scale), _i(window), _i(split_tokens), _i(max_runs),
          _stream(), kernels=2 if max_runs > 1 else 1)
    return out


def attn_decode_fused(qkv: torch.Tensor, q_weight, k_weight, cos, sin, eps: float, k_pool, v_pool, page_table, seq_len,
                      scale: float, max_len: int, n_heads: int, n_kv_heads: int, head_dim: int, window: int = 0,
                      store_kv: bool = True, scratch: torch.Tensor | None = None,
                      runs_target: int = MMA_RUNS_TARGET, run_pages_max: int = MMA_RUN_PAGES_MAX) -> torch.Tensor:
    """``qk_norm_rope_store`` and ``attn_decode`` in one kernel, for a step of one token per sequence on the tensor-core
    path (bfloat16 cache, head size 64 or 128, rotation over the whole head or none): ``qkv`` float32
    [B, (Hq + 2 Hkv) * hd] is the q/k/v projection's output; the new keys and values are written into the cache at
    position ``seq_len - 1`` (unless ``store_kv`` is False).  Returns [B, Hq * hd] bfloat16."""
    _need(qkv, "qkv", torch.float32, 2)
    _need(k_pool, "k_pool", torch.bfloat16, 4)
    _need(v_pool, "v_pool", torch.bfloat16, 4)
    _need(page_table, "page_table", torch.int32, 2)
    _need(seq_len, "seq_len", torch.int32, 1)
    B = qkv.shape[0]
    if qkv.shape[1] != (n_heads + 2 * n_kv_heads) * head_dim or seq_len.numel() != B or page_table.shape[0] != B:
        raise KernelError(f"attn_decode_fused: qkv {tuple(qkv.shape)}, {seq_len.numel()} lengths, page table "
                          f"{tuple(page_table.shape)} do not fit {n_heads}+2x{n_kv_heads} heads of {head_dim}")
    if not mma_attention_fits(k_pool.dtype, head_dim, k_pool.shape[2]):
        raise KernelError(f"attn_decode_fused: head size {head_dim} with pages of {k_pool.shape[2]} is not taken")
    if tuple(k_pool.shape[1:]) != (n_kv_heads, k_pool.shape[2], head_dim) or v_pool.shape != k_pool.shape:
        raise KernelError(f"attn_decode_fused: cache pool {tuple(k_pool.shape)} does not fit {n_kv_heads} heads of {head_dim}")
    for name, t in (("q_weight", q_weight), ("k_weight", k_weight)):
        if t is not None:
            _need(t, name, torch.float32, 1)
            if t.numel() != head_dim:
                raise KernelError(f"attn_decode_fused: {name} has {t.numel()} entries for heads of {head_dim}")
    if (q_weight is None) != (k_weight is None):
        raise KernelError("attn_decode_fused: the norm weights of q and k come together")
    if cos is not None:
        _need(cos, "cos", torch.float32, 2)
        _need(sin, "sin", torch.float32, 2)
        if tuple(cos.shape) != (B, head_dim // 2) or sin.shape != cos.shape:
            raise KernelError(f"attn_decode_fused: cos/sin {tuple(cos.shape)} do not fit {B} tokens and a rotation "
                              f"over all {head_dim} values")
    max_runs = max(1, mma_decode_runs(max_len, runs_target, run_pages_max))
    need = attn_decode_scratch_floats(B, n_heads, head_dim, max_runs) if max_runs > 1 else 0
    if need and (scratch is None or scratch.numel() < need):
        scratch = torch.empty(need, dtype=torch.float32, device=qkv.device)
    out = torch.empty((B, n_heads * head_dim), dtype=torch.bfloat16, device=qkv.device)
    _call("attention_mma", "qwb_attn_mma_decode_fused", _ptr(qkv), _ptr(q_weight), _ptr(k_weight), _ptr(cos), _ptr(sin),
          _f(eps), _i(1 if store_kv else 0), _ptr(k_pool), _ptr(v_pool), _ptr(page_table), _ptr(seq_len), _ptr(scratch),
          _ptr(out), _i(B), _i(n_heads), _i(n_kv_heads), _i(head_dim), _i(k_pool.shape[2]), _i(page_table.shape[1]),
          _f(scale), _i(window), _i(runs_target), _i(run_pages_max), _i(max_len), _stream(),
          kernels=2 if max_runs > 1 else 1)
    return out


# ----------------------------------------------------------------------------- matrix products
SMALL_M = 16            # at most this many rows go to the weight-streaming kernel


def gemm_small(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor | None = None,
               out: torch.Tensor | None = None) -> torch.Tensor:
    """x [M, K] times weight [N, K] transposed, as float32 [M, N] (+ residual), for few rows."""
    _need(x, "x", weight.dtype, 2)
    _need(weight, "weight", ndim=2)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError(f"gemm_small: x has {K} columns, the weight {weight.shape[1]}")
    if out is None:
        out = residual if residual is not None else torch.empty((M, N), dtype=torch.float32, device=x.device)
    _need(out, "out", torch.float32, 2)
    if residual is not None:
        _need(residual, "residual", torch.float32, 2)
    _call("gemm_small", "qwb_gemm_small", _ptr(x), _ptr(weight), _ptr(residual), _ptr(out), _i(_dt(x.dtype)),
          _i(M), _i(N), _i(K), _stream(), kernels=(M + 7) // 8)
    return out


STREAM_M = 16           # at most this many bfloat16 rows go to the tensor-core weight-streaming kernel


STREAM_CONFIGS = ((2, 8), (4, 8), (8, 8), (2, 16), (4, 16), (2, 32))   # (blocks of 32 k in flight per warp, warps) that exist


def gemm_stream(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor | None = None,
                out: torch.Tensor | None = None, config: tuple | None = None) -> torch.Tensor:
    """bfloat16 x [M, K] times bfloat16 weight [N, K] transposed, as float32 [M, N] (+ residual), M <= 16.
    ``config``: one of ``STREAM_CONFIGS`` (default: the kernel's own choice by shape)."""
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError(f"gemm_stream: x has {K} columns, the weight {weight.shape[1]}")
    if out is None:
        out = residual if residual is not None else torch.empty((M, N), dtype=torch.float32, device=x.device)
    _need(out, "out", torch.float32, 2)
    if residual is not None:
        _need(residual, "residual", torch.float32, 2)
    u, w = config or (0, 0)
    _call("gemm_stream", "qwb_gemm_stream", _ptr(x), _ptr(weight), _ptr(residual), _ptr(out), _i(M), _i(N), _i(K),
          _i(u), _i(w), _stream())
    return out


def gemm_stream_swiglu(x: torch.Tensor, weight: torch.Tensor, config: tuple | None = None) -> torch.Tensor:
    """silu(x gate^T) * (x up^T) as bfloat16 [M, F] for bfloat16 x [M, K], M <= 16, and the weight [2F, K] with gate and up
    rows interleaved in groups of 8 features (``interleave_gate_up``)."""
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    M, K = x.shape
    if weight.shape[1] != K or weight.shape[0] % 2:
        raise KernelError(f"gemm_stream_swiglu: x is {tuple(x.shape)}, the weight {tuple(weight.shape)}")
    F = weight.shape[0] // 2
    out = torch.empty((M, F), dtype=torch.bfloat16, device=x.device)
    u, w = config or (0, 0)
    _call("gemm_stream", "qwb_gemm_stream_swiglu", _ptr(x), _ptr(weight), _ptr(out), _i(M), _i(F), _i(K), _i(u), _i(w), _stream())
    return out


RING_STAGE_K = 256              # k per stage of gemm_ring's ring; with 8 or 16 stages a row of W (rows of up to 2,048 or 4,096
RING_KEEPS_X_STAGES = (1, 2, 4, 8, 16)   # values) a warp meets the same k in every tile and keeps its pieces of x in registers


def gemm_ring(x: torch.Tensor, weight: torch.Tensor, residual: torch.Tensor | None = None,
              out: torch.Tensor | None = None) -> torch.Tensor:
    """As ``gemm_stream``, by the kernel that streams W through a ring in shared memory filled by bulk copies and is built
    to overlap with the kernels before and after it.  A wait that gave up shows in ``gemm_tc_check``."""
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError(f"gemm_ring: x has {K} columns, the weight {weight.shape[1]}")
    if out is None:
        out = residual if residual is not None else torch.empty((M, N), dtype=torch.float32, device=x.device)
    _need(out, "out", torch.float32, 2)
    if residual is not None:
        _need(residual, "residual", torch.float32, 2)
    _call("gemm_ring", "qwb_gemm_ring", _ptr(x), _ptr(weight), _ptr(residual), _ptr(out), _i(M), _i(N), _i(K),
          _ptr(gemm_tc_error_word(x.device)), _stream())
    return out


class SplitSum:
    """A product [T, D] that its kernel left as sums over pieces of k: ``planes`` float32 [P, T, D], of which columns
    16 t .. 16 t + 15 have ``plane_count[t]`` (uint8); the product is the sum of a column's planes in their order.
    The kernel that consumes it adds them (``rmsnorm`` does; ``add_onto`` for any other consumer)."""
    __slots__ = ("planes", "plane_count")

    def __init__(self, planes: torch.Tensor, plane_count: torch.Tensor):
        self.planes, self.plane_count = planes, plane_count

    def add_onto(self, x: torch.Tensor) -> torch.Tensor:
        """x += the product, in place."""
        _need(x, "x", torch.float32, 2)
        if tuple(self.planes.shape[1:]) != tuple(x.shape):
            raise KernelError(f"SplitSum: planes {tuple(self.planes.shape)} do not match x {tuple(x.shape)}")
        _call("elementwise", "qwb_add_planes", _ptr(x), _ptr(self.planes), _ptr(self.plane_count), _i(x.shape[0]),
              _i(x.shape[1]), _stream())
        return x

    def total(self) -> torch.Tensor:
        """The product as one tensor (a new one)."""
        return self.add_onto(torch.zeros(self.planes.shape[1:], dtype=torch.float32, device=self.planes.device))


RING_TILE_ROWS = 16             # rows of W per tile of gemm_ring
RING_SPLIT_MAX_PLANES = 4       # the most planes that the consumers of a SplitSum add
RING_SPLIT_BELOW = 0.8          # the split form is used when whole tiles would keep the SMs busy for less than this share of
                                # their rounds (5,120 rows on 148 SMs: 0.72, where it takes 16.0 and 42.4 us for the o and down
                                # projections of the Qwen3-32B sizes against 19.5 and 54.4 us; 4,096 rows: 0.86, where the
                                # pieces' extra epilogues cost what the even shares save: 7.8 and 18.2 against 6.9 and 18.8 us,
                                # and a step with the down projection alone split 2,457 against 2,485 tokens/s)
_RING_PLANS: dict = {}


def ring_split_plan(N: int, K: int, device):
    """How gemm_ring's split form cuts an [N, K] matrix on this device: ``(blocks, n_planes, plane_count)``, or None when
    whole tiles are as good (they fill the SMs' rounds to RING_SPLIT_BELOW or more, or a tile would be cut into more
    than RING_SPLIT_MAX_PLANES pieces).  Block b takes stages [b * all / blocks, (b + 1) * all / blocks) of the
    ceil(N / 16) * ceil(K / 256) stages, counted tile by tile; a tile's planes are the blocks that hold a part of it."""
    dev = torch.device(device)
    key = (N, K, dev.index or 0)
    if key not in _RING_PLANS:
        n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
        _RING_PLANS[key] = _ring_split_plan(N, K, n_sm, dev)
    return _RING_PLANS[key]


def ring_split_counts(N: int, K: int, blocks: int):
    """plane_count of every tile (a list), for ``blocks`` blocks: pure arithmetic, the same as the kernel's."""
    n_tiles, n_stages = -(-N // RING_TILE_ROWS), -(-K // RING_STAGE_K)
    all_stages = n_tiles * n_stages
    counts = []
    for t in range(n_tiles):
        first = ((t * n_stages + 1) * blocks - 1) // all_stages            # the block that holds the tile's first stage
        last = (((t + 1) * n_stages - 1 + 1) * blocks - 1) // all_stages   # ... and its last
        counts.append(last - first + 1)
    return counts


def _ring_split_plan(N: int, K: int, n_sm: int, device):
    n_tiles, n_stages = -(-N // RING_TILE_ROWS), -(-K // RING_STAGE_K)
    rounds = -(-n_tiles // n_sm)
    if n_tiles <= n_sm or n_tiles / (rounds * n_sm) >= RING_SPLIT_BELOW:
        return None
    counts = ring_split_counts(N, K, n_sm)
    if max(counts) > RING_SPLIT_MAX_PLANES:
        return None
    return n_sm, max(counts), torch.tensor(counts, dtype=torch.uint8, device=device)


def gemm_ring_split(x: torch.Tensor, weight: torch.Tensor, plan=None) -> SplitSum:
    """x W^T by the ring kernel's split form: every block streams an equal share of W and leaves its sums over pieces of
    tiles as planes (see ``SplitSum``).  ``plan``: from ``ring_split_plan`` (default: for this weight, which must have one)."""
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    M, K = x.shape
    N = weight.shape[0]
    if weight.shape[1] != K:
        raise KernelError(f"gemm_ring_split: x has {K} columns, the weight {weight.shape[1]}")
    if plan is None:
        plan = ring_split_plan(N, K, x.device)
        if plan is None:
            raise KernelError(f"gemm_ring_split: no split plan for a weight of {N} x {K}")
    blocks, n_planes, plane_count = plan
    planes = torch.empty((n_planes, M, N), dtype=torch.float32, device=x.device)
    _call("gemm_ring", "qwb_gemm_ring_split", _ptr(x), _ptr(weight), _ptr(planes), _i(M), _i(N), _i(K), _i(blocks),
          _ptr(gemm_tc_error_word(x.device)), _stream())
    return SplitSum(planes, plane_count)


def gemm_ring_swiglu(x: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """As ``gemm_stream_swiglu``, by the ring kernel (see ``gemm_ring``)."""
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    M, K = x.shape
    if weight.shape[1] != K or weight.shape[0] % 2:
        raise KernelError(f"gemm_ring_swiglu: x is {tuple(x.shape)}, the weight {tuple(weight.shape)}")
    F = weight.shape[0] // 2
    out = torch.empty((M, F), dtype=torch.bfloat16, device=x.device)
    _call("gemm_ring", "qwb_gemm_ring_swiglu", _ptr(x), _ptr(weight), _ptr(out), _i(M), _i(F), _i(K),
          _ptr(gemm_tc_error_word(x.device)), _stream())
    return out


_TC_ERROR: dict = {}    # device -> one int32 that a gemm_tc kernel sets when one of its waits gives up
TC_EPILOGUES = {"store": 0, "add": 1, "swiglu": 2}


def gemm_tc_error_word(device) -> torch.Tensor:
    key = torch.device(device).index or 0
    if key not in _TC_ERROR:
        _TC_ERROR[key] = torch.zeros((1,), dtype=torch.int32, device=device)
    return _TC_ERROR[key]


def gemm_tc_check(device) -> None:
    """Raise if a tcgen05 kernel (product or attention) on this device gave up a wait since the last check (reads one
    int: synchronises)."""
    word = gemm_tc_error_word(device)
    code = int(word.item())
    if code:
        word.zero_()
        where = {1: "the loader waiting for a free stage", 2: "the tensor-core issuer waiting for its operands",
                 3: "the epilogue or softmax warps waiting for the tensor core",
                 7: "shared memory was not aligned to 1024 bytes"}.get(code, f"code {code}")
        raise KernelError(f"a bounded wait in a tcgen05 kernel ran out ({where}); that kernel's result is not valid")


def gemm_tc(x: torch.Tensor, weight: torch.Tensor, epilogue: str = "store", out: torch.Tensor | None = None,
            tile_n: int | None = None) -> torch.Tensor:
    """bfloat16 x [M, K] times bfloat16 weight transposed on the tcgen05 tensor cores.

    "store": weight [N, K] -> float32 [M, N].  "add": the same, added onto ``out``.
    "swiglu": weight [2F, K] (gate and up rows interleaved in groups of 8 features, ``interleave_gate_up``)
    -> bfloat16 [M, F] = silu(gate) * up.
    """
    _need(x, "x", torch.bfloat16, 2)
    _need(weight, "weight", torch.bfloat16, 2)
    M, K = x.shape
    if weight.shape[1] != K:
        raise KernelError(f"gemm_tc: x has {K} columns, the weight {weight.shape[1]}")
    if epilogue not in TC_EPILOGUES:
        raise KernelError(f"gemm_tc: unknown epilogue '{epilogue}'")
    if epilogue == "swiglu":
        if weight.shape[0] % 2:
            raise KernelError(f"gemm_tc: {weight.shape[0]} rows cannot be split into gate and up")
        N = weight.shape[0] // 2
        out_dtype = torch.bfloat16
    else:
        N = weight.shape[0]
        out_dtype = torch.float32
    if out is None:
        if epilogue == "add":
            raise KernelError("gemm_tc: the 'add' epilogue needs the tensor to add onto")
        out = torch.empty((M, N), dtype=out_dtype, device=x.device)
    _need(out, "out", out_dtype, 2)
    if tuple(out.shape) != (M, N):
        raise KernelError(f"gemm_tc: out is {tuple(out.shape)}, expected {(M, N)}")
    if tile_n is None:
        tile_n = 128 if epilogue == "swiglu" else (128 if N >= 1024 else 64)
    _call("gemm_tc", "qwb_gemm_tc", _ptr(x), _ptr(weight), _ptr(out), _i(TC_EPILOGUES[epilogue]), _i(M), _i(N), _i(K),
          _i(tile_n), _ptr(gemm_tc_error_word(x.device)), _stream())
    return out


# ----------------------------------------------------------------------------- sampling
def sample(logits: torch.Tensor, temperature: float, top_k: int = 0, top_p: float = 1.0, seed: int = 0,
           sequence_index: torch.Tensor | None = None, step: int = 0, recent: torch.Tensor | None = None,
           repeat_penalty: float = 1.0, presence_penalty: float = 0.0, frequency_penalty: float = 0.0,
           out_u: torch.Tensor | None = None, step_add: torch.Tensor | None = None,
           out: torch.Tensor | None = None, split: bool = True, seed_from: torch.Tensor | None = None) -> torch.Tensor:
    """One token id per row of float32 ``logits`` [B, V] (changed in place by penalties).
    ``seed_from``: one int64 on the device that holds the seed (``seed`` is then not used); ``step_add``: one int32 on
    the device that is added to ``step``.  With both, a captured graph holds neither the seed nor the step.
    ``split`` False: one block per row whatever the sizes (the result is the same).  With few rows the kernels cut
    every row into chunks and count into one buffer per device: such calls must follow one another on one stream."""
    _need(logits, "logits", torch.float32, 2)
    B, V = logits.shape
    window = 0
    if recent is not None:
        _need(recent, "recent", torch.int32, 2)
        window = recent.shape[1]
    if sequence_index is not None:
        _need(sequence_index, "sequence_index", torch.int32, 1)
    if out_u is not None:
        _need(out_u, "out_u", torch.float64, 1)
    if seed_from is not None:
        _need(seed_from, "seed_from", torch.int64, 1)
    if out is None:
        out = torch.empty((B,), dtype=torch.int32, device=logits.device)
    # few rows and a small top-k: the kernels cut every row into chunks and want scratch memory for what the chunks find
    scratch_bytes = (_lookup("sampling", "qwb_sample_scratch_bytes")[1](_i(B), _i(V), _f(temperature), _i(top_k), _f(top_p))
                     if split else 0)
    scratch = counters = None
    if scratch_bytes:
        scratch = torch.empty((scratch_bytes,), dtype=torch.uint8, device=logits.device)
        if temperature > 0:
            counters = _sample_counters(logits.device, B)
    _call("sampling", "qwb_sample", _ptr(logits), _i(B), _i(V), _ptr(recent), _i(window), _f(repeat_penalty),
          _f(presence_penalty), _f(frequency_penalty), _f(temperature), _i(top_k), _f(top_p),
          ctypes.c_ulonglong(seed & (2 ** 64 - 1)), _ptr(seed_from), _ptr(sequence_index), ctypes.c_uint(step & 0xFFFFFFFF),
          _ptr(step_add), _ptr(out), _ptr(out_u), _ptr(scratch), _ptr(counters), _stream(),
          kernels=(3 if temperature > 0 else 2) if scratch_bytes else 1)
    return out


SAMPLE_SPLIT_MAX_ROWS = 592     # the split sampling kernels are used for fewer rows than this (four blocks an SM, two chunks a row)
_SAMPLE_COUNTERS: dict = {}     # device -> zeros [SAMPLE_SPLIT_MAX_ROWS * 1025]: the split sampling kernels count into them (a
                                # counter and 1,024 bins a row) and leave them zero; made once and kept, since captured
                                # graphs hold their address


def _sample_counters(device, rows: int) -> torch.Tensor:
    if rows > SAMPLE_SPLIT_MAX_ROWS:
        raise KernelError(f"sample: {rows} rows cannot be cut into chunks (at most {SAMPLE_SPLIT_MAX_ROWS})")
    key = torch.device(device).index or 0
    have = _SAMPLE_COUNTERS.get(key)
    if have is None:
        have = _SAMPLE_COUNTERS[key] = torch.zeros((SAMPLE_SPLIT_MAX_ROWS * 1025,), dtype=torch.int32, device=device)
    return have


def decode_advance(sampled, token_ids, tok_pos, pos0, seq_len, step_counter=None, recent=None, n_seen=None) -> None:
    """The sampled ids become the next inputs; positions and lengths go up by one."""
    B = sampled.numel()
    window = recent.shape[1] if recent is not None else 0
    _call("elementwise", "qwb_decode_advance", _ptr(sampled), _ptr(token_ids), _ptr(tok_pos), _ptr(pos0),
          _ptr(seq_len), _ptr(step_counter), _ptr(recent), _ptr(n_seen), _i(window), _i(B), _stream())
