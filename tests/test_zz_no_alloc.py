"""The entry point that allocates nothing: qwb_attn_decode_noalloc (csrc/attention_noalloc.h).

Some callers of the decode attention kernel cannot give it scratch memory, because they may not call an
allocator where they run: between the steps of a latency-critical loop (cudaMalloc stalls the device), in a
process that gave all device memory to a pool of its own, or as a plugin inside someone else's process.
For them the library has a variant whose scratch is a fixed 16 MiB array inside the loaded module.  This
test calls that variant through its exported C symbol, twice in a row with different inputs (the second
call finds the first call's leftovers in the array), and checks both results against the ordinary entry
point.  It also checks that a problem too large for the array is refused with a message.  The file is
named so that pytest collects it last.
"""
import ctypes
import math

import pytest
import torch

from questwend_b200.kernels import ops
from questwend_b200.kernels.build import load_module

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _inputs(seed, dtype, lens, Hq=8, Hkv=2, hd=64, page=64):
    g = torch.Generator().manual_seed(seed)
    n_pages = sum(-(-n // page) for n in lens) + 2
    k_pool = torch.randn(n_pages, Hkv, page, hd, generator=g).to(dtype).to(DEV)
    v_pool = torch.randn(n_pages, Hkv, page, hd, generator=g).to(dtype).to(DEV)
    order = torch.randperm(n_pages, generator=g).tolist()
    width = max(-(-n // page) for n in lens)
    table = torch.zeros(len(lens), width, dtype=torch.int32)
    for b, n in enumerate(lens):
        for p in range(-(-n // page)):
            table[b, p] = order.pop()
    q = torch.randn(len(lens), Hq, hd, generator=g).to(dtype).to(DEV)
    return q, k_pool, v_pool, table.to(DEV), torch.tensor(lens, dtype=torch.int32, device=DEV)


def _noalloc(lib, q, k_pool, v_pool, table, seq_len, scale, max_len, split):
    B, Hq, hd = q.shape
    out = torch.empty((B, Hq * hd), dtype=q.dtype, device=q.device)
    max_runs = max(1, math.ceil(max_len / split))
    p = lambda t: ctypes.c_void_p(t.data_ptr())
    rc = lib.qwb_attn_decode_noalloc(p(q), p(k_pool), p(v_pool), p(table), p(seq_len), p(out),
                                     ctypes.c_int(0 if q.dtype == torch.float32 else 1), ctypes.c_int(B),
                                     ctypes.c_int(Hq), ctypes.c_int(k_pool.shape[1]), ctypes.c_int(hd),
                                     ctypes.c_int(k_pool.shape[2]), ctypes.c_int(table.shape[1]), ctypes.c_float(scale),
                                     ctypes.c_int(0), ctypes.c_int(split), ctypes.c_int(max_runs),
                                     ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
    return rc, out


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_two_calls_in_a_row_match_the_ordinary_entry_point(dtype):
    lib = load_module("attention")
    lib.qwb_attn_decode_noalloc_capacity.restype = ctypes.c_longlong
    assert lib.qwb_attn_decode_noalloc_capacity() == 4 * 1024 * 1024
    tol = 5e-6 if dtype == torch.float32 else 2.0 ** -7
    for seed, lens in ((1, [700, 130, 64, 1]), (2, [300, 650, 90])):          # several runs per sequence
        q, k_pool, v_pool, table, seq_len = _inputs(seed, dtype, lens)
        scale = 1 / math.sqrt(q.shape[-1])
        want = ops.attn_decode(q, k_pool, v_pool, table, seq_len, scale, max(lens), split_tokens=128)
        rc, got = _noalloc(lib, q, k_pool, v_pool, table, seq_len, scale, max(lens), 128)
        torch.cuda.synchronize()
        assert rc == 0, lib.qwb_last_error().decode()
        err = (got.double() - want.double()).abs().max().item() / want.double().abs().max().item()
        assert err <= tol


def test_a_problem_beyond_the_array_is_refused():
    lib = load_module("attention")
    q, k_pool, v_pool, table, seq_len = _inputs(3, torch.float32, [100, 100], Hq=8, Hkv=2, hd=64)
    rc, _ = _noalloc(lib, q, k_pool, v_pool, table, seq_len, 1.0, 64 * 4 * 1024 * 1024, 64)   # an absurd bound on the length
    assert rc != 0
    msg = lib.qwb_last_error().decode()
    assert "built-in array holds" in msg and "scratch of your own" in msg


def test_too_few_runs_cut_the_sequence_and_touch_nothing_beyond_the_scratch():
    """``max_runs`` must cover the longest sequence; the lengths are on the device, so the launcher cannot check that.  A
    caller that gives too few gets the attention over the first ``max_runs`` runs of keys, not a read or write beyond
    the scratch that it sized by ``max_runs``."""
    lib = load_module("attention")
    q, k_pool, v_pool, table, seq_len = _inputs(4, torch.float32, [300, 40])
    scale = 1 / math.sqrt(q.shape[-1])
    rc, got = _noalloc(lib, q, k_pool, v_pool, table, seq_len, scale, 256, 128)          # 2 runs where 300 keys need 3
    torch.cuda.synchronize()
    assert rc == 0, lib.qwb_last_error().decode()
    cut = torch.tensor([256, 40], dtype=torch.int32, device=DEV)
    want = ops.attn_decode(q, k_pool, v_pool, table, cut, scale, 256, split_tokens=128)
    assert (got - want).abs().max().item() <= 5e-6 * want.abs().max().item()
