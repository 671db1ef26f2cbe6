"""Each kernel alone against a plain reference of the same operation, at sizes other than the
engine's (needs a B200)."""
import math

import numpy as np
import pytest
import torch

import plain_model as pm
from questwend_b200.kernels import ops
from questwend_b200.kernels.ops import KernelError

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = [torch.float32, torch.bfloat16]


def tol(dtype):
    return 5e-6 if dtype == torch.float32 else 2.0 ** -7


def close(got, ref, dtype, scale=None):
    got = got.detach().to(torch.float64).cpu().numpy()
    ref = np.asarray(ref, dtype=np.float64)
    s = np.abs(ref).max() if scale is None else scale
    err = np.abs(got - ref).max() / s
    assert err <= tol(dtype), f"relative error {err:.3e} above {tol(dtype):.1e}"


def f64(t):
    return t.detach().to(torch.float64).cpu().numpy()


# ----------------------------------------------------------------------------- elementwise
@pytest.mark.parametrize("dtype", DTYPES)
def test_embed_gather(dtype):
    g = torch.Generator().manual_seed(0)
    table = torch.randn(37, 100, generator=g).to(dtype).to(DEV)
    ids = torch.tensor([5, 0, 36, 5, 17], dtype=torch.int32, device=DEV)
    out = ops.embed_gather(ids, table)
    assert out.dtype == torch.float32 and torch.equal(out, table[ids.long()].float())
    bad = torch.full((1,), -1, dtype=torch.int32, device=DEV)
    out = ops.embed_gather(torch.tensor([1, 99, 2], dtype=torch.int32, device=DEV), table, bad_token=bad)
    assert int(bad) == 1 and float(out[1].abs().sum()) == 0.0


@pytest.mark.parametrize("D", [100, 1000, 4100, 13000])
@pytest.mark.parametrize("out_dtype", DTYPES)
def test_rmsnorm(D, out_dtype):
    g = torch.Generator().manual_seed(D)
    x = (torch.randn(7, D, generator=g) * 3).to(DEV)
    delta = torch.randn(7, D, generator=g).to(DEV)
    w = (1 + 0.1 * torch.randn(D, generator=g)).to(DEV)
    eps = 1e-5
    close(ops.rmsnorm(x, w, eps, out_dtype), pm.rms_norm(f64(x), f64(w), eps), out_dtype)
    x2 = x.clone()
    out = ops.rmsnorm(x2, w, eps, out_dtype, delta=delta, write_sum=True)
    assert torch.equal(x2, x + delta)                                  # the residual sum, in 32-bit
    close(out, pm.rms_norm(f64(x) + f64(delta), f64(w), eps), out_dtype)
    x3 = x.clone()
    rows = torch.tensor([6, 0, 3], dtype=torch.int32, device=DEV)
    out = ops.rmsnorm(x3, w, eps, out_dtype, delta=delta, rows=rows)
    assert torch.equal(x3, x) and out.shape == (3, D)
    close(out, pm.rms_norm((f64(x) + f64(delta))[[6, 0, 3]], f64(w), eps), out_dtype)


def test_rmsnorm_refuses_a_row_that_does_not_fit():
    with pytest.raises(KernelError, match="shared memory"):
        ops.rmsnorm(torch.zeros(1, 60000, device=DEV), torch.ones(60000, device=DEV), 1e-6, torch.float32)
    with pytest.raises(KernelError, match="CUDA"):
        ops.rmsnorm(torch.zeros(1, 8), torch.ones(8), 1e-6, torch.float32)


@pytest.mark.parametrize("out_dtype", DTYPES)
def test_silu_mul(out_dtype):
    gu = (torch.randn(5, 2 * 77, generator=torch.Generator().manual_seed(1)) * 4).to(DEV)
    close(ops.silu_mul(gu, out_dtype), pm.swiglu(f64(gu)[:, :77], f64(gu)[:, 77:]), out_dtype)
    # the same with gates and ups interleaved in groups of 7 features
    inter = gu.reshape(5, 2, 11, 7).permute(0, 2, 1, 3).reshape(5, 2 * 77).contiguous()
    assert torch.equal(ops.silu_mul(inter, out_dtype, interleave=7), ops.silu_mul(gu, out_dtype))
    with pytest.raises(KernelError, match="interleaved"):
        ops.silu_mul(gu, out_dtype, interleave=8)
    # in eights, the layout of the fused products (a kernel of its own: a thread takes 8 features), many rows and few
    for T, F in ((5, 80), (70, 1000)):
        gu8 = (torch.randn(T, 2 * F, generator=torch.Generator().manual_seed(T)) * 4).to(DEV)
        inter8 = gu8.reshape(T, 2, F // 8, 8).permute(0, 2, 1, 3).reshape(T, 2 * F).contiguous()
        got = ops.silu_mul(inter8, out_dtype, interleave=8)
        close(got, pm.swiglu(f64(gu8)[:, :F], f64(gu8)[:, F:]), out_dtype)
        assert torch.equal(got, ops.silu_mul(gu8, out_dtype))


def test_add_inplace_and_decode_advance():
    a, b = torch.randn(3, 11, device=DEV), torch.randn(3, 11, device=DEV)
    want = a + b
    assert torch.equal(ops.add_inplace(a, b), want)
    sampled = torch.tensor([7, 8, 9], dtype=torch.int32, device=DEV)
    st = [torch.tensor(v, dtype=torch.int32, device=DEV) for v in ([1, 2, 3], [10, 20, 30], [10, 20, 30], [11, 21, 31])]
    counter = torch.tensor([4], dtype=torch.int32, device=DEV)
    recent = torch.full((3, 2), -1, dtype=torch.int32, device=DEV)
    n_seen = torch.tensor([0, 1, 5], dtype=torch.int32, device=DEV)
    ops.decode_advance(sampled, *st, step_counter=counter, recent=recent, n_seen=n_seen)
    assert st[0].tolist() == [7, 8, 9] and st[1].tolist() == [11, 21, 31] and st[3].tolist() == [12, 22, 32]
    assert int(counter) == 5 and recent.tolist() == [[7, -1], [-1, 8], [-1, 9]] and n_seen.tolist() == [1, 2, 6]


# ----------------------------------------------------------------------------- rotation and cache write
def test_rope_table_keeps_digits_at_far_positions():
    pos = torch.tensor([0, 1, 4095, 131071, 1000003], dtype=torch.int32, device=DEV)
    inv = (1e6 ** (-2.0 * torch.arange(24, dtype=torch.float64) / 48)).to(DEV)
    cos, sin = ops.rope_table(pos, inv)
    ang = pm.rope_angles(pos.cpu().numpy(), 48, 1e6)
    assert np.abs(f64(cos) - np.cos(ang)).max() < 1e-7 and np.abs(f64(sin) - np.sin(ang)).max() < 1e-7


def paged(dense, n_kv_heads, head_dim, dtype, page_size=64, seed=0, extra_pages=3):
    """Put per-sequence [len, Hkv, hd] arrays into a pool with shuffled page ids; returns pool, table."""
    n_pages = sum(-(-len(d) // page_size) for d in dense) + extra_pages
    order = np.random.default_rng(seed).permutation(n_pages)
    pool = torch.full((n_pages, n_kv_heads, page_size, head_dim), 1e4, dtype=dtype)   # junk where nothing is stored
    width = max(-(-len(d) // page_size) for d in dense) + 1
    table = np.zeros((len(dense), width), dtype=np.int32)
    nxt = 0
    for b, d in enumerate(dense):
        for p in range(-(-len(d) // page_size)):
            pid = int(order[nxt]); nxt += 1
            table[b, p] = pid
            chunk = torch.as_tensor(d[p * page_size:(p + 1) * page_size]).to(dtype)    # [n, Hkv, hd]
            pool[pid, :, :chunk.shape[0]] = chunk.permute(1, 0, 2)
    return pool.to(DEV), torch.from_numpy(table).to(DEV)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,hd,rot,norm", [(5, 1, 48, 32, True), (4, 2, 16, 16, True), (3, 3, 80, 80, False),
                                                (2, 1, 32, 0, True), (6, 2, 128, 128, True), (3, 1, 128, 128, False),
                                                (2, 2, 128, 64, True)])
def test_qk_norm_rope_store(dtype, Hq, Hkv, hd, rot, norm):
    rng = np.random.default_rng(hd)
    page = 64
    # two sequences: tokens at positions 60..69 of row 0 (crossing a page edge) and 0..2 of row 1
    tok_seq = np.array([0] * 10 + [1] * 3, dtype=np.int32)
    tok_pos = np.array(list(range(60, 70)) + [0, 1, 2], dtype=np.int32)
    T = len(tok_seq)
    qkv = rng.normal(size=(T, (Hq + 2 * Hkv) * hd)).astype(np.float32)
    qw = (1 + 0.1 * rng.normal(size=hd)).astype(np.float32) if norm else None
    kw = (1 + 0.1 * rng.normal(size=hd)).astype(np.float32) if norm else None
    eps = 1e-5
    table = torch.tensor([[4, 1, 0], [2, 0, 0]], dtype=torch.int32, device=DEV)
    k_pool = torch.full((6, Hkv, page, hd), 777.0, dtype=dtype, device=DEV)
    v_pool = torch.full((6, Hkv, page, hd), 777.0, dtype=dtype, device=DEV)
    cos = sin = None
    if rot:
        inv = (1e4 ** (-2.0 * torch.arange(rot // 2, dtype=torch.float64) / rot)).to(DEV)
        cos, sin = ops.rope_table(torch.from_numpy(tok_pos).to(DEV), inv)
    dev = lambda a: None if a is None else torch.from_numpy(a).to(DEV)
    q_out = ops.qk_norm_rope_store(dev(qkv), dev(qw), dev(kw), cos, sin, dev(tok_seq), dev(tok_pos), table, k_pool, v_pool,
                                   Hq, Hkv, hd, rot, eps)
    x = qkv.astype(np.float64)
    q = x[:, :Hq * hd].reshape(T, Hq, hd)
    k = x[:, Hq * hd:(Hq + Hkv) * hd].reshape(T, Hkv, hd)
    v = x[:, (Hq + Hkv) * hd:].reshape(T, Hkv, hd)
    if norm:
        q, k = pm.rms_norm(q, qw.astype(np.float64), eps), pm.rms_norm(k, kw.astype(np.float64), eps)
    if rot:
        ang = pm.rope_angles(tok_pos, rot, 1e4)
        q, k = pm.apply_rope_neox(q, ang, rot), pm.apply_rope_neox(k, ang, rot)
    close(q_out, q, dtype)
    for t in range(T):
        pid = int(table[tok_seq[t], tok_pos[t] // page])
        close(k_pool[pid, :, tok_pos[t] % page], k[t], dtype, scale=np.abs(k).max())
        close(v_pool[pid, :, tok_pos[t] % page], v[t], dtype, scale=np.abs(v).max())
    written = torch.zeros_like(k_pool, dtype=torch.bool)
    for t in range(T):
        written[int(table[tok_seq[t], tok_pos[t] // page]), :, tok_pos[t] % page] = True
    assert bool((k_pool[~written] == 777.0).all()) and bool((v_pool[~written] == 777.0).all())
    # a run that reads another run's cache stores nothing
    k2 = torch.full_like(k_pool, 5.0)
    ops.qk_norm_rope_store(dev(qkv), dev(qw), dev(kw), cos, sin, dev(tok_seq), dev(tok_pos), table, k2, k2.clone(),
                           Hq, Hkv, hd, rot, eps, store_kv=False)
    assert bool((k2 == 5.0).all())


# ----------------------------------------------------------------------------- attention
ATTN_SHAPES = [(4, 2, 16), (6, 1, 32), (3, 3, 48), (8, 2, 64), (8, 1, 128), (2, 1, 256), (12, 1, 16)]


def make_qkv(lens, Hq, Hkv, hd, seed):
    rng = np.random.default_rng(seed)
    q = [rng.normal(size=(n, Hq, hd)) for n in lens]
    k = [rng.normal(size=(n, Hkv, hd)) for n in lens]
    v = [rng.normal(size=(n, Hkv, hd)) for n in lens]
    return q, k, v


def rounded(arrs, dtype):
    return [pm.round_bf16(a) if dtype == torch.bfloat16 else a for a in arrs]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,hd", ATTN_SHAPES)
@pytest.mark.parametrize("window", [0, 37])
def test_attn_prefill(dtype, Hq, Hkv, hd, window):
    _attn_prefill_case(dtype, Hq, Hkv, hd, window, "plain")


@pytest.mark.parametrize("Hq,Hkv,hd", [(8, 2, 64), (8, 1, 128), (4, 4, 128), (12, 1, 64), (32, 1, 128), (6, 2, 128)])
@pytest.mark.parametrize("window", [0, 37])
def test_attn_prefill_tensor_cores(Hq, Hkv, hd, window):
    _attn_prefill_case(torch.bfloat16, Hq, Hkv, hd, window, "mma")


@pytest.mark.parametrize("Hq,Hkv,hd", [(8, 2, 64), (8, 1, 128), (4, 4, 128), (16, 1, 64), (32, 8, 128), (4, 2, 128),
                                       # heads per key/value head that do not divide the block's 128 rows
                                       (6, 2, 128), (40, 8, 128), (7, 1, 64), (12, 1, 64), (33, 1, 128)])
@pytest.mark.parametrize("window", [0, 37])
def test_attn_prefill_tcgen05(Hq, Hkv, hd, window):
    _attn_prefill_case(torch.bfloat16, Hq, Hkv, hd, window, "tc")
    ops.gemm_tc_check(DEV)


def _attn_prefill_case(dtype, Hq, Hkv, hd, window, impl):
    lens = [1, 17, 70, 150, 64]
    new = [1, 17, 33, 22, 64]                       # the last `new` tokens of each sequence are this step's
    q, k, v = (rounded(a, dtype) for a in make_qkv(lens, Hq, Hkv, hd, hd + Hq))
    k_pool, table = paged(k, Hkv, hd, dtype, seed=1)
    v_pool, _ = paged(v, Hkv, hd, dtype, seed=1)
    q_new = torch.cat([torch.as_tensor(qq[n - m:]) for qq, n, m in zip(q, lens, new)]).to(dtype).to(DEV)
    cu = torch.tensor(np.cumsum([0] + new), dtype=torch.int32, device=DEV)
    pos0 = torch.tensor([n - m for n, m in zip(lens, new)], dtype=torch.int32, device=DEV)
    out = ops.attn_prefill(q_new, k_pool, v_pool, table, cu, pos0, max(new), 1 / math.sqrt(hd), window=window, impl=impl)
    ref = np.concatenate([pm.attention_causal(qq, kk, vv, window=window or None)[n - m:].reshape(m, Hq * hd)
                          for qq, kk, vv, n, m in zip(q, k, v, lens, new)])
    close(out, ref, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("Hq,Hkv,hd", ATTN_SHAPES)
@pytest.mark.parametrize("window,split,page", [(0, 128, 64), (100, 64, 64), (0, 256, 64), (0, 128, 32), (50, 64, 16),
                                               (0, 128, 128)])
def test_attn_decode(dtype, Hq, Hkv, hd, window, split, page):
    _attn_decode_case(dtype, Hq, Hkv, hd, window, split, page, "plain")


@pytest.mark.parametrize("Hq,Hkv,hd", [(8, 2, 64), (8, 1, 128), (4, 4, 128), (12, 1, 64), (32, 1, 128), (6, 2, 128)])
@pytest.mark.parametrize("window,runs_target,run_pages_max", [
    (0, 1, 2), (100, 1, 1), (0, 1, 1), (0, 1, 4), (0, 1, 8), (300, 1, 4),      # runs of a fixed number of pages
    (0, 16, 8), (0, 4, 2), (100, 3, 8), (0, 2, 1), (0, 5, 3)])                  # by the sequence's length
def test_attn_decode_tensor_cores(Hq, Hkv, hd, window, runs_target, run_pages_max):
    _attn_decode_case(torch.bfloat16, Hq, Hkv, hd, window, 64 * run_pages_max, 64, "mma",
                      dict(runs_target=runs_target, run_pages_max=run_pages_max))


@pytest.mark.parametrize("Hq,Hkv,hd", [(8, 2, 128), (4, 4, 64)])
def test_attn_decode_merges_many_runs(Hq, Hkv, hd):
    """The merge of the runs' partial results with 18 runs (more than the 16 whose loads make one round) and 35 (more than
    a warp has lanes), beside a sequence of one run: runs of one page, sequences of 1,100, 2,200 and 40 keys."""
    lens = [1100, 2200, 40]
    q, k, v = (rounded(a, torch.bfloat16) for a in make_qkv(lens, Hq, Hkv, hd, 7))
    k_pool, table = paged(k, Hkv, hd, torch.bfloat16, seed=3)
    v_pool, _ = paged(v, Hkv, hd, torch.bfloat16, seed=3)
    q_last = torch.stack([torch.as_tensor(qq[-1]) for qq in q]).to(torch.bfloat16).to(DEV)
    seq_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    out = ops.attn_decode(q_last, k_pool, v_pool, table, seq_len, 1 / math.sqrt(hd), max(lens), impl="mma", runs_target=1,
                          run_pages_max=1)
    ref = np.stack([pm.attention_causal(qq, kk, vv)[-1].reshape(Hq * hd) for qq, kk, vv in zip(q, k, v)])
    close(out, ref, torch.bfloat16)
    alone = ops.attn_decode(q_last[1:2], k_pool, v_pool, table[1:2], seq_len[1:2], 1 / math.sqrt(hd), 4096, impl="mma",
                            runs_target=1, run_pages_max=1)
    assert torch.equal(alone[0], out[1])


def test_attn_decode_runs_by_length():
    """How the tensor-core kernel cuts a sequence of p pages: clamp(ceil(p / target), 1, most) pages a run."""
    def runs(pages, target, most):
        per = min(most, max(1, -(-pages // target)))
        return -(-pages // per)
    for target, most in ((16, 8), (1, 4), (3, 2), (5, 1)):
        for max_pages in (1, 2, 15, 16, 17, 31, 33, 128, 129, 1000):
            want = max(runs(p, target, most) for p in range(1, max_pages + 1))
            assert ops.mma_decode_runs(64 * max_pages, target, most) == want
            assert ops.mma_decode_runs(64 * max_pages - 63, target, most) == want


def _attn_decode_case(dtype, Hq, Hkv, hd, window, split, page, impl, how=None):
    how = dict(split_tokens=split) if how is None else how
    if page == 128 and hd == 256 and dtype == torch.float32:
        pytest.skip("refused: see test_attention_refusals")
    lens = [1, 64, 65, 300, 129, 700]
    q, k, v = (rounded(a, dtype) for a in make_qkv(lens, Hq, Hkv, hd, hd + split))
    k_pool, table = paged(k, Hkv, hd, dtype, page_size=page, seed=2)
    v_pool, _ = paged(v, Hkv, hd, dtype, page_size=page, seed=2)
    q_last = torch.stack([torch.as_tensor(qq[-1]) for qq in q]).to(dtype).to(DEV)
    seq_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    out = ops.attn_decode(q_last, k_pool, v_pool, table, seq_len, 1 / math.sqrt(hd), max(lens), window=window,
                          impl=impl, **how)
    ref = np.stack([pm.attention_causal(qq, kk, vv, window=window or None)[-1].reshape(Hq * hd)
                    for qq, kk, vv in zip(q, k, v)])
    close(out, ref, dtype)
    # more runs than the longest sequence needs (a graph's bucket) change nothing
    again = ops.attn_decode(q_last, k_pool, v_pool, table, seq_len, 1 / math.sqrt(hd), max(lens) + 3 * split,
                            window=window, impl=impl, **how)
    assert torch.equal(out, again)
    # a sequence's result does not depend on the rest of the batch
    alone = ops.attn_decode(q_last[3:4], k_pool, v_pool, table[3:4], seq_len[3:4], 1 / math.sqrt(hd), lens[3],
                            window=window, impl=impl, **how)
    assert torch.equal(alone[0], out[3])


@pytest.mark.parametrize("Hq,Hkv,hd", [(8, 2, 128), (4, 4, 64), (32, 1, 128), (6, 2, 64)])
@pytest.mark.parametrize("norm,rotate,window", [(True, True, 0), (False, True, 0), (True, False, 90), (False, False, 0)])
def test_attn_decode_with_norm_rotation_and_cache_write_inside(Hq, Hkv, hd, norm, rotate, window):
    """The kernel that does the q/k norm, the rotation and the cache write itself against the two kernels it replaces:
    the same attention output, and the same new keys and values in the cache (also where the new token opens a page)."""
    lens = [1, 64, 65, 300, 129, 700, 128]
    B = len(lens)
    rng = np.random.default_rng(Hq + hd)
    _, k, v = (rounded(a, torch.bfloat16) for a in make_qkv(lens, Hq, Hkv, hd, hd + Hq))
    k_pool, table = paged(k, Hkv, hd, torch.bfloat16, seed=4)
    v_pool, _ = paged(v, Hkv, hd, torch.bfloat16, seed=4)
    qkv = torch.from_numpy(rng.normal(size=(B, (Hq + 2 * Hkv) * hd)).astype(np.float32)).to(DEV)
    qw = torch.from_numpy(1 + 0.1 * rng.normal(size=hd).astype(np.float32)).to(DEV) if norm else None
    kw = torch.from_numpy(1 + 0.1 * rng.normal(size=hd).astype(np.float32)).to(DEV) if norm else None
    seq_len = torch.tensor(lens, dtype=torch.int32, device=DEV)
    tok_seq = torch.arange(B, dtype=torch.int32, device=DEV)
    tok_pos = (seq_len - 1).contiguous()
    cos = sin = None
    if rotate:
        inv = torch.tensor(1e4 ** (-2.0 * np.arange(hd // 2) / hd), dtype=torch.float64, device=DEV)
        cos, sin = ops.rope_table(tok_pos, inv)
    scale = 1 / math.sqrt(hd)
    k1, v1 = k_pool.clone(), v_pool.clone()
    q = ops.qk_norm_rope_store(qkv, qw, kw, cos, sin, tok_seq, tok_pos, table, k1, v1, Hq, Hkv, hd, hd if rotate else 0, 1e-5)
    want = ops.attn_decode(q, k1, v1, table, seq_len, scale, max(lens), window=window)
    k2, v2 = k_pool.clone(), v_pool.clone()
    got = ops.attn_decode_fused(qkv, qw, kw, cos, sin, 1e-5, k2, v2, table, seq_len, scale, max(lens), Hq, Hkv, hd, window=window)
    close(got, f64(want), torch.bfloat16)
    assert (f64(k2) - f64(k1)).__abs__().max() <= 2.0 ** -7 * np.abs(f64(k1)[f64(k1) < 1e3]).max()     # a bfloat16 step at most
    assert torch.equal(v2, v1)
    # the cache of another layer's run is read, not written
    k3, v3 = k1.clone(), v1.clone()
    again = ops.attn_decode_fused(qkv, qw, kw, cos, sin, 1e-5, k3, v3, table, seq_len, scale, max(lens), Hq, Hkv, hd,
                                  window=window, store_kv=False)
    assert torch.equal(k3, k1) and torch.equal(v3, v1)
    close(again, f64(want), torch.bfloat16)


@pytest.mark.parametrize("dtype", DTYPES)
def test_one_far_key_among_hundreds(dtype):
    """Random scores hide a key that is read from the wrong place: make one far key's score stand out,
    so that the output must be that key's value."""
    Hq, Hkv, hd, n = 4, 2, 64, 900
    for far in (3, 63, 64, 511, 640):
        q, k, v = make_qkv([n], Hq, Hkv, hd, far)
        q[0][-1] = 0.0
        q[0][-1, :, 5] = 30.0
        k[0][:, :, 5] = 0.0
        k[0][far, :, 5] = 30.0                       # score 900/8 above every other key's
        q, k, v = (rounded(a, dtype) for a in (q, k, v))
        k_pool, table = paged(k, Hkv, hd, dtype, seed=far)
        v_pool, _ = paged(v, Hkv, hd, dtype, seed=far)
        want = np.stack([v[0][far, h // 2] for h in range(Hq)]).reshape(1, Hq * hd)
        seq_len = torch.tensor([n], dtype=torch.int32, device=DEV)
        out = ops.attn_decode(torch.as_tensor(q[0][-1:]).to(dtype).to(DEV), k_pool, v_pool, table, seq_len,
                              1 / math.sqrt(hd), n, split_tokens=128)
        close(out, want, dtype)
        out = ops.attn_prefill(torch.as_tensor(q[0][-5:]).to(dtype).to(DEV), k_pool, v_pool, table,
                               torch.tensor([0, 5], dtype=torch.int32, device=DEV),
                               torch.tensor([n - 5], dtype=torch.int32, device=DEV), 5, 1 / math.sqrt(hd))
        close(out[-1:], want, dtype)


def test_window_edge():
    """With a window of w the key at distance w is hidden and the key at distance w - 1 is seen."""
    Hq = Hkv = 1
    hd, n, w = 16, 200, 70
    q, k, v = make_qkv([n], Hq, Hkv, hd, 9)
    q[0][-1] = 0.0
    q[0][-1, :, 0] = 20.0
    k[0][:, :, 0] = 0.0
    for dist, seen in ((w, False), (w - 1, True)):
        kk = [k[0].copy()]
        kk[0][n - 1 - dist, :, 0] = 20.0
        k_pool, table = paged(kk, Hkv, hd, torch.float32)
        v_pool, _ = paged(v, Hkv, hd, torch.float32)
        seq_len = torch.tensor([n], dtype=torch.int32, device=DEV)
        qd = torch.as_tensor(q[0][-1:]).float().to(DEV)
        out_d = ops.attn_decode(qd, k_pool, v_pool, table, seq_len, 1.0, n, window=w, split_tokens=64)
        out_p = ops.attn_prefill(qd, k_pool, v_pool, table, torch.tensor([0, 1], dtype=torch.int32, device=DEV),
                                 torch.tensor([n - 1], dtype=torch.int32, device=DEV), 1, 1.0, window=w)
        target = v[0][n - 1 - dist, 0]
        for out in (out_d, out_p):
            hit = np.abs(f64(out)[0] - target).max() < 1e-3
            assert hit == seen


def test_attention_refusals():
    q = torch.zeros(1, 4, 24, device=DEV)
    pool = torch.zeros(2, 2, 64, 24, device=DEV)
    table = torch.zeros(1, 2, dtype=torch.int32, device=DEV)
    one = torch.ones(1, dtype=torch.int32, device=DEV)
    with pytest.raises(KernelError, match="multiple of 16"):
        ops.attn_decode(q, pool, pool, table, one, 1.0, 1)
    with pytest.raises(KernelError, match="multiple of 16"):
        ops.attn_prefill(q, pool, pool, table, torch.tensor([0, 1], dtype=torch.int32, device=DEV), one, 1, 1.0)
    q = torch.zeros(1, 3, 32, device=DEV)
    pool = torch.zeros(2, 2, 64, 32, device=DEV)
    with pytest.raises(KernelError, match="not a multiple"):
        ops.attn_decode(q, pool, pool, table, one, 1.0, 1)
    q = torch.zeros(1, 1, 256, device=DEV)
    pool = torch.zeros(2, 1, 128, 256, device=DEV)
    with pytest.raises(KernelError, match="shared memory"):
        ops.attn_decode(q, pool, pool, table, one, 1.0, 1)
    pool = torch.zeros(2, 1, 48, 256, device=DEV)
    with pytest.raises(KernelError, match="page size"):
        ops.attn_decode(q, pool, pool, table, one, 1.0, 1)


# ----------------------------------------------------------------------------- matrix product for few rows
@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("M", [1, 2, 3, 5, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(37, 96), (200, 200), (11, 100), (5, 4100)])
def test_gemm_small(dtype, M, N, K):
    g = torch.Generator().manual_seed(M * 1000 + K)
    x = torch.randn(M, K, generator=g).to(dtype).to(DEV)
    w = torch.randn(N, K, generator=g).to(dtype).to(DEV)
    ref = f64(x) @ f64(w).T
    out = ops.gemm_small(x, w)
    assert out.dtype == torch.float32
    close(out, ref, torch.float32, scale=np.abs(ref).max() * 4)          # 32-bit sums of exact products
    res = torch.randn(M, N, generator=g).to(DEV)
    want = f64(res) + ref
    close(ops.gemm_small(x, w, residual=res.clone()), want, torch.float32, scale=np.abs(want).max() * 4)
    # a row's result does not depend on how many rows come with it
    assert torch.equal(ops.gemm_small(x[:1], w)[0], out[0])


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(37, 96), (200, 200), (16, 4104), (129, 1024), (5000, 8200)])
def test_gemm_stream(M, N, K):
    g = torch.Generator().manual_seed(M * 1000 + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16).to(DEV)
    ref = f64(x) @ f64(w).T
    out = ops.gemm_stream(x, w)
    close(out, ref, torch.float32, scale=np.abs(ref).max() * 4)          # 32-bit sums of exact products
    res = torch.randn(M, N, generator=g).to(DEV)
    want = f64(res) + ref
    close(ops.gemm_stream(x, w, residual=res.clone()), want, torch.float32, scale=np.abs(want).max() * 4)
    assert torch.equal(ops.gemm_stream(x[:1], w)[0], out[0])             # a row does not depend on the others
    with pytest.raises(KernelError, match="multiple of 8"):
        ops.gemm_stream(x[:, :K - 4].contiguous(), w[:, :K - 4].contiguous())
    with pytest.raises(KernelError, match="at most 16"):
        ops.gemm_stream(torch.zeros(17, K, dtype=torch.bfloat16, device=DEV), w)


@pytest.mark.parametrize("M", [1, 3, 8, 9, 16])
@pytest.mark.parametrize("N,K", [(37, 96), (200, 200), (16, 4104), (129, 1024), (5000, 8200), (2400, 512), (4096, 520),
                                 (304, 4096), (2400, 2048), (5008, 3848)])
def test_gemm_ring(M, N, K):
    """The few-rows product that streams W through a ring of TMA boxes: tiles of 16 rows and stages of 256 k that the
    sizes do not fill, more tiles than blocks (5000 rows), one stage and many; rows of 8 or 16 stages, where the warps keep
    their pieces of x in registers (K 2,048, 4,096 and 3,848: the last stage is not full); plain, residual-add and SwiGLU."""
    g = torch.Generator().manual_seed(M * 1000 + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16).to(DEV)
    ref = f64(x) @ f64(w).T
    out = ops.gemm_ring(x, w)
    ops.gemm_tc_check(DEV)
    close(out, ref, torch.float32, scale=np.abs(ref).max() * 4)          # 32-bit sums of exact products
    res = torch.randn(M, N, generator=g).to(DEV)
    want = f64(res) + ref
    close(ops.gemm_ring(x, w, residual=res.clone()), want, torch.float32, scale=np.abs(want).max() * 4)
    assert torch.equal(ops.gemm_ring(x[:1], w)[0], out[0])               # a row does not depend on the others
    assert torch.equal(ops.gemm_ring(x, w), out)                         # nor on timing
    if N % 16 == 0:
        F = N // 2
        xs, ws = (x.float() * 0.3).to(torch.bfloat16), (w.float() * 0.3).to(torch.bfloat16)
        gu = f64(xs) @ f64(ws).T
        act = ops.gemm_ring_swiglu(xs, ops.interleave_gate_up(ws[:F], ws[F:]))
        close(act, pm.swiglu(gu[:, :F], gu[:, F:]), torch.bfloat16)
        assert torch.equal(act, ops.silu_mul(ops.gemm_ring(xs, ws), torch.bfloat16))
    ops.gemm_tc_check(DEV)
    with pytest.raises(KernelError, match="multiple of 8"):
        ops.gemm_ring(x[:, :K - 4].contiguous(), w[:, :K - 4].contiguous())
    with pytest.raises(KernelError, match="at most 16"):
        ops.gemm_ring(torch.zeros(17, K, dtype=torch.bfloat16, device=DEV), w)


@pytest.mark.parametrize("M", [1, 8, 13])
@pytest.mark.parametrize("N,K,blocks", [(4096, 4096, 148), (4096, 12288, 148), (2400, 2048, 148), (5008, 3848, 148),
                                        (5120, 8200, 148), (200, 1000, 7), (37, 4096, 5), (64, 520, 11), (1000, 96, 13)])
def test_gemm_ring_split(M, N, K, blocks):
    """The ring product's split form: every block an equal share of all stages, tiles cut between blocks, their pieces
    left as planes.  The planes add up to the product (by ``SplitSum.total``, and inside the norm), a tile has as many
    planes as the host's table says and the others are never written, and the same call gives the same bits.  With rows
    of 8 or 16 stages (x kept in registers) and others, shares that begin in the middle of a tile, more blocks than
    tiles (a tile in up to 4 pieces) and fewer."""
    g = torch.Generator().manual_seed(M * 1000 + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16).to(DEV)
    ref = f64(x) @ f64(w).T
    counts = ops.ring_split_counts(N, K, blocks)
    assert max(counts) <= ops.RING_SPLIT_MAX_PLANES
    plan = (blocks, max(counts), torch.tensor(counts, dtype=torch.uint8, device=DEV))
    split = ops.gemm_ring_split(x, w, plan)
    ops.gemm_tc_check(DEV)
    close(split.total(), ref, torch.float32, scale=np.abs(ref).max() * 4)
    assert torch.equal(ops.gemm_ring_split(x, w, plan).total(), split.total())          # the same bits at every call
    # planes beyond a tile's count stay as they were: fill them with a mark and look
    marked = ops.SplitSum(torch.full_like(split.planes, 777.0), split.plane_count)
    ops._call("gemm_ring", "qwb_gemm_ring_split", ops._ptr(x), ops._ptr(w), ops._ptr(marked.planes), ops._i(M), ops._i(N),
              ops._i(K), ops._i(blocks), ops._ptr(ops.gemm_tc_error_word(DEV)), ops._stream())
    per_column = torch.tensor(counts, device=DEV).repeat_interleave(16)[:N]
    for p in range(marked.planes.shape[0]):
        untouched = (marked.planes[p] == 777.0).all(dim=0)
        assert torch.equal(untouched, per_column <= p), f"plane {p}"
    # inside the norm: h + planes, written back and normed
    h = torch.randn(M, N, generator=g).to(DEV)
    wn = (torch.rand(N, generator=g) + 0.5).to(DEV)
    want_sum = f64(h) + ref
    h2 = h.clone()
    out = ops.rmsnorm(h2, wn, 1e-6, torch.float32, delta=split, write_sum=True)
    close(h2, want_sum, torch.float32, scale=np.abs(want_sum).max() * 4)
    close(out, pm.rms_norm(f64(h2), f64(wn), 1e-6), torch.float32)
    rows = torch.tensor([M - 1, 0], dtype=torch.int32, device=DEV)
    some = ops.rmsnorm(h.clone(), wn, 1e-6, torch.bfloat16, delta=split, rows=rows)
    close(some, pm.rms_norm(f64(h2), f64(wn), 1e-6)[[M - 1, 0]], torch.bfloat16)
    h3 = h.clone()
    split.add_onto(h3)
    assert torch.equal(h3, h2)                                            # the same sums in the same order


def test_ring_split_plan_on_this_device():
    """Which matrices the split form is chosen for: those whose whole tiles leave the SMs' last round mostly empty."""
    n_sm = torch.cuda.get_device_properties(DEV).multi_processor_count
    assert ops.ring_split_plan(16 * n_sm, 4096, DEV) is None             # one full round
    assert ops.ring_split_plan(16 * n_sm * 20, 4096, DEV) is None        # twenty
    plan = ops.ring_split_plan(16 * (n_sm + n_sm // 2), 4096, DEV)      # a round and a half
    assert plan is not None and plan[0] == n_sm and plan[1] == 2 and plan[2].numel() == n_sm + n_sm // 2
    assert ops.ring_split_plan(16 * (n_sm + 1), 256 * 600, DEV) is None or ops.ring_split_plan(16 * (n_sm + 1), 256 * 600, DEV)[1] <= 4


@pytest.mark.parametrize("config", ops.STREAM_CONFIGS)
@pytest.mark.parametrize("M", [2, 8, 13])
def test_gemm_stream_in_every_form(M, config):
    """Every (loads in flight, warps) form of the few-rows product, chosen by hand as the measuring in ``parts.linear`` may
    choose it: plain, residual-add and SwiGLU, at a width and a length that are no multiples of the forms' tiles."""
    N, K = 1200, 4136
    g = torch.Generator().manual_seed(M)
    x = (torch.randn(M, K, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    w = (torch.randn(N, K, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    ref = f64(x) @ f64(w).T
    close(ops.gemm_stream(x, w, config=config), ref, torch.float32, scale=np.abs(ref).max() * 4)
    res = torch.randn(M, N, generator=g).to(DEV)
    close(ops.gemm_stream(x, w, residual=res.clone(), config=config), f64(res) + ref, torch.float32,
          scale=np.abs(ref).max() * 4)
    F = N // 2
    out = ops.gemm_stream_swiglu(x, ops.interleave_gate_up(w[:F], w[F:]), config=config)
    close(out, pm.swiglu(ref[:, :F], ref[:, F:]), torch.bfloat16)
    assert torch.equal(ops.gemm_stream(x[:1], w, config=config)[0], ops.gemm_stream(x, w, config=config)[0])


@pytest.mark.parametrize("M,N,K", [(128, 128, 64), (128, 256, 256), (300, 200, 200), (17, 96, 1032), (512, 1024, 4096),
                                   (1, 64, 64), (129, 136, 72)])
@pytest.mark.parametrize("tile_n", [64, 128, 256])
def test_gemm_tc(M, N, K, tile_n):
    g = torch.Generator().manual_seed(M + N + K)
    x = torch.randn(M, K, generator=g).to(torch.bfloat16).to(DEV)
    w = torch.randn(N, K, generator=g).to(torch.bfloat16).to(DEV)
    ref = f64(x) @ f64(w).T
    out = ops.gemm_tc(x, w, tile_n=tile_n)
    ops.gemm_tc_check(DEV)
    close(out, ref, torch.float32, scale=np.abs(ref).max() * 4)          # 32-bit sums of exact products
    base = torch.randn(M, N, generator=g).to(DEV)
    added = ops.gemm_tc(x, w, epilogue="add", out=base.clone(), tile_n=tile_n)
    ops.gemm_tc_check(DEV)
    close(added, f64(base) + ref, torch.float32, scale=np.abs(ref).max() * 4)


@pytest.mark.parametrize("M", [1, 5, 8, 11, 16])
@pytest.mark.parametrize("F,K", [(8, 64), (104, 200), (1000, 1024), (24, 4104), (2504, 8200)])
def test_gemm_stream_swiglu(M, F, K):
    g = torch.Generator().manual_seed(M * 1000 + F)
    x = (torch.randn(M, K, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * F, K, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    gu = f64(x) @ f64(w).T
    out = ops.gemm_stream_swiglu(x, ops.interleave_gate_up(w[:F], w[F:]))
    assert out.dtype == torch.bfloat16 and tuple(out.shape) == (M, F)
    close(out, pm.swiglu(gu[:, :F], gu[:, F:]), torch.bfloat16)
    # the same numbers as the product followed by the separate kernel, and a row does not depend on the others
    assert torch.equal(out, ops.silu_mul(ops.gemm_stream(x, w), torch.bfloat16))
    assert torch.equal(ops.gemm_stream_swiglu(x[:1], ops.interleave_gate_up(w[:F], w[F:]))[0], out[0])
    with pytest.raises(KernelError, match="multiple of 8"):
        ops.gemm_stream_swiglu(x, w[:2 * F - 4])
    with pytest.raises(KernelError, match="interleave_gate_up"):
        ops.interleave_gate_up(w[:F - 1], w[F:2 * F - 1])


@pytest.mark.parametrize("M,F,K", [(128, 128, 64), (200, 200, 96), (64, 1000, 512), (300, 64, 4096)])
@pytest.mark.parametrize("tile_n", [128, 256])
def test_gemm_tc_swiglu(M, F, K, tile_n):
    g = torch.Generator().manual_seed(M + F + K)
    x = (torch.randn(M, K, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    w = (torch.randn(2 * F, K, generator=g) * 0.3).to(torch.bfloat16).to(DEV)
    gu = f64(x) @ f64(w).T
    ref = pm.swiglu(gu[:, :F], gu[:, F:])
    out = ops.gemm_tc(x, ops.interleave_gate_up(w[:F], w[F:]), epilogue="swiglu", tile_n=tile_n)
    ops.gemm_tc_check(DEV)
    assert out.dtype == torch.bfloat16
    close(out, ref, torch.bfloat16)


# ----------------------------------------------------------------------------- sampling
def test_greedy_takes_the_lowest_id_among_equals():
    lg = torch.zeros(3, 1000, device=DEV)
    lg[0, [400, 17, 900]] = 5.0
    lg[1, 999] = 1.0
    lg[2] = -3.0
    assert ops.sample(lg, 0.0).tolist() == [17, 999, 0]


@pytest.mark.parametrize("top_k,top_p,temp", [(0, 1.0, 1.0), (40, 0.95, 0.8), (5, 1.0, 1.3), (0, 0.5, 0.7), (1, 1.0, 1.0)])
def test_sample_draws_from_the_reference_distribution(top_k, top_p, temp):
    V, n = 1500, 6000
    rng = np.random.default_rng(top_k)
    row = (rng.normal(size=V) * 2.5).astype(np.float32)
    probs = pm.candidate_probabilities(row, temp, top_k=top_k, top_p=top_p)
    lg = torch.from_numpy(row).to(DEV).repeat(n, 1)
    seq = torch.arange(n, dtype=torch.int32, device=DEV)
    u = torch.zeros(n, dtype=torch.float64, device=DEV)
    ids = ops.sample(lg, temp, top_k=top_k, top_p=top_p, seed=11, sequence_index=seq, step=3, out_u=u).cpu().numpy()
    support = set(np.nonzero(probs)[0])
    assert set(ids) <= support                                           # never outside top-k / top-p
    counts = np.bincount(ids, minlength=V)
    sigma = np.sqrt(n * probs * (1 - probs)) + 1e-9
    assert (np.abs(counts - n * probs) <= 5 * sigma + 2).all()           # the right frequencies
    un = u.cpu().numpy()
    assert (un > 0).all() and (un < 1).all() and abs(un.mean() - 0.5) < 0.02
    # each draw is the walk through the kept tokens in id order with that uniform number
    cum = np.cumsum(probs)
    walk = np.searchsorted(cum, un * cum[-1], side="left")
    assert (walk == ids).mean() > 0.999
    # the same (seed, sequence, step) gives the same token wherever the row is in the batch
    again = ops.sample(lg[:7].clone().flip(0), temp, top_k=top_k, top_p=top_p, seed=11,
                       sequence_index=seq[:7].flip(0).contiguous(), step=3).cpu().numpy()
    assert (again[::-1] == ids[:7]).all()
    other = ops.sample(lg, temp, top_k=top_k, top_p=top_p, seed=11, sequence_index=seq, step=4).cpu().numpy()
    assert top_k == 1 or (other != ids).any()
    # a step counter on the device adds to the step
    counter = torch.tensor([1], dtype=torch.int32, device=DEV)
    same = ops.sample(lg, temp, top_k=top_k, top_p=top_p, seed=11, sequence_index=seq, step=2, step_add=counter)
    assert (same.cpu().numpy() == ids).all()


def test_ties_at_the_cut_go_to_the_lower_ids():
    V = 300
    row = np.full(V, -5.0, dtype=np.float32)
    row[[10, 20, 30, 40]] = 2.0                                          # four equal logits, top_k = 2
    lg = torch.from_numpy(row).to(DEV).repeat(500, 1)
    seq = torch.arange(500, dtype=torch.int32, device=DEV)
    ids = set(ops.sample(lg, 1.0, top_k=2, top_p=1.0, seed=1, sequence_index=seq).tolist())
    assert ids == {10, 20}
    ids = set(ops.sample(lg, 1.0, top_k=0, top_p=0.6, seed=1, sequence_index=seq).tolist())
    assert ids == {10, 20, 30}                                           # 3 of 4 equal shares reach 0.6


@pytest.mark.parametrize("case", ["spread", "one_binade", "tie_in_the_gathered", "negative"])
def test_small_top_k_on_a_large_vocabulary(case):
    """A small top-k settles the cut on the tokens whose key shares the cut's top byte, gathered once, when they are few
    (spread), and by the general selection when they are many (all logits in [2, 8): one top byte)."""
    V, n, k = 40003, 3000, 37
    rng = np.random.default_rng(len(case))
    if case == "spread":
        row = (rng.normal(size=V) * 2.5).astype(np.float32)
    elif case == "one_binade":
        row = rng.uniform(2.0, 7.9, size=V).astype(np.float32)
    elif case == "negative":
        row = (-rng.uniform(2.0, 7.9, size=V)).astype(np.float32)
    else:
        row = np.full(V, -5.0, dtype=np.float32)
        row[rng.choice(V, size=3000, replace=False)] = 3.0               # the cut falls among 3000 equal logits
        row[[5, 20000, 39999]] = 4.0
    probs = pm.candidate_probabilities(row, 0.9, top_k=k, top_p=0.97)
    lg = torch.from_numpy(row).to(DEV).repeat(n, 1)
    seq = torch.arange(n, dtype=torch.int32, device=DEV)
    u = torch.zeros(n, dtype=torch.float64, device=DEV)
    ids = ops.sample(lg, 0.9, top_k=k, top_p=0.97, seed=5, sequence_index=seq, out_u=u).cpu().numpy()
    cum = np.cumsum(probs)
    walk = np.searchsorted(cum, u.cpu().numpy() * cum[-1], side="left")
    assert set(ids) <= set(np.nonzero(probs)[0])
    assert (walk == ids).mean() > 0.999
    only_k = ops.sample(lg, 0.9, top_k=k, top_p=1.0, seed=6, sequence_index=seq).cpu().numpy()
    kept = set(np.nonzero(pm.candidate_probabilities(row, 0.9, top_k=k, top_p=1.0))[0])
    assert set(only_k) <= kept and len(set(only_k)) > len(kept) // 2


@pytest.mark.parametrize("B,V", [(1, 151936), (5, 40003), (8, 36000), (30, 70001), (64, 20000)])
@pytest.mark.parametrize("case", ["spread", "one_binade", "tie_in_the_gathered"])
@pytest.mark.parametrize("k,p", [(29, 0.97), (0, 0.5), (0, 0.9), (0, 1.0)])
def test_few_rows_cut_into_chunks_sample_the_same(B, V, case, k, p):
    """Few rows and a small top-k, or top-p alone (tried on the 1,024 most likely tokens, and done the general way when
    it needs more), or temperature alone: every row is cut into chunks for more blocks than rows.  Same ids as one block per row, the same
    logits after the penalties, and the draw is the walk through the plain implementation's candidates."""
    rng = np.random.default_rng(B + len(case))
    if case == "spread":
        rows = (rng.normal(size=(B, V)) * 2.5).astype(np.float32)
    elif case == "one_binade":
        rows = rng.uniform(2.0, 7.9, size=(B, V)).astype(np.float32)        # too many tokens share the cut's top byte
    else:
        rows = np.full((B, V), -5.0, dtype=np.float32)
        for r in rows:
            r[rng.choice(V, size=2000, replace=False)] = 3.0
            r[rng.choice(V, size=3, replace=False)] = 4.0
    recent = rng.integers(0, V, size=(B, 12)).astype(np.int32)
    recent[:, 3] = recent[:, 7]                                             # a token seen twice
    recent[:, 5] = -1
    recent[0, 0] = int(np.argmax(rows[0]))                                  # the mode itself is penalized
    pen = dict(repeat_penalty=1.2, presence_penalty=0.3, frequency_penalty=0.1)
    seq = torch.arange(B, dtype=torch.int32, device=DEV)
    rec = torch.from_numpy(recent).to(DEV)
    for step in range(6):
        a, b = torch.from_numpy(rows).to(DEV), torch.from_numpy(rows).to(DEV)
        u = torch.zeros(B, dtype=torch.float64, device=DEV)
        ids = ops.sample(a, 0.9, top_k=k, top_p=p, seed=3, sequence_index=seq, step=step, recent=rec, out_u=u, **pen)
        one = ops.sample(b, 0.9, top_k=k, top_p=p, seed=3, sequence_index=seq, step=step, recent=rec, split=False, **pen)
        assert torch.equal(ids, one) and torch.equal(a, b)
        for r in range(B):
            want = pm.penalized_logits(rows[r], [t for t in recent[r] if t >= 0], repeat_penalty=1.2, presence=0.3, frequency=0.1)
            assert np.abs(f64(a[r]) - want).max() < 1e-5
            probs = pm.candidate_probabilities(f64(a[r]).astype(np.float32), 0.9, top_k=k, top_p=p)
            cum = np.cumsum(probs)
            assert int(np.searchsorted(cum, float(u[r]) * cum[-1], side="left")) == int(ids[r])
    # the counters are back at zero: the next call, with other sizes, starts clean
    assert int(ops._sample_counters(DEV, B).abs().sum()) == 0


@pytest.mark.parametrize("B,V", [(1, 151936), (8, 36000), (30, 70001), (64, 40003)])
def test_greedy_over_chunks_of_a_row(B, V):
    """Greedy sampling with few rows cuts every row into chunks (two kernels); with 64 rows a block takes a whole row.
    The same ids as the one-block way and as the plain argmax of the penalized logits, the lowest id among equals - also
    when the equals lie in different chunks - and the same logits after the penalties."""
    rng = np.random.default_rng(B)
    rows = (rng.normal(size=(B, V)) * 2.0).astype(np.float32)
    for r in range(B):
        top = rows[r].max() + 1.0
        rows[r, rng.choice(V, size=3, replace=False)] = top              # three equal maxima, anywhere in the row
    rows[0, 5] = rows[0].max() + 2.0                                        # the mode of row 0 is penalized below it
    recent = rng.integers(0, V, size=(B, 9)).astype(np.int32)
    recent[0, 0] = 5
    pen = dict(repeat_penalty=1.3, presence_penalty=2.5, frequency_penalty=0.2)
    rec = torch.from_numpy(recent).to(DEV)
    a, b = torch.from_numpy(rows).to(DEV), torch.from_numpy(rows).to(DEV)
    ids = ops.sample(a, 0.0, recent=rec, **pen)
    one = ops.sample(b, 0.0, recent=rec, split=False, **pen)
    assert torch.equal(ids, one) and torch.equal(a, b)
    for r in range(B):
        want = pm.penalized_logits(rows[r], list(recent[r]), repeat_penalty=1.3, presence=2.5, frequency=0.2)
        assert np.abs(f64(a[r]) - want).max() < 1e-5
        assert int(ids[r]) == int(np.argmax(f64(a[r])))                     # numpy's argmax: the first of the equals
    assert int(ids[0]) != 5


def test_penalties():
    V = 200
    rng = np.random.default_rng(5)
    row = (rng.normal(size=V) * 2).astype(np.float32)
    recent = [7, 7, 150, 3, 7, -1, -1, 199]
    want = pm.penalized_logits(row, [t for t in recent if t >= 0], repeat_penalty=1.3, presence=0.4, frequency=0.2)
    lg = torch.from_numpy(row).to(DEV).reshape(1, V).clone()
    ids = ops.sample(lg, 0.0, recent=torch.tensor([recent], dtype=torch.int32, device=DEV), repeat_penalty=1.3,
                     presence_penalty=0.4, frequency_penalty=0.2)
    assert np.abs(f64(lg)[0] - want).max() < 1e-5 and int(ids[0]) == int(np.argmax(want))
