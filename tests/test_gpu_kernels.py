"""Each CUDA kernel alone against a plain float64 reference of the same operation, at sizes other
than the tiny models': widths that are no power of two, head sizes 16..256, odd head counts."""
import math

import numpy as np
import pytest
import torch

from plain import model as pm

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16}


def ops():
    from xeno_rt_b200.csrc import ops as o
    return o


def rel(got, want):
    got = got.detach().double().cpu().numpy() if isinstance(got, torch.Tensor) else got
    return float(np.abs(got - want).max() / max(np.abs(want).max(), 1e-30))


def f64(t):
    return t.detach().double().cpu().numpy()


@pytest.mark.parametrize("table_dtype", ["float32", "bfloat16"])
def test_embedding(table_dtype):
    table = torch.randn(203, 100, device=DEV).to(DT[table_dtype])
    ids = torch.tensor([0, 202, 5, 5, 100], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 100, device=DEV)
    flag = torch.zeros(1, dtype=torch.int32, device=DEV)
    ops().embedding(out, table, ids, flag)
    assert torch.equal(out, table[ids.long()].float()) and int(flag) == 0
    bad = torch.tensor([1, 203], dtype=torch.int32, device=DEV)
    out2 = torch.ones(2, 100, device=DEV)
    ops().embedding(out2, table, bad, flag)
    assert int(flag) == 1 and float(out2[1].abs().sum()) == 0.0 and torch.equal(out2[0], table[1].float())


@pytest.mark.parametrize("width", [1, 7, 100, 4100])
@pytest.mark.parametrize("out_dtype,w_dtype", [("float32", "float32"), ("bfloat16", "bfloat16"), ("bfloat16", "float32")])
def test_rmsnorm(width, out_dtype, w_dtype):
    x = torch.randn(9, width, device=DEV) * 3
    w = (1 + 0.1 * torch.randn(width, device=DEV)).to(DT[w_dtype])
    out = torch.empty(9, width, device=DEV, dtype=DT[out_dtype])
    ops().rmsnorm(out, x, w, 3e-6)
    want = pm.rmsnorm(f64(x), f64(w), 3e-6)
    assert rel(out, want) < (1e-6 if out_dtype == "float32" else 5e-3)
    rows = torch.tensor([8, 0, 3], dtype=torch.int32, device=DEV)
    gathered = torch.empty(3, width, device=DEV, dtype=DT[out_dtype])
    ops().rmsnorm(gathered, x, w, 3e-6, rows)
    assert torch.equal(gathered, out[rows.long()])


def test_swiglu():
    gu = torch.randn(5, 2 * 136, device=DEV) * 4
    out = torch.empty(5, 136, device=DEV)
    ops().swiglu(out, gu)
    assert rel(out, pm.swiglu(f64(gu[:, :136]), f64(gu[:, 136:]))) < 1e-6
    out_b = torch.empty(5, 136, device=DEV, dtype=torch.bfloat16)
    ops().swiglu(out_b, gu)
    assert rel(out_b, pm.swiglu(f64(gu[:, :136]), f64(gu[:, 136:]))) < 5e-3


@pytest.mark.parametrize("half,base,scale", [(8, 10000.0, 1.0), (24, 1e6, 1.0), (64, 500000.0, 0.5)])
def test_rope_table(half, base, scale):
    pos = torch.tensor([0, 1, 17, 4095, 100000], dtype=torch.int32, device=DEV)
    freq = torch.from_numpy(pm.rope_frequencies(2 * half, base)).to(DEV)
    table = torch.empty(5, half, 2, device=DEV)
    ops().rope_table(table, pos, freq, scale)
    angle = (pos.cpu().numpy().astype(np.float32)[:, None] * np.float32(scale) / freq.cpu().numpy()[None]).astype(np.float32)
    assert np.abs(f64(table[..., 0]) - np.cos(angle.astype(np.float64))).max() < 2e-7
    assert np.abs(f64(table[..., 1]) - np.sin(angle.astype(np.float64))).max() < 2e-7


def _cache_for(seq_lens, n_kv, hd, dtype, shuffle_seed=0):
    """Pools and a block table whose blocks are deliberately out of order."""
    blocks_per = [(n + 63) // 64 for n in seq_lens]
    total = sum(blocks_per) + 3
    perm = np.random.default_rng(shuffle_seed).permutation(total)
    table = np.full((len(seq_lens) + 1, max(blocks_per)), -1, dtype=np.int32)
    at = 0
    for s, n in enumerate(blocks_per):
        table[s + 1, :n] = perm[at:at + n]  # slot s + 1 holds sequence s; slot 0 stays empty
        at += n
    k = torch.zeros(total, n_kv, 64, hd, device=DEV, dtype=dtype)
    v = torch.zeros_like(k)
    return k, v, torch.from_numpy(table).to(DEV)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd,rope_dim,qk_norm", [(5, 1, 48, 48, True), (4, 2, 16, 16, False),
                                                        (3, 3, 256, 64, True), (8, 2, 80, 80, False),
                                                        (12, 4, 128, 128, True), (7, 1, 128, 128, False),
                                                        (4, 2, 128, 64, False)])
@pytest.mark.parametrize("pairing", ["split_half", "interleaved"])
def test_qk_rope_kv_write(dtype, nh, nkv, hd, rope_dim, qk_norm, pairing):
    """Head norms, rotation of the first ``rope_dim`` dims (pairs (i, i + rope_dim / 2) or (2i, 2i + 1);
    the rest of the head untouched, crates/xrt-kernels/src/cpu/rope.rs:19-35), q output and cache write."""
    seq_lens = [70, 3]
    starts = [60, 0]  # the first sequence continues at position 60 and crosses a block edge
    new = [10, 3]
    T = sum(new)
    qw, kw = nh * hd, nkv * hd
    qkv = torch.randn(T, qw + 2 * kw, device=DEV)
    tok_pos = torch.tensor([starts[0] + i for i in range(new[0])] + list(range(new[1])), dtype=torch.int32, device=DEV)
    tok_slot = torch.tensor([1] * new[0] + [2] * new[1], dtype=torch.int32, device=DEV)
    k_pool, v_pool, table = _cache_for(seq_lens, nkv, hd, DT[dtype])
    qn = (1 + 0.1 * torch.randn(hd, device=DEV)) if qk_norm else None
    kn = (1 + 0.1 * torch.randn(hd, device=DEV)) if qk_norm else None
    freq = torch.from_numpy(pm.rope_frequencies(rope_dim, 10000.0)).to(DEV)
    cs = torch.empty(T, rope_dim // 2, 2, device=DEV)
    ops().rope_table(cs, tok_pos, freq, 1.0)
    q_out = torch.empty(T, qw, device=DEV, dtype=DT[dtype])
    ops().qk_rope_kv_write(q_out, k_pool, v_pool, qkv, qw, qw + kw, qn, kn, 1e-6, cs, tok_slot, tok_pos, table,
                           nh, nkv, hd, pairing=pairing)
    q, k, v = f64(qkv[:, :qw]), f64(qkv[:, qw:qw + kw]), f64(qkv[:, qw + kw:])
    if qk_norm:
        q = pm.head_rmsnorm(q, f64(qn), nh, hd, 1e-6)
        k = pm.head_rmsnorm(k, f64(kn), nkv, hd, 1e-6)
    pos = tok_pos.cpu().numpy()
    if rope_dim < hd:  # the dims beyond rope_dim are what the norm left
        untouched = q.reshape(T, nh, hd)[:, :, rope_dim:].copy()
    q = pm.rope(q, pos, nh, hd, rope_dim, 10000.0, 1.0, pairing)
    k = pm.rope(k, pos, nkv, hd, rope_dim, 10000.0, 1.0, pairing)
    tol = 2e-6 if dtype == "float32" else 5e-3
    assert rel(q_out, q) < tol
    if rope_dim < hd:
        assert rel(q_out.reshape(T, nh, hd)[:, :, rope_dim:], untouched) < tol
    tab = table.cpu().numpy()
    for t in range(T):
        slot, p = int(tok_slot[t]), int(pos[t])
        blk = tab[slot, p // 64]
        assert rel(k_pool[blk, :, p % 64, :].reshape(-1), k[t]) < tol
        assert rel(v_pool[blk, :, p % 64, :].reshape(-1), v[t]) < tol
    # nothing else in the pools was touched
    assert int((k_pool != 0).any(dim=-1).sum()) == T * nkv


def _fill_cache(k_pool, v_pool, table, slot, k, v):
    """k, v: [S, n_kv, hd] for the sequence of ``slot``."""
    tab = table.cpu().numpy()
    for p in range(k.shape[0]):
        blk = tab[slot, p // 64]
        k_pool[blk, :, p % 64, :] = k[p].to(k_pool.dtype)
        v_pool[blk, :, p % 64, :] = v[p].to(v_pool.dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (5, 1, 48), (6, 3, 128), (2, 2, 256)])
def test_attention_reference_kernel(dtype, nh, nkv, hd):
    """Two sequences: one whole (130 tokens, every position a query) and one continuing at position
    199 with a single token."""
    torch.manual_seed(nh * hd)
    lens = [130, 200]
    k_pool, v_pool, table = _cache_for(lens, nkv, hd, DT[dtype], shuffle_seed=hd)
    ks = [torch.randn(n, nkv, hd, device=DEV) for n in lens]
    vs = [torch.randn(n, nkv, hd, device=DEV) for n in lens]
    for s in range(2):
        _fill_cache(k_pool, v_pool, table, s + 1, ks[s], vs[s])
    q = torch.randn(131, nh * hd, device=DEV).to(DT[dtype])
    tok_pos = torch.tensor(list(range(130)) + [199], dtype=torch.int32, device=DEV)
    tok_slot = torch.tensor([1] * 130 + [2], dtype=torch.int32, device=DEV)
    out = torch.empty_like(q)
    ops().attention_reference(out, q, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd))
    def cached(x):
        return f64(x.to(DT[dtype])).reshape(x.shape[0], -1)
    want0 = pm.causal_gqa_attention(f64(q[:130]), cached(ks[0]), cached(vs[0]), nh, nkv, hd)
    q_last = np.zeros((200, nh * hd))
    q_last[199] = f64(q[130])
    want1 = pm.causal_gqa_attention(q_last, cached(ks[1]), cached(vs[1]), nh, nkv, hd)[199]
    tol = 2e-6 if dtype == "float32" else 1e-2
    assert rel(out[:130], want0) < tol
    assert rel(out[130], want1) < tol


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_attention_finds_a_far_key_and_respects_the_window(dtype):
    """One key among 700 is made to stand out; the result must be that key's value.  With a window
    that excludes it, it must not be."""
    nh, nkv, hd, S = 4, 2, 64, 700
    k_pool, v_pool, table = _cache_for([S], nkv, hd, DT[dtype], shuffle_seed=1)
    k = torch.randn(S, nkv, hd, device=DEV) * 0.1
    v = torch.randn(S, nkv, hd, device=DEV)
    q = torch.randn(1, nh, hd, device=DEV) * 0.1
    far = 13  # in the first block, 686 positions back
    k[far, 1] = q[0, 3] * 400  # head 3 reads kv head 1
    _fill_cache(k_pool, v_pool, table, 1, k, v)
    qf = q.reshape(1, nh * hd).to(DT[dtype])
    tok_pos = torch.tensor([S - 1], dtype=torch.int32, device=DEV)
    tok_slot = torch.tensor([1], dtype=torch.int32, device=DEV)
    out = torch.empty_like(qf)
    ops().attention_reference(out, qf, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd))
    got = out.float().reshape(nh, hd)
    assert torch.allclose(got[3], v[far, 1].to(DT[dtype]).float(), atol=2e-2)
    assert not torch.allclose(got[2], v[far, 1].to(DT[dtype]).float(), atol=0.2)
    ops().attention_reference(out, qf, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd),
                              window=S - far - 1)  # keys far+1 .. S-1: the far key is just outside
    assert not torch.allclose(out.float().reshape(nh, hd)[3], v[far, 1].float(), atol=0.2)
    ops().attention_reference(out, qf, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd),
                              window=S - far)  # the far key is the window's first
    assert torch.allclose(out.float().reshape(nh, hd)[3], v[far, 1].to(DT[dtype]).float(), atol=2e-2)


@pytest.mark.parametrize("xd,wd,od", [("float32", "float32", "float32"), ("bfloat16", "bfloat16", "float32"),
                                      ("bfloat16", "bfloat16", "bfloat16")])
@pytest.mark.parametrize("m,n,k", [(1, 203, 100), (7, 64, 17), (130, 136, 96), (65, 320, 260)])
def test_gemm_reference(xd, wd, od, m, n, k):
    x = torch.randn(m, k, device=DEV).to(DT[xd])
    w = (torch.randn(n, k, device=DEV) * 0.1).to(DT[wd])
    out = torch.empty(m, n, device=DEV, dtype=DT[od])
    ops().gemm_reference(out, x, w)
    want = f64(x) @ f64(w).T
    assert rel(out, want) < (2e-6 if od == "float32" else 5e-3)
    if od == "float32":
        base = torch.randn(m, n, device=DEV)
        acc = base.clone()
        ops().gemm_reference(acc, x, w, accumulate=True)
        assert rel(acc, f64(base) + want) < 2e-6


def test_gemm_rows_do_not_depend_on_the_batch():
    x = torch.randn(70, 100, device=DEV)
    w = torch.randn(203, 100, device=DEV)
    whole = torch.empty(70, 203, device=DEV)
    ops().gemm_reference(whole, x, w)
    one = torch.empty(1, 203, device=DEV)
    ops().gemm_reference(one, x[69:70].contiguous(), w)
    assert torch.equal(one[0], whole[69])


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_fill_normal_matches_the_host_generator(dtype):
    from xeno_rt_b200.weights import normal_values, tensor_key
    key = tensor_key(3, "model.layers.0.mlp.up_proj.weight")
    out = torch.empty(1000, 37, device=DEV, dtype=DT[dtype])
    ops().fill_normal(out, key, 0.0, 0.02)
    host = torch.from_numpy(normal_values(key, 37000, 0.0, 0.02)).to(DT[dtype]).reshape(1000, 37)
    same = (out.cpu() == host).float().mean()
    assert same > 0.999  # identical but for rare last-bit differences of log and cos
    assert torch.allclose(out.cpu().float(), host.float(), atol=1e-4)


@pytest.mark.parametrize("m", [1, 3, 8, 16, 17, 40, 64])
@pytest.mark.parametrize("n,k", [(203, 104), (64, 4096), (136, 96), (8, 40), (24, 1544), (5000, 264), (4744, 1032)])
def test_gemm_stream(m, n, k):
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.1).to(torch.bfloat16)
    want = f64(x) @ f64(w).T
    out = torch.empty(m, n, device=DEV)
    ops().gemm_stream(out, x, w)
    assert rel(out, want) < 1e-5  # bfloat16 operands are exact in float64; only the sum's order differs
    out_b = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    ops().gemm_stream(out_b, x, w)
    assert rel(out_b, want) < 5e-3
    base = torch.randn(m, n, device=DEV)
    acc = base.clone()
    ops().gemm_stream(acc, x, w, "accumulate")
    assert rel(acc, f64(base) + want) < 1e-5
    # a row's result does not depend on how many rows the call carries
    one = torch.empty(1, n, device=DEV)
    ops().gemm_stream(one, x[m - 1:m].contiguous(), w)
    assert torch.equal(one[0], out[m - 1])


@pytest.mark.parametrize("m,inner,k", [(1, 136, 96), (9, 203, 104), (33, 64, 4096)])
def test_gemm_stream_swiglu(m, inner, k):
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * inner, k, device=DEV) * 0.1).to(torch.bfloat16)
    out = torch.empty(m, inner, device=DEV, dtype=torch.bfloat16)
    ops().gemm_stream(out, x, w, "swiglu", up_rows=inner)
    want = pm.swiglu(f64(x) @ f64(w[:inner]).T, f64(x) @ f64(w[inner:]).T)
    assert rel(out, want) < 5e-3


def test_gemm_stream_refuses_what_it_cannot_take():
    from xeno_rt_b200.core import KernelError
    x = torch.randn(2, 100, device=DEV).to(torch.bfloat16)  # K = 100 is no multiple of 8
    w = torch.randn(16, 100, device=DEV).to(torch.bfloat16)
    with pytest.raises(KernelError, match="outside what the kernel handles"):
        ops().gemm_stream(torch.empty(2, 16, device=DEV), x, w)


@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (5, 1, 48), (32, 8, 128), (6, 3, 80), (16, 1, 256), (8, 8, 64)])
@pytest.mark.parametrize("chunk,n_splits,fused", [(64, 11, True), (64, 11, False), (256, 3, True), (704, 1, True)])
def test_attention_decode_kernel(nh, nkv, hd, chunk, n_splits, fused):
    """Five sequences of unequal lengths (one of a single token, one ending at a block edge, one a
    padding row), one token each, against the plain attention of the full sequences."""
    torch.manual_seed(nh + hd + chunk)
    lens = [1, 64, 65, 300, 700]
    k_pool, v_pool, table = _cache_for(lens, nkv, hd, torch.bfloat16, shuffle_seed=hd)
    ks = [torch.randn(n, nkv, hd, device=DEV) for n in lens]
    vs = [torch.randn(n, nkv, hd, device=DEV) for n in lens]
    for s in range(len(lens)):
        _fill_cache(k_pool, v_pool, table, s + 1, ks[s], vs[s])
    order = [3, 0, -1, 4, 1, 2]  # token rows: sequences in another order, and a padding row
    q = torch.randn(len(order), nh * hd, device=DEV).to(torch.bfloat16)
    tok_slot = torch.tensor([s + 1 if s >= 0 else -1 for s in order], dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([lens[s] - 1 if s >= 0 else 0 for s in order], dtype=torch.int32, device=DEV)
    out = torch.full_like(q, 7.0)
    ops().attention_decode(out, q, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd), 0,
                           chunk, n_splits, fused=fused)
    if fused:  # the merge by the last block gives the bits of the merge by the second kernel, and leaves the counters zero
        two = torch.full_like(q, 7.0)
        ops().attention_decode(two, q, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd), 0,
                               chunk, n_splits, fused=False)
        assert torch.equal(out, two)
        from xeno_rt_b200.csrc import ops as o
        assert int(o.device_state(DEV)[1].abs().sum()) == 0
    bf = lambda x: f64(x.to(torch.bfloat16)).reshape(x.shape[0], -1)
    for row, s in enumerate(order):
        if s < 0:
            assert float(out[row].float().abs().sum()) == 0.0
            continue
        n = lens[s]
        q_full = np.zeros((n, nh * hd))
        q_full[n - 1] = f64(q[row])
        want = pm.causal_gqa_attention(q_full, bf(ks[s]), bf(vs[s]), nh, nkv, hd)[n - 1]
        assert rel(out[row], want) < 1.5e-2, (row, s)


@pytest.mark.parametrize("nh,nkv,hd,qk_norm,rotate", [(8, 2, 128, True, True), (4, 4, 64, False, True), (6, 1, 128, False, False),
                                                      (2, 1, 256, True, True), (32, 8, 128, False, True)])
@pytest.mark.parametrize("chunk,n_splits,fused", [(704, 1, True), (128, 6, True), (128, 6, False), (64, 11, True)])
def test_attention_decode_from_the_product_of_q_k_v(nh, nkv, hd, qk_norm, rotate, chunk, n_splits, fused):
    """The decode attention that does the step before it itself: from the 32-bit q/k/v rows it norms
    and rotates q and k, writes the newest key and value into the cache (nothing else in the pools
    changes) and attends over the old keys and the newest one.  Sequences whose newest position is the
    first of a block, the last of a block, the very first, and a padding row; against the plain
    functions, and against the two kernels it replaces."""
    torch.manual_seed(nh + hd + chunk + n_splits)
    lens = [1, 64, 65, 300, 700]  # lengths AFTER the step: the newest position is len - 1
    k_pool, v_pool, table = _cache_for(lens, nkv, hd, torch.bfloat16, shuffle_seed=hd + 1)
    ks = [torch.randn(n, nkv, hd, device=DEV) for n in lens]
    vs = [torch.randn(n, nkv, hd, device=DEV) for n in lens]
    for s in range(len(lens)):  # the cache holds all positions but the newest
        _fill_cache(k_pool, v_pool, table, s + 1, ks[s][:-1], vs[s][:-1])
    order = [3, 0, -1, 4, 1, 2]
    T, qw, kw = len(order), nh * hd, nkv * hd
    qkv = torch.randn(T, qw + 2 * kw + 8, device=DEV)  # a row longer than q, k, v
    tok_slot = torch.tensor([s + 1 if s >= 0 else -1 for s in order], dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([lens[s] - 1 if s >= 0 else 0 for s in order], dtype=torch.int32, device=DEV)
    qn = (1 + 0.1 * torch.randn(hd, device=DEV)) if qk_norm else None
    kn = (1 + 0.1 * torch.randn(hd, device=DEV)) if qk_norm else None
    cs = None
    if rotate:
        freq = torch.from_numpy(pm.rope_frequencies(hd, 10000.0)).to(DEV)
        cs = torch.empty(T, hd // 2, 2, device=DEV)
        ops().rope_table(cs, tok_pos, freq, 1.0)
    from xeno_rt_b200.csrc import ops as o
    assert o.attention_decode_takes_qkv(nh, nkv, hd, hd // 2 if rotate else 0, "split_half")
    # the two kernels it replaces, on copies of the pools
    k2, v2 = k_pool.clone(), v_pool.clone()
    q2 = torch.empty(T, qw, device=DEV, dtype=torch.bfloat16)
    ops().qk_rope_kv_write(q2, k2, v2, qkv, qw, qw + kw, qn, kn, 1e-6, cs, tok_slot, tok_pos, table, nh, nkv, hd)
    two = torch.full((T, qw), 7.0, device=DEV, dtype=torch.bfloat16)
    ops().attention_decode(two, q2, k2, v2, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd), 0, chunk, n_splits,
                           fused=fused)
    out = torch.full((T, qw), 7.0, device=DEV, dtype=torch.bfloat16)
    ops().attention_decode_qkv(out, qkv, qw, qw + kw, qn, kn, 1e-6, cs, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd,
                               1 / math.sqrt(hd), 0, chunk, n_splits, fused=fused)
    o.check_error_flag(DEV)
    assert int(o.device_state(DEV)[1].abs().sum()) == 0
    # the cache: the same rows were written as by the kernel it replaces (norm sums differ in their order)
    assert int((k_pool != 0).any(dim=-1).sum()) == int((k2 != 0).any(dim=-1).sum())
    assert rel(k_pool, f64(k2)) < 1e-2 and torch.equal(v_pool, v2)
    live = [r for r, s in enumerate(order) if s >= 0]
    assert rel(out[live], f64(two[live])) < 2e-2
    pos = tok_pos.cpu().numpy()
    q, k = f64(qkv[:, :qw]), f64(qkv[:, qw:qw + kw])
    if qk_norm:
        q, k = pm.head_rmsnorm(q, f64(qn), nh, hd, 1e-6), pm.head_rmsnorm(k, f64(kn), nkv, hd, 1e-6)
    if rotate:
        q, k = pm.rope(q, pos, nh, hd, hd, 10000.0, 1.0), pm.rope(k, pos, nkv, hd, hd, 10000.0, 1.0)
    bf = lambda x, width: f64(torch.as_tensor(x).to(torch.bfloat16)).reshape(len(x), width)
    for row, s in enumerate(order):
        if s < 0:
            assert float(out[row].float().abs().sum()) == 0.0
            continue
        n = lens[s]
        keys = np.concatenate([bf(ks[s][:-1], kw), bf(k[row:row + 1], kw)])
        values = np.concatenate([bf(vs[s][:-1], kw), bf(f64(qkv[row:row + 1, qw + kw:qw + 2 * kw]), kw)])
        q_full = np.zeros((n, qw))
        q_full[n - 1] = bf(q[row:row + 1], qw)[0]
        want = pm.causal_gqa_attention(q_full, keys, values, nh, nkv, hd)[n - 1]
        assert rel(out[row], want) < 1.5e-2, (row, s)
    # a layer that reads another layer's cache: nothing is written, the newest key is there already
    before_k, before_v = k_pool.clone(), v_pool.clone()
    again = torch.full((T, qw), 7.0, device=DEV, dtype=torch.bfloat16)
    ops().attention_decode_qkv(again, qkv[:, :qw].contiguous(), qw, qw + kw, qn, kn, 1e-6, cs, k_pool, v_pool, tok_slot,
                               tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd), 0, chunk, n_splits, write_kv=False, fused=fused)
    assert torch.equal(k_pool, before_k) and torch.equal(v_pool, before_v)
    assert rel(again[live], f64(out[live])) < 1e-2
    # a window of 100 keys (the newest key is its last): against the two kernels on the same cache
    ops().attention_decode(two, q2, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd), 100, chunk,
                           n_splits, fused=fused)
    ops().attention_decode_qkv(again, qkv, qw, qw + kw, qn, kn, 1e-6, cs, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd,
                               1 / math.sqrt(hd), 100, chunk, n_splits, write_kv=False, fused=fused)
    assert rel(again[live], f64(two[live])) < 2e-2
    ref = torch.empty_like(two)
    ops().attention_reference(ref, q2, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd), window=100)
    assert rel(again[live], f64(ref[live])) < 2e-2


def test_attention_decode_finds_a_far_key_and_respects_the_window():
    nh, nkv, hd, S = 8, 2, 128, 1500
    k_pool, v_pool, table = _cache_for([S], nkv, hd, torch.bfloat16, shuffle_seed=2)
    k = torch.randn(S, nkv, hd, device=DEV) * 0.1
    v = torch.randn(S, nkv, hd, device=DEV)
    q = torch.randn(1, nh, hd, device=DEV) * 0.1
    far = 70  # second block, 1429 positions back
    k[far, 1] = q[0, 6] * 400  # head 6 reads kv head 1
    _fill_cache(k_pool, v_pool, table, 1, k, v)
    qf = q.reshape(1, nh * hd).to(torch.bfloat16)
    tok_pos = torch.tensor([S - 1], dtype=torch.int32, device=DEV)
    tok_slot = torch.tensor([1], dtype=torch.int32, device=DEV)
    target = v[far, 1].to(torch.bfloat16).float()
    for chunk, n_splits in ((128, 12), (1536, 1)):
        out = torch.empty_like(qf)
        run = lambda window: ops().attention_decode(out, qf, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd,
                                                    1 / math.sqrt(hd), window, chunk, n_splits)
        run(0)
        assert torch.allclose(out.float().reshape(nh, hd)[6], target, atol=3e-2)
        assert not torch.allclose(out.float().reshape(nh, hd)[5], target, atol=0.2)
        run(S - far - 1)  # the far key is just outside the window
        assert not torch.allclose(out.float().reshape(nh, hd)[6], target, atol=0.2)
        run(S - far)  # the far key is the window's first
        assert torch.allclose(out.float().reshape(nh, hd)[6], target, atol=3e-2)
        ref = torch.empty_like(qf)
        ops().attention_reference(ref, qf, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd),
                                  window=S - far)
        assert torch.allclose(out.float(), ref.float(), atol=3e-2)


@pytest.mark.parametrize("hd", [128, 64])
def test_attention_decode_launches_of_many_blocks(hd):
    """The kernel fed by TMA keeps three tile buffers where two blocks a multiprocessor hold the launch and two
    where more blocks have to be resident: 48 tokens x 2 kv heads x 4 splits are 384 blocks (two buffers), 6 tokens 48
    (three).  The 48 slots read prefixes of different lengths of the same cache blocks; the reference kernel says what
    must come out, with the splits merged as clusters, by the last block and by the second kernel."""
    nh, nkv, S, T = 8, 2, 520, 48
    torch.manual_seed(hd + 5)
    k_pool, v_pool, table = _cache_for([S], nkv, hd, torch.bfloat16, shuffle_seed=5)
    _fill_cache(k_pool, v_pool, table, 1, torch.randn(S, nkv, hd, device=DEV), torch.randn(S, nkv, hd, device=DEV))
    table = torch.cat([table[:1], table[1:2].repeat(T, 1)])  # slots 1 .. T share the sequence's blocks
    tok_slot = torch.arange(1, T + 1, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([60 + (457 * i) % 460 for i in range(T)], dtype=torch.int32, device=DEV)
    q = (torch.randn(T, nh * hd, device=DEV) * 0.3).to(torch.bfloat16)
    ref = torch.empty_like(q)
    ops().attention_reference(ref, q, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd))
    for tokens in (T, 6):
        for fused, clusters in ((True, True), (True, False), (False, False)):
            out = torch.full_like(q, 7.0)
            ops().attention_decode(out[:tokens], q[:tokens], k_pool, v_pool, tok_slot[:tokens], tok_pos[:tokens], table, nh, nkv,
                                   hd, 1 / math.sqrt(hd), 0, 192, 3 if tokens == 6 else 4, fused=fused, clusters=clusters)
            assert rel(out[:tokens], f64(ref[:tokens])) < 1.5e-2, (tokens, fused, clusters)
            assert float((out[tokens:].float() - 7.0).abs().max()) == 0.0 if tokens < T else True


@pytest.mark.parametrize("hd,rise", [(128, 0.07), (80, 0.07), (128, 0.2), (64, -0.05)])
def test_attention_decode_scores_that_rise_slowly(hd, rise):
    """The decode kernels move the reference value of a head's exponents only when a score has outgrown it by more
    than 8 in base 2.  Scores that rise (or fall) by ``rise`` a key make the reference lag behind the maximum for
    tiles on end (0.07 a key: 6.5 in base 2 between the 16 keys a warp sees in one tile and in the next), or jump at
    every tile (0.2): the result must be the plain one either way, for one split and for several."""
    nh, nkv, S = 8, 2, 900
    torch.manual_seed(7)
    k_pool, v_pool, table = _cache_for([S], nkv, hd, torch.bfloat16, shuffle_seed=4)
    u = torch.randn(nkv, hd, device=DEV)
    u = u / u.norm(dim=-1, keepdim=True)
    ramp = torch.arange(S, device=DEV, dtype=torch.float32)[:, None, None] * rise * math.sqrt(hd)
    k = (u[None] * ramp / 4 + torch.randn(S, nkv, hd, device=DEV) * 0.05)
    v = torch.randn(S, nkv, hd, device=DEV)
    q = (u.repeat_interleave(nh // nkv, dim=0) * 4)[None]  # head h reads kv head h // 4: score = rise * position + noise
    _fill_cache(k_pool, v_pool, table, 1, k, v)
    qf = q.reshape(1, nh * hd).to(torch.bfloat16)
    tok_pos = torch.tensor([S - 1], dtype=torch.int32, device=DEV)
    tok_slot = torch.tensor([1], dtype=torch.int32, device=DEV)
    bf = lambda x: f64(x.to(torch.bfloat16))
    q_full = np.zeros((S, nh * hd))
    q_full[S - 1] = bf(qf)[0]
    want = pm.causal_gqa_attention(q_full, bf(k).reshape(S, nkv * hd), bf(v).reshape(S, nkv * hd), nh, nkv, hd)[S - 1]
    for chunk, n_splits in ((960, 1), (256, 4), (64, 15)):
        for fused in (False, True):
            out = torch.full_like(qf, 7.0)
            ops().attention_decode(out, qf, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd), 0,
                                   chunk, n_splits, fused=fused)
            assert rel(out[0], want) < 1.5e-2, (chunk, n_splits, fused)


@pytest.mark.parametrize("hd", [128, 80])
def test_attention_decode_window_splits_start_at_the_window(hd):
    """A windowed layer's splits are counted from the cache block of its first visible key, so three splits
    of 64 keys cover a window of 150 keys at the end of 1,500 (keys 1,350 .. 1,499, from block key 1,344).
    The window's first key is made to stand out; one key less in the window and it is gone."""
    nh, nkv, S, window = 8, 2, 1500, 150
    torch.manual_seed(hd)
    k_pool, v_pool, table = _cache_for([S, 40], nkv, hd, torch.bfloat16, shuffle_seed=3)
    k = torch.randn(S, nkv, hd, device=DEV) * 0.1
    v = torch.randn(S, nkv, hd, device=DEV)
    q = torch.randn(2, nh, hd, device=DEV) * 0.1
    first = S - window
    k[first, 1] = q[0, 6] * 400  # head 6 reads kv head 1
    _fill_cache(k_pool, v_pool, table, 1, k, v)
    _fill_cache(k_pool, v_pool, table, 2, k[:40].contiguous(), v[:40].contiguous())  # shorter than the window
    qf = q.reshape(2, nh * hd).to(torch.bfloat16)
    tok_pos = torch.tensor([S - 1, 39], dtype=torch.int32, device=DEV)
    tok_slot = torch.tensor([1, 2], dtype=torch.int32, device=DEV)
    target = v[first, 1].to(torch.bfloat16).float()
    ref = torch.empty_like(qf)
    ops().attention_reference(ref, qf, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd), window=window)
    assert torch.allclose(ref.float().reshape(2, nh, hd)[0, 6], target, atol=3e-2)
    for chunk, n_splits in ((64, 3), (128, 2), (256, 1)):
        for fused in (False, True):
            for clusters in (False, True):
                out = torch.full_like(qf, 7.0)
                ops().attention_decode(out, qf, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd),
                                       window, chunk, n_splits, fused=fused, clusters=clusters)
                assert torch.allclose(out.float(), ref.float(), atol=3e-2), (chunk, fused, clusters)
                ops().attention_decode(out, qf, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd),
                                       window - 1, chunk, n_splits, fused=fused, clusters=clusters)
                assert not torch.allclose(out.float().reshape(2, nh, hd)[0, 6], target, atol=0.2)


@pytest.mark.parametrize("nh,nkv,hd", [(4, 2, 16), (5, 1, 48), (8, 2, 128), (6, 3, 80), (2, 1, 256)])
def test_attention_prefill_kernel(nh, nkv, hd):
    """Four sequences end to end: a whole prompt of 150 tokens, one of a single token, one that
    continues at position 100 with 70 more tokens (across a block edge), and a skipped one."""
    torch.manual_seed(nh * hd + 1)
    totals = [150, 1, 170, 64]
    starts = [0, 0, 100, 0]
    new = [150, 1, 70, 5]
    k_pool, v_pool, table = _cache_for(totals, nkv, hd, torch.bfloat16, shuffle_seed=hd + 1)
    ks = [torch.randn(n, nkv, hd, device=DEV) for n in totals]
    vs = [torch.randn(n, nkv, hd, device=DEV) for n in totals]
    for s in range(4):
        _fill_cache(k_pool, v_pool, table, s + 1, ks[s], vs[s])
    T = sum(new)
    q = torch.randn(T, nh * hd, device=DEV).to(torch.bfloat16)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(new)]), dtype=torch.int32, device=DEV)
    seq_slot = torch.tensor([1, 2, 3, -1], dtype=torch.int32, device=DEV)
    seq_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
    out = torch.full_like(q, 5.0)
    ops().attention_prefill(out, q, k_pool, v_pool, cu, seq_slot, seq_start, table, max(new), nh, nkv, hd,
                            1 / math.sqrt(hd))
    bf = lambda x: f64(x.to(torch.bfloat16)).reshape(x.shape[0], -1)
    at = 0
    for s in range(3):
        q_full = np.zeros((totals[s], nh * hd))
        q_full[starts[s]:] = f64(q[at:at + new[s]])
        want = pm.causal_gqa_attention(q_full, bf(ks[s]), bf(vs[s]), nh, nkv, hd)[starts[s]:]
        assert rel(out[at:at + new[s]], want) < 1.5e-2, s
        at += new[s]
    assert bool((out[at:] == 5.0).all())  # the skipped sequence's rows are untouched
    # the same rows through the kernel that takes any case
    ref = torch.empty_like(q)
    tok_slot = torch.tensor([1] * 150 + [2] + [3] * 70 + [-1] * 5, dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor(list(range(150)) + [0] + list(range(100, 170)) + [0] * 5, dtype=torch.int32, device=DEV)
    ops().attention_reference(ref, q, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd))
    assert torch.allclose(out[:221].float(), ref[:221].float(), atol=3e-2)


def test_attention_prefill_window_edge():
    """With a window of 70 keys, row i sees keys i-69 .. i: the kernel must agree with the plain
    windowed attention at every row, in particular where the window's edge crosses a block edge."""
    nh, nkv, hd, S, window = 4, 2, 64, 200, 70
    k_pool, v_pool, table = _cache_for([S], nkv, hd, torch.bfloat16, shuffle_seed=5)
    k = torch.randn(S, nkv, hd, device=DEV)
    v = torch.randn(S, nkv, hd, device=DEV)
    _fill_cache(k_pool, v_pool, table, 1, k, v)
    q = (torch.randn(S, nh * hd, device=DEV) * 2).to(torch.bfloat16)
    cu = torch.tensor([0, S], dtype=torch.int32, device=DEV)
    one = lambda x: torch.tensor([x], dtype=torch.int32, device=DEV)
    out = torch.empty_like(q)
    ops().attention_prefill(out, q, k_pool, v_pool, cu, one(1), one(0), table, S, nh, nkv, hd, 1 / math.sqrt(hd), window)
    bf = lambda x: f64(x.to(torch.bfloat16)).reshape(x.shape[0], -1)
    want = pm.causal_gqa_attention(f64(q), bf(k), bf(v), nh, nkv, hd, window=window)
    assert rel(out, want) < 1.5e-2
    full = pm.causal_gqa_attention(f64(q), bf(k), bf(v), nh, nkv, hd)
    assert np.abs(want[150] - full[150]).max() > 0.05  # the window matters in this case


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (65, 8, 8), (200, 300, 136), (129, 513, 1032), (1000, 136, 96)])
def test_gemm_tcgen05(m, n, k):
    """Sizes that are no multiple of the 128 x 256 x 64 tile: TMA zero-fills what reaches beyond."""
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.1).to(torch.bfloat16)
    want = f64(x) @ f64(w).T
    out = torch.full((m, n), 7.0, device=DEV)
    ops().gemm_tcgen05(out, x, w)
    assert rel(out, want) < 1e-5
    out_b = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    ops().gemm_tcgen05(out_b, x, w)
    assert rel(out_b, want) < 5e-3
    base = torch.randn(m, n, device=DEV)
    acc = base.clone()
    ops().gemm_tcgen05(acc, x, w, "accumulate")
    assert rel(acc, f64(base) + want) < 1e-5
    from xeno_rt_b200.csrc import ops as o
    o.check_error_flag(DEV)


def test_gemm_tcgen05_many_tiles_and_row_invariance():
    """More tiles than multiprocessors (the persistent loop and both accumulators are used), and a
    row's result is the same bits whatever the number of rows."""
    m, n, k = 700, 2100, 520
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.1).to(torch.bfloat16)
    out = torch.empty(m, n, device=DEV)
    ops().gemm_tcgen05(out, x, w)
    assert rel(out, f64(x) @ f64(w).T) < 1e-5
    part = torch.empty(70, n, device=DEV)
    ops().gemm_tcgen05(part, x[300:370].contiguous(), w)
    assert torch.equal(part, out[300:370])


@pytest.mark.parametrize("m,inner,k", [(128, 128, 64), (130, 203, 104), (300, 136, 96)])
def test_gemm_tcgen05_swiglu(m, inner, k):
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * inner, k, device=DEV) * 0.1).to(torch.bfloat16)
    out = torch.empty(m, inner, device=DEV, dtype=torch.bfloat16)
    ops().gemm_tcgen05(out, x, w, "swiglu", up_rows=inner)
    want = pm.swiglu(f64(x) @ f64(w[:inner]).T, f64(x) @ f64(w[inner:]).T)
    assert rel(out, want) < 5e-3


@pytest.mark.parametrize("m", [1, 8, 16, 17, 40, 64, 100, 128])
@pytest.mark.parametrize("n,k", [(203, 104), (4096, 512), (136, 96), (8, 40), (300, 2056)])
def test_gemm_decode_tcgen05(m, n, k):
    """Swapped-operand product: any N (tiles of 128 weight rows), K split across blocks or not."""
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(n, k, device=DEV) * 0.1).to(torch.bfloat16)
    want = f64(x) @ f64(w).T
    out = torch.full((m, n), 7.0, device=DEV)
    ops().gemm_decode_tcgen05(out, x, w)
    assert rel(out, want) < 1e-5
    out_b = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    ops().gemm_decode_tcgen05(out_b, x, w)
    assert rel(out_b, want) < 5e-3
    base = torch.randn(m, n, device=DEV)
    acc = base.clone()
    ops().gemm_decode_tcgen05(acc, x, w, "accumulate")
    assert rel(acc, f64(base) + want) < 1e-5
    lo = m - max(1, (m + 15) // 16 * 16 - 15)  # the smallest batch that is padded to the same size
    few = torch.empty(m - lo, n, device=DEV)
    ops().gemm_decode_tcgen05(few, x[lo:m].contiguous(), w)
    assert torch.equal(few[-1], out[m - 1])  # a row's result does not depend on the other rows
    again = torch.empty_like(out)
    ops().gemm_decode_tcgen05(again, x, w)
    assert torch.equal(again, out)  # nor on which block finished a tile last
    from xeno_rt_b200.csrc import ops as o
    o.check_error_flag(DEV)


@pytest.mark.parametrize("m,inner,k", [(1, 136, 96), (9, 203, 104), (64, 256, 4096), (33, 1000, 520)])
def test_gemm_decode_tcgen05_swiglu(m, inner, k):
    x = torch.randn(m, k, device=DEV).to(torch.bfloat16)
    w = (torch.randn(2 * inner, k, device=DEV) * 0.1).to(torch.bfloat16)
    out = torch.empty(m, inner, device=DEV, dtype=torch.bfloat16)
    ops().gemm_decode_tcgen05(out, x, w, "swiglu", up_rows=inner)
    want = pm.swiglu(f64(x) @ f64(w[:inner]).T, f64(x) @ f64(w[inner:]).T)
    assert rel(out, want) < 5e-3


@pytest.mark.parametrize("nh,nkv", [(8, 2), (5, 1), (4, 4), (6, 3)])
def test_attention_prefill_tcgen05_kernel(nh, nkv):
    """The tcgen05 attention (head size 128) on the case of the mma.sync kernel's test: a whole prompt of 150 tokens,
    one of a single token, one that continues at position 100 with 70 more (across a block edge), a skipped one;
    plus a prompt of 300 tokens (three query tiles, five key blocks)."""
    hd = 128
    torch.manual_seed(nh * 7 + nkv)
    totals = [150, 1, 170, 64, 300]
    starts = [0, 0, 100, 0, 0]
    new = [150, 1, 70, 5, 300]
    slots = [1, 2, 3, -1, 5]
    k_pool, v_pool, table = _cache_for(totals, nkv, hd, torch.bfloat16, shuffle_seed=nh)
    ks = [torch.randn(n, nkv, hd, device=DEV) for n in totals]
    vs = [torch.randn(n, nkv, hd, device=DEV) for n in totals]
    for s in range(5):
        _fill_cache(k_pool, v_pool, table, s + 1, ks[s], vs[s])
    T = sum(new)
    q = torch.randn(T, nh * hd, device=DEV).to(torch.bfloat16)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(new)]), dtype=torch.int32, device=DEV)
    seq_slot = torch.tensor(slots, dtype=torch.int32, device=DEV)
    seq_start = torch.tensor(starts, dtype=torch.int32, device=DEV)
    out = torch.full_like(q, 5.0)
    ops().attention_prefill_tcgen05(out, q, k_pool, v_pool, cu, seq_slot, seq_start, table, max(new), nh, nkv, hd,
                                    1 / math.sqrt(hd))
    from xeno_rt_b200.csrc import ops as o
    o.check_error_flag(DEV)
    bf = lambda x: f64(x.to(torch.bfloat16)).reshape(x.shape[0], -1)
    at = 0
    for s in range(5):
        if slots[s] >= 0:
            q_full = np.zeros((totals[s], nh * hd))
            q_full[starts[s]:] = f64(q[at:at + new[s]])
            want = pm.causal_gqa_attention(q_full, bf(ks[s]), bf(vs[s]), nh, nkv, hd)[starts[s]:]
            assert rel(out[at:at + new[s]], want) < 1.5e-2, s
        else:
            assert bool((out[at:at + new[s]] == 5.0).all())  # the skipped sequence's rows are untouched
        at += new[s]


@pytest.mark.parametrize("m", [1, 3, 8, 16])
@pytest.mark.parametrize("width,inner,out_rows,norm_dtype", [(1032, 2760, 1536, torch.float32), (256, 520, 392, torch.bfloat16),
                                                            (4096, 1024, 4096, torch.bfloat16), (5120, 264, 5000, torch.float32)])
def test_a_product_prepares_the_norm_that_follows_and_the_next_product_finishes_it(m, width, inner, out_rows, norm_dtype):
    """(The widest case has more weight rows than the kernel's blocks of 8 rows can all run at once: blocks of 16.)
    residual += act . down^T by the cp.async kernel, which also leaves residual * norm weight in
    bfloat16 and every row's partial sums of squares; then the tcgen05 few-row product of that with
    another matrix, which multiplies row m by 1 / sqrt(mean square + eps).  Against the plain
    functions (norm, then product), store and SwiGLU, and the residual against the plain sum."""
    from xeno_rt_b200.csrc import ops as o
    torch.manual_seed(m + width + inner)
    eps = 1e-5
    resid = torch.randn(m, width, device=DEV) * 2
    act = (torch.randn(m, inner, device=DEV)).to(torch.bfloat16)
    w_down = (torch.randn(width, inner, device=DEV) * 0.05).to(torch.bfloat16)
    w_norm = (1 + 0.1 * torch.randn(width, device=DEV)).to(norm_dtype)
    w_next = (torch.randn(2 * out_rows, width, device=DEV) * 0.05).to(torch.bfloat16)
    want_resid = f64(resid) + f64(act) @ f64(w_down).T
    x = resid.clone()
    scaled = torch.full((m, width), 9.0, device=DEV, dtype=torch.bfloat16)
    squares = torch.full((o.gemm_stream_norm_parts(m, width), m), 9.0, device=DEV)
    o.gemm_stream(x, act, w_down, "accumulate", norm=(scaled, w_norm, squares))
    assert rel(x, want_resid) < 1e-5
    plain = resid.clone()
    o.gemm_stream(plain, act, w_down, "accumulate")
    assert torch.equal(x, plain)  # the residual itself is what the product without the norm writes
    assert rel(scaled, f64(x) * f64(w_norm)) < 5e-3
    assert rel(squares.sum(0), (f64(x) ** 2).sum(1)) < 1e-5
    normed = pm.rmsnorm(f64(x), f64(w_norm), eps)
    out = torch.empty(m, 2 * out_rows, device=DEV)
    o.gemm_decode_tcgen05(out, scaled, w_next, "store", squares=squares, eps=eps)
    assert rel(out, normed @ f64(w_next).T) < 6e-3
    act2 = torch.empty(m, out_rows, device=DEV, dtype=torch.bfloat16)
    o.gemm_decode_tcgen05(act2, scaled, w_next, "swiglu", up_rows=out_rows, squares=squares, eps=eps)
    gate_up = normed @ f64(w_next).T
    assert rel(act2, pm.swiglu(gate_up[:, :out_rows], gate_up[:, out_rows:])) < 1.2e-2
    # the cp.async kernel finishes a pending norm too
    out.fill_(7.0)
    o.gemm_stream(out, scaled, w_next, "store", squares=squares, eps=eps)
    assert rel(out, normed @ f64(w_next).T) < 6e-3
    act2.fill_(7.0)
    o.gemm_stream(act2, scaled, w_next, "swiglu", up_rows=out_rows, squares=squares, eps=eps)
    assert rel(act2, pm.swiglu(gate_up[:, :out_rows], gate_up[:, out_rows:])) < 1.2e-2
    o.check_error_flag(DEV)
    with pytest.raises(Exception):
        o.gemm_stream(x, act, w_down, "store", norm=(scaled, w_norm, squares))
    with pytest.raises(Exception):
        o.gemm_stream(x, act, w_down, "accumulate", squares=squares, eps=eps)


@pytest.mark.parametrize("m", [5, 17, 40, 64, 128])
@pytest.mark.parametrize("width,inner,out_rows,norm_dtype", [(1032, 2760, 392, torch.float32), (256, 4096, 1536, torch.bfloat16),
                                                            (4096, 4096, 1024, torch.bfloat16), (5120, 4096, 256, torch.float32),
                                                            (3072, 2760, 256, torch.bfloat16)])
def test_a_clustered_few_row_product_prepares_the_norm_that_follows(m, width, inner, out_rows, norm_dtype):
    """The same by the tcgen05 few-row product where its splits of K run as clusters: the blocks that finish
    a tile's rows leave residual * norm weight and one partial sum of squares a block.  Widths that end
    inside a tile (1032 = 8 tiles of 128 and 8 rows) and splits whose rows do not divide evenly (three
    splits: 44, 44 and 40 rows; six: five of 24 and one of 8) are among the cases, if the device holds
    their clusters."""
    from xeno_rt_b200.csrc import ops as o
    torch.manual_seed(m + width + inner)
    eps = 1e-5
    parts = o.gemm_decode_tcgen05_norm_parts(m, width, inner, DEV)
    if parts == 0:
        assert width not in (1032, 256, 4096), "these sizes split K into clusters of 4 and 8 on a B200"
        pytest.skip("the device does not hold this product's clusters all at once")
    resid = torch.randn(m, width, device=DEV) * 2
    act = (torch.randn(m, inner, device=DEV)).to(torch.bfloat16)
    w_down = (torch.randn(width, inner, device=DEV) * 0.05).to(torch.bfloat16)
    w_norm = (1 + 0.1 * torch.randn(width, device=DEV)).to(norm_dtype)
    w_next = (torch.randn(2 * out_rows, width, device=DEV) * 0.05).to(torch.bfloat16)
    x = resid.clone()
    scaled = torch.full((m, width), 9.0, device=DEV, dtype=torch.bfloat16)
    squares = torch.full((parts, m), 9.0, device=DEV)
    o.gemm_decode_tcgen05(x, act, w_down, "accumulate", norm=(scaled, w_norm, squares))
    plain = resid.clone()
    o.gemm_decode_tcgen05(plain, act, w_down, "accumulate")
    assert torch.equal(x, plain) and rel(x, f64(resid) + f64(act) @ f64(w_down).T) < 1e-5
    assert rel(scaled, f64(x) * f64(w_norm)) < 5e-3
    assert rel(squares.sum(0), (f64(x) ** 2).sum(1)) < 1e-5
    again = torch.full_like(squares, 7.0)
    y = resid.clone()
    o.gemm_decode_tcgen05(y, act, w_down, "accumulate", norm=(torch.empty_like(scaled), w_norm, again))
    assert torch.equal(again, squares)  # a fixed order of addition
    normed = pm.rmsnorm(f64(x), f64(w_norm), eps)
    out = torch.empty(m, 2 * out_rows, device=DEV)
    o.gemm_decode_tcgen05(out, scaled, w_next, "store", squares=squares, eps=eps)
    assert rel(out, normed @ f64(w_next).T) < 6e-3
    o.check_error_flag(DEV)
    with pytest.raises(Exception):
        o.gemm_decode_tcgen05(x, act, w_down, "store", norm=(scaled, w_norm, squares))


@pytest.mark.parametrize("m", [129, 300, 1000])
@pytest.mark.parametrize("width,inner,out_rows,norm_dtype", [(1032, 520, 392, torch.float32), (256, 2760, 1536, torch.bfloat16),
                                                            (4096, 1024, 2048, torch.bfloat16)])
def test_a_prompt_product_prepares_the_norm_that_follows_and_the_next_finishes_it(m, width, inner, out_rows, norm_dtype):
    """The same for prompts: the tiled tcgen05 product adds into the residual and leaves residual * norm
    weight and one partial sum of squares a tile of 256 columns; the next tiled product scales its rows."""
    from xeno_rt_b200.csrc import ops as o
    torch.manual_seed(m + width + inner)
    eps = 1e-6
    resid = torch.randn(m, width, device=DEV) * 2
    act = (torch.randn(m, inner, device=DEV)).to(torch.bfloat16)
    w_down = (torch.randn(width, inner, device=DEV) * 0.05).to(torch.bfloat16)
    w_norm = (1 + 0.1 * torch.randn(width, device=DEV)).to(norm_dtype)
    w_next = (torch.randn(2 * out_rows, width, device=DEV) * 0.05).to(torch.bfloat16)
    x = resid.clone()
    scaled = torch.full((m, width), 9.0, device=DEV, dtype=torch.bfloat16)
    squares = torch.full((o.gemm_tcgen05_norm_parts(width), m), 9.0, device=DEV)
    o.gemm_tcgen05(x, act, w_down, "accumulate", norm=(scaled, w_norm, squares))
    plain = resid.clone()
    o.gemm_tcgen05(plain, act, w_down, "accumulate")
    assert torch.equal(x, plain) and rel(x, f64(resid) + f64(act) @ f64(w_down).T) < 1e-5
    assert rel(scaled, f64(x) * f64(w_norm)) < 5e-3
    assert rel(squares.sum(0), (f64(x) ** 2).sum(1)) < 1e-5
    normed = pm.rmsnorm(f64(x), f64(w_norm), eps)
    out = torch.empty(m, 2 * out_rows, device=DEV)
    o.gemm_tcgen05(out, scaled, w_next, "store", squares=squares, eps=eps)
    assert rel(out, normed @ f64(w_next).T) < 6e-3
    act2 = torch.empty(m, out_rows, device=DEV, dtype=torch.bfloat16)
    o.gemm_tcgen05(act2, scaled, w_next, "swiglu", up_rows=out_rows, squares=squares, eps=eps)
    gate_up = normed @ f64(w_next).T
    assert rel(act2, pm.swiglu(gate_up[:, :out_rows], gate_up[:, out_rows:])) < 1.2e-2
    o.check_error_flag(DEV)


def test_attention_prefill_tcgen05_scores_that_jump():
    """The kernel takes its exponents against a reference value that moves only when a row's maximum
    has outgrown it by more than 8 (in base 2), and then rescales what it has accumulated.  Here the
    scores stay small for the first key blocks, then one key far along (position 200) and a still larger
    one (position 330) stand out for the later rows, by scaling those keys: rows before them must not
    feel them, rows after them must be dominated by them, and every row must match the plain attention."""
    nh, nkv, hd, S = 4, 2, 128, 400
    torch.manual_seed(11)
    k = torch.randn(S, nkv, hd, device=DEV) * 0.3
    v = torch.randn(S, nkv, hd, device=DEV)
    q = torch.randn(S, nh * hd, device=DEV) * 0.3
    direction = torch.randn(hd, device=DEV)
    direction /= direction.norm()
    q = (q.view(S, nh, hd) + 6.0 * direction).reshape(S, nh * hd)  # every query leans towards `direction`
    k[200] += 20.0 * direction  # its score is 6 * 20 / sqrt(128) = 10.6 above the others': a factor e^10.6
    k[330] += 45.0 * direction  # and a much larger one later: 23.9
    k_pool, v_pool, table = _cache_for([S], nkv, hd, torch.bfloat16, shuffle_seed=3)
    _fill_cache(k_pool, v_pool, table, 1, k, v)
    qb = q.to(torch.bfloat16)
    cu = torch.tensor([0, S], dtype=torch.int32, device=DEV)
    one = lambda x: torch.tensor([x], dtype=torch.int32, device=DEV)
    out = torch.empty_like(qb)
    ops().attention_prefill_tcgen05(out, qb, k_pool, v_pool, cu, one(1), one(0), table, S, nh, nkv, hd, 1 / math.sqrt(hd))
    from xeno_rt_b200.csrc import ops as o
    o.check_error_flag(DEV)
    bf = lambda x: f64(x.to(torch.bfloat16)).reshape(x.shape[0], -1)
    want = pm.causal_gqa_attention(f64(qb), bf(k), bf(v), nh, nkv, hd)
    assert rel(out, want) < 1.5e-2
    vb = bf(v)
    # after position 330 a row's output is almost exactly the value at 330
    assert np.abs(f64(out[399]).reshape(nh, hd)[0] - vb[330].reshape(nkv, hd)[0]).max() < 0.05
    # and between 200 and 329 mostly the value at 200
    assert np.abs(f64(out[300]).reshape(nh, hd)[0] - vb[200].reshape(nkv, hd)[0]).max() < 0.3
