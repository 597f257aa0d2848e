"""The decode attention entry point that allocates nothing, called through its exported C symbol.

Why it exists: some callers of the kernel library cannot call cudaMalloc when they need the
kernel (allocation is forbidden or too slow where they run, or their memory was handed out in
full at start-up), and split decode attention needs scratch for its partial results.
``xrt_attention_decode_static`` keeps that scratch in a fixed 8 MiB array inside the library.
This test calls it with plain pointers, twice in a row on different inputs (the array keeps the
first call's contents, which must not leak into the second), compares with the ordinary entry
point, and checks that a call beyond the array's size is refused with a message that says why.
The file's name makes pytest collect it last.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _entry():
    from xeno_rt_b200.csrc import build
    lib = ctypes.CDLL(build.build())
    fn = lib.xrt_attention_decode_static
    P, I = ctypes.c_void_p, ctypes.c_int
    fn.argtypes = [P, P, P, P, P, P, P, I, I, I, I, I, ctypes.c_float, I, I, I, P, ctypes.c_char_p, I]
    fn.restype = I
    return fn


def _case(seed, lens, nh, nkv, hd, n_blocks=40):
    g = torch.Generator(device="cpu").manual_seed(seed)
    k_pool = torch.randn(n_blocks, nkv, 64, hd, generator=g).to(DEV).to(torch.bfloat16)
    v_pool = torch.randn(n_blocks, nkv, 64, hd, generator=g).to(DEV).to(torch.bfloat16)
    per_seq = max((n + 63) // 64 for n in lens)
    perm = torch.randperm(n_blocks, generator=g)
    table = torch.full((len(lens), per_seq), -1, dtype=torch.int32)
    at = 0
    for s, n in enumerate(lens):
        nb = (n + 63) // 64
        table[s, :nb] = perm[at:at + nb].to(torch.int32)
        at += nb
    q = torch.randn(len(lens), nh * hd, generator=g).to(DEV).to(torch.bfloat16)
    tok_slot = torch.arange(len(lens), dtype=torch.int32, device=DEV)
    tok_pos = torch.tensor([n - 1 for n in lens], dtype=torch.int32, device=DEV)
    return q, k_pool, v_pool, tok_slot, tok_pos, table.to(DEV)


def test_static_scratch_entry_point_matches_the_ordinary_one_twice_in_a_row():
    from xeno_rt_b200.csrc import ops
    fn = _entry()
    nh, nkv, hd, chunk, n_splits = 8, 2, 128, 128, 6
    message = ctypes.create_string_buffer(512)
    stream = torch.cuda.current_stream().cuda_stream
    for seed, lens in ((1, [700, 64, 65, 1]), (2, [130, 768, 5, 300])):
        q, k_pool, v_pool, tok_slot, tok_pos, table = _case(seed, lens, nh, nkv, hd)
        want = torch.empty_like(q)
        ops.attention_decode(want, q, k_pool, v_pool, tok_slot, tok_pos, table, nh, nkv, hd, 1 / math.sqrt(hd), 0,
                             chunk, n_splits)
        got = torch.full_like(q, 9.0)
        status = fn(got.data_ptr(), q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), tok_slot.data_ptr(),
                    tok_pos.data_ptr(), table.data_ptr(), table.shape[1], len(lens), nh, nkv, hd,
                    1 / math.sqrt(hd), 0, chunk, n_splits, stream, message, 512)
        assert status == 0, message.value
        torch.cuda.synchronize()
        # same kernels, same split: the tolerance of the decode attention tests is far from needed
        assert torch.allclose(got.float(), want.float(), atol=1.5e-2)
        assert torch.equal(got, want)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    fn = _entry()
    nh, nkv, hd = 32, 8, 128
    q, k_pool, v_pool, tok_slot, tok_pos, table = _case(3, [100] * 64, nh, nkv, hd, n_blocks=130)
    out = torch.full_like(q, 3.0)
    message = ctypes.create_string_buffer(512)
    # 64 tokens x 32 heads x 16 splits x 130 floats = 17 MB: more than the 8 MiB the library holds
    status = fn(out.data_ptr(), q.data_ptr(), k_pool.data_ptr(), v_pool.data_ptr(), tok_slot.data_ptr(),
                tok_pos.data_ptr(), table.data_ptr(), table.shape[1], 64, nh, nkv, hd, 0.1, 0, 64, 16,
                torch.cuda.current_stream().cuda_stream, message, 512)
    assert status == -3
    text = message.value.decode()
    assert "bytes of scratch" in text and "8388608" in text
    torch.cuda.synchronize()
    assert bool((out == 3.0).all())  # nothing was launched
