"""The decode-attention entry point that allocates nothing (mlxone_attention_decode_static),
called through its exported C symbol as an embedder would call it, against the ordinary entry
point, whose caller provides the scratch. This file is collected last on purpose: if it
fails, a run that stops at the first failure has already run every other test."""

import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"


def library():
    from mlx_one_b200.kernels.build import library_path
    lib = ctypes.CDLL(str(library_path()))
    lib.mlxone_last_error.restype = ctypes.c_char_p
    lib.mlxone_attention_decode_static_capacity.restype = ctypes.c_longlong
    lib.mlxone_attention_decode_scratch.restype = ctypes.c_longlong
    return lib


def case(requests, context, heads, kv_heads, head_dim, page_size, seed):
    generator = torch.Generator().manual_seed(seed)
    blocks = -(-(context + 1) // page_size)
    pages = requests * blocks + 2
    order = torch.randperm(pages, generator=generator)[:requests * blocks].to(torch.int32)
    table = order.view(requests, blocks).contiguous().to(DEVICE)
    kv = torch.randn(2, pages, kv_heads, page_size, head_dim, generator=generator).bfloat16().to(DEVICE)
    q = torch.randn(requests, heads, head_dim, generator=generator).bfloat16().to(DEVICE)
    positions = torch.full((requests,), context, dtype=torch.int32, device=DEVICE)
    return q, kv, table, positions, pages, blocks


def empty_output(q):
    requests, heads, head_dim = q.shape
    return torch.full((requests, heads * head_dim), float("nan"), dtype=torch.bfloat16,
                      device=DEVICE)


def call(lib, name, q, kv, table, positions, pages, blocks, page_size, splits, partial=None,
         out=None):
    requests, heads, head_dim = q.shape
    kv_heads = kv.shape[2]
    out = empty_output(q) if out is None else out
    ptr = lambda t: ctypes.c_void_p(t.data_ptr())
    stream = ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)
    head = [ptr(q), ptr(kv), ptr(table), ctypes.c_int(blocks), ctypes.c_int(page_size),
            ctypes.c_int(pages), ptr(positions), ptr(out)]
    tail = [ctypes.c_int(requests), ctypes.c_int(heads), ctypes.c_int(kv_heads),
            ctypes.c_int(head_dim), ctypes.c_int(splits), ctypes.c_float(head_dim ** -0.5),
            ctypes.c_int(0), stream]
    middle = [] if partial is None else [ptr(partial)]
    code = getattr(lib, name)(*head, *middle, *tail)
    return code, out


def plain_attention(q, kv, table, positions, page_size):
    """softmax(q k^T / sqrt(d)) v over each request's pages, in 64-bit on the host."""
    requests, heads, head_dim = q.shape
    group = heads // kv.shape[2]
    out = torch.empty(requests, heads * head_dim, dtype=torch.float64)
    kv, q, table = kv.double().cpu(), q.double().cpu(), table.cpu()
    for r in range(requests):
        length = int(positions[r]) + 1
        pages = table[r, :-(-length // page_size)].long()
        keys = kv[0, pages].permute(1, 0, 2, 3).reshape(kv.shape[2], -1, head_dim)[:, :length]
        values = kv[1, pages].permute(1, 0, 2, 3).reshape(kv.shape[2], -1, head_dim)[:, :length]
        for h in range(heads):
            scores = keys[h // group] @ q[r, h] * head_dim ** -0.5
            out[r, h * head_dim:(h + 1) * head_dim] = torch.softmax(scores, 0) @ values[h // group]
    return out


def free_bytes():
    """Free device memory as the driver counts it: an allocation by anyone in this process,
    the library included, lowers it (torch's own counters would not see the library's)."""
    torch.cuda.synchronize()
    return torch.cuda.mem_get_info()[0]


def test_static_scratch_entry_point_matches_the_allocating_one():
    lib = library()
    assert lib.mlxone_attention_decode_static_capacity() == 2 * 1024 * 1024
    # calls in a row: each is of another shape than the one before, so the array still holds
    # partial results that this call does not overwrite. The third nearly fills the array
    # (2,095,104 of 2,097,152 floats), the fourth has a single split and needs no scratch.
    for number, (requests, context, heads, kv_heads, head_dim, page, splits, seed) in enumerate((
            (8, 1500, 32, 8, 64, 16, 4, 0), (3, 700, 6, 2, 48, 8, 3, 1),
            (8, 4100, 32, 8, 64, 16, 124, 2), (2, 90, 4, 4, 32, 4, 1, 3))):
        q, kv, table, positions, pages, blocks = case(requests, context, heads, kv_heads,
                                                      head_dim, page, seed)
        floats = lib.mlxone_attention_decode_scratch(requests, heads, head_dim, splits)
        assert floats <= lib.mlxone_attention_decode_static_capacity()
        partial = torch.empty(max(floats, 1), dtype=torch.float32, device=DEVICE)
        code, want = call(lib, "mlxone_attention_decode", q, kv, table, positions, pages, blocks,
                          page, splits, partial)
        assert code == 0, lib.mlxone_last_error().decode()
        got = empty_output(q)                   # the caller's buffers exist before the call
        before = (free_bytes(), torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
        code, got = call(lib, "mlxone_attention_decode_static", q, kv, table, positions, pages,
                         blocks, page, splits, out=got)
        assert code == 0, lib.mlxone_last_error().decode()
        after = (free_bytes(), torch.cuda.memory_allocated(), torch.cuda.memory_reserved())
        if number:
            # (the very first call may make the driver load the library's device image, array
            # included; from the second call on nothing in the process may take device memory)
            assert after == before
        assert not torch.isnan(got.float()).any()
        torch.testing.assert_close(got.float(), want.float(), atol=2e-2, rtol=2e-2)
        assert torch.equal(got, want)          # same kernel, same order of operations
        if requests * context <= 8 * 1500:
            plain = plain_attention(q, kv, table, positions, page)
            torch.testing.assert_close(got.double().cpu(), plain, atol=2e-2, rtol=2e-2)


def test_static_scratch_entry_point_refuses_what_does_not_fit():
    lib = library()
    q, kv, table, positions, pages, blocks = case(64, 300, 64, 8, 128, 16, 2)
    code, out = call(lib, "mlxone_attention_decode_static", q, kv, table, positions, pages,
                     blocks, 16, 8)
    assert code != 0
    message = lib.mlxone_last_error().decode()
    assert "scratch" in message and "fewer splits" in message
    torch.cuda.synchronize()
    assert torch.isnan(out.float()).all()       # nothing was launched
    # one split more than the array holds for this shape (124 fit, see the test above)
    q, kv, table, positions, pages, blocks = case(8, 4100, 32, 8, 64, 16, 4)
    assert lib.mlxone_attention_decode_scratch(8, 32, 64, 125) > \
        lib.mlxone_attention_decode_static_capacity()
    code, out = call(lib, "mlxone_attention_decode_static", q, kv, table, positions, pages,
                     blocks, 16, 125)
    assert code != 0 and "125 splits" in lib.mlxone_last_error().decode()
    torch.cuda.synchronize()
    assert torch.isnan(out.float()).all()
