"""The entry point for callers that cannot allocate device memory, called the way such a
caller would: through its exported C symbol, with nothing but raw pointers.  Its output
must equal the engine's own decode attention (whose scratch PyTorch's allocator provides)
on two calls in a row that share the built-in scratch array, and both must agree with the
plain PyTorch statement of attention.  A table that lacks a page for a visible key must show
in the status word, not in a fault.  Collected last, so that a failure here cannot keep any
other test from running."""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def c_entry():
    from dlm_b200.build import kernels_library_path
    lib = ctypes.CDLL(kernels_library_path())
    fn = lib.dlm_b200_decode_attention_noalloc
    fn.restype = ctypes.c_int
    vp, i32, f32 = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    fn.argtypes = [vp, vp, vp, vp, i32, vp, vp, vp, i32, i32, i32, i32, i32, i32, i32, f32, i32, vp,
                   ctypes.c_char_p, ctypes.c_size_t]
    return fn


def c_status():
    from dlm_b200.build import kernels_library_path
    lib = ctypes.CDLL(kernels_library_path())
    fn = lib.dlm_b200_noalloc_status
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p]
    return fn


def read_status():
    word = torch.full((1,), -1, dtype=torch.int32).pin_memory()
    assert c_status()(word.data_ptr(), torch.cuda.current_stream().cuda_stream) == 0
    torch.cuda.synchronize()
    return int(word[0])


def plain_attention(case, nh, nkv, hd, window):
    from plain_ops import PlainOps
    q, k, v, table, cu_q, kv_len = case
    longest = int(kv_len.max())
    spans = (cu_q[1:] - cu_q[:-1]).tolist()
    return PlainOps().attention(q, k, v, table, cu_q, kv_len, window, 1 / math.sqrt(hd), nh, nkv, hd,
                                max(spans), longest)


def make_case(seed, reqs, nh, nkv, hd, ps):
    g = torch.Generator(device="cuda").manual_seed(seed)
    pages = sum(-(-n // ps) for n in reqs) + 2
    k = torch.randn((pages, nkv, ps, hd), generator=g, device="cuda").to(torch.bfloat16)
    v = torch.randn((pages, nkv, ps, hd), generator=g, device="cuda").to(torch.bfloat16)
    width = max(-(-n // ps) for n in reqs) + 1
    table = torch.full((len(reqs), width), -1, dtype=torch.int32)
    order = torch.randperm(pages, generator=torch.Generator().manual_seed(seed)).tolist()
    it = iter(order)
    for r, n in enumerate(reqs):
        for i in range(-(-n // ps)):
            table[r, i] = next(it)
    R = len(reqs)
    q = torch.randn((R, nh * hd), generator=g, device="cuda").to(torch.bfloat16)
    cu_q = torch.arange(R + 1, dtype=torch.int32, device="cuda")
    kv_len = torch.tensor(reqs, dtype=torch.int32, device="cuda")
    return q, k, v, table.cuda(), cu_q, kv_len


def run_both(fn, ops, case, nh, nkv, hd, ps, window):
    q, k, v, table, cu_q, kv_len = case
    R, longest = table.shape[0], int(kv_len.max())
    scale = 1 / math.sqrt(hd)
    want = ops.attention(q, k, v, table, cu_q, kv_len, window, scale, nh, nkv, hd, 1, longest, R)
    out = torch.zeros_like(q)
    msg = ctypes.create_string_buffer(256)
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.shape[1], cu_q.data_ptr(),
            kv_len.data_ptr(), out.data_ptr(), R, nh, nkv, hd, ps, k.shape[0], window, scale, longest,
            torch.cuda.current_stream().cuda_stream, msg, 256)
    assert rc == 0, msg.value.decode()
    torch.cuda.synchronize()
    return out, want


def test_no_alloc_entry_matches_engine_kernel_twice():
    from dlm_b200.ops import native_ops
    ops = native_ops(fast=True)
    fn = c_entry()
    # head_dim 72 has no tensor-core decode kernel, so the engine's own call runs the same FMA kernel
    nh, nkv, hd, ps = 8, 2, 72, 16
    first = make_case(1, [300, 17, 1, 130], nh, nkv, hd, ps)
    out1, want1 = run_both(fn, ops, first, nh, nkv, hd, ps, 0)
    # the same tolerance as the kernel tests use for bfloat16 attention
    torch.testing.assert_close(out1.float(), want1.float(), rtol=2e-2, atol=1e-2)
    # a second call with other inputs (and a window) reuses the array with the first call's leftovers in it
    second = make_case(2, [64, 257, 33], nh, nkv, hd, ps)
    out2, want2 = run_both(fn, ops, second, nh, nkv, hd, ps, 40)
    torch.testing.assert_close(out2.float(), want2.float(), rtol=2e-2, atol=1e-2)
    # both paths run the same kernels in the same order: the results are in fact identical
    assert torch.equal(out1, want1) and torch.equal(out2, want2)
    # and both are attention: the plain statement of it gives the same numbers (request lengths from 1 to
    # 300 under one max_kv_len, so some key splits are empty and are merged as such)
    torch.testing.assert_close(out1.float(), plain_attention(first, nh, nkv, hd, 0).float(), rtol=2e-2, atol=1e-2)
    torch.testing.assert_close(out2.float(), plain_attention(second, nh, nkv, hd, 40).float(), rtol=2e-2, atol=1e-2)
    assert read_status() == 0


def test_no_alloc_entry_skips_requests_with_other_than_one_token():
    """A request that brings two tokens to the step is not this kernel's: its output rows stay as they were."""
    fn = c_entry()
    nh, nkv, hd, ps = 4, 2, 64, 16
    q, k, v, table, _, kv_len = make_case(3, [90, 40, 200], nh, nkv, hd, ps)
    cu_q = torch.tensor([0, 1, 3, 4], dtype=torch.int32, device="cuda")        # the middle request has 2 tokens
    g = torch.Generator(device="cuda").manual_seed(9)
    q = torch.randn((4, nh * hd), generator=g, device="cuda").to(torch.bfloat16)
    out = torch.full_like(q, 7.0)
    msg = ctypes.create_string_buffer(256)
    rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), table.shape[1], cu_q.data_ptr(),
            kv_len.data_ptr(), out.data_ptr(), 3, nh, nkv, hd, ps, k.shape[0], 0, 1 / math.sqrt(hd), 200,
            torch.cuda.current_stream().cuda_stream, msg, 256)
    assert rc == 0, msg.value.decode()
    torch.cuda.synchronize()
    assert bool((out[1:3] == 7.0).all())
    want = plain_attention((q, k, v, table, cu_q, kv_len), nh, nkv, hd, 0)
    torch.testing.assert_close(out[[0, 3]].float(), want[[0, 3]].float(), rtol=2e-2, atol=1e-2)
    assert read_status() == 0


def test_no_alloc_status_reports_a_missing_page():
    """A visible key whose table entry is -1: the kernel skips the page (no fault), the call still returns
    0 ("launched"), and the status word says 3 until the next call clears it."""
    fn = c_entry()
    nh, nkv, hd, ps = 4, 2, 64, 16
    case = make_case(4, [100, 50], nh, nkv, hd, ps)
    q, k, v, table, cu_q, kv_len = case
    good_out = torch.zeros_like(q)
    msg = ctypes.create_string_buffer(256)

    def call(tbl, out):
        rc = fn(q.data_ptr(), k.data_ptr(), v.data_ptr(), tbl.data_ptr(), tbl.shape[1], cu_q.data_ptr(),
                kv_len.data_ptr(), out.data_ptr(), 2, nh, nkv, hd, ps, k.shape[0], 0, 1 / math.sqrt(hd), 100,
                torch.cuda.current_stream().cuda_stream, msg, 256)
        assert rc == 0, msg.value.decode()

    broken = table.clone()
    broken[0, 2] = -1                       # keys 32..47 of the first request have no page
    bad_out = torch.zeros_like(q)
    call(broken, bad_out)
    assert read_status() == 3
    call(table, good_out)
    assert read_status() == 0               # cleared by the next call
    torch.testing.assert_close(good_out.float(), plain_attention(case, nh, nkv, hd, 0).float(), rtol=2e-2, atol=1e-2)
    # the other request of the broken call was not affected
    assert torch.equal(bad_out[1], good_out[1])
    assert c_status()(None, None) == 1


def test_no_alloc_entry_refuses_what_does_not_fit():
    fn = c_entry()
    msg = ctypes.create_string_buffer(256)
    # 512 requests x 64 heads x splits x 130 floats is far beyond the built-in 4 MiB: refused, nothing launched
    rc = fn(0, 0, 0, 0, 4, 0, 0, 0, 512, 64, 8, 128, 16, 1, 0, 0.1, 4096, 0, msg, 256)
    assert rc == 1 and b"exceed the built-in maximum" in msg.value
    rc = fn(0, 0, 0, 0, 4, 0, 0, 0, 2, 8, 2, 12, 16, 1, 0, 0.1, 64, 0, msg, 256)
    assert rc == 1 and b"head_dim" in msg.value
