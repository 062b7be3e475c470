"""Allocation-free decode-attention entry point, called through its exported C symbol and compared with the
ordinary entry point (caller-supplied scratch) on two calls in a row.  Collected last on purpose: it must hold
both in a fresh process and after every other GPU test has used the library."""
import ctypes as C
import gc

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(seed, R, H, Hkv, D, ctx_max, split_len):
    from hipengine_b200.ops import kernels as K
    g = torch.Generator(device="cuda").manual_seed(seed)
    page = 16
    max_pages = (ctx_max + page - 1) // page
    n_pages = R * max_pages + 1
    cache = (torch.randn(n_pages, 2, Hkv, page, D, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    perm = torch.randperm(n_pages - 1, device="cuda", generator=g).to(torch.int32) + 1
    bt = perm[: R * max_pages].reshape(R, max_pages).contiguous()
    slot = torch.arange(R, device="cuda", dtype=torch.int32)
    ctx = torch.randint(1, ctx_max + 1, (R,), device="cuda", generator=g).to(torch.int32)
    ctx[0] = ctx_max
    q = torch.randn(R, H, D, device="cuda", generator=g).to(torch.bfloat16)
    gate = torch.randn(R, H, D, device="cuda", generator=g).to(torch.bfloat16)
    max_splits = (ctx_max + split_len - 1) // split_len
    a = K._AttnDecArgs()
    a.q, a.gate, a.kv_cache = q.data_ptr(), gate.data_ptr(), cache.data_ptr()
    a.block_table, a.slot, a.ctx_len = bt.data_ptr(), slot.data_ptr(), ctx.data_ptr()
    a.R, a.H, a.Hkv, a.D, a.page, a.max_pages = R, H, Hkv, D, page, max_pages
    a.split_len, a.max_splits, a.window, a.scale = split_len, max_splits, 0, D ** -0.5
    keep = (cache, bt, slot, ctx, q, gate)
    return a, keep, max_splits


def test_noalloc_matches_regular_entry_point_twice():
    from hipengine_b200.core import native as N
    from hipengine_b200.ops import kernels as K
    lib = N.lib()
    fn = lib.he_attn_decode_noalloc
    fn.restype = C.c_int
    cap = lib.he_attn_decode_noalloc_capacity
    cap.restype = C.c_longlong
    assert cap() == 2 * 1024 * 1024
    stream = C.c_void_p(torch.cuda.current_stream().cuda_stream)
    for call, (seed, R, H, Hkv, D, ctx_max, split_len) in enumerate([(1, 3, 8, 2, 128, 200, 64),
                                                                     (2, 2, 24, 4, 256, 333, 128)]):
        a, keep, max_splits = _case(seed, R, H, Hkv, D, ctx_max, split_len)
        ref = torch.zeros(R, H * D, device="cuda", dtype=torch.bfloat16)
        out = torch.zeros_like(ref)
        part = torch.empty(K.attn_decode_scratch_floats(R, H, max_splits, D), device="cuda")
        a.partial, a.out = part.data_ptr(), ref.data_ptr()
        assert lib.he_attn_decode(C.byref(a), stream) == 0
        a.partial, a.out = None, out.data_ptr()
        # count allocator calls, not live bytes: objects of earlier tests may be garbage-collected (and their
        # memory freed) at any moment, which says nothing about this call
        gc.collect()
        torch.cuda.synchronize()
        before = torch.cuda.memory_stats().get("allocation.all.allocated", 0)
        assert fn(C.byref(a), stream) == 0, f"call {call}"
        torch.cuda.synchronize()
        assert torch.cuda.memory_stats().get("allocation.all.allocated", 0) == before
        torch.testing.assert_close(out.float(), ref.float(), atol=2e-2, rtol=2e-2)
        assert out.float().abs().max() > 0


def test_noalloc_rejects_oversized_request():
    from hipengine_b200.core import native as N
    lib = N.lib()
    fn = lib.he_attn_decode_noalloc
    fn.restype = C.c_int
    a, keep, _ = _case(3, 2, 8, 2, 128, 64, 64)
    a.R, a.max_splits = 64, 4096      # 64 * 8 * 4096 * 130 floats: far beyond the built-in scratch
    out = torch.zeros(2, 8 * 128, device="cuda", dtype=torch.bfloat16)
    a.out = out.data_ptr()
    assert fn(C.byref(a), C.c_void_p(torch.cuda.current_stream().cuda_stream)) == -3
    torch.cuda.synchronize()
    assert float(out.float().abs().max()) == 0.0
