"""The entry point that allocates nothing (nanoinfer_b200/csrc/no_alloc.h), called as a C program would
call it: through its exported symbol, with raw device pointers.

Some hosts of this library cannot allocate device memory when they need attention (an allocator they
must not enter, no torch at all), so the split decode attention also exists with its scratch built into
the library. This test makes the calls such a host makes and checks the result against the ordinary
entry point, which gets its scratch from the caller. It is collected last on purpose: a run that stops
at the first failure has then already run every other test. It passes alone in a fresh process and after
the other tests alike, since the only state it relies on is the library's own array.
"""
import ctypes
import math
from ctypes import c_float, c_int, c_void_p

import pytest
import torch

from gpu_util import assert_close, make_paged_batch

pytestmark = pytest.mark.gpu


def _call(lib, fn, qkv, out, ctx, bt, page, kp, vp, heads, kv_heads, hd, window, splits, scratch=None):
    args = [c_void_p(qkv.data_ptr()), c_int(qkv.stride(0)), c_void_p(out.data_ptr()), c_void_p(ctx.ctx_lens.data_ptr()),
            c_void_p(bt.data_ptr()), c_int(bt.stride(0)), c_int(page), c_void_p(kp.data_ptr()), c_void_p(vp.data_ptr()),
            c_int(kp.shape[0]), c_int(qkv.shape[0]), c_int(heads), c_int(kv_heads), c_int(hd),
            c_float(1.0 / math.sqrt(hd)), c_int(window), c_int(splits)]
    if scratch is not None:
        args += [c_void_p(scratch[0].data_ptr()), c_void_p(scratch[1].data_ptr()), c_void_p(0)]
    args.append(c_void_p(torch.cuda.current_stream().cuda_stream))
    return fn(*args)


def test_no_alloc_decode_attention_matches_the_ordinary_entry_point_twice():
    from nanoinfer_b200.csrc import build
    lib = ctypes.CDLL(build.build(verbose=False))          # the exported C symbols, nothing else
    lib.nib_last_error.restype = ctypes.c_char_p
    noalloc, ordinary = lib.nib_attention_decode_noalloc, lib.nib_attention_decode_mma
    noalloc.restype = ordinary.restype = c_int

    heads, kv_heads, hd, page = 14, 2, 64, 16
    for round_, (seed, before, splits, window) in enumerate([(1, [0, 63, 700, 2999, 1500], 6, 0),
                                                             (2, [4000, 17, 64], 9, 900)]):
        g = torch.Generator().manual_seed(seed)
        n = len(before)
        ctx, bt = make_paged_batch([1] * n, before, page, 640, "cuda", seed=seed)
        shape = (640, kv_heads, page, hd)
        kp = torch.randn(shape, generator=g).to(torch.bfloat16).cuda()
        vp = torch.randn(shape, generator=g).to(torch.bfloat16).cuda()
        qkv = torch.randn(n, (heads + 2 * kv_heads) * hd, generator=g).to(torch.bfloat16).cuda()
        got = torch.full((n, heads * hd), float("nan"), dtype=torch.bfloat16, device="cuda")
        ref = torch.empty_like(got)
        scratch = (torch.empty(n * heads * splits * hd, device="cuda"), torch.empty(n * heads * splits * 2, device="cuda"))
        torch.cuda.synchronize()
        before_bytes = torch.cuda.memory_allocated()
        rc = _call(lib, noalloc, qkv, got, ctx, bt, page, kp, vp, heads, kv_heads, hd, window, splits)
        assert rc == 0, lib.nib_last_error().decode()
        assert torch.cuda.memory_allocated() == before_bytes
        # the driver's own count of free device memory sees what torch's allocator cannot (a cudaMalloc inside
        # the library); the call above has loaded the kernels' module, so this one can add nothing
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        rc = _call(lib, noalloc, qkv, got, ctx, bt, page, kp, vp, heads, kv_heads, hd, window, splits)
        torch.cuda.synchronize()
        assert rc == 0, lib.nib_last_error().decode()
        assert torch.cuda.mem_get_info()[0] == free_before, "device memory was taken during the call"
        rc = _call(lib, ordinary, qkv, ref, ctx, bt, page, kp, vp, heads, kv_heads, hd, window, splits, scratch)
        assert rc == 0, lib.nib_last_error().decode()
        torch.cuda.synchronize()
        assert_close(got, ref.double(), torch.bfloat16, f"no-alloc call {round_}")
        assert torch.equal(got, ref)       # same kernels, same order of sums

    # more scratch than the library owns: refused with a clear message, nothing launched
    big = 4096
    ctx, bt = make_paged_batch([1] * big, [0] * big, page, big, "cuda", seed=3)
    kp = torch.zeros((big, kv_heads, page, hd), dtype=torch.bfloat16, device="cuda")
    qkv = torch.zeros(big, (heads + 2 * kv_heads) * hd, dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(big, heads * hd, dtype=torch.bfloat16, device="cuda")
    rc = _call(lib, noalloc, qkv, out, ctx, bt, page, kp, kp, heads, kv_heads, hd, 0, 16)
    assert rc != 0 and "need" in lib.nib_last_error().decode() and "built-in array" in lib.nib_last_error().decode()
