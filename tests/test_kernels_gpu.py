"""Each CUDA kernel alone against its plain PyTorch statement (tests/torch_ops.py), at sizes other
than the engine's test models: widths and vocabularies that are no power of two, head sizes in steps
of 16, odd head counts and groups, page sizes 8 and 16, rows that do not fill a tile."""
import math

import pytest
import torch

from gpu_util import assert_close, make_paged_batch
from torch_ops import TorchOps

pytestmark = pytest.mark.gpu
DTYPES = [torch.float32, torch.bfloat16]
REF = TorchOps()


@pytest.fixture(scope="module")
def K():
    from nanoinfer_b200.csrc.lib import load_kernels
    return load_kernels()


def rnd(shape, dtype, seed, scale=1.0, device="cuda"):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype).to(device)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,hidden,vocab", [(1, 40, 11), (37, 896, 1000), (5, 1000, 503)])
def test_embed(K, dtype, m, hidden, vocab):
    table = rnd((vocab, hidden), dtype, 1)
    ids = torch.randint(0, vocab, (m,), generator=torch.Generator().manual_seed(2)).int().cuda()
    out, ref = torch.empty(m, hidden, device="cuda"), torch.empty(m, hidden, device="cuda")
    K.embed(ids, table, out)
    REF.embed(ids, table, ref)
    assert torch.equal(out, ref)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden,eps", [(1, 64, 1e-6), (33, 896, 1e-5), (7, 1000, 1e-3), (300, 24, 1e-6)])
def test_rmsnorm(K, dtype, rows, hidden, eps):
    x = rnd((rows, hidden), torch.float32, 3, scale=3.0)
    gain = 1 + 0.1 * rnd((hidden,), torch.float32, 4)
    out, ref = torch.empty(rows, hidden, dtype=dtype, device="cuda"), torch.empty(rows, hidden, dtype=dtype, device="cuda")
    K.rmsnorm(x, gain, eps, out, None)
    REF.rmsnorm(x, gain, eps, ref, None)
    assert_close(out, ref, dtype, "rmsnorm")
    sel = torch.tensor([rows - 1, 0, rows // 2], dtype=torch.int32, device="cuda")
    out2, ref2 = torch.empty(3, hidden, dtype=dtype, device="cuda"), torch.empty(3, hidden, dtype=dtype, device="cuda")
    K.rmsnorm(x, gain, eps, out2, sel)
    REF.rmsnorm(x, gain, eps, ref2, sel)
    assert_close(out2, ref2, dtype, "rmsnorm rows")
    assert torch.equal(out2, out[sel.long()])   # a row's result does not depend on the batch


def _ref_linear_f64(a, w, bias):
    y = a.double() @ w.double().t()
    return y if bias is None else y + bias.double()


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,n,k", [(1, 503, 192), (3, 64, 64), (65, 130, 72), (200, 896, 896), (17, 1000, 344), (2, 9, 5)])
def test_linear_modes(K, dtype, m, n, k):
    a, w = rnd((m, k), dtype, 5), rnd((n, k), dtype, 6, scale=0.05)
    bias = rnd((n,), torch.float32, 7)
    ref = _ref_linear_f64(a, w, bias)
    out = torch.empty(m, n, dtype=dtype, device="cuda")
    K.linear(a, w, bias, out, "store")
    assert_close(out, ref.to(dtype) if dtype == torch.bfloat16 else ref, dtype, "linear store")
    out32 = torch.empty(m, n, device="cuda")
    K.linear(a, w, None, out32, "f32")
    assert_close(out32, _ref_linear_f64(a, w, None), torch.float32, "linear f32")
    res = rnd((m, n), torch.float32, 8)
    acc = res.clone()
    K.linear(a, w, None, acc, "add")
    assert_close(acc, res.double() + _ref_linear_f64(a, w, None), torch.float32, "linear add")


@pytest.mark.parametrize("dtype", DTYPES)
def test_linear_rows_do_not_depend_on_batch(K, dtype):
    a, w = rnd((77, 200), dtype, 9), rnd((150, 200), dtype, 10, scale=0.05)
    full = torch.empty(77, 150, device="cuda")
    K.linear(a, w, None, full, "f32")
    for lo, hi in ((0, 1), (5, 8), (60, 77)):
        part = torch.empty(hi - lo, 150, device="cuda")
        K.linear(a[lo:hi].contiguous(), w, None, part, "f32")
        assert torch.equal(part, full[lo:hi])


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("m,inter,k", [(1, 320, 192), (70, 200, 144), (9, 4864, 896)])
def test_linear_swiglu(K, dtype, m, inter, k):
    a, w = rnd((m, k), dtype, 11), rnd((2 * inter, k), dtype, 12, scale=0.08)
    out, ref = torch.empty(m, inter, dtype=dtype, device="cuda"), torch.empty(m, inter, dtype=dtype, device="cuda")
    K.linear_swiglu(a, w, out)
    REF.linear_swiglu(a, w, ref)
    assert_close(out, ref, dtype, "swiglu")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,hd,rot,page", [(4, 2, 16, 16, 16), (6, 1, 32, 32, 8), (3, 3, 48, 48, 8),
                                                        (14, 2, 64, 64, 16), (5, 5, 80, 32, 4), (2, 1, 128, 128, 64)])
def test_rope_store(K, dtype, heads, kv_heads, hd, rot, page):
    from nanoinfer_b200.parts.position import rotary_tables
    q_lens, before = [5, 1, 19], [0, 37, 11]
    num_pages = 40
    ctx, bt = make_paged_batch(q_lens, before, page, num_pages, "cuda", seed=1)
    m = sum(q_lens)
    cos, sin = rotary_tables(128, rot, 10000.0)
    rotary = (cos.cuda(), sin.cuda(), rot)
    qkv = rnd((m, (heads + 2 * kv_heads) * hd), dtype, 13)
    qkv_ref = qkv.clone()
    shape = (num_pages, kv_heads, page, hd)
    kp, vp = torch.zeros(shape, dtype=dtype, device="cuda"), torch.zeros(shape, dtype=dtype, device="cuda")
    kr, vr = torch.zeros_like(kp), torch.zeros_like(vp)
    K.rope_store(qkv, heads, kv_heads, hd, ctx.positions, ctx.req_index, rotary, bt, page, kp, vp, True)
    REF.rope_store(qkv_ref, heads, kv_heads, hd, ctx.positions, ctx.req_index, rotary, bt, page, kr, vr, True)
    assert_close(qkv, qkv_ref, dtype, "rope qkv")
    assert_close(kp, kr, dtype, "k pages")
    assert torch.equal(vp, vr)
    # without writing, pages stay as they are
    kp2 = torch.zeros_like(kp)
    q2 = qkv_ref.clone()
    K.rope_store(q2, heads, kv_heads, hd, ctx.positions, ctx.req_index, None, bt, page, kp2, kp2, False)
    assert torch.equal(q2, qkv_ref) and not kp2.any()


def _fill_cache(ctx, bt, page, num_pages, kv_heads, hd, dtype, seed):
    """Random keys and values for every position of every request, in pages."""
    shape = (num_pages, kv_heads, page, hd)
    kp, vp = rnd(shape, dtype, seed), rnd(shape, dtype, seed + 1)
    return kp, vp


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("heads,kv_heads,hd,page,window", [
    (4, 2, 16, 16, 0), (6, 1, 32, 8, 0), (3, 3, 48, 8, 24), (14, 2, 64, 16, 0), (7, 7, 80, 4, 0),
    (8, 2, 128, 16, 100), (2, 1, 256, 16, 0), (5, 1, 96, 32, 7), (4, 4, 64, 16, 0), (2, 2, 128, 8, 30), (1, 1, 64, 32, 0),
    (32, 2, 64, 16, 0)])
def test_attention_mixed_batch(K, dtype, heads, kv_heads, hd, page, window):
    q_lens, before = [1, 33, 2, 1], [130, 0, 77, 0]
    num_pages = 64
    ctx, bt = make_paged_batch(q_lens, before, page, num_pages * (16 // min(page, 16)), "cuda", seed=2)
    kp, vp = _fill_cache(ctx, bt, page, kp_pages := bt.max().item() + 1, kv_heads, hd, dtype, 20)
    m = sum(q_lens)
    qkv = rnd((m, (heads + 2 * kv_heads) * hd), dtype, 22)
    out, ref = (torch.empty(m, heads * hd, dtype=dtype, device="cuda") for _ in range(2))
    scale = 1.0 / math.sqrt(hd)
    K.attention(qkv, out, heads, kv_heads, hd, scale, window, ctx, bt, page, kp, vp)
    REF.attention(qkv, ref, heads, kv_heads, hd, scale, window, ctx, bt, page, kp, vp)
    assert_close(out, ref, dtype, "attention")


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("window", [0, 50])
def test_attention_finds_one_far_key(K, dtype, window):
    """One key among hundreds carries the whole score: the result must be that key's value. Placed at
    the first position, at page edges, at the window's first key, at the query's own position; and just
    outside the window, where it must NOT be seen."""
    heads, kv_heads, hd, page = 4, 2, 64, 16
    ctx_len = 403
    ctx, bt = make_paged_batch([1], [ctx_len - 1], page, 40, "cuda", seed=3)
    pos = ctx_len - 1
    lo = max(0, pos - window + 1) if window else 0
    spots = [lo, lo + 1, pos, pos - 1, (pos // page) * page, (pos // page) * page - 1]
    if window:
        spots.append(lo - 1)            # invisible
    else:
        spots += [0, 15, 16, 17, 255, 256]
    for spot in spots:
        kp, vp = _fill_cache(ctx, bt, page, 40, kv_heads, hd, dtype, 30)
        kp.mul_(0.05)
        qkv = rnd((1, (heads + 2 * kv_heads) * hd), dtype, 31)
        phys = bt[0, spot // page].item()
        qv = qkv.view(1, heads + 2 * kv_heads, hd)
        # key at `spot` of kv head 1 is 12 * (query head 3) / |q|: score ~ 12 * |q| * sqrt... dominates
        q3 = qv[0, 3].float()
        kp[phys, 1, spot % page] = (q3 / q3.norm() * 40.0).to(dtype)
        out, ref = (torch.empty(1, heads * hd, dtype=dtype, device="cuda") for _ in range(2))
        scale = 1.0 / math.sqrt(hd)
        K.attention(qkv, out, heads, kv_heads, hd, scale, window, ctx, bt, page, kp, vp)
        REF.attention(qkv, ref, heads, kv_heads, hd, scale, window, ctx, bt, page, kp, vp)
        assert_close(out, ref, dtype, f"far key at {spot}")
        o3 = out.view(heads, hd)[3].float()
        v_spot = vp[phys, 1, spot % page].float()
        seen = (o3 - v_spot).abs().max().item() < 0.05
        assert seen == (spot >= lo), f"key at {spot}: seen={seen}, window starts at {lo}"


@pytest.mark.parametrize("window", [0, 50])
@pytest.mark.parametrize("route,hd,q_len,options", [
    ("tcgen05 prefill", 64, 2, {}), ("tcgen05 prefill", 64, 33, {}), ("tcgen05 prefill", 128, 2, {}), ("tcgen05 prefill", 128, 33, {}),
    ("mma.sync prefill", 48, 2, {}), ("mma.sync prefill", 48, 33, {}), ("mma.sync prefill", 64, 33, {"force_mma_prefill": True}),
    ("cp.async decode", 64, 1, {"decode_tma": False}), ("cp.async decode", 128, 1, {"decode_tma": False})])
def test_attention_routes_find_one_far_key(K, route, hd, q_len, options, window):
    """The far-key check on the other attention kernels (bfloat16): a prompt portion that starts inside a page on the
    tcgen05 and the mma.sync prefill kernels, and a decoded token on the cp.async decode kernel. For the first and
    the last query of the portion, one key carries the whole score: the window's first key, the query's own
    position, the first position of all (no window), and the key just before the window, which must NOT be seen."""
    dtype = torch.bfloat16
    heads, kv_heads, page = 4, 2, 16
    before = 305                                   # 305 % 16 == 1: the portion starts inside a page
    ctx_len = before + q_len
    K = K.with_options(**options)
    ctx, bt = make_paged_batch([q_len], [before], page, 40, "cuda", seed=3)
    scale = 1.0 / math.sqrt(hd)
    for r in sorted({0, q_len - 1}):
        pos = before + r
        lo = max(0, pos - window + 1) if window else 0
        spots = [lo, pos] + ([lo - 1] if window else [0, before - 1, before])
        for spot in spots:
            kp, vp = _fill_cache(ctx, bt, page, 40, kv_heads, hd, dtype, 30)
            kp.mul_(0.05)
            qkv = rnd((q_len, (heads + 2 * kv_heads) * hd), dtype, 31)
            phys = bt[0, spot // page].item()
            q3 = qkv.view(q_len, heads + 2 * kv_heads, hd)[r, 3].float()
            kp[phys, 1, spot % page] = (q3 / q3.norm() * 40.0).to(dtype)     # aligned with query head 3 of row r
            out, ref = (torch.empty(q_len, heads * hd, dtype=dtype, device="cuda") for _ in range(2))
            K.attention(qkv, out, heads, kv_heads, hd, scale, window, ctx, bt, page, kp, vp)
            REF.attention(qkv, ref, heads, kv_heads, hd, scale, window, ctx, bt, page, kp, vp)
            assert_close(out, ref, dtype, f"{route}: far key at {spot}, query {r}")
            o3 = out.view(q_len, heads, hd)[r, 3].float()
            seen = (o3 - vp[phys, 1, spot % page].float()).abs().max().item() < 0.05
            assert seen == (lo <= spot <= pos), f"{route}: key at {spot}, query at {pos}: seen={seen}, window starts at {lo}"
    assert K.attention_tc_error() == 0 and K.attention_decode_tma_error() == 0


@pytest.mark.parametrize("rows", [5, 200])
@pytest.mark.parametrize("vocab", [11, 503, 4099, 151936])
def test_argmax_first_maximum(K, vocab, rows):
    """One CTA per row, or (few rows of a large vocabulary) many CTAs per row with the pieces' results
    merged by the last one: ties across pieces go to the first index, NaN never wins, an all-negative
    row works, and two calls in a row agree (the counters are left ready)."""
    logits = rnd((rows, vocab), torch.float32, 40)
    logits[1, vocab // 2] = 50.0
    logits[2, 3] = 60.0
    logits[2, vocab - 1] = 60.0      # a tie: the first wins
    logits[3, vocab - 1] = 70.0
    logits[4] = -logits[4].abs() - 1.0
    logits[4, vocab // 3] = float("nan")
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    K.argmax(logits, out)
    ref = logits.cpu().clone()
    ref[4, vocab // 3] = -float("inf")
    assert out.tolist() == torch.argmax(ref, dim=-1).tolist()
    assert out[2].item() == 3 and out[3].item() == vocab - 1
    again = torch.empty_like(out)
    K.argmax(logits, again)
    assert torch.equal(out, again)


@pytest.mark.parametrize("tma", [True, False])
@pytest.mark.parametrize("splits", [0, 1, 3, 8])
@pytest.mark.parametrize("heads,kv_heads,hd,window,page", [
    (14, 2, 64, 0, 16), (16, 1, 64, 0, 16), (12, 1, 32, 700, 16), (20, 1, 16, 0, 16), (8, 8, 128, 0, 16), (9, 3, 112, 0, 16),
    (14, 2, 64, 700, 8), (8, 2, 128, 100, 32), (7, 1, 64, 0, 64), (4, 2, 128, 0, 8)])
def test_attention_decode_long_context_split_over_ctas(K, heads, kv_heads, hd, window, page, splits, tma):
    """Single decoded tokens at contexts from 1 to 3000 keys (tile edges 63, 64, 65), any number of
    splits, up to 16 query heads per kv head on the decode kernels (20: the prefill kernel takes them);
    with the pages fetched by TMA (head sizes 64 and 128, pages of 8..64) and by cp.async."""
    dtype = torch.bfloat16
    before = [0, 62, 63, 64, 2999, 1500]
    q_lens = [1] * len(before)
    n_pages = 6 * (3000 // page + 2)
    ctx, bt = make_paged_batch(q_lens, before, page, n_pages, "cuda", seed=5)
    if window:      # pages that the window has passed are given back: the table no longer names them
        for i, b in enumerate(before):
            bt[i, :max(0, b - window + 1) // page] = -1
    kp, vp = _fill_cache(ctx, bt, page, n_pages, kv_heads, hd, dtype, 50)
    qkv = rnd((len(before), (heads + 2 * kv_heads) * hd), dtype, 52)
    out, ref = (torch.empty(len(before), heads * hd, dtype=dtype, device="cuda") for _ in range(2))
    scale = 1.0 / math.sqrt(hd)
    K = K.with_options(fixed_decode_splits=splits, decode_tma=tma)
    two = torch.empty_like(out)
    K.attention(qkv, out, heads, kv_heads, hd, scale, window, ctx, bt, page, kp, vp)
    K = K.with_options(separate_combine=False)          # the splits merged by the CTA that finishes last: the same sums in the same order
    K.attention(qkv, two, heads, kv_heads, hd, scale, window, ctx, bt, page, kp, vp)
    assert K.attention_decode_tma_error() == 0
    REF.attention(qkv, ref, heads, kv_heads, hd, scale, window, ctx, bt, page, kp, vp)
    assert_close(out, ref, dtype, "decode attention")
    assert_close(two, ref, dtype, "decode attention, merged by the last CTA")


@pytest.mark.parametrize("heads,kv_heads,hd,page", [(14, 2, 64, 16), (12, 2, 128, 16), (4, 4, 64, 8), (7, 1, 128, 64)])
@pytest.mark.parametrize("splits", [0, 1, 4, 8])
def test_attention_decode_takes_the_own_key_and_value_from_the_row(K, heads, kv_heads, hd, page, splits):
    """With own_kv the TMA decode kernel reads every page before the step's earlier kernels have finished and takes
    the token's own key and value from its row of the activation buffer: the page's slot for that position may
    still hold anything (here: large finite junk). Positions at tile and page edges, first token of a request."""
    dtype = torch.bfloat16
    before = [0, 1, 15, 16, 127, 128, 129, 1000, 2047, 2048]
    n = len(before)
    ctx, bt = make_paged_batch([1] * n, before, page, sum(b // page + 2 for b in before), "cuda", seed=9)
    pages = int(bt.max().item()) + 1
    kp, vp = _fill_cache(ctx, bt, page, pages, kv_heads, hd, dtype, 60)
    qkv = rnd((n, (heads + 2 * kv_heads) * hd), dtype, 62)
    rows = qkv.view(n, heads + 2 * kv_heads, hd)
    pos = ctx.positions.long()
    phys = bt[torch.arange(n, device="cuda"), pos // page].long()
    true_k, true_v = kp.clone(), vp.clone()
    true_k[phys, :, pos % page, :] = rows[:, heads:heads + kv_heads]
    true_v[phys, :, pos % page, :] = rows[:, heads + kv_heads:]
    kp[phys, :, pos % page, :] = 77.0            # what a copy taken too early would see
    vp[phys, :, pos % page, :] = -55.0
    got, ref = (torch.empty(n, heads * hd, dtype=dtype, device="cuda") for _ in range(2))
    scale = 1.0 / math.sqrt(hd)
    K = K.with_options(fixed_decode_splits=splits)
    K.attention(qkv, got, heads, kv_heads, hd, scale, 0, ctx, bt, page, kp, vp, own_kv=True)
    assert K.attention_decode_tma_error() == 0
    REF.attention(qkv, ref, heads, kv_heads, hd, scale, 0, ctx, bt, page, true_k, true_v)
    assert_close(got, ref, dtype, "decode attention, own key and value from the row")


@pytest.mark.parametrize("heads,kv_heads,hd,page,window", [(14, 2, 64, 16, 0), (6, 1, 32, 8, 0), (3, 3, 48, 8, 24), (8, 2, 128, 16, 0)])
def test_attention_tensor_core_kernels_agree_with_the_general_kernel(K, heads, kv_heads, hd, page, window):
    """bfloat16: the same batch through the tensor-core kernels and through the general kernel."""
    dtype = torch.bfloat16
    q_lens, before = [1, 1, 150, 7, 1], [500, 0, 100, 0, 64]
    ctx, bt = make_paged_batch(q_lens, before, page, 200, "cuda", seed=6)
    kp, vp = _fill_cache(ctx, bt, page, 200, kv_heads, hd, dtype, 60)
    m = sum(q_lens)
    qkv = rnd((m, (heads + 2 * kv_heads) * hd), dtype, 62)
    fast, general = (torch.empty(m, heads * hd, dtype=dtype, device="cuda") for _ in range(2))
    scale = 1.0 / math.sqrt(hd)
    K.attention(qkv, fast, heads, kv_heads, hd, scale, window, ctx, bt, page, kp, vp)
    K = K.with_options(force_general_attention=True)
    K.attention(qkv, general, heads, kv_heads, hd, scale, window, ctx, bt, page, kp, vp)
    assert_close(fast, general.double(), dtype, "tensor-core vs general attention")


@pytest.mark.parametrize("tile", [0, 16, 32, 64, 128, 256])
@pytest.mark.parametrize("m,n,k", [(1, 503, 192), (7, 128, 64), (65, 130, 72), (200, 896, 896), (130, 1000, 344),
                                   (300, 311, 4864), (17, 9, 8)])
def test_tensor_core_gemm_tiles_and_ragged_shapes(K, m, n, k, tile):
    """The tcgen05 kernel at every token tile, with rows, features and K that do not fill a tile, in all
    four epilogues, against float64; and against the CUDA-core kernel row by row."""
    dtype = torch.bfloat16
    a, w = rnd((m, k), dtype, 70), rnd((n, k), dtype, 71, scale=0.05)
    bias = rnd((n,), torch.float32, 72)
    K = K.with_options(tc_token_tile=tile)
    out = torch.empty(m, n, dtype=dtype, device="cuda")
    K.linear(a, w, bias, out, "store")
    assert_close(out, _ref_linear_f64(a, w, bias), dtype, "tc store")
    out32 = torch.empty(m, n, device="cuda")
    K.linear(a, w, None, out32, "f32")
    assert_close(out32, _ref_linear_f64(a, w, None), torch.float32, "tc f32")
    res = rnd((m, n), torch.float32, 73)
    acc = res.clone()
    K.linear(a, w, bias, acc, "add")
    assert_close(acc, res.double() + _ref_linear_f64(a, w, bias), torch.float32, "tc add")
    inter = max(1, n // 2)
    sw, ref = (torch.empty(m, inter, dtype=dtype, device="cuda") for _ in range(2))
    if tile == 256:
        K = K.with_options(tc_token_tile=128)      # two accumulators, double buffered: up to 128 tokens per tile
    K.linear_swiglu(a, w[:2 * inter].contiguous(), sw)
    REF.linear_swiglu(a, w[:2 * inter].contiguous(), ref)
    assert_close(sw, ref, dtype, "tc swiglu")
    assert K.gemm_tc_error() == 0


@pytest.mark.parametrize("splits", [0, 2, 5, 64])
@pytest.mark.parametrize("m,n,k", [(1, 896, 4864), (8, 130, 1000), (16, 503, 328), (40, 896, 896), (64, 200, 2048)])
def test_tensor_core_gemm_split_k(K, m, n, k, splits):
    """K cut into work items that different CTAs run: partial sums through the scratch and the last
    warp (store, f32, swiglu; the same bits on every call) or added in memory (add); more splits than
    blocks of K, a ragged last split, and the counters left ready for the next call."""
    dtype = torch.bfloat16
    a, w = rnd((m, k), dtype, 74), rnd((n, k), dtype, 75, scale=0.05)
    bias = rnd((n,), torch.float32, 76)
    K = K.with_options(gemm_route="tc", tc_splits=splits)
    for _ in range(2):
        out = torch.empty(m, n, dtype=dtype, device="cuda")
        K.linear(a, w, bias, out, "store")
        assert_close(out, _ref_linear_f64(a, w, bias), dtype, "split store")
        out32 = torch.empty(m, n, device="cuda")
        K.linear(a, w, None, out32, "f32")
        assert_close(out32, _ref_linear_f64(a, w, None), torch.float32, "split f32")
        again = torch.empty_like(out32)
        K.linear(a, w, None, again, "f32")
        assert torch.equal(out32, again)
        res = rnd((m, n), torch.float32, 77)
        acc = res.clone()
        K.linear(a, w, bias, acc, "add")
        assert_close(acc, res.double() + _ref_linear_f64(a, w, bias), torch.float32, "split add")
        inter = n // 2
        sw, ref = (torch.empty(m, inter, dtype=dtype, device="cuda") for _ in range(2))
        K.linear_swiglu(a, w[:2 * inter].contiguous(), sw)
        REF.linear_swiglu(a, w[:2 * inter].contiguous(), ref)
        assert_close(sw, ref, dtype, "split swiglu")
    assert K.gemm_tc_error() == 0


@pytest.mark.parametrize("tile", [0, 128, 256])
@pytest.mark.parametrize("m,n,k", [(256, 512, 128), (300, 896, 896), (130, 1000, 344), (1, 256, 64), (700, 130, 72),
                                   (2048, 1152, 896), (515, 311, 200), (4096, 4864, 896)])
def test_tensor_core_gemm_on_pairs_of_sms(K, m, n, k, tile):
    """tcgen05.mma.cta_group::2: tiles of 256 tokens on two SMs, each CTA holding half of the tile's weight
    rows; features, tokens and K that do not fill a tile (and rows of the output that rule out 16-byte
    stores); all four epilogues; several tiles per cluster."""
    dtype = torch.bfloat16
    a, w = rnd((m, k), dtype, 170), rnd((n, k), dtype, 171, scale=0.05)
    bias = rnd((n,), torch.float32, 172)
    K = K.with_options(gemm_route="tc_pair", pair_n_tile=tile)
    for splits in (2, 5):       # K split over clusters, partial sums added in memory
        K = K.with_options(tc_splits=splits)
        res = rnd((m, n), torch.float32, 174)
        acc = res.clone()
        K.linear(a, w, bias, acc, "add")
        assert_close(acc, res.double() + _ref_linear_f64(a, w, bias), torch.float32, f"pair add, {splits} splits")
    K = K.with_options(tc_splits=0)
    out = torch.empty(m, n, dtype=dtype, device="cuda")
    K.linear(a, w, bias, out, "store")
    assert_close(out, _ref_linear_f64(a, w, bias), dtype, "pair store")
    out32 = torch.empty(m, n, device="cuda")
    K.linear(a, w, None, out32, "f32")
    assert_close(out32, _ref_linear_f64(a, w, None), torch.float32, "pair f32")
    res = rnd((m, n), torch.float32, 173)
    acc = res.clone()
    K.linear(a, w, bias, acc, "add")
    assert_close(acc, res.double() + _ref_linear_f64(a, w, bias), torch.float32, "pair add")
    inter = n // 2
    sw, ref = (torch.empty(m, inter, dtype=dtype, device="cuda") for _ in range(2))
    K.linear_swiglu(a, w[:2 * inter].contiguous(), sw)
    REF.linear_swiglu(a, w[:2 * inter].contiguous(), ref)
    assert_close(sw, ref, dtype, "pair swiglu")
    assert K.gemm_tc_error() == 0


def test_tensor_core_gemm_refuses_what_it_cannot_take(K):
    from nanoinfer_b200.csrc.lib import KernelError
    a, w = rnd((4, 20), torch.bfloat16, 80), rnd((6, 20), torch.bfloat16, 81)      # K = 20: rows are not 16-byte multiples
    out = torch.empty(4, 6, device="cuda")
    K.linear(a, w, None, out, "f32")                      # the dispatcher falls back to the CUDA-core kernel
    assert_close(out, _ref_linear_f64(a, w, None), torch.float32, "odd K")
    with pytest.raises(KernelError, match="multiples of 8"):
        K._check(K._lib.nib_gemm_tc(a.data_ptr(), w.data_ptr(), None, out.data_ptr(), 4, 6, 20, 20, 6, 2, 0, None), "direct")


@pytest.mark.parametrize("ksplit,cross", [(0, 0), (1, 0), (8, 1), (8, 3), (8, 16)])
@pytest.mark.parametrize("m,n,k", [(1, 503, 192), (8, 896, 896), (9, 130, 64), (16, 1000, 4864), (33, 311, 320), (64, 72, 128)])
def test_small_m_gemm(K, m, n, k, ksplit, cross):
    """The decode GEMM (weights streamed into mma.sync fragments) for 1..64 tokens, both K splits, all
    epilogues; a row's result does not depend on how many rows are in the call."""
    dtype = torch.bfloat16
    a, w = rnd((m, k), dtype, 90), rnd((n, k), dtype, 91, scale=0.05)
    bias = rnd((n,), torch.float32, 92)
    K = K.with_options(smallm_ksplit=ksplit, smallm_cross=cross, gemm_route="smallm")
    out = torch.empty(m, n, dtype=dtype, device="cuda")
    K.linear(a, w, bias, out, "store")
    assert_close(out, _ref_linear_f64(a, w, bias), dtype, "smallm store")
    again = torch.empty_like(out)
    K.linear(a, w, bias, again, "store")
    assert torch.equal(out, again)            # the split over CTAs is summed in a fixed order
    out32 = torch.empty(m, n, device="cuda")
    K.linear(a, w, None, out32, "f32")
    assert_close(out32, _ref_linear_f64(a, w, None), torch.float32, "smallm f32")
    res = rnd((m, n), torch.float32, 93)
    acc = res.clone()
    K.linear(a, w, bias, acc, "add")
    assert_close(acc, res.double() + _ref_linear_f64(a, w, bias), torch.float32, "smallm add")
    inter = n // 2
    sw, ref = (torch.empty(m, inter, dtype=dtype, device="cuda") for _ in range(2))
    K.linear_swiglu(a, w[:2 * inter].contiguous(), sw)
    REF.linear_swiglu(a, w[:2 * inter].contiguous(), ref)
    assert_close(sw, ref, dtype, "smallm swiglu")
    one = torch.empty(1, n, device="cuda")
    K.linear(a[m - 1:m].contiguous(), w, None, one, "f32")
    assert torch.equal(one[0], out32[m - 1])


@pytest.mark.parametrize("m,n,k,eps", [(1, 1152, 896, 1e-6), (8, 320, 192, 1e-5), (20, 200, 64, 1e-3), (64, 503, 320, 1e-6)])
def test_small_m_gemm_with_fused_rmsnorm(K, m, n, k, eps):
    """The decode GEMM that reads the 32-bit residual stream and applies RMSNorm on the fly, against the
    separate norm kernel followed by the same GEMM, and against float64."""
    from nanoinfer_b200.parts.base import FoldedNorm, LazyNorm

    class _Norm:
        def forward(self_, x32, rows=None):
            out = torch.empty(x32.shape, dtype=torch.bfloat16, device="cuda")
            K.rmsnorm(x32, gain, eps, out, rows)
            return out

    x32 = rnd((m, k), torch.float32, 95, scale=2.5)
    gain = 1 + 0.1 * rnd((k,), torch.float32, 96)
    w = rnd((n, k), torch.bfloat16, 97, scale=0.05)
    fused, two_step = torch.empty(m, n, device="cuda"), torch.empty(m, n, device="cuda")
    K = K.with_options(gemm_route="smallm_fused")
    K.linear(LazyNorm(_Norm(), FoldedNorm(x32, gain, eps), torch.bfloat16), w, None, fused, "f32")
    K = K.with_options(gemm_route="smallm")
    h = _Norm().forward(x32)
    K.linear(h, w, None, two_step, "f32")
    ref = _ref_linear_f64(h, w, None)
    assert_close(two_step, ref, torch.float32, "norm then gemm")
    # the fused kernel sums x^2 in another order: its bfloat16 inputs may differ by one rounding
    exact = (x32.double() * torch.rsqrt(x32.double().pow(2).mean(-1, keepdim=True) + eps) * gain.double()) @ w.double().t()
    assert_close(fused, exact, torch.bfloat16, "fused norm gemm")
    inter = n // 2
    sw, sw_ref = (torch.empty(m, inter, dtype=torch.bfloat16, device="cuda") for _ in range(2))
    K = K.with_options(gemm_route="smallm_fused")
    K.linear_swiglu(LazyNorm(_Norm(), FoldedNorm(x32, gain, eps), torch.bfloat16), w[:2 * inter].contiguous(), sw)
    K = K.with_options(gemm_route=None)
    REF.linear_swiglu(h, w[:2 * inter].contiguous(), sw_ref)
    assert_close(sw, sw_ref, torch.bfloat16, "fused norm swiglu")


def test_other_norms_use_the_fold_hook_without_a_change_to_the_library(K):
    """Two norms the library has never seen, defined here. One stores its gain as ``g`` and multiplies with ``1 + g``:
    it hands over the vector it multiplies with and is applied inside the small-M product like the built-in norm.
    The other subtracts the mean first (kind "layer"): the library does not know that kind and lets the norm compute
    itself. Both against float64."""
    from nanoinfer_b200.parts.base import FoldedNorm, LazyNorm
    m, n, k, eps = 5, 320, 192, 1e-5
    x32 = rnd((m, k), torch.float32, 151, scale=2.0)
    g = 0.1 * rnd((k,), torch.float32, 152)
    w = rnd((n, k), torch.bfloat16, 153, scale=0.05)
    calls = []

    class OnePlusGain:
        def forward(self, x, rows=None):
            calls.append("one_plus")
            out = torch.empty(x.shape, dtype=torch.bfloat16, device="cuda")
            K.rmsnorm(x, 1 + g, eps, out, rows)
            return out

    class MeanFree:
        def forward(self, x, rows=None):
            calls.append("layer")
            xd = x.double() - x.double().mean(-1, keepdim=True)
            return (xd * torch.rsqrt(xd.pow(2).mean(-1, keepdim=True) + eps) * (1 + g).double()).to(torch.bfloat16)

    out = torch.empty(m, n, device="cuda")
    K = K.with_options(gemm_route="smallm_fused")
    K.linear(LazyNorm(OnePlusGain(), FoldedNorm(x32, 1 + g, eps, "rms"), torch.bfloat16), w, None, out, "f32")
    assert calls == [], "applied inside the product"
    xd = x32.double()
    exact = (xd * torch.rsqrt(xd.pow(2).mean(-1, keepdim=True) + eps) * (1 + g).double()) @ w.double().t()
    assert_close(out, exact, torch.bfloat16, "1 + g norm folded")
    K.linear(LazyNorm(MeanFree(), FoldedNorm(x32, 1 + g, eps, "layer"), torch.bfloat16), w, None, out, "f32")
    assert calls == ["layer"], "computed by the norm itself"
    xd = xd - xd.mean(-1, keepdim=True)
    exact = (xd * torch.rsqrt(xd.pow(2).mean(-1, keepdim=True) + eps) * (1 + g).double()) @ w.double().t()
    assert_close(out, exact, torch.bfloat16, "mean-free norm resolved")


@pytest.mark.parametrize("heads,kv_heads,hd,page,window", [
    (14, 2, 64, 16, 0), (12, 2, 128, 16, 0), (4, 4, 64, 8, 0), (7, 1, 64, 64, 0), (16, 2, 128, 32, 200),
    (3, 1, 64, 16, 100), (28, 4, 128, 128, 0)])
def test_attention_tcgen05_prefill(K, heads, kv_heads, hd, page, window):
    """Prompt portions on the tcgen05 kernel (head sizes 64 and 128): portions that start at position 0
    and inside a context, one token, tile edges at 127/128/129 keys, several requests, pages handed out
    in shuffled order; against float64 and against the mma.sync kernel."""
    dtype = torch.bfloat16
    q_lens, before = [300, 1, 129, 40, 128], [0, 127, 200, 515, 0]
    total = sum(a + b for a, b in zip(q_lens, before))
    pages = total // page + 8
    ctx, bt = make_paged_batch(q_lens, before, page, pages, "cuda", seed=7)
    kp, vp = _fill_cache(ctx, bt, page, pages, kv_heads, hd, dtype, 110)
    m = sum(q_lens)
    qkv = rnd((m, (heads + 2 * kv_heads) * hd), dtype, 112)
    fast, legacy, ref = (torch.empty(m, heads * hd, dtype=dtype, device="cuda") for _ in range(3))
    scale = 1.0 / math.sqrt(hd)
    K.attention(qkv, fast, heads, kv_heads, hd, scale, window, ctx, bt, page, kp, vp)
    assert K.attention_tc_error() == 0
    K = K.with_options(force_mma_prefill=True)
    K.attention(qkv, legacy, heads, kv_heads, hd, scale, window, ctx, bt, page, kp, vp)
    assert_close(fast, legacy.double(), dtype, "tcgen05 vs mma.sync attention")
    REF.attention(qkv, ref, heads, kv_heads, hd, scale, window, ctx, bt, page, kp, vp)
    assert_close(fast, ref, dtype, "tcgen05 attention")


def _ref_attention_masked(qkv, heads, kv_heads, hd, scale, window, q_lens, before, bt, page, kp, vp):
    """The same formula as ``TorchOps.attention`` (float64, keys lo..own position), one masked softmax per
    request instead of a loop over tokens: for portions of thousands of tokens."""
    m = qkv.shape[0]
    q_all = qkv.view(m, heads + 2 * kv_heads, hd)[:, :heads].double()
    out = torch.empty(m, heads, hd, dtype=torch.float64, device=qkv.device)
    n_rep = heads // kv_heads
    row = 0
    for r, (ql, b) in enumerate(zip(q_lens, before)):
        n = b + ql
        idx = torch.arange(n, device=qkv.device)
        pages = bt[r, idx // page].long()
        held = pages >= 0
        k = kp[pages.clamp(min=0), :, idx % page, :].double()      # [n, kv_heads, hd]
        v = vp[pages.clamp(min=0), :, idx % page, :].double()
        pos = torch.arange(b, n, device=qkv.device)[:, None]
        visible = idx[None, :] <= pos
        if window:
            visible &= idx[None, :] > pos - window
        assert bool((held[None, :] | ~visible).all()), "read of a position without a page"
        q = q_all[row:row + ql]
        s = torch.einsum("thd,nhd->htn", q, k.repeat_interleave(n_rep, dim=1)) * scale
        s = s.masked_fill(~visible[None], float("-inf"))
        out[row:row + ql] = torch.einsum("htn,nhd->thd", torch.softmax(s, dim=-1), v.repeat_interleave(n_rep, dim=1))
        row += ql
    return out.view(m, heads * hd)


@pytest.mark.parametrize("heads,kv_heads,hd,page,window,q_lens,before", [
    (14, 2, 64, 16, 0, [2048], [0]), (14, 2, 64, 16, 0, [2048, 1000], [2048, 3096]), (12, 2, 128, 16, 0, [4096], [0]),
    (12, 2, 128, 16, 0, [2048, 2], [2048, 4094]), (4, 1, 64, 32, 1500, [2048], [2048]), (28, 4, 128, 16, 0, [2048], [0])])
def test_attention_prefill_at_benchmark_lengths(K, heads, kv_heads, hd, page, window, q_lens, before):
    """Prompt portions of 2,048 and 4,096 tokens, from position 0 and behind 2,048 cached keys: the tcgen05
    kernel walks 16 to 32 key blocks per tile."""
    dtype = torch.bfloat16
    total = sum(a + b for a, b in zip(q_lens, before))
    pages = total // page + 8
    ctx, bt = make_paged_batch(q_lens, before, page, pages, "cuda", seed=17)
    kp, vp = _fill_cache(ctx, bt, page, pages, kv_heads, hd, dtype, 210)
    m = sum(q_lens)
    qkv = rnd((m, (heads + 2 * kv_heads) * hd), dtype, 212)
    got = torch.empty(m, heads * hd, dtype=dtype, device="cuda")
    scale = 1.0 / math.sqrt(hd)
    K.attention(qkv, got, heads, kv_heads, hd, scale, window, ctx, bt, page, kp, vp)
    assert K.attention_tc_error() == 0
    ref = _ref_attention_masked(qkv, heads, kv_heads, hd, scale, window, q_lens, before, bt, page, kp, vp)
    assert_close(got, ref, dtype, "prefill attention at benchmark lengths")


@pytest.mark.parametrize("heads,kv_heads,hd,page", [(14, 2, 64, 16), (12, 2, 128, 16), (28, 4, 128, 64)])
@pytest.mark.parametrize("n_req", [1, 8, 64])
def test_attention_decode_at_benchmark_lengths(K, heads, kv_heads, hd, page, n_req):
    """Single decoded tokens over 4,096 and 8,192 cached keys (and shorter neighbours in the same batch), with
    the number of splits that the engine chooses for the batch size."""
    dtype = torch.bfloat16
    before = [(8191 if i % 4 == 0 else 4095 if i % 4 == 1 else 4096 if i % 4 == 2 else 3000 + 7 * i) for i in range(n_req)]
    q_lens = [1] * n_req
    pages = sum(-(-(b + 1) // page) for b in before) + 8
    ctx, bt = make_paged_batch(q_lens, before, page, pages, "cuda", seed=18)
    kp, vp = _fill_cache(ctx, bt, page, pages, kv_heads, hd, dtype, 220)
    qkv = rnd((n_req, (heads + 2 * kv_heads) * hd), dtype, 222)
    got = torch.empty(n_req, heads * hd, dtype=dtype, device="cuda")
    scale = 1.0 / math.sqrt(hd)
    K.attention(qkv, got, heads, kv_heads, hd, scale, 0, ctx, bt, page, kp, vp)
    assert K.attention_decode_tma_error() == 0
    ref = _ref_attention_masked(qkv, heads, kv_heads, hd, scale, 0, q_lens, before, bt, page, kp, vp)
    assert_close(got, ref, dtype, "decode attention at benchmark lengths")


@pytest.mark.parametrize("heads,kv_heads,hd,rot,page,hidden,fused", [
    (14, 2, 64, 64, 16, 896, True), (12, 2, 128, 128, 16, 1536, True), (3, 1, 64, 0, 8, 72, True), (5, 5, 128, 128, 32, 200, True),
    (7, 1, 64, 32, 16, 128, False), (3, 3, 48, 48, 8, 160, False)])
def test_qkv_projection_of_a_prompt_portion_with_rotation_and_cache_write(K, heads, kv_heads, hd, rot, page, hidden, fused):
    """A prompt portion's q/k/v product on the tcgen05 kernel whose epilogue adds the bias, rotates whole heads and
    writes keys and values into the pages: the rows against float64, the pages against the rows. Several requests,
    portions that start inside a page and inside a tile of 128 tokens, a request of one token between them, a row
    without a page; heads of 64 and 128, no rotation at all. Shapes the fused form does not take (half-rotated heads,
    heads of 48) run the product and the rotation kernel and must give the same."""
    from nanoinfer_b200.parts.position import rotary_tables
    dtype = torch.bfloat16
    q_lens, before = [150, 1, 70, 2, 130], [0, 63, 61, 300, 17]
    m = sum(q_lens)
    ctx, bt = make_paged_batch(q_lens, before, page, 800 // page * 2, "cuda", seed=18)
    pages = int(bt.max().item()) + 1
    shape = (pages, kv_heads, page, hd)
    rotary = None
    if rot:
        cos, sin = rotary_tables(600, rot, 10000.0)
        rotary = (cos.cuda(), sin.cuda(), rot)
    n = (heads + 2 * kv_heads) * hd
    w = rnd((n, hidden), dtype, 221, scale=0.05)
    bias = rnd((n,), torch.float32, 222)
    h = rnd((m, hidden), dtype, 224, scale=1.0)
    kp, vp = torch.zeros(shape, dtype=dtype, device="cuda"), torch.zeros(shape, dtype=dtype, device="cuda")
    qkv = torch.empty(m, n, dtype=dtype, device="cuda")
    before_launches = K.launches
    K.qkv_project(h, w, bias, qkv, heads, kv_heads, hd, ctx.positions, ctx.req_index, rotary, bt, page, kp, vp, True)
    assert K.launches == before_launches + (1 if fused else 2)
    assert K.gemm_tc_error() == 0
    ref = (h.double() @ w.double().t() + bias.double()).view(m, heads + 2 * kv_heads, hd)
    if rot:
        half = rot // 2
        c = rotary[0][ctx.positions.long()].double()[:, None, :]
        sn = rotary[1][ctx.positions.long()].double()[:, None, :]
        qk = ref[:, :heads + kv_heads]
        x1, x2 = qk[..., :half].clone(), qk[..., half:rot].clone()
        qk[..., :half] = x1 * c - x2 * sn
        qk[..., half:rot] = x2 * c + x1 * sn
    assert_close(qkv, ref.view(m, n), dtype, "q/k/v rows of a portion")
    kr, vr = torch.zeros_like(kp), torch.zeros_like(vp)
    pos = ctx.positions.long()
    page_of = bt[ctx.req_index.long(), pos // page].long()
    got = qkv.view(m, heads + 2 * kv_heads, hd)
    kr[page_of, :, pos % page, :] = got[:, heads:heads + kv_heads]
    vr[page_of, :, pos % page, :] = got[:, heads + kv_heads:]
    assert torch.equal(kp, kr) and torch.equal(vp, vr)
    # without writing, pages stay as they are; a request without pages (-1 in its table) writes nothing
    kp2 = torch.zeros_like(kp)
    q2 = torch.empty_like(qkv)
    K.qkv_project(h, w, bias, q2, heads, kv_heads, hd, ctx.positions, ctx.req_index, rotary, bt, page, kp2, kp2, False)
    assert torch.equal(q2, qkv) and not kp2.any()
    bt_pad = bt.clone()
    bt_pad[2] = -1
    kp3, vp3 = torch.zeros_like(kp), torch.zeros_like(vp)
    K.qkv_project(h, w, bias, q2, heads, kv_heads, hd, ctx.positions, ctx.req_index, rotary, bt_pad, page, kp3, vp3, True)
    rows2 = (ctx.req_index == 2)
    keep = torch.ones(pages, dtype=torch.bool, device="cuda")
    keep[page_of[rows2]] = False
    assert torch.equal(kp3[keep], kr[keep]) and not kp3[~keep].any() and torch.equal(q2, qkv)
    # the same rows from the product followed by the rotation kernel (one more rounding: to bfloat16 before the rotation)
    two = torch.empty_like(qkv)
    K.with_options(fuse_qkv=False).qkv_project(h, w, bias, two, heads, kv_heads, hd, ctx.positions, ctx.req_index, rotary,
                                               bt, page, torch.zeros_like(kp), torch.zeros_like(vp), True)
    assert_close(two, ref.view(m, n), dtype, "q/k/v rows, product then rotation")


@pytest.mark.parametrize("q_lens,before", [([1, 1, 2, 1, 1], [0, 63, 64, 300, 17]),
                                           ([1] * 23 + [3] + [1] * 20, [7 * i % 311 for i in range(44)]),        # 46 tokens: six tiles of 8
                                           ([1] * 64, [(13 * i + 5) % 389 for i in range(64)])])
@pytest.mark.parametrize("with_norm", [False, True])
@pytest.mark.parametrize("heads,kv_heads,hd,rot,page,hidden", [(14, 2, 64, 64, 16, 896), (6, 1, 32, 32, 8, 192), (3, 3, 48, 48, 8, 160),
                                                               (16, 1, 128, 64, 16, 1536), (4, 2, 16, 16, 16, 64), (28, 4, 128, 128, 32, 3584),
                                                               (5, 5, 80, 0, 4, 96), (2, 1, 128, 32, 16, 256)])
def test_qkv_projection_with_rotation_and_cache_write(K, heads, kv_heads, hd, rot, page, hidden, with_norm, q_lens, before):
    """The decode step's q/k/v product with the norm as its prologue and bias, rotation and the write of keys and
    values into the pages as its epilogue, in one kernel: against float64 for the whole row, and the pages
    against the separate rotation kernel's pages (which other tests hold against float64). Tokens of several
    requests at different positions, one request with two tokens, pages in shuffled order."""
    from nanoinfer_b200.parts.base import FoldedNorm, LazyNorm
    from nanoinfer_b200.parts.position import rotary_tables
    dtype = torch.bfloat16
    m = sum(q_lens)
    ctx, bt = make_paged_batch(q_lens, before, page, (sum(b // page + 2 for b in before) + 8), "cuda", seed=8)
    pages = int(bt.max().item()) + 1
    shape = (pages, kv_heads, page, hd)
    rotary = None
    if rot:
        cos, sin = rotary_tables(400, rot, 10000.0)
        rotary = (cos.cuda(), sin.cuda(), rot)
    n = (heads + 2 * kv_heads) * hd
    w = rnd((n, hidden), dtype, 121, scale=0.05)
    bias = rnd((n,), torch.float32, 122)
    eps = 1e-6
    gain = 1 + 0.1 * rnd((hidden,), torch.float32, 123)
    x32 = rnd((m, hidden), torch.float32, 124, scale=2.0)

    class _Norm:
        def forward(self_, x, rows=None):
            out = torch.empty(x.shape, dtype=dtype, device="cuda")
            K.rmsnorm(x, gain, eps, out, rows)
            return out

    h = _Norm().forward(x32)
    a = LazyNorm(_Norm(), FoldedNorm(x32, gain, eps), dtype) if with_norm else h
    kp, vp = torch.zeros(shape, dtype=dtype, device="cuda"), torch.zeros(shape, dtype=dtype, device="cuda")
    qkv = torch.empty(m, n, dtype=dtype, device="cuda")
    before_launches = K.launches
    K.qkv_project(a, w, bias, qkv, heads, kv_heads, hd, ctx.positions, ctx.req_index, rotary, bt, page, kp, vp, True)
    norm_alone = with_norm and not (m <= 8 or (m <= 16 and hidden <= 1024))        # the norm is folded in for few tokens only
    assert K.launches == before_launches + (2 if norm_alone else 1), "one kernel for the whole of it"
    # float64: product (+ norm), bias, rotation
    hh = (x32.double() * torch.rsqrt(x32.double().pow(2).mean(-1, keepdim=True) + eps) * gain.double()) if (with_norm and not norm_alone) else h.double()
    ref = (hh @ w.double().t() + bias.double()).view(m, heads + 2 * kv_heads, hd)
    if rot:
        half = rot // 2
        c = rotary[0][ctx.positions.long()].double()[:, None, :]
        sn = rotary[1][ctx.positions.long()].double()[:, None, :]
        qk = ref[:, :heads + kv_heads]
        x1, x2 = qk[..., :half].clone(), qk[..., half:rot].clone()
        qk[..., :half] = x1 * c - x2 * sn
        qk[..., half:rot] = x2 * c + x1 * sn
    assert_close(qkv, ref.view(m, n), dtype, "q/k/v row")
    # the pages hold exactly the row's keys and values, at the tokens' positions, and nothing else
    kr, vr = torch.zeros_like(kp), torch.zeros_like(vp)
    pos = ctx.positions.long()
    page_of = bt[ctx.req_index.long(), pos // page].long()
    got = qkv.view(m, heads + 2 * kv_heads, hd)
    kr[page_of, :, pos % page, :] = got[:, heads:heads + kv_heads]
    vr[page_of, :, pos % page, :] = got[:, heads + kv_heads:]
    assert torch.equal(kp, kr) and torch.equal(vp, vr)
    # without writing, pages stay as they are
    kp2 = torch.zeros_like(kp)
    q2 = torch.empty_like(qkv)
    K.qkv_project(a, w, bias, q2, heads, kv_heads, hd, ctx.positions, ctx.req_index, rotary, bt, page, kp2, kp2, False)
    assert torch.equal(q2, qkv) and not kp2.any()
    # a row of a padded batch (no page: -1 in the table) writes nothing
    bt_pad = bt.clone()
    bt_pad[1] = -1
    kp3, vp3 = torch.zeros_like(kp), torch.zeros_like(vp)
    K.qkv_project(a, w, bias, q2, heads, kv_heads, hd, ctx.positions, ctx.req_index, rotary, bt_pad, page, kp3, vp3, True)
    keep = torch.ones(pages, dtype=torch.bool, device="cuda")
    keep[page_of[1]] = False
    assert torch.equal(kp3[keep], kr[keep]) and not kp3[page_of[1]].any()
