"""Helpers of the GPU tests: tolerances, paged-cache fixtures, comparison with NaN awareness."""
from types import SimpleNamespace

import torch

# Tolerances, stated once. 32-bit: kernels accumulate in float32 in a different order than the
# float64 reference. bfloat16: every stored activation is rounded to 8 bits of mantissa (relative
# half-ulp 2^-9); errors are judged against the root mean square of the reference values.
F32_REL = 2e-5      # max |err| <= F32_REL * max(1, max |ref|)
BF16_RMS = 0.015    # rms(err) <= BF16_RMS * rms(ref)
BF16_MAX = 0.06     # |err| <= BF16_MAX * rms(ref) + BF16_ULP * |ref| for every element
BF16_ULP = 2.0 ** -7  # a result stored in bfloat16 may differ by one unit in the last place of its own value


def assert_close(got: torch.Tensor, ref: torch.Tensor, dtype: torch.dtype, what: str = ""):
    got, ref = got.detach().double().cpu(), ref.detach().double().cpu()
    assert got.shape == ref.shape, (what, got.shape, ref.shape)
    assert not torch.isnan(got).any() and not torch.isinf(got).any(), f"{what}: NaN or inf in the result"
    err = (got - ref).abs()
    if dtype == torch.float32:
        bound = F32_REL * max(1.0, ref.abs().max().item())
        assert err.max().item() <= bound, f"{what}: max err {err.max().item():.3e} > {bound:.3e}"
    else:
        rms = ref.pow(2).mean().sqrt().item()
        e_rms = err.pow(2).mean().sqrt().item()
        assert e_rms <= BF16_RMS * rms + 1e-12, f"{what}: rms err {e_rms:.3e} > {BF16_RMS * rms:.3e}"
        excess = (err - (BF16_MAX * rms + BF16_ULP * ref.abs() + 1e-12)).max().item()
        assert excess <= 0, f"{what}: max err {err.max().item():.3e} exceeds {BF16_MAX * rms:.3e} + one ulp by {excess:.3e}"


def bf16_slack(row: torch.Tensor) -> float:
    """How far below the best logit of ``row`` (the plain model's, float64) a token may lie and still be the
    best one for an engine whose logits carry bfloat16's rounding: twice the element tolerance."""
    row = row.double()
    return 2 * (BF16_MAX * row.pow(2).mean().sqrt().item() + BF16_ULP * row.abs().max().item())


def assert_diverges_only_at_a_close_call(plain, prompt, a, b, what=""):
    """Two greedy continuations of one prompt in bfloat16 (another batch, another cut): they are equal, or at
    the first place where they differ BOTH tokens are within rounding of the plain model's best logit, given
    the tokens both have read so far. After that place the two runs read different contexts."""
    for i, (x, y) in enumerate(zip(a, b)):
        if x != y:
            row = plain.logits(list(prompt) + list(a[:i]))[-1].double()
            slack = bf16_slack(row)
            best = row.max().item()
            assert best - row[x].item() <= slack and best - row[y].item() <= slack, \
                f"{what}: token {i}: {x} ({row[x].item():.4f}) against {y} ({row[y].item():.4f}), best {best:.4f}, slack {slack:.4f}"
            return
    assert len(a) == len(b), f"{what}: lengths {len(a)} and {len(b)}"


def make_paged_batch(q_lens, ctx_before, page_size, num_pages, device, seed=0, shuffle=True):
    """A batch description like the engine builds, with pages handed out in a shuffled order so that
    logical and physical order differ. Returns (ctx, block_table)."""
    g = torch.Generator().manual_seed(seed)
    r = len(q_lens)
    ctx_lens = [c + q for c, q in zip(ctx_before, q_lens)]
    order = torch.randperm(num_pages, generator=g).tolist() if shuffle else list(range(num_pages))
    width = max(-(-c // page_size) for c in ctx_lens)
    bt = torch.full((r, width), -1, dtype=torch.int32)
    for i, c in enumerate(ctx_lens):
        for p in range(-(-c // page_size)):
            bt[i, p] = order.pop()
    positions = torch.cat([torch.arange(c, c + q, dtype=torch.int32) for c, q in zip(ctx_before, q_lens)])
    req_index = torch.cat([torch.full((q,), i, dtype=torch.int32) for i, q in enumerate(q_lens)])
    q_start = torch.zeros(r + 1, dtype=torch.int32)
    q_start[1:] = torch.tensor(q_lens).cumsum(0)
    ctx = SimpleNamespace(
        num_tokens=int(sum(q_lens)), positions=positions.to(device), req_index=req_index.to(device),
        q_start=q_start.to(device), ctx_lens=torch.tensor(ctx_lens, dtype=torch.int32, device=device),
        host=SimpleNamespace(q_lens=list(q_lens), ctx_lens=ctx_lens, num_requests=r,
                             max_q_len=max(q_lens), max_ctx_len=max(ctx_lens)))
    return ctx, bt.to(device)
