"""Plain PyTorch statements of what each CUDA kernel of the engine computes, with the kernels'
own signatures. Used by the tests only: as the reference each kernel is compared with, and to run
the engine's host-side logic (cache, batching, scheduler) on a machine without a GPU.
Math is done in float64 and rounded once to the output's dtype.
"""
from __future__ import annotations


import torch

from nanoinfer_b200.parts.base import as_tensor


class TorchOps:
    name = "torch-reference"

    def embed(self, ids, table, out32):
        out32.copy_(table[ids.long()].to(torch.float32))

    def rmsnorm(self, x32, gain32, eps, out, rows=None):
        x = x32.double() if rows is None else x32[rows.long()].double()
        y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * gain32.double()
        out.copy_(y.to(out.dtype))

    def linear(self, a, w, bias32, out, mode):
        a = as_tensor(a)
        y = a.double() @ w.double().t()
        if bias32 is not None:
            y = y + bias32.double()
        if mode == "add":
            out.copy_((out.double() + y).to(out.dtype))
        elif mode in ("store", "f32"):
            out.copy_(y.to(out.dtype))
        else:
            raise ValueError(mode)

    def linear_swiglu(self, a, w_gate_up, out):
        a = as_tensor(a)
        inter = w_gate_up.shape[0] // 2
        g = a.double() @ w_gate_up[:inter].double().t()
        u = a.double() @ w_gate_up[inter:].double().t()
        out.copy_((g / (1.0 + torch.exp(-g)) * u).to(out.dtype))

    def qkv_project(self, a, w_qkv, bias32, qkv, heads, kv_heads, head_dim, positions, req_index, rotary,
                    block_table, page_size, k_pages, v_pages, writes):
        self.linear(a, w_qkv, bias32, qkv, "store")
        self.rope_store(qkv, heads, kv_heads, head_dim, positions, req_index, rotary, block_table, page_size,
                        k_pages, v_pages, writes)

    def rope_store(self, qkv, heads, kv_heads, head_dim, positions, req_index, rotary, block_table,
                   page_size, k_pages, v_pages, writes):
        m = qkv.shape[0]
        x = qkv.double().view(m, heads + 2 * kv_heads, head_dim)
        if rotary is not None:
            cos, sin, dim = rotary
            half = dim // 2
            c = cos[positions.long()].double()[:, None, :]
            s = sin[positions.long()].double()[:, None, :]
            qk = x[:, :heads + kv_heads, :]
            x1, x2 = qk[..., :half].clone(), qk[..., half:dim].clone()
            qk[..., :half] = x1 * c - x2 * s
            qk[..., half:dim] = x2 * c + x1 * s
        qkv.copy_(x.view(m, -1).to(qkv.dtype))
        if not writes:
            return
        pos = positions.long()
        page = block_table[req_index.long(), pos // page_size].long()
        assert (page >= 0).all(), "write to a position without a page"
        off = pos % page_size
        k = qkv.view(m, heads + 2 * kv_heads, head_dim)[:, heads:heads + kv_heads]
        v = qkv.view(m, heads + 2 * kv_heads, head_dim)[:, heads + kv_heads:]
        k_pages[page, :, off, :] = k
        v_pages[page, :, off, :] = v

    def attention(self, qkv, out, heads, kv_heads, head_dim, scale, window, ctx, block_table,
                  page_size, k_pages, v_pages, own_kv=False):
        m = qkv.shape[0]
        q = qkv.view(m, heads + 2 * kv_heads, head_dim)[:, :heads].double()
        n_rep = heads // kv_heads
        res = torch.zeros(m, heads, head_dim, dtype=torch.float64, device=qkv.device)
        positions = ctx.positions.tolist()
        req_index = ctx.req_index.tolist()
        for t in range(m):
            p, r = positions[t], req_index[t]
            lo = max(0, p - window + 1) if window else 0
            idx = torch.arange(lo, p + 1, device=qkv.device)
            pages = block_table[r, idx // page_size].long()
            assert (pages >= 0).all(), "read of a position without a page"
            k = k_pages[pages, :, idx % page_size, :].double()   # [n, kv_heads, d]
            v = v_pages[pages, :, idx % page_size, :].double()
            for h in range(heads):
                s = (k[:, h // n_rep, :] @ q[t, h]) * scale
                e = torch.exp(s - s.max())
                res[t, h] = (e / e.sum()) @ v[:, h // n_rep, :]
        out.copy_(res.view(m, -1).to(out.dtype))

    def argmax(self, logits, out):
        out.copy_(torch.argmax(logits, dim=-1).to(out.dtype))

    def repetition_penalty(self, logits, seen, seen_start, penalty, pending=None):
        starts = seen_start.tolist()
        for r in range(logits.shape[0]):
            p = float(penalty[r])
            if p == 1.0:
                continue
            ids = seen[starts[r]:starts[r + 1]].long()
            if pending is not None and int(pending[r]) not in ids.tolist():
                ids = torch.cat([ids, pending[r:r + 1].long()])
            s = logits[r, ids]
            logits[r, ids] = torch.where(s > 0, s / p, s * p)

    def sample(self, logits, temperature, top_k, top_p, uniform, out):
        """Inverse CDF in vocabulary order over the distribution of tests/plain_qwen2.py."""
        import numpy as np
        from plain_qwen2 import sampling_distribution
        for r in range(logits.shape[0]):
            probs = sampling_distribution(logits[r].double().cpu().numpy(), [], float(temperature[r]),
                                          int(top_k[r]), float(top_p[r]), 1.0)
            cdf = np.cumsum(probs)
            i = int(np.searchsorted(cdf, float(uniform[r]) * cdf[-1], side="right"))
            kept = np.nonzero(probs > 0)[0]
            i = min(i, int(kept[-1]))
            while probs[i] == 0:
                i += 1
            out[r] = i
