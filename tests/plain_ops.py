"""Plain torch restatements of every kernel, with the kernels' own signatures.

Two uses: the ``-m gpu`` tests compare each CUDA kernel with the function of the same name
here, and the CPU tests put this class in the place of the CUDA kernel set so that the
engine's bookkeeping (batches, block tables, slots, the scheduler) can be run without a GPU.
It is test code: the engine itself never falls back to it.
"""

from __future__ import annotations

import torch


class PlainOps:
    name = "plain"

    def __init__(self, device="cpu"):
        self.device = torch.device(device)
        self.launches = 0
        # stands in for the kernels' device flag: a test sets it to see the engine react
        self.error_flag = torch.zeros(1, dtype=torch.int32, device=self.device)

    def describe_error(self, code):
        return RuntimeError(f"a kernel reported code {code}")

    def check_errors(self):
        code = int(self.error_flag.item())
        if code:
            self.error_flag.zero_()
            raise self.describe_error(code)

    def check_attention_sizes(self, heads, kv_heads, head_dim):
        assert heads % kv_heads == 0

    def embedding(self, ids, table):
        return table[ids.long()].float()

    def add_rmsnorm(self, residual, delta, weight, eps, dtype):
        if delta is not None:
            residual += delta.float()
        inv = torch.rsqrt(residual.pow(2).mean(dim=-1, keepdim=True) + eps)
        return (residual * inv * weight).to(dtype)

    def gather_rows(self, residual, delta, rows):
        index = rows.long()
        return residual[index].clone(), None if delta is None else delta[index].clone()

    def linear(self, a, w, bias=None, out_dtype=None):
        out = a.float() @ w.float().T
        if out_dtype != torch.float32:
            out = out.to(a.dtype).float()
        if bias is not None:
            out = out + bias
        return out.to(out_dtype or a.dtype)

    def linear_swiglu(self, a, gate_up):
        return self.swiglu(self.linear(a, gate_up))

    def linear_add(self, a, w, bias, residual):
        return self.linear(a, w, bias)

    def swiglu(self, gate_up):
        width = gate_up.shape[1] // 2
        gate, up = gate_up[:, :width].float(), gate_up[:, width:].float()
        return (gate / (1 + torch.exp(-gate)) * up).to(gate_up.dtype)

    def short_conv(self, bcx, *, kernel, bias, taps, ctx, view, write):
        hidden = bcx.shape[1] // 3
        dtype = bcx.dtype
        gate_b, gate_c, x = bcx[:, :hidden].float(), bcx[:, hidden:2 * hidden].float(), \
            bcx[:, 2 * hidden:].float()
        g = (gate_b * x).to(dtype).float()
        out = torch.empty_like(g)
        starts = ctx.request_start.tolist()
        history = ctx.history.tolist()
        slots = view.slots.tolist()
        for r in range(ctx.requests):
            first, last = starts[r], starts[r + 1]
            n = last - first
            state = view.state[slots[r]].float()                    # [taps-1, hidden]
            if taps > 1:
                valid = torch.arange(taps - 1) + history[r] - (taps - 1) >= 0
                state = state * valid[:, None].to(state.dtype)
                padded = torch.cat((state[:taps - 1], g[first:last]), dim=0)
            else:
                padded = g[first:last]
            y = torch.zeros(n, hidden)
            for k in range(taps):
                y = y + padded[k:k + n] * kernel[:, k]
            if bias is not None:
                y = y + bias
            out[first:last] = gate_c[first:last] * y
            if write and taps > 1:
                view.state[slots[r]][:taps - 1] = padded[n:n + taps - 1].to(view.state.dtype)
        return out.to(dtype)

    def linear_short_conv(self, a, w, w_bias, *, kernel, bias, taps, ctx, view, write):
        return self.short_conv(self.linear(a, w, w_bias), kernel=kernel, bias=bias, taps=taps,
                               ctx=ctx, view=view, write=write)

    def qk_norm_rope_store(self, qkv, *, heads, kv_heads, head_dim, q_weight, k_weight, eps,
                           rotary, ctx, view, write):
        tokens = qkv.shape[0]
        dtype = qkv.dtype
        split = qkv.float().view(tokens, heads + 2 * kv_heads, head_dim)
        q, k, v = split[:, :heads], split[:, heads:heads + kv_heads], split[:, heads + kv_heads:]

        def norm(x, weight):
            if weight is None:
                return x
            return x * torch.rsqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps) * weight

        def rotate(x):
            if rotary is None:
                return x
            inv_freq, rotary_dim = rotary
            half = rotary_dim // 2
            angles = ctx.positions.float()[:, None] * inv_freq[None, :]
            cos, sin = torch.cos(angles)[:, None, :], torch.sin(angles)[:, None, :]
            a, b = x[..., :half], x[..., half:rotary_dim]
            return torch.cat((a * cos - b * sin, b * cos + a * sin, x[..., rotary_dim:]), dim=-1)

        q = rotate(norm(q, q_weight)).to(dtype)
        k = rotate(norm(k, k_weight)).to(dtype)
        if write:
            positions = ctx.positions.tolist()
            requests = ctx.token_request.tolist()
            table = view.block_table.tolist()
            for t in range(tokens):
                page = table[requests[t]][positions[t] // view.page_size]
                assert page >= 0, "a key is written to a position without a page"
                offset = positions[t] % view.page_size
                view.kv[0, page, :, offset] = k[t]
                view.kv[1, page, :, offset] = v[t].to(dtype)
        return q.contiguous()

    def qkv_attention(self, qkv, *, heads, kv_heads, head_dim, q_weight, k_weight, eps, rotary,
                      scale, window, ctx, view, write):
        q = self.qk_norm_rope_store(qkv, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                    q_weight=q_weight, k_weight=k_weight, eps=eps, rotary=rotary,
                                    ctx=ctx, view=view, write=write)
        return self.paged_attention(q, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                    scale=scale, window=window, ctx=ctx, view=view)

    def paged_attention(self, q, *, heads, kv_heads, head_dim, scale, window, ctx, view):
        tokens = q.shape[0]
        out = torch.empty(tokens, heads, head_dim)
        positions = ctx.positions.tolist()
        requests = ctx.token_request.tolist()
        table = view.block_table.tolist()
        group = heads // kv_heads
        for t in range(tokens):
            p = positions[t]
            lowest = max(p - window + 1, 0) if window else 0
            keys = list(range(lowest, p + 1))
            pages = [table[requests[t]][key // view.page_size] for key in keys]
            assert min(pages) >= 0, "a key is read from a position without a page"
            offsets = [key % view.page_size for key in keys]
            k = view.kv[0, pages, :, offsets].float()            # [keys, kv_heads, head_dim]
            v = view.kv[1, pages, :, offsets].float()
            k = k.repeat_interleave(group, dim=1)
            v = v.repeat_interleave(group, dim=1)
            scores = torch.einsum("hd,khd->hk", q[t].float(), k) * scale
            out[t] = torch.einsum("hk,khd->hd", torch.softmax(scores, dim=-1), v)
        return out.reshape(tokens, heads * head_dim).to(q.dtype)

    def argmax(self, logits):
        return torch.argmax(logits, dim=-1).to(torch.int32)

    def decode_advance(self, chosen, token_ids, positions, history, record, counter):
        token_ids.copy_(chosen)
        positions += 1
        history += 1
        step = int(counter)
        if step < record.shape[0]:
            record[step] = chosen
        counter += 1

    def publish_tokens(self, chosen, index, published):
        published[index.long()] = chosen
        return torch.cat([chosen.to(torch.int32), self.error_flag.to(torch.int32)])

    def resolve_tokens(self, token_ids, source, published):
        taken = source >= 0
        token_ids[taken] = published[source[taken].long()]

    def reserve_sample_scratch(self, rows, vocab):
        pass

    def sample(self, logits, temperature, top_k, top_p, seed, step):
        """Token-order draw over the reference's kept set, in float64."""
        rows, vocab = logits.shape
        out = torch.empty(rows, dtype=torch.int32)
        probabilities = torch.empty(rows, vocab, dtype=torch.float32)
        for r in range(rows):
            if float(temperature[r]) <= 0:                   # greedy row
                out[r] = int(torch.argmax(logits[r]))
                probabilities[r] = 0
                probabilities[r, int(out[r])] = 1
                continue
            scaled = (logits[r] - logits[r].max()) * (1.0 / temperature[r])
            p = torch.exp(scaled.float())
            probabilities[r] = p
            kept = kept_set(p, int(top_k[r]), float(top_p[r]))
            weights = torch.zeros(vocab, dtype=torch.float64)
            weights[kept] = p[kept].double()
            running = torch.cumsum(weights, dim=0)
            target = uniform(int(seed[r]), int(step[r])) * float(weights.sum())
            hit = torch.nonzero((running >= target) & (weights > 0))
            out[r] = int(hit[0]) if len(hit) else int(kept.max())
        return out, probabilities


def kept_set(p, top_k, top_p):
    """Indices that the reference's rule keeps (src/mlx_one/text/sampling.py:56-81): stable
    descending order, first top_k, then the shortest prefix reaching top_p of their mass."""
    order = torch.sort(p.double(), descending=True, stable=True).indices
    if top_k > 0:
        order = order[:top_k]
    ranked = p.double()[order]
    if top_p < 1.0:
        running = torch.cumsum(ranked, dim=0)
        cutoff = top_p * float(ranked.sum())
        count = min(int(torch.searchsorted(running, torch.tensor(cutoff, dtype=torch.float64))) + 1,
                    len(order))
        order = order[:count]
    return order


def uniform(seed, step):
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + (step + 1) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)
