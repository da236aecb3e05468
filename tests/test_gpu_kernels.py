"""Each CUDA kernel alone against its plain restatement (tests/plain_ops.py), at sizes other
than the engine's tiny models: head sizes in steps of 16, odd head counts and groups, widths
and vocabularies that are no power of two."""

import math

import pytest
import torch

from plain_ops import PlainOps, kept_set, uniform
from mlx_one_b200.parts.base import FixedState, PagedKeyValues, PagedView, StateView, StepContext

pytestmark = pytest.mark.gpu
DEVICE = "cuda:0"


@pytest.fixture(scope="module")
def ops():
    from mlx_one_b200.kernels import default_ops
    return default_ops(DEVICE)


@pytest.fixture(scope="module")
def plain():
    return PlainOps()


def tolerance(dtype):
    return dict(atol=2e-5, rtol=2e-5) if dtype == torch.float32 else dict(atol=2e-2, rtol=2e-2)


def make_batch(portions, histories, page_size, device, extra_pages=3, seed=0):
    """A ragged batch and block tables with shuffled pages. Returns (ctx, table, pages)."""
    generator = torch.Generator().manual_seed(seed)
    requests = len(portions)
    blocks = [-(-(h + n) // page_size) for h, n in zip(histories, portions)]
    pages = sum(blocks) + extra_pages
    order = torch.randperm(pages, generator=generator).tolist()
    width = max(blocks) + 2
    table = torch.full((requests, width), -1, dtype=torch.int32)
    for r, count in enumerate(blocks):
        for b in range(count):
            table[r, b] = order.pop()
    positions, token_request, starts = [], [], [0]
    for r, (h, n) in enumerate(zip(histories, portions)):
        positions += list(range(h, h + n))
        token_request += [r] * n
        starts.append(starts[-1] + n)
    as_int = lambda values: torch.tensor(values, dtype=torch.int32, device=device)
    ctx = StepContext(tokens=len(positions), requests=requests,
                      token_ids=as_int([0] * len(positions)), positions=as_int(positions),
                      token_request=as_int(token_request), request_start=as_int(starts),
                      history=as_int(histories), max_portion=max(portions),
                      max_context=max(h + n for h, n in zip(histories, portions)))
    return ctx, table.to(device), pages


def on_cpu(ctx):
    return StepContext(tokens=ctx.tokens, requests=ctx.requests, token_ids=ctx.token_ids.cpu(),
                       positions=ctx.positions.cpu(), token_request=ctx.token_request.cpu(),
                       request_start=ctx.request_start.cpu(), history=ctx.history.cpu(),
                       max_portion=ctx.max_portion, max_context=ctx.max_context)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,vocab", [(80, 333), (2048, 1000), (1000, 50)])
@pytest.mark.parametrize("rows", [37, 1600])      # a block per row; a warp per row
def test_embedding_and_norm(ops, plain, dtype, hidden, vocab, rows):
    torch.manual_seed(0)
    table = torch.randn(vocab, hidden).to(dtype)
    ids = torch.randint(0, vocab, (rows,), dtype=torch.int32)
    got = ops.embedding(ids.to(DEVICE), table.to(DEVICE))
    assert torch.equal(got.cpu(), plain.embedding(ids, table))
    residual = torch.randn(rows, hidden)
    delta = torch.randn(rows, hidden).to(dtype)
    weight = 1 + 0.1 * torch.randn(hidden)
    for use_delta in (True, False):
        res_gpu = residual.clone().to(DEVICE)
        res_cpu = residual.clone()
        got = ops.add_rmsnorm(res_gpu, delta.to(DEVICE) if use_delta else None,
                              weight.to(DEVICE), 1e-5, dtype)
        want = plain.add_rmsnorm(res_cpu, delta if use_delta else None, weight, 1e-5, dtype)
        torch.testing.assert_close(res_gpu.cpu(), res_cpu, atol=1e-6, rtol=1e-6)
        torch.testing.assert_close(got.cpu().float(), want.float(), **tolerance(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gather_swiglu_bias(ops, plain, dtype):
    torch.manual_seed(1)
    residual, delta = torch.randn(29, 112), torch.randn(29, 112).to(dtype)
    rows = torch.tensor([3, 28, 0, 3], dtype=torch.int32)
    picked, picked_delta = ops.gather_rows(residual.to(DEVICE), delta.to(DEVICE), rows.to(DEVICE))
    assert torch.equal(picked.cpu(), residual[rows.long()])
    assert torch.equal(picked_delta.cpu(), delta[rows.long()])
    gate_up = torch.randn(29, 2 * 77).to(dtype)
    torch.testing.assert_close(ops.swiglu(gate_up.to(DEVICE)).cpu().float(),
                               plain.swiglu(gate_up).float(), **tolerance(dtype))


@pytest.mark.parametrize("m,n,k", [(1, 5, 7), (37, 333, 130), (64, 96, 288), (130, 1000, 96)])
def test_matrix_product_float32(ops, plain, m, n, k):
    """True 32-bit: compared with a float64 product at float32 rounding, no tensor-core mode."""
    torch.manual_seed(2)
    a, w, bias = torch.randn(m, k), torch.randn(n, k), torch.randn(n)
    got = ops.linear(a.to(DEVICE), w.to(DEVICE), bias.to(DEVICE)).cpu()
    want = (a.double() @ w.double().T + bias.double()).float()
    torch.testing.assert_close(got, want, atol=1e-5 * math.sqrt(k), rtol=1e-6)
    # a row's result does not depend on which other rows the call has
    alone = ops.linear(a[:1].contiguous().to(DEVICE), w.to(DEVICE), bias.to(DEVICE)).cpu()
    assert torch.equal(alone[0], got[0])


@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (8, 333, 136), (130, 1000, 96)])
def test_matrix_product_bfloat16(ops, plain, m, n, k):
    """Whatever kernel the sizes select (skinny, tcgen05 or the library) gives the product."""
    torch.manual_seed(3)
    a, w = torch.randn(m, k).bfloat16(), torch.randn(n, k).bfloat16()
    bias = torch.randn(n)
    got = ops.linear(a.to(DEVICE), w.to(DEVICE), bias.to(DEVICE)).cpu().float()
    want = a.float() @ w.float().T + bias
    torch.testing.assert_close(got, want, atol=0.02 * math.sqrt(k), rtol=2e-2)
    logits = ops.linear(a.to(DEVICE), w.to(DEVICE), out_dtype=torch.float32).cpu()
    torch.testing.assert_close(logits, a.float() @ w.float().T, atol=1e-3 * math.sqrt(k), rtol=1e-3)


@pytest.mark.parametrize("m", [1, 7, 8, 9, 16, 17, 32])
@pytest.mark.parametrize("n,k", [(16, 64), (333, 136), (1000, 2048), (96, 8192), (50, 8)])
def test_skinny_product(ops, m, n, k):
    """The weight-streaming product for few rows (up to the 32 that the kernel takes, not only
    the 8 that the engine sends it), all four epilogues, against float64."""
    ops.skinny_max_rows = 32
    try:
        _skinny_product_case(ops, m, n, k)
    finally:
        ops.skinny_max_rows = 8


def _skinny_product_case(ops, m, n, k):
    torch.manual_seed(m * 1000 + n + k)
    a = torch.randn(m, k).bfloat16()
    w = (torch.randn(n, k) / math.sqrt(k)).bfloat16()
    bias = torch.randn(n)
    want = a.double() @ w.double().T
    assert ops._skinny(a.to(DEVICE), w.to(DEVICE))
    before = ops.launches
    got = ops.linear(a.to(DEVICE), w.to(DEVICE), bias.to(DEVICE))
    assert ops.launches == before + 1          # one kernel, no library call plus bias kernel
    torch.testing.assert_close(got.cpu().double(), want + bias.double(), atol=2e-2, rtol=2e-2)
    logits = ops.linear(a.to(DEVICE), w.to(DEVICE), out_dtype=torch.float32)
    torch.testing.assert_close(logits.cpu().double(), want, atol=1e-3, rtol=1e-3)
    residual = torch.randn(m, n)
    on_gpu = residual.clone().to(DEVICE)
    assert ops.linear_add(a.to(DEVICE), w.to(DEVICE), bias.to(DEVICE), on_gpu) is None
    torch.testing.assert_close(on_gpu.cpu().double(), residual.double() + want + bias.double(),
                               atol=1e-3, rtol=1e-3)
    if n % 2 == 0:
        gated = ops.linear_swiglu(a.to(DEVICE), w.to(DEVICE))
        gate, up = want[:, :n // 2], want[:, n // 2:]
        torch.testing.assert_close(gated.cpu().double(), gate * torch.sigmoid(gate) * up,
                                   atol=2e-2, rtol=2e-2)
    # a token's result does not depend on the other tokens of the call
    alone = ops.linear(a[:1].contiguous().to(DEVICE), w.to(DEVICE), out_dtype=torch.float32)
    assert torch.equal(alone[0].cpu(), logits[0].cpu())
    # the same product with the RMSNorm of 32-bit rows applied while they are loaded
    from mlx_one_b200.parts import NormedInput
    rows = torch.randn(m, k).to(DEVICE)
    kept = (ops.fused_norms, ops.fused_norm_max_rows)
    ops.fused_norms, ops.fused_norm_max_rows = True, 16       # as many rows as the kernel takes
    fits = ops.can_fuse_norm(rows, torch.bfloat16)
    ops.fused_norms, ops.fused_norm_max_rows = kept
    assert fits or m > 16 or k > 4000
    if fits:
        scale = (1 + 0.1 * torch.randn(k)).to(DEVICE)
        lazy = NormedInput(rows, scale, 1e-5, torch.bfloat16, ops)
        normed = lazy.materialize()
        fused = ops.linear(lazy, w.to(DEVICE), out_dtype=torch.float32)
        apart = ops.linear(normed, w.to(DEVICE), out_dtype=torch.float32)
        torch.testing.assert_close(fused, apart, atol=2e-2, rtol=2e-2)
        if n % 2 == 0:
            torch.testing.assert_close(ops.linear_swiglu(lazy, w.to(DEVICE)).float(),
                                       ops.linear_swiglu(normed, w.to(DEVICE)).float(),
                                       atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("m", [33, 128, 200, 777])
@pytest.mark.parametrize("n,k", [(128, 64), (334, 136), (1000, 2048), (2048, 520), (50, 8)])
def test_tcgen05_product(ops, m, n, k):
    """The tensor-memory product for many rows: all four epilogues, ragged edges in M, N, K."""
    assert ops.enable_tcgen05(True)
    least, ops.tcgen05_min_rows = ops.tcgen05_min_rows, 1
    ops.tcgen05_always = True
    try:
        torch.manual_seed(m + n + k)
        a = torch.randn(m, k).bfloat16()
        w = (torch.randn(n, k) / math.sqrt(k)).bfloat16()
        bias = torch.randn(n)
        want = a.double() @ w.double().T
        assert ops._tcgen05(a.to(DEVICE), w.to(DEVICE)) and not ops._skinny(a.to(DEVICE), w.to(DEVICE))
        got = ops.linear(a.to(DEVICE), w.to(DEVICE), bias.to(DEVICE))
        torch.testing.assert_close(got.cpu().double(), want + bias.double(), atol=2e-2, rtol=2e-2)
        logits = ops.linear(a.to(DEVICE), w.to(DEVICE), out_dtype=torch.float32)
        torch.testing.assert_close(logits.cpu().double(), want, atol=1e-3, rtol=1e-3)
        residual = torch.randn(m, n)
        on_gpu = residual.clone().to(DEVICE)
        assert ops.linear_add(a.to(DEVICE), w.to(DEVICE), bias.to(DEVICE), on_gpu) is None
        torch.testing.assert_close(on_gpu.cpu().double(), residual.double() + want + bias.double(),
                                   atol=1e-3, rtol=1e-3)
        gated = ops.linear_swiglu(a.to(DEVICE), w.to(DEVICE))
        gate, up = want[:, :n // 2], want[:, n // 2:]
        torch.testing.assert_close(gated.cpu().double(), gate * torch.sigmoid(gate) * up,
                                   atol=2e-2, rtol=2e-2)
        ops.check_errors()
    finally:
        ops.enable_tcgen05(True)
        ops.tcgen05_min_rows = least
        ops.tcgen05_always = False


@pytest.mark.parametrize("m", [33, 64, 65, 100, 128])
@pytest.mark.parametrize("n,k", [(128, 128), (334, 136), (2048, 2048), (2048, 8192), (6144, 520),
                                 (50, 64), (16384, 2048)])
def test_tcgen05_swapped_product(ops, m, n, k):
    """The product for 33 to 128 rows with the weights as the 128-row operand: all four
    epilogues, ragged edges in M, N and K, clusters of 1 to 8 blocks that split K."""
    assert ops.enable_tcgen05(True)
    ops.swapped_products = True
    try:
        _swapped_product_case(ops, m, n, k)
    finally:
        ops.swapped_products = False


def _swapped_product_case(ops, m, n, k):
    torch.manual_seed(m + n + k)
    a = torch.randn(m, k).bfloat16()
    w = (torch.randn(n, k) / math.sqrt(k)).bfloat16()
    bias = torch.randn(n)
    want = a.double() @ w.double().T
    assert ops._swapped(a.to(DEVICE), w.to(DEVICE))
    got = ops.linear(a.to(DEVICE), w.to(DEVICE), bias.to(DEVICE))
    torch.testing.assert_close(got.cpu().double(), want + bias.double(), atol=2e-2, rtol=2e-2)
    logits = ops.linear(a.to(DEVICE), w.to(DEVICE), out_dtype=torch.float32)
    torch.testing.assert_close(logits.cpu().double(), want, atol=1e-3, rtol=1e-3)
    again = ops.linear(a.to(DEVICE), w.to(DEVICE), out_dtype=torch.float32)
    assert torch.equal(logits, again)                      # the same sum whatever the timing
    residual = torch.randn(m, n)
    on_gpu = residual.clone().to(DEVICE)
    assert ops.linear_add(a.to(DEVICE), w.to(DEVICE), bias.to(DEVICE), on_gpu) is None
    torch.testing.assert_close(on_gpu.cpu().double(), residual.double() + want + bias.double(),
                               atol=1e-3, rtol=1e-3)
    gated = ops.linear_swiglu(a.to(DEVICE), w.to(DEVICE))
    gate, up = want[:, :n // 2], want[:, n // 2:]
    torch.testing.assert_close(gated.cpu().double(), gate * torch.sigmoid(gate) * up,
                               atol=2e-2, rtol=2e-2)
    ops.check_errors()


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hidden,taps,bias", [(48, 3, False), (200, 4, True), (64, 2, True),
                                              (32, 1, False), (96, 7, False), (204, 3, True)])
@pytest.mark.parametrize("decode", [False, True, "long"])
def test_short_conv(ops, plain, dtype, hidden, taps, bias, decode):
    """Portions that start at position 0, in the middle, shorter than the kernel is wide; single
    tokens (the fused decode kernel) at positions 0, 1 and beyond; and so many tokens that the
    kernel for runs of tokens is taken, with requests that begin inside a run."""
    torch.manual_seed(4)
    if decode == "long":
        portions, histories = [301, 1, 2, 43, 1], [0, 7, 0, 1, 0]
    else:
        portions, histories = ([1] * 5, [0, 7, 3, 1, 2]) if decode else ([5, 1, 9, 2, 1], [0, 7, 3, 0, 1])
    ctx, _, _ = make_batch(portions, histories, 4, DEVICE)
    slots = torch.tensor([4, 0, 2, 5, 1], dtype=torch.int32)
    state = torch.randn(6, max(taps - 1, 1), hidden).to(dtype)
    bcx = torch.randn(ctx.tokens, 3 * hidden).to(dtype)
    kernel = torch.randn(hidden, taps)
    conv_bias = torch.randn(hidden) if bias else None
    need = FixedState((max(taps - 1, 1), hidden))
    state_gpu = state.clone().to(DEVICE)
    got = ops.short_conv(bcx.to(DEVICE), kernel=kernel.to(DEVICE),
                         bias=None if conv_bias is None else conv_bias.to(DEVICE), taps=taps,
                         ctx=ctx, view=StateView(state_gpu, slots.to(DEVICE), need), write=True)
    state_cpu = state.clone()
    want = plain.short_conv(bcx, kernel=kernel, bias=conv_bias, taps=taps, ctx=on_cpu(ctx),
                            view=StateView(state_cpu, slots, need), write=True)
    torch.testing.assert_close(got.cpu().float(), want.float(), **tolerance(dtype))
    if taps > 1:
        # rows of positions before 0 are never read, so they need not agree
        for r, (h, n) in enumerate(zip(histories, portions)):
            valid = [s for s in range(taps - 1) if h + n - (taps - 1) + s >= 0]
            torch.testing.assert_close(state_gpu.cpu()[slots[r], valid].float(),
                                       state_cpu[slots[r], valid].float(), **tolerance(dtype))


@pytest.mark.parametrize("rows,hidden,k,taps,bias", [
    (5, 40, 64, 3, True), (1, 2048, 2048, 3, False), (8, 136, 200, 4, False), (3, 24, 72, 1, True),
    (17, 600, 96, 2, True), (32, 48, 2048, 3, False), (4, 40, 64, 5, True),
    (12, 2048, 2048, 3, True), (16, 136, 264, 3, False),
    (5, 40, 6144, 3, True), (7, 2048, 4096, 3, False)])      # rows too long for shared memory
def test_linear_short_conv(ops, plain, rows, hidden, k, taps, bias):
    """The product with the convolution's decode update as its epilogue, against the plain
    convolution of the product that the kernel without that epilogue gives (the same sums in
    the same order, so B, C and x round alike and what is compared is the epilogue): positions
    0, 1 and later, slots in any order, more taps than it fuses (5)."""
    ops.skinny_max_rows = 32
    try:
        _linear_short_conv_case(ops, plain, rows, hidden, k, taps, bias)
    finally:
        ops.skinny_max_rows = 8


def _linear_short_conv_case(ops, plain, rows, hidden, k, taps, bias):
    torch.manual_seed(14)
    dtype = torch.bfloat16
    histories = [(3 * r) % 7 if r % 3 else r % 2 for r in range(rows)]
    ctx, _, _ = make_batch([1] * rows, histories, 4, DEVICE)
    slots = torch.randperm(rows + 2)[:rows].to(torch.int32)
    state = torch.randn(rows + 2, max(taps - 1, 1), hidden).to(dtype)
    a = torch.randn(rows, k).to(dtype)
    w = (torch.randn(3 * hidden, k) / k ** 0.5).to(dtype)
    w_bias = torch.randn(3 * hidden) if bias else None
    kernel = torch.randn(hidden, taps)
    conv_bias = torch.randn(hidden) if bias else None
    need = FixedState((max(taps - 1, 1), hidden))
    to = lambda t: None if t is None else t.to(DEVICE)
    state_gpu = state.clone().to(DEVICE)
    before = ops.launches
    got = ops.linear_short_conv(to(a), to(w), to(w_bias), kernel=to(kernel), bias=to(conv_bias),
                                taps=taps, ctx=ctx, view=StateView(state_gpu, to(slots), need),
                                write=True)
    assert ops.launches - before == (1 if taps <= 4 else 2)
    state_cpu = state.clone()
    bcx = ops.linear(to(a), to(w), to(w_bias)).cpu()
    torch.testing.assert_close(bcx.float(), plain.linear(a, w, w_bias).float(), **tolerance(dtype))
    want = plain.short_conv(bcx, kernel=kernel, bias=conv_bias, taps=taps, ctx=on_cpu(ctx),
                            view=StateView(state_cpu, slots, need), write=True)
    torch.testing.assert_close(got.cpu().float(), want.float(), **tolerance(dtype))
    if taps > 1:
        for r, h in enumerate(histories):
            valid = [s for s in range(taps - 1) if h + 1 - (taps - 1) + s >= 0]
            torch.testing.assert_close(state_gpu.cpu()[slots[r], valid].float(),
                                       state_cpu[slots[r], valid].float(), **tolerance(dtype))
    untouched = [s for s in range(rows + 2) if s not in slots.tolist()]
    assert torch.equal(state_gpu.cpu()[untouched], state[untouched])
    # the same with the RMSNorm of 32-bit rows applied while they are loaded: still one kernel
    from mlx_one_b200.parts import NormedInput
    source = torch.randn(rows, k).to(DEVICE)
    kept = (ops.fused_norms, ops.fused_norm_max_rows)
    ops.fused_norms, ops.fused_norm_max_rows = True, 16       # as many rows as the kernel takes
    fits = ops.can_fuse_norm(source, dtype)
    ops.fused_norms, ops.fused_norm_max_rows = kept
    assert fits or rows > 16 or k > 4000
    if fits and taps <= 4:
        lazy = NormedInput(source, (1 + 0.1 * torch.randn(k)).to(DEVICE), 1e-5, dtype, ops)
        states = [state.clone().to(DEVICE) for _ in range(2)]
        results = []
        for given, held in zip((lazy, lazy.materialize()), states):
            before = ops.launches
            results.append(ops.linear_short_conv(given, to(w), to(w_bias), kernel=to(kernel),
                                                 bias=to(conv_bias), taps=taps, ctx=ctx,
                                                 view=StateView(held, to(slots), need), write=True))
            assert ops.launches - before == 1
        torch.testing.assert_close(results[0].float(), results[1].float(), **tolerance(dtype))
        torch.testing.assert_close(states[0].float(), states[1].float(), **tolerance(dtype))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,rotary_dim,norm", [
    (4, 2, 16, 16, True), (3, 1, 32, 32, True), (6, 3, 48, 24, False), (5, 5, 80, 80, True),
    (2, 1, 256, 256, True), (8, 2, 64, 64, True), (4, 4, 128, 128, False), (3, 3, 64, 32, True)])
def test_qk_norm_rope_store(ops, plain, dtype, heads, kv_heads, head_dim, rotary_dim, norm):
    torch.manual_seed(5)
    page_size = 8
    ctx, table, pages = make_batch([6, 1, 11], [0, 100_000, 13], page_size, DEVICE)
    qkv = torch.randn(ctx.tokens, (heads + 2 * kv_heads) * head_dim).to(dtype)
    q_weight = (1 + 0.1 * torch.randn(head_dim)) if norm else None
    k_weight = (1 + 0.1 * torch.randn(head_dim)) if norm else None
    half = rotary_dim // 2
    inv_freq = torch.pow(torch.tensor(10000.0), -torch.arange(half, dtype=torch.float32) / half)
    need = PagedKeyValues(kv_heads, head_dim)
    kv_gpu = torch.zeros(2, pages, kv_heads, page_size, head_dim, dtype=dtype, device=DEVICE)
    kv_cpu = torch.zeros(2, pages, kv_heads, page_size, head_dim, dtype=dtype)
    to = lambda t: None if t is None else t.to(DEVICE)
    got = ops.qk_norm_rope_store(
        qkv.to(DEVICE), heads=heads, kv_heads=kv_heads, head_dim=head_dim, q_weight=to(q_weight),
        k_weight=to(k_weight), eps=1e-5, rotary=(inv_freq.to(DEVICE), rotary_dim), ctx=ctx,
        view=PagedView(kv_gpu, table, page_size, need), write=True)
    want = plain.qk_norm_rope_store(
        qkv, heads=heads, kv_heads=kv_heads, head_dim=head_dim, q_weight=q_weight,
        k_weight=k_weight, eps=1e-5, rotary=(inv_freq, rotary_dim), ctx=on_cpu(ctx),
        view=PagedView(kv_cpu, table.cpu(), page_size, need), write=True)
    # at position 100000 a 32-bit angle is exact to ~1e-2 rad only in its last bits; both sides
    # compute position * inv_freq in 32-bit, so they agree far better than that
    torch.testing.assert_close(got.cpu().float(), want.float(), **tolerance(dtype))
    torch.testing.assert_close(kv_gpu.cpu().float(), kv_cpu.float(), **tolerance(dtype))
    ops.check_errors()


def attention_case(ops, plain, dtype, heads, kv_heads, head_dim, page_size, portions, histories,
                   window, tensor_cores, seed=6, spike=None, tcgen05=False, ramp=None):
    torch.manual_seed(seed)
    ctx, table, pages = make_batch(portions, histories, page_size, DEVICE, seed=seed)
    kv = torch.randn(2, pages, kv_heads, page_size, head_dim).to(dtype)
    q = torch.randn(ctx.tokens, heads, head_dim).to(dtype)
    if ramp is not None:
        # every query's scores rise by `ramp` (in units of e) per 64 keys along the context, so
        # that the running maximum keeps moving and earlier keys still weigh in
        scale = head_dim ** -0.5
        direction = torch.zeros(head_dim)
        direction[::2] = 1.0
        direction /= direction.norm()
        q = (q.float() * 0.3 + direction * 4.0).to(dtype)
        for request, (portion, history) in enumerate(zip(portions, histories)):
            for position in range(history + portion):
                page = int(table[request, position // page_size])
                rise = ramp * position / 64 / (4.0 * scale)
                kv[0, page, :, position % page_size] = (
                    kv[0, page, :, position % page_size].float() * 0.3 + direction * rise).to(dtype)
    if spike is not None:
        # one far key and the last query are scaled so that this key's score stands out:
        # an error in finding its page or position would change the output visibly
        request, key_position = spike
        page = int(table[request, key_position // page_size])
        kv[0, page, :, key_position % page_size] *= 4
        last = int(ctx.request_start[request + 1]) - 1
        q[last] = kv[0, page, :, key_position % page_size].repeat_interleave(
            heads // kv_heads, dim=0).float().to(dtype) * 2
    need = PagedKeyValues(kv_heads, head_dim, window)
    scale = head_dim ** -0.5
    ops.tensor_core_attention = tensor_cores
    ops.tcgen05_attention = tcgen05
    try:
        got = ops.paged_attention(q.to(DEVICE), heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                  scale=scale, window=window, ctx=ctx,
                                  view=PagedView(kv.to(DEVICE), table, page_size, need))
    finally:
        ops.tensor_core_attention = True
        ops.tcgen05_attention = True
    want = plain.paged_attention(q, heads=heads, kv_heads=kv_heads, head_dim=head_dim,
                                 scale=scale, window=window, ctx=on_cpu(ctx),
                                 view=PagedView(kv, table.cpu(), page_size, need))
    ops.check_errors()
    torch.testing.assert_close(got.cpu().float(), want.float(), **tolerance(dtype))


SHAPES = [(4, 2, 16, 4), (3, 1, 32, 8), (6, 2, 48, 16), (8, 8, 64, 16), (32, 8, 64, 16),
          (5, 5, 80, 32), (4, 1, 128, 64), (2, 2, 96, 1), (34, 2, 112, 16)]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("heads,kv_heads,head_dim,page_size", SHAPES)
@pytest.mark.parametrize("window", [None, 37])
def test_attention_general(ops, plain, dtype, heads, kv_heads, head_dim, page_size, window):
    attention_case(ops, plain, dtype, heads, kv_heads, head_dim, page_size,
                   portions=[7, 1, 70, 2], histories=[0, 200, 31, 64], window=window,
                   tensor_cores=False, spike=(1, 3 if window is None else 180))


@pytest.mark.parametrize("heads,kv_heads,head_dim,page_size", SHAPES)
@pytest.mark.parametrize("window", [None, 37, 64, 1])
def test_attention_prefill_tensor_cores(ops, plain, heads, kv_heads, head_dim, page_size, window):
    """Portions beside single tokens; a portion that crosses tiles of 64 rows and 64 keys; a
    window's edge at 37, exactly at a tile (64) and of one key."""
    attention_case(ops, plain, torch.bfloat16, heads, kv_heads, head_dim, page_size,
                   portions=[7, 1, 150, 2, 64], histories=[0, 200, 31, 64, 64], window=window,
                   tensor_cores=True, spike=(1, 3 if window is None else 200))


@pytest.mark.parametrize("heads,kv_heads,head_dim,page_size", SHAPES)
@pytest.mark.parametrize("window", [None, 37])
@pytest.mark.parametrize("histories", [[0, 1, 63, 64, 65], [700, 3, 255, 256, 1030]])
@pytest.mark.parametrize("cluster", [False, True])
def test_attention_decode_tensor_cores(ops, plain, heads, kv_heads, head_dim, page_size, window,
                                       histories, cluster):
    """One token per request: contexts at the edges of tiles, split over several blocks, which
    are merged by a kernel of its own or, as a thread-block cluster, among themselves."""
    far = (0, 5) if histories[0] > 100 and window is None else None
    kept = (ops.cluster_merge, ops.cluster_merge_max_splits)
    ops.cluster_merge, ops.cluster_merge_max_splits = cluster, 8       # clusters of every size
    try:
        attention_case(ops, plain, torch.bfloat16, heads, kv_heads, head_dim, page_size,
                       portions=[1] * 5, histories=histories, window=window, tensor_cores=True,
                       spike=far)
    finally:
        ops.cluster_merge, ops.cluster_merge_max_splits = kept


@pytest.mark.parametrize("heads,kv_heads,page_size", [
    (8, 8, 16), (32, 8, 16), (4, 2, 8), (16, 2, 64), (3, 3, 128), (8, 1, 256), (64, 1, 32),
    (24, 8, 16), (6, 2, 8), (5, 1, 64), (7, 1, 16)])       # groups of 3, 5, 7 do not divide 128 rows
@pytest.mark.parametrize("window", [None, 37, 128, 300])
def test_attention_prefill_tcgen05(ops, plain, heads, kv_heads, page_size, window):
    """The tcgen05 kernel (head size 64): query heads of a group stacked in one block; portions
    that end inside a block of rows, cross tiles of 128 keys and start deep in a context; single
    tokens beside them; windows inside a tile, of exactly a tile and over several."""
    assert ops.lib.mlxone_attention_tcgen05_supports(64, heads, kv_heads, page_size)
    before = ops.launches
    attention_case(ops, plain, torch.bfloat16, heads, kv_heads, 64, page_size,
                   portions=[7, 1, 300, 2, 128, 33], histories=[0, 200, 500, 64, 128, 1000],
                   window=window, tensor_cores=True, tcgen05=True,
                   spike=(2, 5 if window is None else 700))
    assert ops.launches - before <= 2           # with few key heads: cut by keys, and a merge


@pytest.mark.parametrize("heads,kv_heads,page_size", [(24, 8, 16), (32, 8, 16), (4, 2, 8), (5, 1, 64)])
@pytest.mark.parametrize("window", [None, 300, 1000])
@pytest.mark.parametrize("portions,histories", [([512], [1100]), ([3, 200, 1], [5000, 0, 77]),
                                                 ([130], [0])])
def test_attention_prefill_tcgen05_key_splits(ops, plain, heads, kv_heads, page_size, window,
                                              portions, histories):
    """Fewer items than SMs (a prompt's portion beside a step's decodes): the items' keys are cut
    into parts that run side by side and a merge kernel adds them up. Parts without keys (rows
    early in a prompt, a window that ends before the part), one far key that must show, and the
    same launch uncut."""
    far = (0, 5) if window is None and histories[0] > 64 else None
    before = ops.launches
    attention_case(ops, plain, torch.bfloat16, heads, kv_heads, 64, page_size, portions=portions,
                   histories=histories, window=window, tensor_cores=True, tcgen05=True, spike=far)
    cut = ops.launches - before
    kept, ops.prefill_key_splits = ops.prefill_key_splits, False
    try:
        before = ops.launches
        attention_case(ops, plain, torch.bfloat16, heads, kv_heads, 64, page_size,
                       portions=portions, histories=histories, window=window, tensor_cores=True,
                       tcgen05=True, spike=far)
        assert ops.launches - before == 1
    finally:
        ops.prefill_key_splits = kept
    assert cut in (1, 2)
    if portions == [512] and window is None:
        assert cut == 2                 # this one is cut: the kernel and the merge


@pytest.mark.parametrize("heads,kv_heads,page_size", [(32, 8, 16), (8, 4, 8), (6, 6, 64),
                                                      (24, 8, 16)])
@pytest.mark.parametrize("window", [None, 300])
def test_attention_prefill_tcgen05_many_items(ops, plain, heads, kv_heads, page_size, window):
    """So many tokens that the kernel takes its shape with tiles of 64 keys and two blocks an
    SM (at least two items of work for every SM)."""
    before = ops.launches
    attention_case(ops, plain, torch.bfloat16, heads, kv_heads, 64, page_size,
                   portions=[2100, 1, 1900, 2, 37], histories=[0, 200, 300, 64, 1000],
                   window=window, tensor_cores=True, tcgen05=True,
                   spike=(2, 5 if window is None else 2000))
    assert ops.launches - before == 1


@pytest.mark.parametrize("ramp", [0.7, 3.0, 12.0])
@pytest.mark.parametrize("portions,histories", [([300, 1, 128], [500, 900, 0]),
                                                 ([2100, 2, 1900], [0, 64, 300])])
def test_attention_prefill_tcgen05_rising_scores(ops, plain, ramp, portions, histories):
    """Scores that rise along the context: the maximum that the exponentials are taken against
    follows the running maximum only from time to time, and the output summed so far is then
    rescaled in tensor memory. Slopes at which that happens every dozen tiles, every other tile
    and at every tile, in both shapes of the kernel."""
    attention_case(ops, plain, torch.bfloat16, 8, 2, 64, 16, portions=portions,
                   histories=histories, window=None, tensor_cores=True, tcgen05=True, ramp=ramp)


@pytest.mark.parametrize("heads,kv_heads,head_dim,page_size", [
    (32, 8, 64, 16), (24, 8, 64, 16), (3, 1, 32, 8), (20, 2, 128, 32), (6, 3, 96, 4), (4, 2, 64, 1)])
@pytest.mark.parametrize("norm,rotate,window", [(True, True, None), (False, True, 70),
                                                 (True, False, None), (False, False, 33)])
@pytest.mark.parametrize("cluster", [False, True])
def test_decode_attention_from_the_fused_projection(ops, plain, heads, kv_heads, head_dim,
                                                    page_size, norm, rotate, window, cluster):
    """A step of single tokens: q/k norm, rotation, the write of key and value into the page and
    attention in one kernel, against the plain preparation followed by plain attention: the
    mixed heads and the cache afterwards. Contexts from one key (the token's own) to several
    splits, positions at the edges of tiles of 32 keys and of pages; one request's query is made
    to pick out its own new key, which only the fused kernel's shared-memory copy can serve."""
    torch.manual_seed(heads * 7 + head_dim)
    histories = [0, 1, 31, 32, 63, 64, 200, 1023, 1500]
    portions = [1] * len(histories)
    ctx, table, pages = make_batch(portions, histories, page_size, DEVICE, seed=3)
    assert ops.lib.mlxone_attention_decode_fused_supports(head_dim)
    kv = torch.randn(2, pages, kv_heads, page_size, head_dim).bfloat16()
    width = (heads + 2 * kv_heads) * head_dim
    qkv = torch.randn(ctx.tokens, width).bfloat16()
    # request 6: the query heads equal the new key (before norm and rotation both are scaled
    # alike), times a large factor, so that its own position dominates the softmax
    group = heads // kv_heads
    for h in range(heads):
        k_at = (heads + h // group) * head_dim
        qkv[6, h * head_dim:(h + 1) * head_dim] = qkv[6, k_at:k_at + head_dim] * 3
    q_weight = (1 + 0.1 * torch.randn(head_dim)) if norm else None
    k_weight = (1 + 0.1 * torch.randn(head_dim)) if norm else None
    rotary = None
    if rotate:
        half = head_dim // 2
        rotary = (torch.pow(torch.tensor(10000.0), -torch.arange(half, dtype=torch.float32) / half),
                  head_dim)
    need = PagedKeyValues(kv_heads, head_dim, window)
    arguments = dict(heads=heads, kv_heads=kv_heads, head_dim=head_dim, eps=1e-5 if norm else None,
                     scale=head_dim ** -0.5, window=window, write=True)
    kv_gpu = kv.clone().to(DEVICE)
    on_gpu = lambda v: None if v is None else v.to(DEVICE)
    kept = (ops.cluster_merge, ops.cluster_merge_max_splits)
    ops.cluster_merge, ops.cluster_merge_max_splits = cluster, 8       # clusters of every size
    before = ops.launches
    try:
        got = ops.qkv_attention(qkv.to(DEVICE), q_weight=on_gpu(q_weight), k_weight=on_gpu(k_weight),
                                rotary=None if rotary is None else (rotary[0].to(DEVICE), head_dim),
                                ctx=ctx, view=PagedView(kv_gpu, table, page_size, need), **arguments)
    finally:
        ops.cluster_merge, ops.cluster_merge_max_splits = kept
    assert ops.launches - before <= 2                   # one kernel, or one and the merge kernel
    kv_cpu = kv.clone()
    want = plain.qkv_attention(qkv, q_weight=q_weight, k_weight=k_weight, rotary=rotary,
                               ctx=on_cpu(ctx), view=PagedView(kv_cpu, table.cpu(), page_size, need),
                               **arguments)
    ops.check_errors()
    torch.testing.assert_close(got.cpu().float(), want.float(), **tolerance(torch.bfloat16))
    # the cache: only the new rows changed, and they hold the plain preparation's keys and values
    assert not torch.equal(kv_cpu, kv)
    torch.testing.assert_close(kv_gpu.cpu().float(), kv_cpu.float(), atol=2e-2, rtol=2e-2)
    # read-only call: nothing is written, and the token's row in the cache is what is attended to
    kv_gpu2 = kv_cpu.clone().to(DEVICE)
    again = ops.qkv_attention(qkv.to(DEVICE), q_weight=on_gpu(q_weight), k_weight=on_gpu(k_weight),
                              rotary=None if rotary is None else (rotary[0].to(DEVICE), head_dim),
                              ctx=ctx, view=PagedView(kv_gpu2, table, page_size, need),
                              **{**arguments, "write": False})
    assert torch.equal(kv_gpu2.cpu(), kv_cpu)
    torch.testing.assert_close(again.cpu().float(), want.float(), **tolerance(torch.bfloat16))


def test_decode_splits_are_used(ops):
    assert ops.decode_splits(1, 32, 8, 64, 4096, None) > 1
    assert ops.decode_splits(64, 32, 8, 64, 4096, None) == 1
    assert ops.decode_splits(1, 32, 8, 64, 4096, 10) == 1


def test_argmax_and_sampling(ops, plain):
    torch.manual_seed(7)
    vocab, rows = 5000, 6
    logits = torch.randn(rows, vocab) * 3
    logits[2, 17] = logits[2, 900] = logits[2].max() + 1     # a tie: the lower index wins
    assert ops.argmax(logits.to(DEVICE)).cpu().tolist() == torch.argmax(logits, -1).tolist()
    assert ops.argmax(logits.to(DEVICE)).cpu()[2] == 17
    temperature = torch.tensor([0.8, 1.0, 0.5, 1.3, 0.0, 0.9])
    top_k = torch.tensor([0, 50, 5, 0, 0, 1], dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 0.9, 0.7, 1.0, 1.0])
    seed = torch.tensor([0, 1, 2, 3, 4, 5], dtype=torch.int64)
    for step in range(20):
        got = check_draws(ops, logits, temperature, top_k, top_p, seed, step, range(4))
        assert got[4] == int(torch.argmax(logits[4]))           # temperature 0 is greedy
        assert got[5] == int(torch.argmax(logits[5]))           # top_k = 1 too


def check_draws(ops, logits, temperature, top_k, top_p, seed, step, sampled_rows):
    """One call of the sampling kernel; every sampled row's token lies in the kept set that the
    reference's rule gives for the kernel's own probabilities, and is the token that the same
    draw in float64, in token order, gives."""
    rows, vocab = logits.shape
    steps = torch.full((rows,), step, dtype=torch.int32)
    got, probabilities = ops.sample(logits.to(DEVICE), temperature.to(DEVICE),
                                    top_k.to(DEVICE), top_p.to(DEVICE), seed.to(DEVICE),
                                    steps.to(DEVICE))
    got = got.cpu().tolist()
    for r in sampled_rows:
        p = probabilities[r].cpu()
        want_p = torch.exp((logits[r] - logits[r].max()) * (1.0 / temperature[r]))
        assert torch.allclose(p, want_p, rtol=1e-5, atol=1e-30)
        kept = set(kept_set(p, int(top_k[r]), float(top_p[r])).tolist())
        assert got[r] in kept, (r, step)
        weights = torch.zeros(vocab, dtype=torch.float64)
        index = torch.tensor(sorted(kept))
        weights[index] = p[index].double()
        running = torch.cumsum(weights, 0)
        target = uniform(int(seed[r]), step) * float(weights.sum())
        want = int(torch.nonzero((running >= target) & (weights > 0))[0])
        if got[r] != want:        # only a draw within rounding of a boundary may differ
            edge = float(running[min(got[r], want)])
            assert abs(edge - target) < 1e-5 * float(weights.sum()), (r, step, got[r], want)
    return got


@pytest.mark.parametrize("vocab", [301, 70001])
def test_sampling_among_equal_probabilities(ops, vocab):
    """Logits on a coarse grid, so that the k-th largest probability and the top-p boundary are
    shared by many tokens, and a row in which all tokens are equal: ties enter in token order."""
    torch.manual_seed(vocab)
    rows = 8
    logits = torch.round(torch.randn(rows, vocab) * 2) * 0.5
    logits[6] = 1.25                                     # all equal
    logits[7] = -40.0
    logits[7, 5::97] = 3.0                               # a few equal tokens far above the rest
    temperature = torch.tensor([0.7, 1.0, 0.6, 1.2, 0.9, 1.0, 1.0, 0.5])
    top_k = torch.tensor([0, 40, 7, 0, 200, 3, 11, 0], dtype=torch.int32)
    top_p = torch.tensor([1.0, 1.0, 0.9, 0.6, 0.5, 0.95, 0.5, 0.8])
    seed = torch.arange(rows, dtype=torch.int64) + 100
    for step in range(12):
        check_draws(ops, logits, temperature, top_k, top_p, seed, step, range(rows))


@pytest.mark.parametrize("rows", [20, 40, 80])
def test_sampling_of_many_rows(ops, rows):
    """More rows than the eight-block clusters have room for: a row is then shared by four, two
    or one block. Every row has options of its own."""
    torch.manual_seed(rows)
    vocab = 4099
    logits = torch.randn(rows, vocab) * 2.5
    logits[1::5] = torch.round(logits[1::5] * 2) * 0.5            # rows full of ties
    temperature = 0.5 + torch.rand(rows)
    temperature[3::7] = 0.0                                        # greedy rows among them
    top_k = torch.tensor([(0, 1, 13, 200, vocab + 5)[i % 5] for i in range(rows)], dtype=torch.int32)
    top_p = torch.tensor([(1.0, 0.9, 0.35, 0.99)[i % 4] for i in range(rows)])
    seed = torch.arange(rows, dtype=torch.int64) * 7 + 1
    sampled = [r for r in range(rows) if float(temperature[r]) > 0]
    for step in range(3):
        got = check_draws(ops, logits, temperature, top_k, top_p, seed, step, sampled)
        for r in range(rows):
            if float(temperature[r]) <= 0:
                assert got[r] == int(torch.argmax(logits[r]))


def test_sampling_distribution(ops):
    """Over many steps the drawn tokens follow softmax(logits / T)."""
    logits = torch.tensor([[2.0, 1.0, 0.0, -1.0, 1.5]])
    counts = torch.zeros(5)
    rows = 1
    for step in range(3000):
        got, _ = ops.sample(logits.to(DEVICE), torch.tensor([0.7], device=DEVICE),
                            torch.zeros(rows, dtype=torch.int32, device=DEVICE),
                            torch.ones(rows, device=DEVICE),
                            torch.tensor([11], dtype=torch.int64, device=DEVICE),
                            torch.tensor([step], dtype=torch.int32, device=DEVICE))
        counts[int(got[0])] += 1
    want = torch.softmax(logits[0] / 0.7, -1)
    assert (counts / counts.sum() - want).abs().max() < 0.03
