"""Each CUDA kernel alone against a plain PyTorch float32 reference of the same operation,
at sizes other than the engine's."""

from __future__ import annotations

import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def ops():
    from mini_engine_b200.csrc import ops as module

    return module


def rel_error(got: torch.Tensor, want: torch.Tensor) -> float:
    return float((got.double() - want.double()).abs().max() / want.double().abs().max().clamp_min(1e-30))


# ------------------------------------------------------------------------------- GEMMs


@pytest.mark.parametrize("tokens,outs,inner", [(1, 5, 3), (7, 96, 100), (65, 130, 257), (300, 70, 64)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_gemm_simt(tokens, outs, inner, dtype):
    torch.manual_seed(0)
    x = torch.randn(tokens, inner, device="cuda").to(dtype)
    w = torch.randn(outs, inner, device="cuda").to(dtype)
    out = torch.empty(tokens, outs, device="cuda")
    ops().gemm_simt(x, w, out)
    want = x.double() @ w.double().T
    assert rel_error(out, want) < 2e-6 * math.sqrt(inner)


def test_gemm_simt_rows_do_not_depend_on_the_batch():
    torch.manual_seed(1)
    x = torch.randn(200, 333, device="cuda")
    w = torch.randn(77, 333, device="cuda")
    full = torch.empty(200, 77, device="cuda")
    ops().gemm_simt(x, w, full)
    for rows in ([0], [5, 6, 7], list(range(63, 130))):
        part = torch.empty(len(rows), 77, device="cuda")
        ops().gemm_simt(x[rows].contiguous(), w, part)
        assert torch.equal(part, full[rows])


TC_SHAPES = [
    (1, 128, 64),  # one token, one tile, one k block
    (8, 384, 4096),  # decode-like, split over k
    (13, 200, 96),  # ragged outputs and a partial k block
    (64, 1000, 520),  # partial k block, several splits
    (100, 256, 256),
    (300, 520, 1160),  # token tile 256 with a ragged second tile
    (700, 130, 72),
    # CTA pairs with a partly filled last wave: its tiles are cut in two (88 tiles) and in four (82)
    (2048, 2600, 128),
    (512, 10496, 72),
    # a few hundred tokens and a long reduction: each split of it runs on CTA pairs
    (300, 4000, 12352),
    (640, 2100, 6200),
]


@pytest.mark.parametrize("tokens,outs,inner", TC_SHAPES)
def test_gemm_tensor_core(tokens, outs, inner):
    from mini_engine_b200.csrc import tensor_core

    torch.manual_seed(2)
    x = torch.randn(tokens, inner, device="cuda").to(torch.bfloat16)
    w = torch.randn(outs, inner, device="cuda").to(torch.bfloat16)
    plan = tensor_core.GemmPlan(w)
    want = x.double() @ w.double().T
    for splits in sorted({1, tensor_core.choose_splits(tokens, outs, inner)}):
        out = torch.full((splits, tokens, outs), float("nan"), device="cuda")
        tensor_core.gemm(plan, x, out, splits)
        assert tensor_core.take_error() == 0
        # float32 accumulation: the error grows with the square root of the reduction's length
        # (as in test_gemm_simt); 1e-5 is the bound up to 4,096, the engine's usual length.
        assert rel_error(out.sum(0), want) < 1e-5 * max(1.0, math.sqrt(inner / 4096)), f"splits={splits}"


@pytest.mark.parametrize("group", [None, 0, 1, 3, 8])
def test_gemm_tensor_core_tile_groups(group):
    """The persistent pair kernel numbers its tiles group by group (so many token tiles wide, all
    feature tiles tall).  Ten token tiles and nine feature tiles, the last group narrower than the
    others and the tiles of the last round cut in four: every width of group gives the product,
    plain and gated (18 token tiles in groups of 16 by the rule)."""
    from mini_engine_b200.csrc import tensor_core

    torch.manual_seed(11)
    tokens, outs, inner = 2321, 2100, 72
    x = torch.randn(tokens, inner, device="cuda").to(torch.bfloat16)
    w = torch.randn(outs, inner, device="cuda").to(torch.bfloat16)
    out = torch.full((1, tokens, outs), float("nan"), device="cuda")
    tensor_core.gemm(tensor_core.GemmPlan(w), x, out, 1, group)
    assert tensor_core.take_error() == 0
    assert rel_error(out[0], x.double() @ w.double().T) < 1e-5
    tokens, inter = 4400, 1300
    x = torch.randn(tokens, inner, device="cuda").to(torch.bfloat16)
    w = (torch.randn(2 * inter, inner, device="cuda") * 0.2).to(torch.bfloat16)
    act = torch.full((tokens, inter), float("nan"), device="cuda", dtype=torch.bfloat16)
    tensor_core.gemm_swiglu(tensor_core.GemmPlan(w, dual_rows=inter), x, act, None, group)
    assert tensor_core.take_error() == 0
    both = x.double() @ w.double().T
    gate, up = both[:, :inter], both[:, inter:]
    assert rel_error(act, gate * torch.sigmoid(gate) * up) < 6e-3


def test_the_tensor_pipe_alone_runs_at_its_nominal_rate():
    """The measuring kernel of `kernel_bench mma-rate`: a CTA, or a CTA pair, that only issues MMAs
    needs 64 cycles for 128 x 128 x 16 and twice that for N = 256 (8,192 flop a cycle and SM)."""
    from mini_engine_b200.cli.kernel_bench import mma_rate

    assert 60 <= mma_rate(0, 0, 0, 128, ctas=4, iters=500) <= 72
    assert 120 <= mma_rate(1, 0, 0, 256, ctas=4, iters=500) <= 144
    assert 60 <= mma_rate(1, 1, 1, 128, ctas=4, iters=500) <= 72


def test_gemm_tensor_core_finds_one_large_product():
    """A single large x[t][k] * w[n][k] among small terms must land in exactly out[t][n]:
    a wrong swizzle, k step or lane mapping would put it elsewhere or drop it."""
    from mini_engine_b200.csrc import tensor_core

    tokens, outs, inner = 40, 300, 200
    for t, n, k in [(0, 0, 0), (39, 299, 199), (17, 131, 77), (5, 128, 64), (33, 127, 63)]:
        x = torch.full((tokens, inner), 0.001, device="cuda").to(torch.bfloat16)
        w = torch.full((outs, inner), 0.001, device="cuda").to(torch.bfloat16)
        x[t, k], w[n, k] = 64.0, 32.0
        out = torch.empty(1, tokens, outs, device="cuda")
        tensor_core.gemm(tensor_core.GemmPlan(w), x, out, 1)
        want = x.double() @ w.double().T
        assert rel_error(out[0], want) < 1e-5
        assert int(out[0].argmax()) == t * outs + n


@pytest.mark.parametrize(
    "tokens,inter,inner",
    [
        (1, 64, 64), (8, 200, 136), (17, 160, 520), (33, 100, 72), (64, 448, 264),  # gate rows stacked on up rows
        (65, 160, 96), (128, 128, 64), (300, 300, 264), (2048, 2600, 136),
    ],
)  # fmt: skip
def test_gemm_tensor_core_swiglu(tokens, inter, inner):
    from mini_engine_b200.csrc import tensor_core

    torch.manual_seed(3)
    x = torch.randn(tokens, inner, device="cuda").to(torch.bfloat16)
    w = (torch.randn(2 * inter, inner, device="cuda") * 0.2).to(torch.bfloat16)
    act = torch.empty(tokens, inter, device="cuda", dtype=torch.bfloat16)
    tensor_core.gemm_swiglu(tensor_core.GemmPlan(w, dual_rows=inter), x, act)
    assert tensor_core.take_error() == 0
    both = x.double() @ w.double().T
    gate, up = both[:, :inter], both[:, inter:]
    want = gate * torch.sigmoid(gate) * up
    assert rel_error(act, want) < 6e-3  # one rounding to bfloat16


@pytest.mark.parametrize(
    "tokens,inter,inner",
    [(1, 64, 128), (8, 200, 136), (16, 130, 200), (5, 12288, 4096), (3, 72, 64), (9, 64, 1096), (16, 100, 72), (12, 3072, 1024)],
)  # fmt: skip
def test_gemm_tensor_core_swiglu_with_the_reduction_in_two_ctas(tokens, inter, inner):
    """Up to 16 tokens the reduction of the stacked gated product may be cut in two halves that
    the two CTAs of a cluster compute, the second adding its sums into the first one's shared
    memory: both forms against float64, over an odd number of k blocks, a last k block that is
    partly empty and a single k block (the second CTA then has nothing to add).  A value that
    stands out in the second half of the reduction must arrive."""
    from mini_engine_b200.csrc import tensor_core

    torch.manual_seed(5)
    x = torch.randn(tokens, inner, device="cuda").to(torch.bfloat16)
    w = (torch.randn(2 * inter, inner, device="cuda") * 0.2).to(torch.bfloat16)
    x[tokens - 1, inner - 1], w[inter - 1, inner - 1], w[2 * inter - 1, inner - 1] = 16.0, 8.0, 8.0
    both = x.double() @ w.double().T
    gate, up = both[:, :inter], both[:, inter:]
    want = gate * torch.sigmoid(gate) * up
    plan = tensor_core.GemmPlan(w, dual_rows=inter)
    for halves in (2, 1, None):
        act = torch.full((tokens, inter), float("nan"), device="cuda", dtype=torch.bfloat16)
        tensor_core.gemm_swiglu(plan, x, act, halves)
        assert tensor_core.take_error() == 0
        assert rel_error(act, want) < 6e-3, halves
        assert int(act.float().abs().argmax()) == (tokens - 1) * inter + inter - 1


# -------------------------------------------------------------------------- elementwise


@pytest.mark.parametrize("hidden", [24, 100, 4096])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_add_rmsnorm(hidden, out_dtype):
    torch.manual_seed(4)
    tokens, eps = 9, 3e-5
    x = torch.randn(tokens, hidden, device="cuda")
    pending = torch.randn(3, tokens, hidden, device="cuda")
    weight = 1 + 0.1 * torch.randn(hidden, device="cuda")
    summed = x.double() + pending.double().sum(0)
    want = weight.double() * summed * torch.rsqrt(summed.pow(2).mean(-1, keepdim=True) + eps)
    out = torch.empty(tokens, hidden, device="cuda", dtype=out_dtype)
    x_run = x.clone()
    ops().add_rmsnorm(x_run, pending, weight, eps, out)
    assert rel_error(x_run, summed) < 1e-6
    assert rel_error(out, want) < (1e-5 if out_dtype == torch.float32 else 5e-3)
    rows = torch.tensor([7, 0, 7], device="cuda", dtype=torch.int32)
    picked = torch.empty(3, hidden, device="cuda", dtype=out_dtype)
    x_keep = x.clone()
    ops().add_rmsnorm(x_keep, pending, weight, eps, picked, rows)
    assert torch.equal(x_keep, x)
    assert rel_error(picked, want[rows.long()]) < (1e-5 if out_dtype == torch.float32 else 5e-3)
    plain = torch.empty(tokens, hidden, device="cuda", dtype=out_dtype)
    ops().add_rmsnorm(x.clone(), None, weight, eps, plain)
    want_plain = weight.double() * x.double() * torch.rsqrt(x.double().pow(2).mean(-1, keepdim=True) + eps)
    assert rel_error(plain, want_plain) < (1e-5 if out_dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("hidden", [136, 1536, 4096, 5120, 2050])
def test_add_rmsnorm_same_bits_for_few_and_many_rows(hidden):
    """Many rows run with fewer threads per row than few rows do; a row's result must not tell."""
    torch.manual_seed(5)
    tokens = 300
    x = torch.randn(tokens, hidden, device="cuda")
    pending = torch.randn(2, tokens, hidden, device="cuda")
    weight = 1 + 0.1 * torch.randn(hidden, device="cuda")
    many = torch.empty(tokens, hidden, device="cuda")
    ops().add_rmsnorm(x.clone(), pending, weight, 1e-6, many)
    few = torch.empty(7, hidden, device="cuda")
    ops().add_rmsnorm(x[:7].clone(), pending[:, :7].contiguous(), weight, 1e-6, few)
    assert torch.equal(few, many[:7])
    rows = torch.tensor([299, 5], device="cuda", dtype=torch.int32)
    picked = torch.empty(2, hidden, device="cuda")
    ops().add_rmsnorm(x.clone(), pending, weight, 1e-6, picked, rows)
    assert torch.equal(picked, many[rows.long()])


def test_embedding():
    table = torch.randn(50, 24, device="cuda").to(torch.bfloat16)
    ids = torch.tensor([3, 49, 0, 3], device="cuda", dtype=torch.int32)
    out = torch.empty(4, 24, device="cuda")
    ops().embedding(table, ids, out)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_swiglu(out_dtype):
    torch.manual_seed(5)
    partials = torch.randn(2, 5, 2 * 37, device="cuda")
    both = partials.double().sum(0)
    gate, up = both[:, :37], both[:, 37:]
    out = torch.empty(5, 37, device="cuda", dtype=out_dtype)
    ops().swiglu(partials, out)
    assert rel_error(out, gate * torch.sigmoid(gate) * up) < (1e-6 if out_dtype == torch.float32 else 5e-3)


def rope_reference(x, positions, theta):
    d = x.shape[-1]
    inv_freq = 1.0 / (theta ** (torch.arange(0, d, 2, dtype=torch.float32) / d))
    angles = positions.float()[:, None] * inv_freq[None, :]
    angles = torch.cat((angles, angles), -1).double()
    half = d // 2
    rotated = torch.cat((-x[..., half:], x[..., :half]), -1)
    return x * angles.cos()[:, None, :] + rotated * angles.sin()[:, None, :]


@pytest.mark.parametrize("heads,kv_heads,head_dim,page", [(3, 1, 16, 4), (6, 3, 48, 8), (4, 2, 128, 16)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_qk_norm_rope_store(heads, kv_heads, head_dim, page, dtype):
    torch.manual_seed(6)
    tokens, pages, eps, theta = 11, 9, 2e-5, 5000.0
    width = (heads + 2 * kv_heads) * head_dim
    qkv = torch.randn(2, tokens, width, device="cuda")
    qw = 1 + 0.1 * torch.randn(head_dim, device="cuda")
    kw = 1 + 0.1 * torch.randn(head_dim, device="cuda")
    positions = torch.randint(0, 3000, (tokens,), dtype=torch.int32)
    slots = torch.randperm(pages * page)[:tokens].to(torch.int32)
    slots[4] = -1  # not stored
    inv_freq = (1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))).cuda()
    cos_sin = torch.empty(tokens, head_dim // 2, 2, device="cuda")
    ops().rope_table(inv_freq, positions.cuda(), cos_sin)
    angles = positions.float()[:, None] * inv_freq.cpu()[None, :]
    assert torch.allclose(cos_sin[..., 0].cpu(), angles.cos(), atol=2e-6) and torch.allclose(cos_sin[..., 1].cpu(), angles.sin(), atol=2e-6)
    q_out = torch.empty(tokens, heads * head_dim, device="cuda", dtype=dtype)
    k_pages = torch.zeros(pages, kv_heads, page, head_dim, device="cuda", dtype=dtype)
    v_pages = torch.zeros_like(k_pages)
    ops().qk_norm_rope_store(
        qkv=qkv, heads=heads, kv_heads=kv_heads, head_dim=head_dim, q_weight=qw, k_weight=kw, eps=eps,
        cos_sin=cos_sin, positions=positions.cuda(), q_out=q_out, page_size=page, slot_mapping=slots.cuda(),
        k_pages=k_pages, v_pages=v_pages,
    )  # fmt: skip
    total = qkv.double().sum(0).cpu()
    q, k, v = total.split([heads * head_dim, kv_heads * head_dim, kv_heads * head_dim], dim=-1)

    def normed(t, w, n):
        t = t.view(tokens, n, head_dim)
        return w.double().cpu() * t * torch.rsqrt(t.pow(2).mean(-1, keepdim=True) + eps)

    q_want = rope_reference(normed(q, qw, heads), positions, theta)
    k_want = rope_reference(normed(k, kw, kv_heads), positions, theta)
    tol = 2e-5 if dtype == torch.float32 else 6e-3
    assert rel_error(q_out.cpu().view(tokens, heads, head_dim), q_want) < tol
    for t in range(tokens):
        s = int(slots[t])
        if s < 0:
            continue
        assert rel_error(k_pages[s // page, :, s % page].cpu(), k_want[t]) < tol
        assert rel_error(v_pages[s // page, :, s % page].cpu(), v.view(tokens, kv_heads, head_dim)[t]) < tol
    written = {int(s) for s in slots if s >= 0}
    for s in range(pages * page):
        if s not in written:
            assert float(k_pages[s // page, :, s % page].abs().max()) == 0.0


# ---------------------------------------------------------------------------- attention


def attention_reference(q, k, v, scale, window=None):
    """q [T, heads, d], k/v [T, kv, d] (float64) of one whole sequence -> [T, heads, d]."""
    t, heads, d = q.shape
    group = heads // k.shape[1]
    pos = torch.arange(t)
    allowed = pos[None, :] <= pos[:, None]
    if window:
        allowed &= pos[None, :] > pos[:, None] - window
    out = torch.empty_like(q)
    for h in range(heads):
        s = (q[:, h] @ k[:, h // group].T) * scale
        s = s.masked_fill(~allowed, float("-inf"))
        out[:, h] = torch.softmax(s, -1) @ v[:, h // group]
    return out


def paged_case(lengths, new_counts, heads, kv_heads, head_dim, page, dtype, seed, spike=None, stale=None, ramp=None,
               window=None):
    """Sequences of the given lengths in scattered pages; the last ``new_counts[i]`` tokens of
    each are the batch's queries.  Returns kernel inputs and the expected output rows.  Slots that
    no sequence owns hold random numbers, or ``stale`` when given.  With ``ramp`` the scores of
    every query grow steadily with the key's position (by ``ramp`` per key before the softmax
    scale), so that a running maximum keeps growing from tile to tile."""
    g = torch.Generator().manual_seed(seed)
    total_pages = sum(-(-n // page) for n in lengths) + 3
    order = torch.randperm(total_pages, generator=g).tolist()
    width = max(-(-n // page) for n in lengths) + 1
    k_pages = torch.randn(total_pages, kv_heads, page, head_dim, generator=g).to(dtype)  # stale data everywhere
    v_pages = torch.randn(total_pages, kv_heads, page, head_dim, generator=g).to(dtype)
    if stale is not None:
        k_pages.fill_(stale)
        v_pages.fill_(stale)
    table = torch.full((len(lengths), width), -1, dtype=torch.int32)
    q_rows, want_rows, entry_of, positions = [], [], [], []
    for b, (n, new) in enumerate(zip(lengths, new_counts)):
        q = torch.randn(n, heads, head_dim, generator=g).to(dtype)
        k = torch.randn(n, kv_heads, head_dim, generator=g).to(dtype)
        v = torch.randn(n, kv_heads, head_dim, generator=g).to(dtype)
        if ramp is not None:
            k[:, :, 0] += ramp * torch.arange(n, dtype=torch.float32)[:, None] / 4.0
            q[:, :, 0] = 4.0
        if spike is not None and n > spike[1]:
            # one far key answers one late query loudly: it must be found among hundreds
            query_pos, key_pos = n - 1, spike[1]
            k[key_pos] = 0
            q[query_pos] = 0
            k[key_pos, :, 0] = 30.0
            q[query_pos, :, 0] = 30.0
            v[key_pos] = 5.0
        for i in range(-(-n // page)):
            table[b, i] = order.pop()
        for p in range(n):
            k_pages[table[b, p // page], :, p % page] = k[p]
            v_pages[table[b, p // page], :, p % page] = v[p]
        want = attention_reference(q.double(), k.double(), v.double(), head_dim**-0.5, window)
        q_rows.append(q[n - new :])
        want_rows.append(want[n - new :])
        entry_of += [b] * new
        positions += list(range(n - new, n))
    return dict(
        q=torch.cat(q_rows).reshape(-1, heads * head_dim).contiguous().cuda(),
        k_pages=k_pages.cuda(), v_pages=v_pages.cuda(), table=table.cuda(),
        entry_of=torch.tensor(entry_of, dtype=torch.int32).cuda(),
        positions=torch.tensor(positions, dtype=torch.int32).cuda(),
        want=torch.cat(want_rows).reshape(-1, heads * head_dim),
        lengths=lengths, new_counts=new_counts,
    )  # fmt: skip


ATTENTION_CASES = [
    # lengths, new tokens of each, heads, kv heads, head_dim, page
    ([1, 16, 17, 33, 100, 255], [1, 1, 1, 1, 1, 1], 4, 2, 16, 16),  # decode at the reference's lengths
    ([7, 9, 13], [7, 1, 5], 4, 2, 32, 4),  # fresh prompt, decode, continuation
    ([300, 64, 2], [300, 33, 2], 6, 1, 48, 8),
    ([513, 40], [2, 40], 8, 8, 80, 16),
]


@pytest.mark.parametrize("case", ATTENTION_CASES)
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_paged_attention_generic(case, dtype):
    lengths, news, heads, kv_heads, head_dim, page = case
    data = paged_case(lengths, news, heads, kv_heads, head_dim, page, dtype, seed=7, spike=(0, 3))
    out = torch.empty_like(data["q"])
    ops().paged_attention_generic(
        data["q"], data["k_pages"], data["v_pages"], data["table"], data["entry_of"], data["positions"], out,
        heads, kv_heads, head_dim, head_dim**-0.5, 0,
    )  # fmt: skip
    assert rel_error(out.cpu(), data["want"]) < (2e-5 if dtype == torch.float32 else 1e-2)


def test_paged_attention_generic_window():
    heads, kv_heads, head_dim, page, window = 4, 2, 16, 4, 10
    data = paged_case([50, 9], [50, 3], heads, kv_heads, head_dim, page, torch.float32, seed=8, window=window)
    out = torch.empty_like(data["q"])
    ops().paged_attention_generic(
        data["q"], data["k_pages"], data["v_pages"], data["table"], data["entry_of"], data["positions"], out,
        heads, kv_heads, head_dim, head_dim**-0.5, window,
    )  # fmt: skip
    assert rel_error(out.cpu(), data["want"]) < 2e-5


BF16_ATTENTION_CASES = [
    # lengths, new tokens of each, heads, kv heads, head_dim, page
    ([1, 16, 17, 33, 100, 255, 256, 257, 600], [1] * 9, 8, 2, 128, 16),  # decode, group 4
    ([64, 65, 300], [1, 1, 1], 4, 4, 64, 4),  # decode, group 1, small pages
    ([700, 3], [1, 1], 16, 1, 64, 16),  # decode, group 16
    ([1, 8, 9, 16, 17, 127, 128, 129, 640], [1] * 9, 8, 1, 128, 8),  # decode, group 8, two pages per 16 keys
    ([5, 250, 1031], [1] * 3, 6, 2, 64, 32),  # decode, group 3, 16 keys are half a page
    ([2000, 77], [1, 1], 4, 1, 128, 128),  # decode, pages as large as a tile
    ([7, 9, 13], [7, 1, 5], 4, 2, 64, 4),  # fresh prompt, decode, continuation
    ([300, 64, 2, 129], [300, 33, 2, 65], 6, 2, 128, 8),
    ([513, 40], [2, 40], 8, 8, 64, 16),
    ([1000], [1000], 2, 1, 128, 16),
    # many (request, KV head) pairs: a decode CTA walks two, then four tiles of 128 keys
    ([1 + (37 * i) % 700 for i in range(40)], [1] * 40, 8, 4, 64, 16),
    ([1 + (53 * i) % 900 for i in range(70)], [1] * 70, 8, 4, 128, 16),
    # 480 (request, KV head) pairs: more than three CTAs of eight warps per SM hold, so six warps by the rule
    ([1 + (29 * i) % 500 for i in range(60)], [1] * 60, 16, 8, 128, 16),
]


@pytest.fixture(params=[None, 6, 8], ids=["by-rule", "six-warps", "eight-warps"])
def decode_warps(request):
    """Warps of a CTA of the TMA decode kernel: by the engine's rule, six (tiles of 96 keys) or eight."""
    return request.param


def fake_context(data):
    """What the attention binding reads of a step context."""
    from types import SimpleNamespace

    from mini_engine_b200.engine.workspace import Workspace

    news, lengths = data["new_counts"], data["lengths"]
    cu = [0]
    for n in news:
        cu.append(cu[-1] + n)
    ones = [b for b, n in enumerate(news) if n == 1]
    more = [b for b, n in enumerate(news) if n > 1]
    return SimpleNamespace(
        num_decode_entries=len(ones), decode_entries=torch.tensor(ones, dtype=torch.int32, device="cuda"),
        portion_entries=torch.tensor(more, dtype=torch.int32, device="cuda"),
        num_entries=len(news), all_decode=max(news) == 1, max_query_len=max(news), max_context_len=max(lengths),
        cu_tokens=torch.tensor(cu, dtype=torch.int32, device="cuda"),
        context_lens=torch.tensor(lengths, dtype=torch.int32, device="cuda"),
        entry_of_token=data["entry_of"], positions=data["positions"], workspace=Workspace(64),
    )  # fmt: skip


@pytest.mark.parametrize("case", BF16_ATTENTION_CASES)
def test_paged_attention_bf16_tensor_core(case, decode_warps):
    from mini_engine_b200.csrc import attention_bf16

    lengths, news, heads, kv_heads, head_dim, page = case
    assert attention_bf16.supports(head_dim, heads, kv_heads)
    data = paged_case(lengths, news, heads, kv_heads, head_dim, page, torch.bfloat16, seed=11, spike=(0, 3))
    out = torch.full_like(data["q"], float("nan"))
    attention_bf16.paged_attention(
        data["q"], data["k_pages"], data["v_pages"], data["table"], fake_context(data), out, heads, kv_heads,
        head_dim, head_dim**-0.5, 0,
    )  # fmt: skip
    assert rel_error(out.cpu(), data["want"]) < 1e-2
    assert attention_bf16.take_error() == 0


@pytest.mark.parametrize("page", [8, 16, 64])
def test_decode_ignores_what_reused_pages_still_hold(page, decode_warps):
    """Slots behind a request's last token (and pages it does not own) hold infinities: none of it
    may reach the output, not even multiplied by a probability of zero."""
    from mini_engine_b200.csrc import attention_bf16

    lengths, heads, kv_heads, head_dim = [1, 7, 19, 130, 257], 8, 2, 128
    news = [1] * len(lengths)
    data = paged_case(lengths, news, heads, kv_heads, head_dim, page, torch.bfloat16, seed=14, stale=float("inf"))
    out = torch.full_like(data["q"], float("nan"))
    attention_bf16.paged_attention(
        data["q"], data["k_pages"], data["v_pages"], data["table"], fake_context(data), out, heads, kv_heads,
        head_dim, head_dim**-0.5, 0,
    )  # fmt: skip
    assert attention_bf16.take_error() == 0
    assert torch.isfinite(out).all()
    assert rel_error(out.cpu(), data["want"]) < 1e-2


TENSOR_MEMORY_CASES = [
    # lengths, new tokens of each, heads, kv heads, page: head_dim 128, portions of 32 tokens and more
    ([128], [128], 2, 1, 16),  # exactly one block and one tile
    ([129, 40], [129, 33], 4, 2, 16),  # a second block of one row; a continuation
    ([700, 64, 300], [700, 64, 45], 8, 2, 8),  # several tiles, small pages, a portion far into its request
    ([1000, 3, 257], [256, 3, 257], 4, 4, 32),  # the last 256 tokens of 1000; a tiny entry in the same launch
    ([500, 90, 300, 64, 17], [1, 90, 1, 64, 1], 8, 2, 16),  # decoded tokens of some beside portions of others
    ([2048], [2048], 2, 1, 128),  # pages as large as a tile
    # groups of an odd number of query heads (and of one) take the kernel with one head per CTA,
    # even groups the one that carries two heads of a KV group per CTA
    ([300, 129], [300, 64], 6, 2, 16),
    ([640], [640], 3, 3, 64),
    ([1500, 200], [1500, 130], 8, 1, 16),  # a group of eight: four CTAs share each block's keys
]


@pytest.mark.parametrize("case", TENSOR_MEMORY_CASES)
def test_paged_attention_tcgen05(case):
    from mini_engine_b200.csrc import attention_bf16

    lengths, news, heads, kv_heads, page = case
    head_dim = 128
    assert attention_bf16.tensor_memory_kernel_takes(head_dim, page, 0, max(news))
    data = paged_case(lengths, news, heads, kv_heads, head_dim, page, torch.bfloat16, seed=13, spike=(0, 3))
    out = torch.full_like(data["q"], float("nan"))
    attention_bf16.paged_attention(
        data["q"], data["k_pages"], data["v_pages"], data["table"], fake_context(data), out, heads, kv_heads,
        head_dim, head_dim**-0.5, 0,
    )  # fmt: skip
    assert attention_bf16.take_error() == 0
    assert rel_error(out.cpu(), data["want"]) < 1e-2


@pytest.mark.parametrize("ramp", [0.04, 0.3, 2.0])
def test_paged_attention_tcgen05_growing_maximum(ramp):
    """The kernel rescales its output lazily, when a row's maximum has outgrown the value its
    probabilities are taken relative to: scores that grow slowly, quickly and very quickly."""
    from mini_engine_b200.csrc import attention_bf16

    lengths, news, heads, kv_heads, head_dim, page = [1500, 300], [1400, 300], 4, 2, 128, 16
    data = paged_case(lengths, news, heads, kv_heads, head_dim, page, torch.bfloat16, seed=15, ramp=ramp)
    out = torch.full_like(data["q"], float("nan"))
    attention_bf16.paged_attention(
        data["q"], data["k_pages"], data["v_pages"], data["table"], fake_context(data), out, heads, kv_heads,
        head_dim, head_dim**-0.5, 0,
    )  # fmt: skip
    assert attention_bf16.take_error() == 0
    assert torch.isfinite(out).all()
    assert rel_error(out.cpu(), data["want"]) < 1e-2


@pytest.mark.parametrize("news", [[1, 1], [90, 5]])
def test_paged_attention_bf16_window(news, decode_warps):
    """A window of 70 keys over contexts of 400 and 90, against attention in float64 with the
    same window (a window edge inside a tile, a tile wholly behind the window)."""
    from mini_engine_b200.csrc import attention_bf16

    heads, kv_heads, head_dim, page, window = 4, 2, 64, 8, 70
    lengths = [400, 90]
    data = paged_case(lengths, news, heads, kv_heads, head_dim, page, torch.bfloat16, seed=12, window=window)
    out = torch.full_like(data["q"], float("nan"))
    attention_bf16.paged_attention(
        data["q"], data["k_pages"], data["v_pages"], data["table"], fake_context(data), out, heads, kv_heads,
        head_dim, head_dim**-0.5, window,
    )  # fmt: skip
    assert torch.isfinite(out).all()
    assert rel_error(out.cpu(), data["want"]) < 1e-2
    assert attention_bf16.take_error() == 0


def test_a_wait_that_runs_out_is_reported_and_leaves_the_device_usable():
    """Every barrier wait of the tensor-core kernels has a limit, after which the kernel records
    an error word, gives its tensor memory back and returns.  The probe is a CTA with the product
    kernels' warp roles whose copies are never issued, so its waits run out after a few thousand
    polls: the error must reach the host, `raise_on_device_error` must raise exactly once, and
    the next ordinary product must be right (tensor memory was freed, the context is intact)."""
    from mini_engine_b200.csrc import ops as kernel_ops
    from mini_engine_b200.csrc import tensor_core

    kernel_ops.raise_on_device_error()  # nothing pending from earlier tests
    assert tensor_core.wait_probe(polls=4096)  # it returned, past its dealloc
    torch.cuda.synchronize()
    with pytest.raises(kernel_ops.KernelError, match="limit of a wait"):
        kernel_ops.raise_on_device_error()
    kernel_ops.raise_on_device_error()  # taken: the word is clear again
    # the code says which wait gave up first: the MMA warp's (40) or the epilogue's (41)
    assert tensor_core.wait_probe(polls=2048)
    assert tensor_core.take_error() >> 8 in (40, 41)
    # many probes in a row leave tensor memory free: 512 columns per SM would be gone after 16 leaks
    for _ in range(40):
        assert tensor_core.wait_probe(polls=64)
    assert tensor_core.take_error() != 0
    torch.manual_seed(5)
    x = torch.randn(40, 256, device="cuda").to(torch.bfloat16)
    w = torch.randn(300, 256, device="cuda").to(torch.bfloat16)
    out = torch.full((1, 40, 300), float("nan"), device="cuda")
    tensor_core.gemm(tensor_core.GemmPlan(w), x, out, 1)
    assert rel_error(out[0], x.double() @ w.double().T) < 1e-5
    assert tensor_core.take_error() == 0


# ----------------------------------------------------------------------------- sampling


def test_sample_greedy_and_temperature():
    torch.manual_seed(9)
    rows, vocab = 6, 5003
    logits = torch.randn(rows, vocab, device="cuda") * 3
    logits[1, 77] = logits[1, 4000] = 50.0  # equal maxima: the lowest index wins
    out = torch.empty(rows, dtype=torch.int32, device="cuda")
    ops().sample(logits, None, None, out)
    want = logits.argmax(-1)
    want[1] = 77
    assert out.tolist() == want.tolist()
    temps = torch.tensor([0.0, 0.0, 0.8, 1.0, 1.5, 0.3], device="cuda")
    uniforms = torch.tensor([0.5, 0.5, 0.0, 0.37, 0.93, 0.999999], device="cuda")
    ops().sample(logits, temps, uniforms, out)
    got = out.tolist()
    assert got[:2] == want.tolist()[:2]
    for r in range(2, rows):
        probs = torch.softmax(logits[r].double() / float(temps[r]), -1).cpu()
        cdf = torch.cumsum(probs, -1)
        target = float(uniforms[r])
        below = float(cdf[got[r] - 1]) if got[r] > 0 else 0.0
        assert below - 1e-4 <= target <= float(cdf[got[r]]) + 1e-4, f"row {r}: token {got[r]} does not hold u={target}"


@pytest.mark.parametrize("vocab", [5, 33, 1000, 40961])
def test_sample_never_draws_a_token_without_probability(vocab):
    """A few tokens hold all the probability; the rest lie so far below that their exponentials
    are zero.  Whatever the uniform number (0, the edges between the few, almost 1), the draw is
    one of the few, and the one that the cumulative sums name."""
    few = sorted({1, vocab // 3, vocab // 2 + 1, vocab - 2})
    uniforms = [0.0, 0.1, 0.2499, 0.2501, 0.5, 0.7499, 0.7501, 0.9, 0.99999994]
    logits = torch.full((len(uniforms), vocab), -1e4, device="cuda")
    logits[:, few] = 3.0
    out = torch.empty(len(uniforms), dtype=torch.int32, device="cuda")
    ops().sample(logits, torch.full((len(uniforms),), 0.9, device="cuda"), torch.tensor(uniforms, device="cuda"), out)
    share = 1.0 / len(few)
    for u, token in zip(uniforms, out.tolist()):
        assert token in few, f"u={u}: token {token} has probability zero"
        k = few.index(token)
        assert k * share - 1e-3 <= u <= (k + 1) * share + 1e-3, f"u={u}: token {token} is number {k} of {len(few)}"


def test_sample_distribution():
    vocab, draws = 7, 4000
    logits = torch.tensor([[2.0, 0.0, 1.0, -1.0, 0.5, 0.0, -3.0]], device="cuda").repeat(draws, 1)
    temps = torch.full((draws,), 0.7, device="cuda")
    uniforms = torch.rand(draws, device="cuda", generator=torch.Generator("cuda").manual_seed(0))
    out = torch.empty(draws, dtype=torch.int32, device="cuda")
    ops().sample(logits, temps, uniforms, out)
    freq = torch.bincount(out.long().cpu(), minlength=vocab).double() / draws
    want = torch.softmax(logits[0].double().cpu() / 0.7, -1)
    assert float((freq - want).abs().max()) < 0.03
