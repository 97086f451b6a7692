"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory when they need attention (a plug-in in
a process that owns all memory, a loop that must not risk the synchronisation an allocation
can cause), so `me_attention_decode_bf16_noalloc` keeps its scratch in a fixed array inside the
library.  Here it must give what plain attention over the same pages gives (a float64
restatement below, so that wrong arithmetic in the split kernel or in its merge would show) and
what the ordinary entry point gives with caller-supplied scratch, on two calls in a row (the
second finds the first call's leftovers in the shared scratch); it must take the largest request
that fits its limit, refuse one beyond it, and report a context that its splits do not cover.
The file sorts last so that a run that stops at the first failure has run everything else before.
"""

from __future__ import annotations

from ctypes import byref, c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

TOO_LARGE = 1003
MAX_FLOATS = 2 * 1024 * 1024
TOLERANCE = 1e-2  # as for the other bfloat16 attention kernels: of the largest output value


def library():
    from mini_engine_b200.csrc.build import load_library

    lib = load_library("attention_bf16")
    lib.me_attention_decode_bf16_noalloc.argtypes = [c_void_p] * 7 + [c_float] + [c_int] * 8 + [c_void_p]
    lib.me_attention_decode_bf16_noalloc.restype = c_int
    lib.me_attention_decode_bf16.argtypes = [c_void_p] * 8 + [c_float] + [c_int] * 8 + [c_void_p]
    lib.me_attention_decode_bf16.restype = c_int
    lib.me_attention_bf16_take_error.restype = c_int
    return lib


def take_error(lib) -> int:
    code = c_int(0)
    assert lib.me_attention_bf16_take_error(byref(code)) == 0
    return code.value


def make_case(seed, lengths, heads, kv_heads, head_dim, page):
    g = torch.Generator().manual_seed(seed)
    pages = sum(-(-n // page) for n in lengths) + 2
    width = max(-(-n // page) for n in lengths)
    order = torch.randperm(pages, generator=g).tolist()
    table = torch.full((len(lengths), width), -1, dtype=torch.int32)
    for b, n in enumerate(lengths):
        for i in range(-(-n // page)):
            table[b, i] = order.pop()
    host = dict(
        q=torch.randn(len(lengths), heads * head_dim, generator=g).to(torch.bfloat16),
        k=torch.randn(pages, kv_heads, page, head_dim, generator=g).to(torch.bfloat16),
        v=torch.randn(pages, kv_heads, page, head_dim, generator=g).to(torch.bfloat16),
        table=table,
        cu=torch.arange(len(lengths) + 1, dtype=torch.int32),
        lens=torch.tensor(lengths, dtype=torch.int32),
    )
    case = {name: tensor.cuda() for name, tensor in host.items()}
    case["host"] = host
    return case


def plain_attention(case, heads, kv_heads, head_dim, page, window=0, visible=None):
    """One query per request at its last position over the request's pages, in float64:
    softmax(q . k / sqrt(d)) v over the keys the query can see (all earlier ones, the last
    `window` of them when a window is set, or only the first `visible` keys)."""
    host = case["host"]
    group = heads // kv_heads
    out = torch.zeros(len(host["lens"]), heads, head_dim, dtype=torch.float64)
    for b, n in enumerate(host["lens"].tolist()):
        pages = host["table"][b, : -(-n // page)].long()
        keys = host["k"][pages].double().permute(1, 0, 2, 3).reshape(kv_heads, -1, head_dim)[:, :n]
        values = host["v"][pages].double().permute(1, 0, 2, 3).reshape(kv_heads, -1, head_dim)[:, :n]
        first = max(n - window, 0) if window else 0
        last = min(n, visible) if visible else n
        q = host["q"][b].double().view(heads, head_dim)
        for h in range(heads):
            k, v = keys[h // group, first:last], values[h // group, first:last]
            out[b, h] = torch.softmax((k @ q[h]) * head_dim**-0.5, 0) @ v
    return out.view(len(host["lens"]), heads * head_dim)


def call_both(lib, case, heads, kv_heads, head_dim, page, splits, window=0):
    entries = case["q"].shape[0]
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    common = [case[k].data_ptr() for k in ("q", "k", "v", "table", "cu", "lens")]
    tail = [head_dim**-0.5, entries, splits, heads, kv_heads, head_dim, page, case["table"].shape[1], window, stream]
    ours = torch.full_like(case["q"], float("nan"))
    theirs = torch.full_like(case["q"], float("nan"))
    scratch = torch.empty(entries * heads * splits * (head_dim + 2), dtype=torch.float32, device="cuda")
    assert lib.me_attention_decode_bf16(*common, theirs.data_ptr(), scratch.data_ptr(), *tail) == 0
    assert lib.me_attention_decode_bf16_noalloc(*common, ours.data_ptr(), *tail) == 0
    torch.cuda.synchronize()
    return ours, theirs


def assert_close(got, want):
    assert torch.isfinite(got.float()).all()
    error = float((got.double().cpu() - want).abs().max()) / float(want.abs().max())
    assert error <= TOLERANCE, f"relative error {error:.3g}"


def test_no_alloc_entry_matches_plain_attention_twice_in_a_row():
    lib = library()
    take_error(lib)
    first = make_case(1, [600, 33, 256, 1], heads=8, kv_heads=2, head_dim=128, page=16)
    ours, theirs = call_both(lib, first, 8, 2, 128, 16, splits=5)  # ceil(600 / 128)
    assert_close(ours, plain_attention(first, 8, 2, 128, 16))
    assert torch.equal(ours, theirs)  # the same kernels, only the scratch lies elsewhere
    # a second call of another shape, right behind the first, on the same scratch
    second = make_case(2, [90, 300], heads=4, kv_heads=4, head_dim=64, page=8)
    ours2, theirs2 = call_both(lib, second, 4, 4, 64, 8, splits=3)
    assert_close(ours2, plain_attention(second, 4, 4, 64, 8))
    assert torch.equal(ours2, theirs2)
    # and the first again: the same bits as before (the kernels are deterministic)
    ours3, _ = call_both(lib, first, 8, 2, 128, 16, splits=5)
    assert torch.equal(ours3, ours)
    assert take_error(lib) == 0


def test_no_alloc_entry_with_a_window():
    """Only the last 200 keys count: the first splits of the long requests have nothing to do and
    the merge starts at the first split that the window reaches."""
    lib = library()
    case = make_case(4, [700, 150, 400], heads=8, kv_heads=4, head_dim=128, page=16)
    ours, theirs = call_both(lib, case, 8, 4, 128, 16, splits=6, window=200)
    assert_close(ours, plain_attention(case, 8, 4, 128, 16, window=200))
    assert torch.equal(ours, theirs)
    assert take_error(lib) == 0


def test_no_alloc_entry_takes_the_most_that_fits_and_refuses_more():
    """The scratch holds 2^21 floats and a request needs entries x heads x splits x (head_dim + 2);
    head_dim + 2 is 66 or 130, which have odd factors, so no request needs exactly 2^21: the
    largest that fits must run and one split more must be refused without a launch."""
    lib = library()
    take_error(lib)
    case = make_case(5, [70] * 32, heads=16, kv_heads=4, head_dim=64, page=16)
    most = MAX_FLOATS // (32 * 16 * 66)  # 62 splits: 2,095,104 floats
    assert 32 * 16 * most * 66 <= MAX_FLOATS < 32 * 16 * (most + 1) * 66
    ours, theirs = call_both(lib, case, 16, 4, 64, 16, splits=most)
    assert_close(ours, plain_attention(case, 16, 4, 64, 16))
    assert torch.equal(ours, theirs)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    out = torch.zeros_like(case["q"])
    code = lib.me_attention_decode_bf16_noalloc(
        *[case[k].data_ptr() for k in ("q", "k", "v", "table", "cu", "lens")], out.data_ptr(), 64**-0.5,
        32, most + 1, 16, 4, 64, 16, case["table"].shape[1], 0, stream,
    )  # fmt: skip
    torch.cuda.synchronize()
    assert code == TOO_LARGE
    assert float(out.float().abs().max()) == 0.0  # nothing was launched
    assert take_error(lib) == 0


def test_too_few_splits_are_reported_and_harmless():
    """`max_splits` one short of what the longest context needs (the host cannot see the lengths):
    the call returns, the keys beyond the covered range are left out (the output is plain
    attention over the covered keys), nothing outside the request's own slots is read, and the
    error word says so once."""
    lib = library()
    take_error(lib)
    case = make_case(6, [300, 100], heads=4, kv_heads=2, head_dim=128, page=16)  # 300 keys need 3 splits
    ours, theirs = call_both(lib, case, 4, 2, 128, 16, splits=2)
    assert take_error(lib) == 2
    assert take_error(lib) == 0  # taken: the word is clear again
    want = plain_attention(case, 4, 2, 128, 16, visible=256)
    assert_close(ours, want)
    assert torch.equal(ours, theirs)
    # with enough splits the next call is whole again
    ours, _ = call_both(lib, case, 4, 2, 128, 16, splits=3)
    assert_close(ours, plain_attention(case, 4, 2, 128, 16))
    assert take_error(lib) == 0
