"""The allocation-free decode-attention entry point, called through its exported C symbol.

Some users of the library cannot allocate device memory when they need attention (a plug-in in
a process that owns all memory, a loop that must not risk the synchronisation an allocation
can cause), so `me_attention_decode_bf16_noalloc` keeps its scratch in a fixed array inside the
library.  Here it must give what the ordinary entry point gives with caller-supplied scratch,
on two calls in a row (the second finds the first call's leftovers in the shared scratch), and
refuse sizes beyond its limit.  The file sorts last so that a run that stops at the first
failure has run everything else before.
"""

from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import pytest
import torch

pytestmark = pytest.mark.gpu

TOO_LARGE = 1003
MAX_FLOATS = 2 * 1024 * 1024


def library():
    from mini_engine_b200.csrc.build import load_library

    lib = load_library("attention_bf16")
    lib.me_attention_decode_bf16_noalloc.argtypes = [c_void_p] * 7 + [c_float] + [c_int] * 8 + [c_void_p]
    lib.me_attention_decode_bf16_noalloc.restype = c_int
    lib.me_attention_decode_bf16.argtypes = [c_void_p] * 8 + [c_float] + [c_int] * 8 + [c_void_p]
    lib.me_attention_decode_bf16.restype = c_int
    return lib


def make_case(seed, lengths, heads, kv_heads, head_dim, page):
    g = torch.Generator().manual_seed(seed)
    pages = sum(-(-n // page) for n in lengths) + 2
    width = max(-(-n // page) for n in lengths)
    order = torch.randperm(pages, generator=g).tolist()
    table = torch.full((len(lengths), width), -1, dtype=torch.int32)
    for b, n in enumerate(lengths):
        for i in range(-(-n // page)):
            table[b, i] = order.pop()
    return dict(
        q=torch.randn(len(lengths), heads * head_dim, generator=g).to(torch.bfloat16).cuda(),
        k=torch.randn(pages, kv_heads, page, head_dim, generator=g).to(torch.bfloat16).cuda(),
        v=torch.randn(pages, kv_heads, page, head_dim, generator=g).to(torch.bfloat16).cuda(),
        table=table.cuda(),
        cu=torch.arange(len(lengths) + 1, dtype=torch.int32).cuda(),
        lens=torch.tensor(lengths, dtype=torch.int32).cuda(),
    )


def call_both(lib, case, heads, kv_heads, head_dim, page, splits):
    entries = case["q"].shape[0]
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    common = [case[k].data_ptr() for k in ("q", "k", "v", "table", "cu", "lens")]
    tail = [head_dim**-0.5, entries, splits, heads, kv_heads, head_dim, page, case["table"].shape[1], 0, stream]
    ours = torch.full_like(case["q"], float("nan"))
    theirs = torch.full_like(case["q"], float("nan"))
    scratch = torch.empty(entries * heads * splits * (head_dim + 2), dtype=torch.float32, device="cuda")
    assert lib.me_attention_decode_bf16(*common, theirs.data_ptr(), scratch.data_ptr(), *tail) == 0
    assert lib.me_attention_decode_bf16_noalloc(*common, ours.data_ptr(), *tail) == 0
    torch.cuda.synchronize()
    return ours, theirs


def test_no_alloc_entry_matches_the_ordinary_one_twice_in_a_row():
    lib = library()
    first = make_case(1, [600, 33, 256, 1], heads=8, kv_heads=2, head_dim=128, page=16)
    ours, theirs = call_both(lib, first, 8, 2, 128, 16, splits=5)  # ceil(600 / 128)
    assert torch.isfinite(ours.float()).all()
    assert float((ours.float() - theirs.float()).abs().max()) <= 1e-2 * float(theirs.float().abs().max())
    # a second call of another shape, right behind the first, on the same scratch
    second = make_case(2, [90, 300], heads=4, kv_heads=4, head_dim=64, page=8)
    ours2, theirs2 = call_both(lib, second, 4, 4, 64, 8, splits=3)
    assert torch.isfinite(ours2.float()).all()
    assert float((ours2.float() - theirs2.float()).abs().max()) <= 1e-2 * float(theirs2.float().abs().max())
    # and the first again: the same bits as before (the kernels are deterministic)
    ours3, _ = call_both(lib, first, 8, 2, 128, 16, splits=5)
    assert torch.equal(ours3, ours)


def test_no_alloc_entry_refuses_what_does_not_fit():
    lib = library()
    case = make_case(3, [40, 40], heads=8, kv_heads=2, head_dim=128, page=16)
    stream = c_void_p(torch.cuda.current_stream().cuda_stream)
    out = torch.zeros_like(case["q"])
    entries, heads, head_dim = 2, 8, 128
    splits = MAX_FLOATS // (entries * heads * (head_dim + 2)) + 1
    code = lib.me_attention_decode_bf16_noalloc(
        *[case[k].data_ptr() for k in ("q", "k", "v", "table", "cu", "lens")], out.data_ptr(), head_dim**-0.5,
        entries, splits, heads, 2, head_dim, 16, case["table"].shape[1], 0, stream,
    )  # fmt: skip
    torch.cuda.synchronize()
    assert code == TOO_LARGE
    assert float(out.float().abs().max()) == 0.0  # nothing was launched
