"""Host side of the bfloat16 tensor-core attention kernels: which kernel a batch takes.

* every entry brings one token and the group has at most 16 query heads: a split decode kernel
  (scratch for the partial results comes from the workspace): with groups of at most 8 heads and
  pages of a power of two of at least 8 keys the one that fetches whole page rows by TMA, else
  the one that gathers keys row by row;
* otherwise, head size 128, no window, pages of 8 to 128 tokens and a portion of at least 32
  tokens in the batch: the tcgen05 kernel (both products on the tensor cores with accumulators in
  tensor memory, keys and values fetched by TMA page by page);
* otherwise: the mma.sync portions kernel, for any mix of portion lengths.

Head sizes 64 and 128 are taken; other sizes use the generic kernel.
"""

from __future__ import annotations

from ctypes import c_float, c_int, c_void_p

import torch

from mini_engine_b200.csrc import ops, tensor_core
from mini_engine_b200.csrc.build import load_library

DECODE_CHUNK = 128
TENSOR_MEMORY_MIN_TOKENS = 32  # portions at least this long take the tcgen05 kernel

def _ops_stream() -> c_void_p:
    return ops._stream()


_lib = None
_tc_lib = None
_page_maps: dict[tuple[int, tuple[int, ...], int], object] = {}
_query_maps: dict[tuple[int, int, int], object] = {}


def _tc_library():
    global _tc_lib
    if _tc_lib is None:
        import ctypes

        lib = load_library("attention_tcgen05")
        lib.me_attention_tcgen05.argtypes = [c_void_p] * 7 + [c_float] + [c_int] * 7 + [c_void_p, c_void_p]
        lib.me_attention_tcgen05.restype = c_int
        lib.me_attention_take_error.argtypes = [ctypes.POINTER(c_int)]
        lib.me_attention_take_error.restype = c_int
        _tc_lib = lib
    return _tc_lib


def take_error() -> int:
    """First failure (a wait that ran out) that an attention kernel recorded since the last call,
    or 0.  Only libraries that were loaded are asked."""
    import ctypes

    found = 0
    for lib, symbol in ((_tc_lib, "me_attention_take_error"), (_lib, "me_attention_bf16_take_error")):
        if lib is None:
            continue
        code = c_int(0)
        status = getattr(lib, symbol)(ctypes.byref(code))
        if status != 0:
            raise RuntimeError(f"could not read the attention kernels' error flag (CUDA error {status})")
        found = found or code.value
    return found


def _page_map(pages: torch.Tensor, box_rows: int | None = None):
    """TMA descriptor of a page array seen as [(pages * kv_heads * page_size), head_dim], with
    boxes of ``box_rows`` rows (a whole page by default)."""
    count, kv_heads, page_size, head_dim = pages.shape
    box_rows = box_rows or page_size
    key = (pages.data_ptr(), tuple(pages.shape), box_rows)
    held = _page_maps.get(key)
    if held is None:
        held = tensor_core._make_map(pages.view(count * kv_heads * page_size, head_dim), box_rows)
        _page_maps[key] = held
    return held


TMA_DECODE_KEYS = 16  # keys of one warp's box in the TMA decode kernel


def tma_decode_kernel_takes(heads: int, kv_heads: int, page_size: int) -> bool:
    return heads // kv_heads <= 8 and page_size >= 8 and page_size & (page_size - 1) == 0


def _query_map(q: torch.Tensor):
    key = (q.data_ptr(), q.shape[0], q.shape[1])
    held = _query_maps.get(key)
    if held is None:
        if len(_query_maps) > 8192:
            _query_maps.clear()
        held = tensor_core._make_map(q, 128)
        _query_maps[key] = held
    return held


def tensor_memory_kernel_takes(head_dim: int, page_size: int, window: int, max_query_len: int) -> bool:
    return (
        head_dim == 128
        and window == 0
        and 8 <= page_size <= 128
        and 128 % page_size == 0
        and max_query_len >= TENSOR_MEMORY_MIN_TOKENS
    )


def _library():
    global _lib
    if _lib is None:
        import ctypes

        lib = load_library("attention_bf16")
        lib.me_attention_portions_bf16.argtypes = [c_void_p] * 7 + [c_float] + [c_int] * 8 + [c_void_p, c_void_p]
        lib.me_attention_portions_bf16.restype = c_int
        lib.me_attention_decode_bf16_tiled.argtypes = [c_void_p] * 9 + [c_float] + [c_int] * 9 + [c_void_p, c_void_p]
        lib.me_attention_decode_bf16_tiled.restype = c_int
        lib.me_attention_decode_bf16_tma.argtypes = [c_void_p] * 9 + [c_float] + [c_int] * 9 + [c_void_p, c_void_p]
        lib.me_attention_decode_bf16_tma.restype = c_int
        lib.me_attention_bf16_take_error.argtypes = [ctypes.POINTER(c_int)]
        lib.me_attention_bf16_take_error.restype = c_int
        _lib = lib
    return _lib


def supports(head_dim: int, heads: int, kv_heads: int) -> bool:
    return head_dim in (64, 128) and kv_heads > 0 and heads % kv_heads == 0


RESIDENT_DECODE_CTAS = 3 * 148  # three CTAs of the decode kernel fit an SM


def decode_tiles_per_cta(entries: int, kv_heads: int, max_context_len: int) -> int:
    """Consecutive 128-key tiles that one CTA walks (1 to 8): as few CTAs as cover the longest
    context the launch may meet in one resident wave, so that every CTA pays its start-up once and
    keeps loads in flight from tile to tile.  The choice changes how partial results are grouped,
    hence the result in its last bits, never which keys are read."""
    tiles = entries * kv_heads * max(1, -(-max_context_len // DECODE_CHUNK))
    return max(1, min(8, -(-tiles // RESIDENT_DECODE_CTAS)))


RESIDENT_DECODE_CTAS_OF_SIX_WARPS = 4 * 148  # four CTAs of six warps fit an SM


def tma_decode_warps(entries: int, kv_heads: int) -> int:
    """Warps of a CTA of the TMA decode kernel: eight (128 keys at a time, three CTAs to an SM,
    444 resident) or six (96 keys at a time, four CTAs to an SM, 592 resident).  Six when one CTA
    per (request, KV head) then needs fewer waves: batch 64 with 8 KV heads is 512 pairs, one wave
    of six-warp CTAs but a full and a nearly empty one of eight-warp CTAs (2,048 keys: 88.7 us
    against 93.2 us with three CTAs per pair; 320 keys: 17.9 us against 22.0 us).  With as many
    waves either way, eight warps are faster (batch 96: 122 us against 137 us)."""
    pairs = max(1, entries * kv_heads)
    waves_of_eight = -(-pairs // RESIDENT_DECODE_CTAS)
    waves_of_six = -(-pairs // RESIDENT_DECODE_CTAS_OF_SIX_WARPS)
    return 6 if waves_of_six < waves_of_eight else 8


def tma_decode_splits(entries: int, kv_heads: int, max_context_len: int, warps: int = 8) -> int:
    """CTAs that share the keys of one (request, KV head) in the TMA decode kernel: as many as
    fill one resident wave, at most one per two tiles of the longest context.  The kernel divides
    each request's own tiles evenly among them (two tiles or more per CTA).

    Long contexts whose one wave would be lopsided (fewer CTAs than three quarters of the slots,
    so that some SMs hold two and some one) take three times as many: with several CTAs per slot
    the SMs that finish early take the next ones, and a CTA of 24 tiles and more hides its
    start-up (batch 32 at 8,192 keys: 199 -> 171 us).  So do batches with a few more (request, KV
    head) pairs than slots, from 16 tiles on: whole pairs would leave a last wave that is nearly
    empty and as long as the first (batch 64 at 2,048 keys: 103 -> 93 us; at 4,096: 194 -> 168 us),
    while with a last wave that is a third full and more, one CTA per pair is faster (batch 80 at
    4,096 keys: 202 us against 208 us)."""
    tiles = max(1, -(-max_context_len // (warps * TMA_DECODE_KEYS)))
    pairs = max(1, entries * kv_heads)
    slots = RESIDENT_DECODE_CTAS if warps == 8 else RESIDENT_DECODE_CTAS_OF_SIX_WARPS
    splits = max(1, min(slots // pairs, -(-tiles // 2), 64))
    if pairs > slots:
        if tiles >= 16 and pairs % slots < 0.25 * slots:
            splits = 3
    elif tiles / splits >= 24 and pairs * splits < 0.75 * slots:
        splits = max(splits, min(3 * splits, tiles // 8, 64))
    return splits


def decode_splits(max_context_len: int, tiles_per_cta: int = 1) -> int:
    return max(1, -(-max_context_len // (DECODE_CHUNK * tiles_per_cta)))


def paged_attention(q, k_pages, v_pages, block_table, ctx, out, heads, kv_heads, head_dim, scale, window,
                    decode_warps: int | None = None, decode_splits_per_pair: int | None = None) -> None:
    """Attention of the batch's new tokens.  Entries that bring one token take the split decode
    kernel, the others a portions kernel; a step that holds both kinds is two launches, each over
    its own list of entries.  ``decode_warps`` (6 or 8) and ``decode_splits_per_pair`` pin the form
    of the TMA decode kernel that the rules above would otherwise choose from the batch: the kernel
    tests run every case in both forms, and the kernel bench times one form against the other."""
    for name, t in (("q", q), ("out", out), ("k_pages", k_pages), ("v_pages", v_pages)):
        if t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise ops.KernelError(f"{name} must be contiguous bfloat16")
    if block_table.dtype != torch.int32 or not block_table.is_contiguous():
        raise ops.KernelError("block_table must be contiguous int32")
    stream = _ops_stream()
    page_size, width = k_pages.shape[2], block_table.shape[1]
    common = (q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(), ctx.cu_tokens.data_ptr(),
              ctx.context_lens.data_ptr(), out.data_ptr())  # fmt: skip
    decode_ok = heads // kv_heads <= 16
    if ctx.all_decode and decode_ok:
        launches = [("decode", ctx.num_entries, None, 1)]
    else:
        decodes = getattr(ctx, "num_decode_entries", 0) if decode_ok else 0
        if decodes and decodes < ctx.num_entries:
            launches = [
                ("decode", decodes, ctx.decode_entries, 1),
                ("portions", ctx.num_entries - decodes, ctx.portion_entries, ctx.max_query_len),
            ]
        else:
            launches = [("portions", ctx.num_entries, None, ctx.max_query_len)]
    for kind, entries, ids, longest in launches:
        ids_ptr = None if ids is None else ids.data_ptr()
        if kind == "decode" and tma_decode_kernel_takes(heads, kv_heads, page_size):
            warps = decode_warps or tma_decode_warps(entries, kv_heads)
            splits = decode_splits_per_pair or tma_decode_splits(entries, kv_heads, ctx.max_context_len, warps)
            partials = counters = None
            if splits > 1:
                partials = ctx.workspace.growing("attn.partials", (ctx.num_entries, heads, splits, head_dim + 2), torch.float32).data_ptr()
                counters = ctx.workspace.zeroed("attn.counters", ctx.num_entries * kv_heads).data_ptr()
            rows = min(page_size, TMA_DECODE_KEYS)
            code = _library().me_attention_decode_bf16_tma(
                _page_map(k_pages, rows), _page_map(v_pages, rows), common[0], *common[3:], partials, counters, scale,
                entries, splits, warps, heads, kv_heads, head_dim, page_size, width, window, ids_ptr, stream,
            )  # fmt: skip
            ops._check(code, "attention_decode_bf16_tma")
        elif kind == "decode":
            tiles = decode_tiles_per_cta(entries, kv_heads, ctx.max_context_len)
            splits = decode_splits(ctx.max_context_len, tiles)
            partials = ctx.workspace.growing("attn.partials", (ctx.num_entries, heads, splits, head_dim + 2), torch.float32)
            counters = ctx.workspace.zeroed("attn.counters", ctx.num_entries * kv_heads)
            code = _library().me_attention_decode_bf16_tiled(
                *common, partials.data_ptr(), counters.data_ptr(), scale, entries, splits, tiles, heads, kv_heads,
                head_dim, page_size, width, window, ids_ptr, stream,
            )  # fmt: skip
            ops._check(code, "attention_decode_bf16")
        elif tensor_memory_kernel_takes(head_dim, page_size, window, longest):
            code = _tc_library().me_attention_tcgen05(
                _query_map(q), _page_map(k_pages), _page_map(v_pages), *common[3:], scale, entries, longest, heads,
                kv_heads, head_dim, page_size, width, ids_ptr, stream,
            )  # fmt: skip
            ops._check(code, "attention_tcgen05")
        else:
            code = _library().me_attention_portions_bf16(
                *common, scale, entries, longest, heads, kv_heads, head_dim, page_size, width, window, ids_ptr, stream
            )
            ops._check(code, "attention_portions_bf16")
