"""The host-side rules that choose how a kernel is launched: pure functions of the sizes, so they
are checked without a GPU.  What they are measured against is written beside each rule."""

from __future__ import annotations

import pytest


def attention():
    from mini_engine_b200.csrc import attention_bf16

    return attention_bf16


@pytest.mark.parametrize("entries", [1, 2, 3, 8, 17, 55, 56, 64, 74, 75, 111, 128, 500])
@pytest.mark.parametrize("kv_heads", [1, 2, 8])
@pytest.mark.parametrize("context", [1, 100, 2048, 8192, 40960])
def test_decode_attention_split_is_launchable(entries, kv_heads, context):
    """Whatever the batch: a warp count that the kernel has, at least one CTA per (request, KV
    head), never more CTAs per pair than tiles of the longest context allow at two tiles each
    (or one CTA), and a grid that CUDA takes."""
    module = attention()
    warps = module.tma_decode_warps(entries, kv_heads)
    assert warps in (6, 8)
    splits = module.tma_decode_splits(entries, kv_heads, context, warps)
    tiles = max(1, -(-context // (warps * module.TMA_DECODE_KEYS)))
    assert 1 <= splits <= 64
    assert splits <= max(1, -(-tiles // 2)) or splits == 3  # three per pair when a last wave would be nearly empty
    if splits == 3 and tiles < 6:
        assert tiles >= 2  # the kernel gives a CTA two tiles at least and leaves the others idle


def test_decode_attention_takes_six_warps_only_to_save_a_wave():
    module = attention()
    eight, six = module.RESIDENT_DECODE_CTAS, module.RESIDENT_DECODE_CTAS_OF_SIX_WARPS
    for pairs in range(1, 4 * six):
        warps = module.tma_decode_warps(pairs, 1)
        fewer_waves = -(-pairs // six) < -(-pairs // eight)
        assert (warps == 6) == fewer_waves
    assert module.tma_decode_warps(64, 8) == 6  # 512 pairs: one wave of 592 slots, two of 444
    assert module.tma_decode_warps(8, 8) == 8
    assert module.tma_decode_warps(96, 8) == 8  # two waves either way


def test_one_wave_of_decode_attention_for_small_batches():
    """Up to as many pairs as resident CTAs, pairs x splits stays within one resident wave unless
    the contexts are long enough for three times as many CTAs to pay."""
    module = attention()
    for entries in (1, 2, 4, 8, 16, 32, 55):
        splits = module.tma_decode_splits(entries, 8, 2048)
        assert entries * 8 * splits <= module.RESIDENT_DECODE_CTAS
    assert module.tma_decode_splits(1, 8, 2048) == 8  # 16 tiles: two per CTA
    assert module.tma_decode_splits(8, 8, 2048) == 6
    assert module.tma_decode_splits(64, 8, 128) == 1  # one tile: nothing to share


@pytest.mark.parametrize("tokens", [1, 5, 16, 17, 64, 65, 200, 1024, 1025, 5000])
@pytest.mark.parametrize("outs", [1, 128, 1000, 4096, 151936])
@pytest.mark.parametrize("inner", [8, 64, 72, 1160, 4096, 12288])
def test_reduction_split_of_the_tensor_core_product(tokens, outs, inner):
    """The split depends on the sizes only, stays within the partial-sum buffers (eight slices)
    and leaves no range of the reduction empty."""
    from mini_engine_b200.csrc import tensor_core

    splits = tensor_core.choose_splits(tokens, outs, inner)
    assert splits == tensor_core.choose_splits(tokens, outs, inner)
    k_blocks = -(-inner // tensor_core.BLOCK_K)
    assert 1 <= splits <= min(8, k_blocks)
    per_split = -(-k_blocks // splits)
    assert (splits - 1) * per_split < k_blocks  # the last range holds at least one block
    if tokens > tensor_core.SPLIT_MAX_TOKENS:
        assert splits == 1


def test_partial_sum_buffer_holds_every_split_of_a_decode_step():
    from mini_engine_b200.parts import linear

    for max_tokens in (1, 8, 64, 100, 2048, 8192):
        rows = linear.partial_rows(max_tokens)
        for tokens in range(1, min(max_tokens, linear.DECODE_TOKENS) + 1):
            assert rows >= linear.MAX_SPLITS * tokens
        assert rows >= max_tokens


def test_a_buffer_that_grows_leaves_the_old_one_alive():
    """A captured graph holds the address of the buffer it was captured with: when a later step
    needs a larger one, the old memory stays with the workspace instead of going back to the
    allocator, where someone else could be given it."""
    import torch

    from mini_engine_b200.engine.workspace import Workspace

    workspace = Workspace(8, device="cpu")
    small = workspace.growing("attn.partials", (4, 2, 3), torch.float32)
    counters = workspace.zeroed("attn.counters", 10)
    addresses = {small.data_ptr(), counters.data_ptr()}
    del small, counters
    large = workspace.growing("attn.partials", (40, 2, 30), torch.float32)
    more = workspace.zeroed("attn.counters", 5000)
    assert {t.data_ptr() for t in workspace._retired} == addresses
    assert large.data_ptr() not in addresses and more.data_ptr() not in addresses
    assert int(more.sum()) == 0
    again = workspace.growing("attn.partials", (40, 2, 30), torch.float32)
    assert again.data_ptr() == large.data_ptr() and len(workspace._retired) == 2  # the same size: no new buffer


@pytest.mark.parametrize("max_batch", [1, 2, 3, 8, 9, 16, 17, 64, 100, 256])
def test_graph_buckets_cover_every_batch_up_to_the_cap(max_batch):
    """Buckets 1, 2, 4, 8, then multiples of 16 up to the request cap (the reference's,
    src/mini_engine/cuda_graphs.py:28-40): ascending, the last one the cap itself, and every batch
    size has a bucket that is at least as large and wastes less than 16 rows (or half the bucket)."""
    from mini_engine_b200.engine.graphs import batch_buckets

    buckets = batch_buckets(max_batch)
    assert buckets == sorted(set(buckets)) and buckets[-1] == max_batch and buckets[0] >= 1
    for batch in range(1, max_batch + 1):
        bucket = next(b for b in buckets if b >= batch)
        assert bucket - batch < max(16, bucket // 2 + 1)
