"""Times one kernel of the engine alone, with CUDA events, at sizes given on the command line.

    python -m mini_engine_b200.cli.kernel_bench gemm --tokens 2048 --outs 6144 --inner 4096
    python -m mini_engine_b200.cli.kernel_bench gemm --tokens 8 --outs 4096 --inner 12288
    python -m mini_engine_b200.cli.kernel_bench swiglu-gemm --tokens 2048 --outs 12288 --inner 4096
    python -m mini_engine_b200.cli.kernel_bench decode-attention --batch 64 --context 2048
    python -m mini_engine_b200.cli.kernel_bench prefill-attention --tokens 2048
    python -m mini_engine_b200.cli.kernel_bench mma-rate     # the tensor pipe alone: cycles per MMA

It is what the profiles under ``profiles/`` were captured with (small cases, a few launches).
Weights are rotated between launches so that every launch reads more than the 126 MB L2 holds.
The reference's counterpart is benchmarks/profile_engine.py of YuvGev00/mini-engine, which
times phases of a step rather than single kernels.
"""

from __future__ import annotations

import argparse
import sys
import time
from types import SimpleNamespace

import torch


GRAPH = False  # set by --graph: launches are captured into one CUDA graph and replayed
WARM_MS = 0.0  # set by --warm-ms


def timed(run, iters: int, warmup: int = 3) -> float:
    """Milliseconds per call of ``run(i)``, device time.  A kernel of a few microseconds is
    launched faster by a graph than by this Python loop; use --graph for those."""
    for i in range(warmup):
        run(i)
    torch.cuda.synchronize()
    # A GPU that was idle runs its first milliseconds below its boost clock (1.5 of 1.9 GHz seen
    # in kernels of 50 us): --warm-ms keeps it busy that long before the timed calls.
    deadline = time.perf_counter() + WARM_MS / 1e3
    while time.perf_counter() < deadline:
        for i in range(8):
            run(i)
        torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    if GRAPH:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            for i in range(iters):
                run(i)
        graph.replay()
        torch.cuda.synchronize()
        start.record()
        graph.replay()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / iters
    start.record()
    for i in range(iters):
        run(i)
    end.record()
    torch.cuda.synchronize()
    return start.elapsed_time(end) / iters


def bench_gemm(args, gated: bool) -> None:
    from mini_engine_b200.csrc import tensor_core as tc

    tokens, outs, inner = args.tokens, args.outs, args.inner
    rows = outs * (2 if gated else 1)
    copies = max(2, min(8, int(300e6 // (rows * inner * 2)) + 1))
    x = torch.randn(tokens, inner, device="cuda").to(torch.bfloat16)
    plans = [
        tc.GemmPlan(torch.randn(rows, inner, device="cuda").to(torch.bfloat16), dual_rows=outs if gated else None)
        for _ in range(copies)
    ]
    splits = 1 if gated else (args.gemm_splits or tc.choose_splits(tokens, outs, inner))
    out = (
        torch.empty(tokens, outs, device="cuda", dtype=torch.bfloat16)
        if gated
        else torch.empty(splits, tokens, outs, device="cuda")
    )

    def run(i: int) -> None:
        if gated:
            tc.gemm_swiglu(plans[i % copies], x, out, args.halves or None, None if args.group < 0 else args.group)
        else:
            tc.gemm(plans[i % copies], x, out, splits, None if args.group < 0 else args.group)

    ms = timed(run, args.iters)
    flops = 2.0 * tokens * rows * inner
    print(
        f"{'swiglu-' if gated else ''}gemm tokens={tokens} outs={outs} inner={inner} splits={splits}: {ms * 1e3:.1f} us, "
        f"{flops / ms / 1e9:.1f} TFLOP/s, weights {rows * inner * 2 / ms / 1e6:.0f} GB/s"
    )
    assert tc.take_error() == 0


MMA_RATE_CASES = [
    # (label, pair, a_in_tensor_memory, b_mn_major, n)
    ("one CTA, both operands in shared memory, N = 64", 0, 0, 0, 64),
    ("one CTA, both operands in shared memory, N = 128", 0, 0, 0, 128),
    ("one CTA, both operands in shared memory, N = 256", 0, 0, 0, 256),
    ("one CTA, A in tensor memory, B MN-major, N = 128", 0, 1, 1, 128),
    ("CTA pair, both operands in shared memory, N = 64", 1, 0, 0, 64),
    ("CTA pair, both operands in shared memory, N = 128", 1, 0, 0, 128),
    ("CTA pair, both operands in shared memory, N = 256", 1, 0, 0, 256),
    ("CTA pair, A in tensor memory, B MN-major, N = 128", 1, 1, 1, 128),
]


def mma_rate(pair: int, a_in_tensor_memory: int, b_mn_major: int, n: int, ctas: int = 148, iters: int = 2000) -> float:
    """Cycles per MMA of K = 16 when nothing but MMAs runs (csrc/mma_rate.cu)."""
    import ctypes

    from mini_engine_b200.csrc.build import load_library

    lib = load_library("mma_rate")
    lib.me_mma_rate.argtypes = [ctypes.c_void_p] + [ctypes.c_int] * 6 + [ctypes.c_void_p]
    lib.me_mma_rate.restype = ctypes.c_int
    cycles = torch.zeros(1, dtype=torch.int64, device="cuda")
    for _ in range(2):
        code = lib.me_mma_rate(cycles.data_ptr(), pair, a_in_tensor_memory, b_mn_major, n, ctas, iters, None)
        if code != 0:
            raise RuntimeError(f"me_mma_rate failed to launch (code {code})")
        torch.cuda.synchronize()
    total = int(cycles.item())
    if total < 0:
        raise RuntimeError("the MMAs' bounded wait ran out")
    return total / (4 * iters)


def bench_mma_rate(args) -> None:
    for label, pair, in_tmem, mn_major, n in MMA_RATE_CASES:
        cycles = mma_rate(pair, in_tmem, mn_major, n)
        m = 256 if pair else 128
        print(f"{label}: {cycles:.1f} cycles per MMA of {m} x {n} x 16, {2 * 128 * n * 16 / cycles:.0f} flop per cycle and SM")


def attention_context(entries: int, new_tokens: int, context: int):
    from mini_engine_b200.engine.workspace import Workspace

    cu = torch.arange(entries + 1, dtype=torch.int32, device="cuda") * new_tokens
    return SimpleNamespace(
        num_entries=entries, all_decode=new_tokens == 1, max_query_len=new_tokens, max_context_len=context,
        cu_tokens=cu.contiguous(), context_lens=torch.full((entries,), context, dtype=torch.int32, device="cuda"),
        workspace=Workspace(64),
    )  # fmt: skip


def bench_attention(args, decode: bool) -> None:
    from mini_engine_b200.csrc import attention_bf16

    heads, kv_heads, d, page = args.heads, args.kv_heads, args.head_dim, args.page
    entries = args.batch if decode else 1
    context = args.context if decode else args.tokens
    new_tokens = 1 if decode else args.tokens
    pages_per = -(-context // page)
    layers = max(1, min(8, int(300e6 // (entries * pages_per * page * kv_heads * d * 4)) + 1)) if decode else 1
    k = [torch.randn(entries * pages_per + 1, kv_heads, page, d, device="cuda", dtype=torch.bfloat16) for _ in range(layers)]
    v = [torch.randn_like(k[0]) for _ in range(layers)]
    table = torch.randperm(entries * pages_per, device="cuda").to(torch.int32).view(entries, pages_per).contiguous()
    q = torch.randn(entries * new_tokens, heads * d, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(q)
    ctx = attention_context(entries, new_tokens, context)

    def run(i: int) -> None:
        attention_bf16.paged_attention(q, k[i % layers], v[i % layers], table, ctx, out, heads, kv_heads, d, d**-0.5, 0,
                                       decode_warps=args.warps or None, decode_splits_per_pair=args.splits or None)  # fmt: skip

    ms = timed(run, args.iters)
    if decode:
        gigabytes = entries * context * kv_heads * d * 2 * 2 / 1e9
        print(f"decode-attention batch={entries} context={context}: {ms * 1e3:.1f} us, {gigabytes / ms * 1e3:.0f} GB/s of keys and values")
    else:
        flops = 4.0 * heads * d * new_tokens * (new_tokens + 1) / 2
        print(f"prefill-attention tokens={new_tokens}: {ms * 1e3:.1f} us, {flops / ms / 1e9:.1f} TFLOP/s (causal)")


def main(argv: list[str] | None = None) -> int:
    parser = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    parser.add_argument("kernel", choices=["gemm", "swiglu-gemm", "decode-attention", "prefill-attention", "mma-rate"])
    parser.add_argument("--tokens", type=int, default=2048)
    parser.add_argument("--outs", type=int, default=4096)
    parser.add_argument("--inner", type=int, default=4096)
    parser.add_argument("--batch", type=int, default=8)
    parser.add_argument("--context", type=int, default=2048)
    parser.add_argument("--heads", type=int, default=32)
    parser.add_argument("--kv-heads", type=int, default=8)
    parser.add_argument("--head-dim", type=int, default=128)
    parser.add_argument("--page", type=int, default=16)
    parser.add_argument("--iters", type=int, default=20)
    parser.add_argument("--splits", type=int, default=0, help="decode-attention: CTAs per (request, KV head); 0: the engine's rule")
    parser.add_argument("--warps", type=int, default=0, choices=[0, 6, 8], help="decode-attention: warps of a CTA; 0: the engine's rule")
    parser.add_argument("--gemm-splits", type=int, default=0, help="gemm: ranges of the reduction axis; 0: the engine's rule")
    parser.add_argument("--halves", type=int, default=0, choices=[0, 1, 2], help="swiglu-gemm of up to 16 tokens: CTAs per reduction; 0: the engine's rule")
    parser.add_argument("--group", type=int, default=-1, help="products of more than 128 tokens: token tiles of a group of the tile list (0: one group); -1: the engine's rule")
    parser.add_argument("--warm-ms", type=float, default=0.0, help="keep the GPU busy this long before the timed calls")
    parser.add_argument("--graph", action="store_true", help="capture the launches into a CUDA graph")
    args = parser.parse_args(argv)
    global GRAPH, WARM_MS
    GRAPH = args.graph
    WARM_MS = args.warm_ms
    if args.kernel == "mma-rate":
        bench_mma_rate(args)
    elif args.kernel in ("gemm", "swiglu-gemm"):
        bench_gemm(args, gated=args.kernel == "swiglu-gemm")
    else:
        bench_attention(args, decode=args.kernel == "decode-attention")
    return 0


if __name__ == "__main__":
    sys.exit(main())
