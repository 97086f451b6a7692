"""Matrix products ``y = x W^T`` as the parts use them.

``Linear`` and ``GatedLinear`` are helpers, not parts: they own a weight ``[out, in]`` in the
torch ``Linear`` layout that checkpoints use (src/mini_engine/model.py:97-100,126-128 of
YuvGev00/mini-engine) and pick the kernel:

* bfloat16 with ``in`` a multiple of 8: the TMA + tcgen05 tensor-core kernel.  The weight
  is the 128-row operand and the tokens are the narrow one, so the same kernel serves a
  2,048-token prompt and a single decoded token; for few tokens the reduction axis is
  split over several CTAs and the result comes back as ``S`` partial sums that the consumer
  adds in a fixed order.
* float32, and bfloat16 shapes that TMA cannot address: a CUDA-core kernel that adds the
  products of one output element in ascending ``k`` with one accumulator, so a row's
  result never depends on which other rows are in the batch.
"""

from __future__ import annotations

import torch

from mini_engine_b200.csrc import ops
from mini_engine_b200.parts.base import StepContext

# A split product returns at most this many partial sums.  Up to DECODE_TOKENS tokens (the steps
# that captured graphs replay) a partial-sum buffer is sized for all of them at once; longer split
# products (a few hundred tokens, too few tiles to fill the GPU otherwise) let it grow on demand.
MAX_SPLITS = 8
DECODE_TOKENS = 64
# The tensor-core gated product runs as one kernel with the activation in its epilogue from this
# many tokens on (4 to 64 tokens: gate rows stacked on up rows, up to 16 tokens with the reduction
# in the two CTAs of a cluster; more: CTA pairs).  Below, all of a step's time is the weight stream
# and 384 short CTAs of a split product followed by the activation kernel stream it as fast or a
# little faster (a decode step of Qwen3-8B sizes, split product against one kernel: batch 1 3.21
# against 3.23 ms, batch 2 3.26 against 3.27, batch 3 3.28 against 3.28, batch 4 3.33 against 3.30).
GATED_FUSED_MIN_TOKENS = 4
# The stacked kernel (4 to 64 tokens) has one CTA (up to 16 tokens: two) per 64 gated features: with
# few features it leaves most SMs idle, and the split product with the activation kernel behind it
# is faster (intermediate size 3,072: a decode step of 28 layers takes 1.11 ms that way against
# 1.15 ms at batch 8, 2.07 against 2.13 ms at batch 32; at 12,288 features the stacked kernel wins).
GATED_STACKED_MIN_FEATURES = 128 * 64


def partial_rows(max_tokens: int) -> int:
    """Rows that a ``[S, T, out]`` partial-sum buffer starts with."""
    return max(max_tokens, MAX_SPLITS * min(max_tokens, DECODE_TOKENS))


class Linear:
    def __init__(self, weight: torch.Tensor):
        self.weight = weight
        self.out_features, self.in_features = weight.shape
        self.tensor_core = weight.dtype == torch.bfloat16 and ops.tensor_core_gemm_supports(
            self.out_features, self.in_features
        )
        self.plan = ops.GemmPlan(weight) if self.tensor_core else None

    def forward(self, x: torch.Tensor, ctx: StepContext, out_name: str, whole: bool = False) -> torch.Tensor:
        """``x [T, in]`` -> ``[S, T, out]`` float32 in the named workspace buffer.  With
        ``whole`` the product is never split (``S == 1``) and the buffer is sized for exactly
        ``T`` rows (the logits: few rows of a very wide output)."""
        tokens = x.shape[0]
        splits = 1
        if self.tensor_core and not whole:
            splits = ops.choose_splits(tokens, self.out_features, self.in_features)
        if whole:
            out = ctx.workspace.growing(out_name, (1, tokens, self.out_features), torch.float32)
        else:
            out = ctx.workspace.partials(out_name, splits, tokens, self.out_features)
        if self.tensor_core:
            ops.gemm_tensor_core(self.plan, x, out, splits)
        else:
            ops.gemm_simt(x, self.weight, out[0])
        return out


class GatedLinear:
    """``silu(x Wg^T) * (x Wu^T)`` from the row-concatenated weight ``[2 * inter, in]``."""

    def __init__(self, gate_up: torch.Tensor):
        self.weight = gate_up
        self.inter = gate_up.shape[0] // 2
        self.in_features = gate_up.shape[1]
        self.tensor_core = gate_up.dtype == torch.bfloat16 and ops.tensor_core_gemm_supports(
            self.inter, self.in_features
        )
        self.linear = Linear(gate_up)
        self.plan = ops.GemmPlan(gate_up, dual_rows=self.inter) if self.tensor_core else None

    def forward(self, x: torch.Tensor, ctx: StepContext, name: str) -> torch.Tensor:
        """``x [T, in]`` -> activated ``[T, inter]`` in the compute dtype."""
        tokens = x.shape[0]
        act = ctx.buffer(name + ".act", (tokens, self.inter), x.dtype)
        fused = tokens >= GATED_FUSED_MIN_TOKENS and (tokens > DECODE_TOKENS or self.inter >= GATED_STACKED_MIN_FEATURES)
        if self.tensor_core and fused:
            ops.gemm_tensor_core_swiglu(self.plan, x, act)
            return act
        both = self.linear.forward(x, ctx, name + ".gate_up")
        ops.swiglu(both, act)
        return act
