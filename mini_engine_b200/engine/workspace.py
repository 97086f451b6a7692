"""Named, persistent device buffers for one step's activations.

Parts ask for a buffer by name and shape; the first request allocates it at the engine's
token capacity and every later request returns a view of the same memory.  Addresses are
therefore stable from step to step, which is what lets a decode step be captured in a CUDA
graph and lets TMA descriptors of activations be made once.
"""

from __future__ import annotations

import math

import torch

from mini_engine_b200.parts.linear import partial_rows


class Workspace:
    def __init__(self, max_tokens: int, device: str | torch.device = "cuda"):
        self.max_tokens = max_tokens
        self.device = torch.device(device)
        self._buffers: dict[tuple[str, torch.dtype], torch.Tensor] = {}
        self.frozen = False  # set while a graph is captured: no new allocation may happen
        # Buffers that were replaced by larger ones.  A captured graph keeps the address of the
        # buffer it was captured with and goes on writing and reading there, so the memory must
        # neither be freed nor given to anyone else.
        self._retired: list[torch.Tensor] = []

    def _flat(self, name: str, elements: int, dtype: torch.dtype) -> torch.Tensor:
        key = (name, dtype)
        held = self._buffers.get(key)
        if held is None or held.numel() < elements:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would have to grow during graph capture")
            if held is not None:
                self._retired.append(held)
            held = torch.empty(elements, dtype=dtype, device=self.device)
            self._buffers[key] = held
        return held

    def get(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """A contiguous view ``shape`` of the named buffer.  The first axis is a token count;
        the buffer is sized for ``max_tokens`` of them."""
        per_row = math.prod(shape[1:])
        rows = max(shape[0], self.max_tokens)
        flat = self._flat(name, rows * per_row, dtype)
        return flat[: shape[0] * per_row].view(shape)

    def partials(self, name: str, splits: int, tokens: int, width: int) -> torch.Tensor:
        """``[splits, tokens, width]`` float32 for the partial sums of a split product."""
        rows = max(partial_rows(self.max_tokens), splits * tokens)
        flat = self._flat(name, rows * width, torch.float32)
        return flat[: splits * tokens * width].view(splits, tokens, width)

    def growing(self, name: str, shape: tuple[int, ...], dtype: torch.dtype) -> torch.Tensor:
        """A buffer of exactly ``shape`` that grows on demand instead of being sized for the
        token capacity (logits: ``[rows, vocab]`` is large and ``rows`` is usually small)."""
        flat = self._flat(name, math.prod(shape), dtype)
        return flat[: math.prod(shape)].view(shape)

    def zeroed(self, name: str, count: int) -> torch.Tensor:
        """``count`` int32 values that are zero when first handed out.  Kernels that use them
        (arrival counters) leave them zero again, so they are never cleared between steps."""
        key = (name, torch.int32)
        held = self._buffers.get(key)
        if held is None or held.numel() < count:
            if self.frozen:
                raise RuntimeError(f"workspace buffer {name!r} would have to grow during graph capture")
            if held is not None:
                self._retired.append(held)
            held = torch.zeros(max(count, 1024), dtype=torch.int32, device=self.device)
            self._buffers[key] = held
        return held[:count]

    def bytes_held(self) -> int:
        return sum(t.numel() * t.element_size() for t in [*self._buffers.values(), *self._retired])
