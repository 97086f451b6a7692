"""Host side of the TMA + tcgen05 matrix product: tensor maps, tile and split choice, launch.

A :class:`GemmPlan` is made once per weight and holds its TMA descriptor.  Descriptors of
activations are cached by (address, rows, width, tile), which is stable because activations
live in the engine's persistent workspace.
"""

from __future__ import annotations

import ctypes
from ctypes import c_int, c_uint, c_ulonglong, c_void_p

import torch

from mini_engine_b200.csrc import ops
from mini_engine_b200.csrc.build import load_library

NUM_SMS = 148
BLOCK_N = 128
BLOCK_K = 64
TOKEN_TILES = (16, 32, 64, 128, 256)
SPLIT_MAX_TOKENS = 1024  # products of more tokens have enough tiles without splitting
MIN_K_BLOCKS_PER_SPLIT = 4
PAIR_MIN_TOKENS = 128  # longer products run on CTA pairs (256 x 256 tiles), unsplit ones in the persistent kernel
# Products of 129 to 1,024 tokens whose reduction is split run on CTA pairs too (each split its own
# pairs) when a split is long: 48 k blocks and more (the down projection of Qwen3-8B: 256 tokens
# 33.1 -> 31.3 us, 512 tokens 48.9 -> 44.2 us); with 16 to 32 k blocks per split the lone CTAs are as
# fast or 2 % faster.
PAIR_SPLIT_MIN_K_BLOCKS = 48
# Up to this many tokens the stacked gated product cuts its reduction in two halves, one per CTA of a
# cluster of two: 384 CTAs of 72 KB, three to an SM, stream the weights at 6.5 TB/s where 192 CTAs
# with the whole reduction reach 5.9 (8 tokens, 12,288 gated features of 4,096: 34.3 us unsplit).
STACKED_HALVES_MAX_TOKENS = 16
# The persistent pair kernel numbers its tiles in groups of this many token tiles (all feature tiles
# of a group before the next group): the pairs that run together then share a block of tiles about
# as tall as it is wide, and a group's activations are read once for all features.  0: one group (the
# token tile fastest over the whole product).  Measured at Qwen3-8B's shapes: nothing changes up to
# 4,096 tokens; 8,192 tokens: q/k/v 317 -> 295 us, o 211 -> 193, down 606 -> 563, gate and up with
# SwiGLU 1,159 -> 1,119 (its groups 16 wide: with 8, 1,130); 16,384 tokens: 697 -> 574, 464 -> 384,
# 1,349 -> 1,125, 2,462 -> 2,247 us (1.43 to 1.47 PFLOP/s).
PAIR_GROUP_TOKEN_TILES = 8
PAIR_GROUP_TOKEN_TILES_GATED = 16
STACKED_MAX_TOKENS = 64  # gated products of up to this many tokens stack gate rows on up rows in one operand


def _ops_stream() -> c_void_p:
    return ops._stream()


_lib = None


def _library():
    global _lib
    if _lib is None:
        lib = load_library("gemm_tcgen05")
        lib.me_make_tensor_map.argtypes = [c_void_p, c_void_p, c_ulonglong, c_ulonglong, c_uint]
        lib.me_make_tensor_map.restype = c_int
        lib.me_gemm_tcgen05.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]
        lib.me_gemm_tcgen05.restype = c_int
        lib.me_gemm_tcgen05_swiglu.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]
        lib.me_gemm_tcgen05_swiglu.restype = c_int
        lib.me_gemm_tcgen05_pair_split.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        lib.me_gemm_tcgen05_pair_split.restype = c_int
        lib.me_gemm_tcgen05_persistent.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p]
        lib.me_gemm_tcgen05_persistent.restype = c_int
        lib.me_gemm_tcgen05_persistent_swiglu.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_void_p]
        lib.me_gemm_tcgen05_persistent_swiglu.restype = c_int
        lib.me_gemm_tcgen05_stacked_swiglu.argtypes = [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_int, c_int, c_void_p]
        lib.me_gemm_tcgen05_stacked_swiglu.restype = c_int
        lib.me_gemm_wait_probe.argtypes = [c_int, c_void_p, c_void_p]
        lib.me_gemm_wait_probe.restype = c_int
        lib.me_gemm_take_error.argtypes = [ctypes.POINTER(c_int)]
        lib.me_gemm_take_error.restype = c_int
        _lib = lib
    return _lib


def supports(outs: int, inner: int) -> bool:
    """TMA wants a 16-byte row pitch: ``inner`` a multiple of 8 bfloat16 values."""
    return inner % 8 == 0 and inner >= 8 and outs >= 1


def token_tile(tokens: int) -> int:
    for tile in TOKEN_TILES:
        if tokens <= tile:
            return tile
    return TOKEN_TILES[-1]


def choose_splits(tokens: int, outs: int, inner: int, max_splits: int = 8) -> int:
    """How many ranges the reduction axis is cut into.  It depends on the sizes only (for a
    given number of tokens the same split is always chosen), and no split is empty."""
    if tokens > SPLIT_MAX_TOKENS:
        return 1
    tile = token_tile(tokens)
    tiles = -(-outs // BLOCK_N) * -(-tokens // tile)
    k_blocks = -(-inner // BLOCK_K)
    slots = NUM_SMS * (3 if tile <= 16 else 2 if tile <= 64 else 1)  # CTAs of this tile size that fit an SM at once (72, 80, 96, 192 KB of shared memory)
    wanted = min(max_splits, max(1, slots // tiles), max(1, k_blocks // MIN_K_BLOCKS_PER_SPLIT))
    per_split = -(-k_blocks // wanted)
    return -(-k_blocks // per_split)


def _make_map(tensor: torch.Tensor, box_rows: int) -> ctypes.Array:
    """TMA descriptor of a contiguous bfloat16 matrix with boxes of ``box_rows`` x 64 elements."""
    if tensor.dtype != torch.bfloat16 or not tensor.is_contiguous() or tensor.dim() != 2:
        raise RuntimeError("TMA descriptors are made for contiguous 2-D bfloat16 tensors")
    rows, inner = tensor.shape
    holder = (ctypes.c_ubyte * 128)()
    code = _library().me_make_tensor_map(holder, tensor.data_ptr(), rows, inner, box_rows)
    if code != 0:
        raise RuntimeError(f"could not make a TMA descriptor for a {rows} x {inner} matrix (code {code})")
    return holder


class GemmPlan:
    def __init__(self, weight: torch.Tensor, dual_rows: int | None = None):
        if weight.dtype != torch.bfloat16 or not weight.is_contiguous() or not weight.is_cuda:
            raise RuntimeError("the tensor-core product takes a contiguous bfloat16 CUDA weight")
        self.weight = weight
        self.rows, self.inner = weight.shape
        self.dual_rows = dual_rows  # gate rows [0, dual_rows), up rows [dual_rows, 2 * dual_rows)
        self.map = _make_map(weight, BLOCK_N)
        # Boxes of 64 rows, for the few-token gated kernel that stacks gate rows on up rows.
        self.map_half = _make_map(weight, BLOCK_N // 2) if dual_rows is not None else None


_activation_maps: dict[tuple[int, int, int, int], ctypes.Array] = {}


def _activation_map(x: torch.Tensor, tile: int) -> ctypes.Array:
    key = (x.data_ptr(), x.shape[0], x.shape[1], tile)
    held = _activation_maps.get(key)
    if held is None:
        if len(_activation_maps) > 8192:
            _activation_maps.clear()
        held = _make_map(x, tile)
        _activation_maps[key] = held
    return held


def _check_x(plan: GemmPlan, x: torch.Tensor) -> None:
    if x.dtype != torch.bfloat16 or not x.is_contiguous() or x.dim() != 2 or x.shape[1] != plan.inner:
        raise RuntimeError(f"activation {tuple(x.shape)} {x.dtype} does not fit a weight of width {plan.inner}")
    if x.data_ptr() % 16:
        raise RuntimeError("activation must be 16-byte aligned for TMA")


def gemm(plan: GemmPlan, x: torch.Tensor, out: torch.Tensor, splits: int, group: int | None = None) -> None:
    """``out[s] = x @ weight^T`` restricted to the k range of split ``s``; float32
    ``[splits, T, rows]``.  ``group`` pins the width of the persistent kernel's tile groups (the
    kernel tests run several; the kernel bench times them)."""
    _check_x(plan, x)
    tokens = x.shape[0]
    if out.dtype != torch.float32 or tuple(out.shape) != (splits, tokens, plan.rows) or not out.is_contiguous():
        raise RuntimeError(f"output {tuple(out.shape)} does not fit [{splits}, {tokens}, {plan.rows}] float32")
    tile = token_tile(tokens)
    stream = _ops_stream()
    if tokens > PAIR_MIN_TOKENS and splits == 1:
        code = _library().me_gemm_tcgen05_persistent(
            plan.map, _activation_map(x, 128), out.data_ptr(), tokens, plan.rows, plan.inner,
            PAIR_GROUP_TOKEN_TILES if group is None else group, stream,
        )  # fmt: skip
    elif tokens > PAIR_MIN_TOKENS and -(-plan.inner // BLOCK_K) >= PAIR_SPLIT_MIN_K_BLOCKS * splits:
        code = _library().me_gemm_tcgen05_pair_split(
            plan.map, _activation_map(x, 128), out.data_ptr(), tokens, plan.rows, plan.inner, splits, stream
        )
    else:
        code = _library().me_gemm_tcgen05(
            plan.map, _activation_map(x, tile), out.data_ptr(), tokens, plan.rows, plan.inner, tile, splits, stream
        )
    _count_launch()
    if code != 0:
        raise RuntimeError(f"tensor-core product failed to launch (code {code})")


def gemm_swiglu(plan: GemmPlan, x: torch.Tensor, act: torch.Tensor, halves: int | None = None, group: int | None = None) -> None:
    """``act = silu(x @ gate^T) * (x @ up^T)`` in bfloat16, gate/up being the halves of the
    plan's weight.  ``halves`` (1 or 2) pins how many CTAs share a reduction of the few-token kernel
    instead of the rule's choice: the kernel tests run both forms, the kernel bench times them."""
    _check_x(plan, x)
    tokens = x.shape[0]
    if plan.dual_rows is None:
        raise RuntimeError("this plan was not made for a gated product")
    if act.dtype != torch.bfloat16 or tuple(act.shape) != (tokens, plan.dual_rows) or not act.is_contiguous():
        raise RuntimeError(f"activation output {tuple(act.shape)} does not fit [{tokens}, {plan.dual_rows}] bfloat16")
    stream = _ops_stream()
    if tokens <= STACKED_MAX_TOKENS:
        tile = token_tile(tokens)
        if halves is None:
            halves = 2 if tokens <= STACKED_HALVES_MAX_TOKENS and plan.inner >= 2 * BLOCK_K else 1
        code = _library().me_gemm_tcgen05_stacked_swiglu(
            plan.map_half, _activation_map(x, tile), act.data_ptr(), tokens, plan.dual_rows, plan.inner, plan.dual_rows,
            tile, halves, stream,
        )  # fmt: skip
    elif tokens > PAIR_MIN_TOKENS:
        code = _library().me_gemm_tcgen05_persistent_swiglu(
            plan.map, _activation_map(x, 128), act.data_ptr(), tokens, plan.dual_rows, plan.inner, plan.dual_rows,
            PAIR_GROUP_TOKEN_TILES_GATED if group is None else group, stream,
        )  # fmt: skip
    else:
        tile = 128  # 65 to 128 tokens: lone CTAs with gate and up sums side by side in tensor memory
        code = _library().me_gemm_tcgen05_swiglu(
            plan.map, _activation_map(x, tile), act.data_ptr(), tokens, plan.dual_rows, plan.inner, plan.dual_rows,
            tile, stream,
        )
    _count_launch()
    if code != 0:
        raise RuntimeError(f"gated tensor-core product failed to launch (code {code})")


def _count_launch() -> None:
    ops._Counter.launches += 1


def wait_probe(polls: int = 4096) -> bool:
    """Launch a CTA whose barrier waits run out after ``polls`` polls because nothing ever arrives
    at them (no fault, trap or endless loop): it records the failure as the product kernels do,
    gives its tensor memory back and returns.  True when it returned; :func:`take_error` then
    reports the recorded code.  Exists so that the give-up path can be tested."""
    lib = _library()
    returned = torch.zeros(1, dtype=torch.int32, device="cuda")
    code = lib.me_gemm_wait_probe(polls, returned.data_ptr(), _ops_stream())
    _count_launch()
    if code != 0:
        raise RuntimeError(f"the wait probe failed to launch (code {code})")
    return bool(returned.item())


def take_error() -> int:
    """The first failure that a tensor-core kernel recorded on the device since the last call
    (a wait that ran into its limit), or 0.  Synchronises the device."""
    if _lib is None:
        return 0
    code = c_int(0)
    status = _lib.me_gemm_take_error(ctypes.byref(code))
    if status != 0:
        raise RuntimeError(f"could not read the kernels' error flag (CUDA error {status})")
    return code.value
