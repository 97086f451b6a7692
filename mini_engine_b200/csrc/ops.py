"""Python bindings of the CUDA kernels.

Each function checks its arguments, passes raw pointers, sizes and the current CUDA stream to
an ``extern "C"`` launcher, and raises if the launcher reports an error.  There is no other
implementation behind these names: without a GPU, a compiler or a successful build they
raise.
"""

from __future__ import annotations

import ctypes
from ctypes import c_float, c_int, c_longlong, c_void_p
from typing import Any

import torch

from mini_engine_b200.csrc.build import load_library

F32, BF16 = 0, 1
_ERRORS = {1001: "sizes not supported by this kernel", 1002: "bad argument"}


class KernelError(RuntimeError):
    pass


def _type_code(dtype: torch.dtype) -> int:
    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    raise KernelError(f"kernels take float32 or bfloat16, got {dtype}")


def _ptr(tensor: torch.Tensor | None) -> c_void_p:
    return c_void_p(0 if tensor is None else tensor.data_ptr())


_scoped_stream: c_void_p | None = None


def _stream() -> c_void_p:
    """The stream that launches go to: torch's current one, looked up once per `stream_scope`
    (the lookup costs about as much as the rest of a launch's Python)."""
    if _scoped_stream is not None:
        return _scoped_stream
    return c_void_p(torch.cuda.current_stream().cuda_stream)


class stream_scope:
    """While open, every launch of this package goes to the stream that was torch's current one
    when the scope was opened.  The model's forward pass opens one: nothing inside it changes the
    current stream (a graph capture changes it around the whole pass)."""

    def __enter__(self) -> None:
        global _scoped_stream
        self.previous = _scoped_stream
        _scoped_stream = c_void_p(torch.cuda.current_stream().cuda_stream)

    def __exit__(self, *exc) -> None:
        global _scoped_stream
        _scoped_stream = self.previous


class _Counter:
    """Kernel launches issued through this package's bindings since import."""

    launches = 0


def launch_count() -> int:
    return _Counter.launches


def _check(code: int, what: str) -> None:
    _Counter.launches += 1
    if code == 0:
        return
    if code in _ERRORS:
        raise KernelError(f"{what}: {_ERRORS[code]}")
    raise KernelError(f"{what}: CUDA error {code} ({_cuda_error_name(code)})")


def raise_on_device_error() -> None:
    """Ask the tensor-core and attention libraries that are loaded whether a kernel gave up a
    bounded wait since the last call, and raise if one did: what such a kernel wrote is invalid.
    Reads a flag from the device, so it waits for the work in flight."""
    for what, code in (("tensor-core product", tensor_core.take_error()), ("attention", attention_bf16.take_error())):
        if code:
            raise KernelError(
                f"a {what} kernel ran into the limit of a wait (code {code}): the results since the last check are invalid"
            )


def _cuda_error_name(code: int) -> str:
    try:
        runtime = ctypes.CDLL("libcudart.so")
        runtime.cudaGetErrorString.restype = ctypes.c_char_p
        return runtime.cudaGetErrorString(code).decode()
    except OSError:
        return "unknown"


def _need(tensor: torch.Tensor, dtype: torch.dtype | None, name: str) -> None:
    if not tensor.is_cuda:
        raise KernelError(f"{name} must be a CUDA tensor")
    if not tensor.is_contiguous():
        raise KernelError(f"{name} must be contiguous")
    if dtype is not None and tensor.dtype != dtype:
        raise KernelError(f"{name} must be {dtype}, got {tensor.dtype}")


_signatures_done: set[str] = set()


def _fn(library: str, name: str, argtypes: list[Any]):
    lib = load_library(library)
    fn = getattr(lib, name)
    if name not in _signatures_done:
        fn.argtypes = argtypes
        fn.restype = c_int
        _signatures_done.add(name)
    return fn


# ------------------------------------------------------------------------------ size rules


def check_attention_sizes(head_dim: int, heads: int, kv_heads: int) -> None:
    """Sizes that some attention kernel of this package takes; a clear error otherwise."""
    if head_dim < 16 or head_dim % 16 or head_dim > 512:
        raise ValueError(f"head_dim must be a multiple of 16 between 16 and 512, got {head_dim}")
    if heads < 1 or kv_heads < 1 or heads % kv_heads:
        raise ValueError(f"heads ({heads}) must be a positive multiple of kv_heads ({kv_heads})")


# ------------------------------------------------------------------------------ elementwise


def embedding(table: torch.Tensor, token_ids: torch.Tensor, out: torch.Tensor, multiplier: float = 1.0) -> None:
    """``out[t] = table[token_ids[t]] * multiplier`` widened to float32."""
    _need(table, None, "table"), _need(token_ids, torch.int32, "token_ids"), _need(out, torch.float32, "out")
    fn = _fn("elementwise", "me_embedding", [c_void_p, c_int, c_void_p, c_void_p, c_int, c_int, c_int, c_float, c_void_p])
    vocab, hidden = table.shape
    code = fn(_ptr(table), _type_code(table.dtype), _ptr(token_ids), _ptr(out), out.shape[0], hidden, vocab,
              float(multiplier), _stream())  # fmt: skip
    _check(code, "embedding")


def logits_finish(logits: torch.Tensor, bias: torch.Tensor | None, scale: float = 1.0, soft_cap: float = 0.0) -> None:
    """In place on float32 ``logits [N, vocab]``: ``y = x * scale + bias``, then ``soft_cap *
    tanh(y / soft_cap)`` when ``soft_cap > 0``."""
    _need(logits, torch.float32, "logits")
    if bias is not None:
        _need(bias, torch.float32, "bias")
        if bias.shape != (logits.shape[1],):
            raise KernelError("the bias must have one value per logit")
    fn = _fn("elementwise", "me_logits_finish", [c_void_p, c_void_p, c_float, c_float, c_int, c_int, c_void_p])
    code = fn(_ptr(logits), _ptr(bias) if bias is not None else None, float(scale), float(soft_cap),
              logits.shape[0], logits.shape[1], _stream())  # fmt: skip
    _check(code, "logits_finish")


def pick_tokens(tokens: torch.Tensor, rows: torch.Tensor, out: torch.Tensor) -> None:
    """``out[i] = tokens[rows[i]]``, all int32 on the device."""
    _need(tokens, torch.int32, "tokens"), _need(rows, torch.int32, "rows"), _need(out, torch.int32, "out")
    if rows.shape[0] != out.shape[0]:
        raise KernelError("one row index per output")
    fn = _fn("sampling", "me_pick_tokens", [c_void_p, c_void_p, c_void_p, c_int, c_void_p])
    _check(fn(_ptr(tokens), _ptr(rows), _ptr(out), out.shape[0], _stream()), "pick_tokens")


def add_rmsnorm(
    x: torch.Tensor,
    pending: torch.Tensor | None,
    weight: torch.Tensor,
    eps: float,
    out: torch.Tensor,
    rows: torch.Tensor | None = None,
) -> None:
    """``x += sum_s pending[s]`` (in place, float32) and ``out = weight * rmsnorm(x)``.

    With ``rows`` only ``x[rows]`` (+ pending) are normalised into ``out[0..len(rows))`` and
    ``x`` is not modified."""
    _need(x, torch.float32, "x"), _need(weight, torch.float32, "weight"), _need(out, None, "out")
    hidden = x.shape[-1]
    splits, stride = 0, 0
    if pending is not None:
        _need(pending, torch.float32, "pending")
        splits, stride = pending.shape[0], pending.stride(0)
        if pending.shape[1:] != x.shape:
            raise KernelError(f"pending {tuple(pending.shape)} does not fit x {tuple(x.shape)}")
    if weight.shape != (hidden,) or out.shape[-1] != hidden:
        raise KernelError("add_rmsnorm: weight/out width does not match x")
    count = x.shape[0] if rows is None else rows.shape[0]
    if rows is not None:
        _need(rows, torch.int32, "rows")
    fn = _fn(
        "elementwise",
        "me_add_rmsnorm",
        [c_void_p, c_void_p, c_int, c_longlong, c_void_p, c_float, c_void_p, c_int, c_void_p, c_int, c_int, c_void_p],
    )
    code = fn(
        _ptr(x), _ptr(pending), splits, stride, _ptr(weight), eps, _ptr(out), _type_code(out.dtype),
        _ptr(rows), count, hidden, _stream(),
    )  # fmt: skip
    _check(code, "add_rmsnorm")


def swiglu(partials: torch.Tensor, out: torch.Tensor) -> None:
    """``out = silu(gate) * up`` where gate/up are the halves of ``sum_s partials[s]``."""
    _need(partials, torch.float32, "partials"), _need(out, None, "out")
    splits, tokens, width = partials.shape
    inter = width // 2
    if out.shape != (tokens, inter):
        raise KernelError(f"swiglu: out {tuple(out.shape)} does not fit partials {tuple(partials.shape)}")
    fn = _fn("elementwise", "me_swiglu", [c_void_p, c_int, c_longlong, c_void_p, c_int, c_int, c_int, c_void_p])
    code = fn(_ptr(partials), splits, partials.stride(0), _ptr(out), _type_code(out.dtype), tokens, inter, _stream())
    _check(code, "swiglu")


def qk_norm_rope_store(
    *,
    qkv: torch.Tensor,
    heads: int,
    kv_heads: int,
    head_dim: int,
    q_weight: torch.Tensor | None,
    k_weight: torch.Tensor | None,
    eps: float,
    cos_sin: torch.Tensor | None,
    positions: torch.Tensor,
    q_out: torch.Tensor,
    page_size: int,
    slot_mapping: torch.Tensor | None = None,
    k_pages: torch.Tensor | None = None,
    v_pages: torch.Tensor | None = None,
    k_dense: torch.Tensor | None = None,
    v_dense: torch.Tensor | None = None,
    bias: torch.Tensor | None = None,
) -> None:
    """Per-head RMSNorm of q and k, rotation, and the write of k and v to their cache slots
    (or to dense ``[T, kv_heads * head_dim]`` buffers when ``slot_mapping`` is ``None``).
    ``qkv`` is ``[S, T, (heads + 2 * kv_heads) * head_dim]`` float32 partial sums; ``bias`` (float32,
    one value per column of ``qkv``) is added to their sum before anything else."""
    _need(qkv, torch.float32, "qkv"), _need(q_out, None, "q_out"), _need(positions, torch.int32, "positions")
    splits, tokens, width = qkv.shape
    if width != (heads + 2 * kv_heads) * head_dim:
        raise KernelError(f"qkv width {width} is not (heads + 2 kv_heads) * head_dim")
    if kv_heads and slot_mapping is None and (k_dense is None or v_dense is None):
        raise KernelError("either slot_mapping with pages or dense outputs must be given")
    if kv_heads and slot_mapping is not None:
        _need(slot_mapping, torch.int32, "slot_mapping")
        if k_pages is None or v_pages is None or k_pages.dtype != q_out.dtype:
            raise KernelError("pages must be given in the dtype of q_out")
        if k_pages.shape[1:] != (kv_heads, page_size, head_dim):
            raise KernelError(f"pages {tuple(k_pages.shape)} do not fit kv_heads/page_size/head_dim")
    rotary_dim = head_dim
    if cos_sin is not None:
        # a rotation of the first rotary_dim <= head_dim elements of every head; the rest pass through
        rotary_dim = 2 * cos_sin.shape[1] if cos_sin.dim() == 3 else -1
        if cos_sin.dim() != 3 or cos_sin.shape[0] != tokens or cos_sin.shape[2] != 2 or not 2 <= rotary_dim <= head_dim:
            raise KernelError(f"cos_sin {tuple(cos_sin.shape)} is not [tokens, rotary_dim / 2, 2] with rotary_dim <= head_dim")
    for w in (q_weight, k_weight, cos_sin, bias):
        if w is not None:
            _need(w, torch.float32, "weight/table")
    if bias is not None and bias.shape != (width,):
        raise KernelError(f"bias {tuple(bias.shape)} does not fit the {width} columns of qkv")
    fn = _fn(
        "elementwise",
        "me_qk_norm_rope_store",
        [c_void_p, c_int, c_longlong] + [c_void_p] * 2 + [c_float] + [c_void_p] * 8 + [c_int] * 7 + [c_void_p, c_void_p],
    )
    code = fn(
        _ptr(qkv), splits, qkv.stride(0), _ptr(q_weight), _ptr(k_weight), eps, _ptr(cos_sin), _ptr(positions),
        _ptr(slot_mapping if kv_heads else None), _ptr(q_out), _ptr(k_pages), _ptr(v_pages), _ptr(k_dense),
        _ptr(v_dense), _type_code(q_out.dtype), tokens, heads, kv_heads, head_dim, page_size, rotary_dim, _ptr(bias), _stream(),
    )  # fmt: skip
    _check(code, "qk_norm_rope_store")


def rope_table(inv_freq: torch.Tensor, positions: torch.Tensor, out: torch.Tensor) -> None:
    """``out[t, i] = (cos, sin)(positions[t] * inv_freq[i])`` in float32, ``[T, rotary_dim / 2, 2]``."""
    _need(inv_freq, torch.float32, "inv_freq"), _need(positions, torch.int32, "positions"), _need(out, torch.float32, "out")
    tokens, half = positions.shape[0], inv_freq.shape[0]
    if tuple(out.shape) != (tokens, half, 2):
        raise KernelError(f"rope_table: out {tuple(out.shape)} is not [{tokens}, {half}, 2]")
    fn = _fn("elementwise", "me_rope_table", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_void_p])
    _check(fn(_ptr(inv_freq), _ptr(positions), _ptr(out), tokens, half, _stream()), "rope_table")


def kv_store(k_dense, v_dense, slot_mapping, k_pages, v_pages, kv_heads: int, head_dim: int, page_size: int) -> None:
    """Dense new keys/values ``[T, kv_heads * head_dim]`` into their cache slots."""
    for name, t in (("k_dense", k_dense), ("v_dense", v_dense), ("k_pages", k_pages), ("v_pages", v_pages)):
        _need(t, k_dense.dtype, name)
    _need(slot_mapping, torch.int32, "slot_mapping")
    fn = _fn("elementwise", "me_kv_store", [c_void_p] * 5 + [c_int] * 5 + [c_void_p])
    code = fn(
        _ptr(k_dense), _ptr(v_dense), _ptr(slot_mapping), _ptr(k_pages), _ptr(v_pages), _type_code(k_dense.dtype),
        k_dense.shape[0], kv_heads, head_dim, page_size, _stream(),
    )  # fmt: skip
    _check(code, "kv_store")


# ----------------------------------------------------------------------------------- GEMMs


def gemm_simt(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor) -> None:
    """``out[T, N] (float32) = x[T, K] @ weight[N, K]^T`` on CUDA cores, ascending-k sums."""
    _need(x, weight.dtype, "x"), _need(weight, None, "weight"), _need(out, torch.float32, "out")
    tokens, inner = x.shape
    outs = weight.shape[0]
    if weight.shape[1] != inner or out.shape != (tokens, outs):
        raise KernelError(f"gemm_simt: shapes {tuple(x.shape)} x {tuple(weight.shape)} -> {tuple(out.shape)}")
    fn = _fn("gemm_simt", "me_gemm_simt", [c_void_p, c_void_p, c_void_p, c_int, c_int, c_int, c_int, c_void_p])
    code = fn(_ptr(x), _ptr(weight), _ptr(out), _type_code(x.dtype), tokens, outs, inner, _stream())
    _check(code, "gemm_simt")


def tensor_core_gemm_supports(outs: int, inner: int) -> bool:
    """TMA addresses rows whose pitch is a multiple of 16 bytes: ``inner % 8 == 0`` for
    bfloat16.  Other shapes take the CUDA-core kernel."""
    return tensor_core.supports(outs, inner)


def choose_splits(tokens: int, outs: int, inner: int, max_splits: int = 8) -> int:
    return tensor_core.choose_splits(tokens, outs, inner, max_splits)


def GemmPlan(weight: torch.Tensor, dual_rows: int | None = None):  # noqa: N802 - constructs a plan object
    return tensor_core.GemmPlan(weight, dual_rows)


def gemm_tensor_core(plan, x: torch.Tensor, out: torch.Tensor, splits: int) -> None:
    tensor_core.gemm(plan, x, out, splits)


def gemm_tensor_core_swiglu(plan, x: torch.Tensor, act: torch.Tensor) -> None:
    tensor_core.gemm_swiglu(plan, x, act)


# -------------------------------------------------------------------------------- attention


def paged_attention_generic(
    q, k_pages, v_pages, block_table, entry_of_token, positions, out, heads, kv_heads, head_dim, scale, window
) -> None:
    _need(q, None, "q"), _need(out, q.dtype, "out"), _need(k_pages, q.dtype, "k_pages"), _need(v_pages, q.dtype, "v_pages")
    _need(block_table, torch.int32, "block_table"), _need(entry_of_token, torch.int32, "entry_of_token")
    _need(positions, torch.int32, "positions")
    fn = _fn(
        "attention_generic",
        "me_paged_attention_generic",
        [c_void_p] * 7 + [c_int, c_float] + [c_int] * 7 + [c_void_p],
    )
    code = fn(
        _ptr(q), _ptr(k_pages), _ptr(v_pages), _ptr(block_table), _ptr(entry_of_token), _ptr(positions), _ptr(out),
        _type_code(q.dtype), scale, q.shape[0], heads, kv_heads, head_dim, k_pages.shape[2], block_table.shape[1],
        window, _stream(),
    )  # fmt: skip
    _check(code, "paged_attention_generic")


def paged_attention(
    *, q, k_pages, v_pages, block_table, ctx, out, heads: int, kv_heads: int, head_dim: int, scale: float, window: int
) -> None:
    """Causal attention of the batch's new tokens over their requests' cached keys (the new
    tokens' own keys are already in the cache).  Chooses the kernel by dtype and sizes."""
    if q.dtype == torch.bfloat16:
        if attention_bf16.supports(head_dim, heads, kv_heads):
            attention_bf16.paged_attention(
                q, k_pages, v_pages, block_table, ctx, out, heads, kv_heads, head_dim, scale, window
            )
            return
    paged_attention_generic(
        q, k_pages, v_pages, block_table, ctx.entry_of_token, ctx.positions, out, heads, kv_heads, head_dim,
        scale, window,
    )  # fmt: skip


# --------------------------------------------------------------------------------- sampling


def sample(logits: torch.Tensor, temperatures: torch.Tensor | None, uniforms: torch.Tensor | None, out: torch.Tensor) -> None:
    """Per row: argmax (lowest index among maxima) when its temperature is 0, else the token
    at which the cumulative distribution of ``softmax(logits / T)`` passes ``uniforms[row]``."""
    _need(logits, torch.float32, "logits"), _need(out, torch.int32, "out")
    rows, vocab = logits.shape
    if temperatures is not None:
        _need(temperatures, torch.float32, "temperatures"), _need(uniforms, torch.float32, "uniforms")
    fn = _fn("sampling", "me_sample", [c_void_p] * 4 + [c_int, c_int, c_void_p])
    code = fn(_ptr(logits), _ptr(temperatures), _ptr(uniforms), _ptr(out), rows, vocab, _stream())
    _check(code, "sample")


# The bindings of the tensor-core and attention libraries use this module's helpers and are used
# by its wrappers: they are imported last, when everything above exists.
from mini_engine_b200.csrc import attention_bf16, tensor_core  # noqa: E402
