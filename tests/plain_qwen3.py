"""Plain, slow Qwen3-dense forward pass: whole sequences, no cache, no batching.

This is the oracle that the engine is compared with.  It shares no code with the
product package: it reads ``config.json`` itself, takes weights as a dict of tensors keyed
by checkpoint name, and is one small function per part.  Every function cites the file
and lines of YuvGev00/mini-engine whose formula it restates (paths are relative to that
project's root).

Precision: ``compute`` is the dtype that matrices and activations are held in (float32
or float64); statistics that the reference computes in 32-bit are computed in ``compute``
here, which for float32 is the reference's own arithmetic and for float64 is an error-free
yardstick.
"""

from __future__ import annotations

import json
from pathlib import Path

import torch


# ------------------------------------------------------------------------- configuration


def read_config(folder: str | Path) -> dict:
    """The numbers of ``config.json`` that the formulas below need.

    Defaults follow src/mini_engine/model.py:35-56: ``head_dim`` defaults to
    ``hidden_size // num_attention_heads`` (:51), ``rope_theta`` comes from
    ``rope_parameters.rope_theta``, else the top-level key, else 10000.0 (:53).
    """
    raw = json.loads((Path(folder) / "config.json").read_text())
    rope = raw.get("rope_parameters") or {}
    heads = raw["num_attention_heads"]
    return {
        "vocab": raw["vocab_size"],
        "hidden": raw["hidden_size"],
        "inter": raw["intermediate_size"],
        "layers": raw["num_hidden_layers"],
        "heads": heads,
        "kv_heads": raw["num_key_value_heads"],
        "head_dim": raw.get("head_dim") or raw["hidden_size"] // heads,
        "eps": raw["rms_norm_eps"],
        "theta": float(rope.get("rope_theta", raw.get("rope_theta", 10000.0))),
        "tied": bool(raw.get("tie_word_embeddings", False)),
    }


# --------------------------------------------------------------------------------- parts


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``w * (x * rsqrt(mean(x^2) + eps))`` over the last axis.

    src/mini_engine/model.py:65-69: statistics in 32-bit, eps inside the root and added
    to the mean, no bias, the weight multiplies the normalised value directly (no 1+w).
    """
    variance = x.pow(2).mean(-1, keepdim=True)
    return weight * (x * torch.rsqrt(variance + eps))


def rope_angles(positions: torch.Tensor, head_dim: int, theta: float, compute: torch.dtype):
    """cos and sin tables ``[T, head_dim]`` for absolute positions.

    src/mini_engine/model.py:75: ``inv_freq[i] = 1 / theta**(2i/d)`` built in float32;
    :81-83: ``angle = pos * inv_freq``, the half-table is repeated twice along the last
    axis.  The frequencies are formed in float32 exactly as there, so that a float32 run
    sees the same table; only the trigonometry is done in ``compute``.
    """
    inv_freq = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32) / head_dim))
    freqs = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    angles = torch.cat((freqs, freqs), dim=-1).to(compute)
    return angles.cos(), angles.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half convention on ``x [T, heads, d]``: ``x*cos + cat(-x2, x1)*sin``.

    src/mini_engine/model.py:86-90; applied to the whole head (no partial rotary).
    """
    half = x.shape[-1] // 2
    x1, x2 = x[..., :half], x[..., half:]
    rotated = torch.cat((-x2, x1), dim=-1)
    return x * cos[:, None, :] + rotated * sin[:, None, :]


def causal_attention(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, window: int | None = None
) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence.

    ``q [T, heads, d]``, ``k, v [T, kv_heads, d]`` -> ``[T, heads, d]``.
    src/mini_engine/attention.py:160-175: query head ``h`` reads KV head ``h // g`` with
    ``g = heads / kv_heads`` (:163), scores are scaled by ``d**-0.5`` (:170), masked
    positions get -inf and the softmax runs over the keys; :84-86: the query at position
    ``p`` sees keys at positions ``<= p``.  ``window`` (not used by Qwen3 dense, whose
    layers are all full attention, src/mini_engine/model.py:42-43) further restricts a query
    to the last ``window`` keys, itself included.
    """
    t, heads, d = q.shape
    kv_heads = k.shape[1]
    group = heads // kv_heads
    out = torch.empty_like(q)
    pos = torch.arange(t)
    allowed = pos[None, :] <= pos[:, None]
    if window is not None:
        allowed &= pos[None, :] > pos[:, None] - window
    for h in range(heads):
        kh = h // group
        scores = (q[:, h, :] @ k[:, kh, :].T) * (d**-0.5)
        scores = scores.masked_fill(~allowed, float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        out[:, h, :] = probs @ v[:, kh, :]
    return out


def attention_block(x: torch.Tensor, w: dict, prefix: str, cfg: dict, positions: torch.Tensor):
    """Projections, per-head q/k norm, RoPE, attention, output projection.

    src/mini_engine/model.py:113-118: q and k are normalised per head over ``head_dim``
    with one weight shared by all heads (:101-103), *before* the rotation (:116); v is
    neither normalised nor rotated; no projection has a bias (:97-100).
    """
    t = x.shape[0]
    d = cfg["head_dim"]
    q = (x @ w[prefix + "q_proj.weight"].T).view(t, cfg["heads"], d)
    k = (x @ w[prefix + "k_proj.weight"].T).view(t, cfg["kv_heads"], d)
    v = (x @ w[prefix + "v_proj.weight"].T).view(t, cfg["kv_heads"], d)
    q = rms_norm(q, w[prefix + "q_norm.weight"], cfg["eps"])
    k = rms_norm(k, w[prefix + "k_norm.weight"], cfg["eps"])
    cos, sin = rope_angles(positions, d, cfg["theta"], x.dtype)
    q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
    out = causal_attention(q, k, v, cfg.get("window"))
    return out.reshape(t, -1) @ w[prefix + "o_proj.weight"].T


def swiglu_mlp(x: torch.Tensor, w: dict, prefix: str) -> torch.Tensor:
    """``down(silu(gate(x)) * up(x))`` with ``silu(a) = a * sigmoid(a)``, no biases.

    src/mini_engine/model.py:122-131.
    """
    gate = x @ w[prefix + "gate_proj.weight"].T
    up = x @ w[prefix + "up_proj.weight"].T
    return ((gate * torch.sigmoid(gate)) * up) @ w[prefix + "down_proj.weight"].T


def decoder_layer(x: torch.Tensor, w: dict, index: int, cfg: dict, positions: torch.Tensor):
    """Pre-norm residual layer: ``h = x + attn(norm(x))``, ``y = h + mlp(norm(h))``.

    src/mini_engine/model.py:149-150.
    """
    p = f"model.layers.{index}."
    h = x + attention_block(
        rms_norm(x, w[p + "input_layernorm.weight"], cfg["eps"]), w, p + "self_attn.", cfg, positions
    )
    return h + swiglu_mlp(rms_norm(h, w[p + "post_attention_layernorm.weight"], cfg["eps"]), w, p + "mlp.")


# --------------------------------------------------------------------------- whole model


def forward_logits(
    weights: dict, cfg: dict, token_ids: list[int], compute: torch.dtype = torch.float32
) -> torch.Tensor:
    """Logits ``[T, vocab]`` at every position of one whole sequence.

    src/mini_engine/model.py:182-187: embedding lookup without scaling, the layers in
    order, the final norm, the LM head without bias; the head is the embedding matrix when
    the embeddings are tied (:169-170).  Positions are 0..T-1
    (src/mini_engine/engine.py:207-209).
    """
    w = {name: t.to(compute) for name, t in weights.items()}
    ids = torch.tensor(token_ids, dtype=torch.long)
    positions = torch.arange(len(token_ids))
    x = w["model.embed_tokens.weight"][ids]
    for index in range(cfg["layers"]):
        x = decoder_layer(x, w, index, cfg, positions)
    x = rms_norm(x, w["model.norm.weight"], cfg["eps"])
    head = w["model.embed_tokens.weight"] if cfg["tied"] else w["lm_head.weight"]
    return x @ head.T


def greedy_generate(weights: dict, cfg: dict, prompt: list[int], steps: int, compute=torch.float32):
    """Greedy continuation by re-running the whole sequence for every new token.

    Returns the new tokens and, for each, the gap between the two largest logits, so that a
    caller can tell a near-tie (rounding) from a real difference
    (the method of benchmarks/gpu_divergence.py:55-65).
    """
    ids = list(prompt)
    tokens: list[int] = []
    gaps: list[float] = []
    for _ in range(steps):
        last = forward_logits(weights, cfg, ids, compute)[-1]
        top = torch.topk(last, 2)
        tokens.append(int(top.indices[0]))
        gaps.append(float(top.values[0] - top.values[1]))
        ids.append(tokens[-1])
    return tokens, gaps


def sample_from_logits(logits: torch.Tensor, temperature: float, uniform: float) -> int:
    """Token for one row of logits given a uniform number in [0, 1).

    src/mini_engine/engine.py:282-291: temperature 0 is argmax (lowest index among equal
    maxima); otherwise ``softmax(logits / max(T, 1e-5))`` in 32-bit and one draw from it.
    The reference draws with ``torch.multinomial``; here the draw is the inverse of the
    cumulative distribution at ``uniform``, which is the same distribution.
    """
    if temperature == 0:
        return int(torch.argmax(logits))
    probs = torch.softmax(logits.double() / max(temperature, 1e-5), dim=-1)
    cdf = torch.cumsum(probs, dim=-1)
    index = int(torch.searchsorted(cdf, torch.tensor(uniform * float(cdf[-1]), dtype=cdf.dtype), right=True))
    return min(index, logits.numel() - 1)


def kv_bytes_per_token(cfg: dict, element_size: int) -> int:
    """``2 * layers * kv_heads * head_dim * element_size`` (src/mini_engine/engine.py:54-56)."""
    return 2 * cfg["layers"] * cfg["kv_heads"] * cfg["head_dim"] * element_size
