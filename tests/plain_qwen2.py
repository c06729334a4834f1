"""A plain, slow implementation of the Qwen2 decoder for the tests to compare with.

Whole sequences, no cache, no batching, one function for each part.  It shares no
code with the package under test: it reads config.json and model.safetensors by
itself (the latter with the ``safetensors`` library) and works on host tensors.

It rests on the reference's formulas, each cited by file:line below.  The
reference's own model code is Rust and reads GGUF files only; neither a Rust
toolchain nor a GGUF model exists on the machines these tests run on, so the
whole model cannot be compared with a run of the reference.  What can be run is
the reference's CUDA port of the small operations of a layer
(crates/vipera-backend-gpu/src/layer.cu, "a straight port of the CPU function of
the same name"): ``tests/golden/make_reference_ops.py`` ran those kernels once on
seeded inputs, ``tests/golden/reference_ops.npz`` holds what they computed, and
``tests/test_golden.py`` holds ``rms_norm``, ``rope_angles`` + ``rope_neox``,
``attention`` and ``silu`` of this file to it (agreement to about 5e-7 of the
largest value).  Embedding, the products and their order are restatements of the
cited lines.

``dtype`` chooses the arithmetic (float64 by default, so that this side of a
comparison adds no rounding of its own).  Rotation angles are always computed in
32-bit as the reference does.  ``round_to`` names a storage dtype (bfloat16) whose
rounding is applied where a bfloat16 engine stores activations: the input of each
matrix product, keys and values in the cache, and the mixer's output.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional, Sequence, Tuple

import torch


# --------------------------------------------------------------------------------------
# configuration and weights
# --------------------------------------------------------------------------------------
def read_config(model_dir: str) -> dict:
    with open(os.path.join(model_dir, "config.json"), "r", encoding="utf-8") as handle:
        raw = json.load(handle)
    heads = raw["num_attention_heads"]
    config = {
        "layers": raw["num_hidden_layers"],
        "hidden": raw["hidden_size"],
        "heads": heads,
        "kv_heads": raw.get("num_key_value_heads", heads),
        "head_dim": raw.get("head_dim") or raw["hidden_size"] // heads,
        "ffn": raw["intermediate_size"],
        "vocab": raw["vocab_size"],
        # defaults as in crates/vipera-backend-cpu/src/model.rs:1397-1398
        "eps": raw.get("rms_norm_eps", 1e-6),
        "rope_base": raw.get("rope_theta", 10000.0),
        "tied": raw.get("tie_word_embeddings", False),
        "windows": [None] * raw["num_hidden_layers"],
    }
    if raw.get("use_sliding_window", False):
        first = raw.get("max_window_layers", config["layers"])
        for layer in range(first, config["layers"]):
            config["windows"][layer] = raw["sliding_window"]
    return config


def read_weights(model_dir: str) -> Dict[str, torch.Tensor]:
    from safetensors.torch import load_file

    return load_file(os.path.join(model_dir, "model.safetensors"))


def _rounded(x: torch.Tensor, round_to: Optional[torch.dtype]) -> torch.Tensor:
    return x if round_to is None else x.to(round_to).to(x.dtype)


# --------------------------------------------------------------------------------------
# parts
# --------------------------------------------------------------------------------------
def embedding(table: torch.Tensor, tokens: Sequence[int], dtype) -> torch.Tensor:
    """Row lookup without scaling (crates/vipera-backend-cpu/src/model.rs:956-966)."""
    index = torch.as_tensor(list(tokens), dtype=torch.long)
    if int(index.max()) >= table.shape[0] or int(index.min()) < 0:
        raise ValueError("token id outside the vocabulary")
    return table[index].to(dtype)


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """``x * (1/sqrt(mean(x^2) + eps)) * w``, in that order of multiplication
    (crates/vipera-backend-cpu/src/model.rs:4282-4288)."""
    mean = (x * x).sum(dim=-1, keepdim=True) / x.shape[-1]
    inverse = 1.0 / torch.sqrt(mean + eps)
    return x * inverse * weight.to(x.dtype)


def rope_angles(positions: Sequence[int], head_dim: int, base: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """``inv_i = 1/base^(2i/d)``, ``angle = position * inv_i``, all in 32-bit
    (crates/vipera-backend-cpu/src/model.rs:4204-4206).  Returns (sin, cos), each
    [tokens, head_dim/2]."""
    half = head_dim // 2
    index = torch.arange(half, dtype=torch.float32)
    exponent = 2.0 * index / torch.tensor(float(head_dim), dtype=torch.float32)
    inverse = 1.0 / torch.pow(torch.tensor(base, dtype=torch.float32), exponent)
    position = torch.as_tensor(list(positions), dtype=torch.float32)
    angle = position[:, None] * inverse[None, :]
    return torch.sin(angle), torch.cos(angle)


def rope_neox(x: torch.Tensor, sin: torch.Tensor, cos: torch.Tensor) -> torch.Tensor:
    """Rotate pairs ``(i, i + d/2)`` of every head: ``low*cos - high*sin`` and
    ``low*sin + high*cos`` (crates/vipera-backend-cpu/src/model.rs:4226-4251).
    ``x`` is [tokens, heads, head_dim]."""
    half = x.shape[-1] // 2
    low, high = x[..., :half], x[..., half:]
    s = sin.to(x.dtype)[:, None, :]
    c = cos.to(x.dtype)[:, None, :]
    return torch.cat([low * c - high * s, low * s + high * c], dim=-1)


def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, scale: Optional[float] = None,
              window: Optional[int] = None, first_position: int = 0) -> torch.Tensor:
    """Causal grouped-query attention by the definition
    (crates/vipera-backend-cpu/src/model.rs:1804-1859): query head ``h`` reads KV head
    ``h // group``; the score is ``(q . k) * scale`` with ``scale = 1/sqrt(d)`` applied
    after the dot; position ``p`` sees keys ``0..p``; weights are ``exp(s - max)`` over
    their sum; the output is the weighted sum of the values.

    ``q`` is [queries, heads, d]; ``k`` and ``v`` are [keys, kv_heads, d]; query ``t``
    stands at position ``first_position + t`` and key ``j`` at position ``j``.  With a
    ``window`` a query at ``p`` sees keys ``p - window + 1 .. p`` only.
    """
    queries, heads, d = q.shape
    keys, kv_heads, _ = k.shape
    group = heads // kv_heads
    if scale is None:
        scale = 1.0 / math.sqrt(d)
    out = torch.zeros_like(q)
    for head in range(heads):
        kv_head = head // group
        for t in range(queries):
            position = first_position + t
            start = 0 if window is None else max(0, position - window + 1)
            visible_k = k[start : position + 1, kv_head]
            visible_v = v[start : position + 1, kv_head]
            scores = (visible_k @ q[t, head]) * scale
            weights = torch.exp(scores - scores.max())
            weights = weights / weights.sum()
            out[t, head] = weights @ visible_v
    return out


def silu(x: torch.Tensor) -> torch.Tensor:
    """``x / (1 + exp(-x))`` (crates/vipera-backend-cpu/src/model.rs:4368-4370)."""
    return x / (1.0 + torch.exp(-x))


def swiglu(h: torch.Tensor, gate_w, up_w, down_w, round_to=None) -> torch.Tensor:
    """``down(up(h) * silu(gate(h)))`` without biases
    (crates/vipera-backend-cpu/src/model.rs:1154-1198)."""
    gate = h @ gate_w.to(h.dtype).T
    up = h @ up_w.to(h.dtype).T
    act = _rounded(up * silu(gate), round_to)
    return act @ down_w.to(h.dtype).T


# --------------------------------------------------------------------------------------
# the model
# --------------------------------------------------------------------------------------
def forward(config: dict, weights: Dict[str, torch.Tensor], tokens: Sequence[int], *,
            dtype=torch.float64, round_to: Optional[torch.dtype] = None,
            schedule: Optional[List[Tuple[int, int, bool]]] = None) -> torch.Tensor:
    """Logits [tokens, vocab] of one whole sequence, in the order of steps of
    crates/vipera-backend-cpu/src/model.rs:521-689: embedding; per layer norm,
    q/k/v products, bias, rotation of q and k, attention, output product and residual,
    norm, SwiGLU and residual; final norm; output product (the embedding matrix when
    the model has no ``lm_head.weight``, model.rs:425).

    ``schedule`` lists (layer, cache slot, writes) in execution order; by default
    every layer runs once with a cache slot of its own.
    """
    heads, kv_heads, d = config["heads"], config["kv_heads"], config["head_dim"]
    count = len(tokens)
    if schedule is None:
        schedule = [(layer, layer, True) for layer in range(config["layers"])]
    x = embedding(weights["model.embed_tokens.weight"], tokens, dtype)
    sin, cos = rope_angles(range(count), d, config["rope_base"])
    slots: Dict[int, Tuple[torch.Tensor, torch.Tensor]] = {}
    for layer, slot, writes in schedule:
        p = f"model.layers.{layer}."
        h = _rounded(rms_norm(x, weights[p + "input_layernorm.weight"], config["eps"]), round_to)

        def project(name):
            y = h @ weights[p + f"self_attn.{name}.weight"].to(dtype).T
            bias = weights.get(p + f"self_attn.{name}.bias")
            return y if bias is None else y + bias.to(dtype)

        q = rope_neox(project("q_proj").view(count, heads, d), sin, cos)
        if writes:
            k = rope_neox(project("k_proj").view(count, kv_heads, d), sin, cos)
            v = project("v_proj").view(count, kv_heads, d)
            slots[slot] = (_rounded(k, round_to), _rounded(v, round_to))
        k, v = slots[slot]
        q = _rounded(q, round_to)
        mixed = attention(q, k, v, window=config["windows"][layer])
        mixed = _rounded(mixed.reshape(count, heads * d), round_to)
        x = x + mixed @ weights[p + "self_attn.o_proj.weight"].to(dtype).T
        h = _rounded(rms_norm(x, weights[p + "post_attention_layernorm.weight"], config["eps"]), round_to)
        x = x + swiglu(h, weights[p + "mlp.gate_proj.weight"], weights[p + "mlp.up_proj.weight"],
                       weights[p + "mlp.down_proj.weight"], round_to)
    h = _rounded(rms_norm(x, weights["model.norm.weight"], config["eps"]), round_to)
    head = weights.get("lm_head.weight")
    if head is None:
        head = weights["model.embed_tokens.weight"]
    return h @ head.to(dtype).T


def greedy_continuation(config, weights, prompt: Sequence[int], steps: int, **kwargs) -> List[int]:
    """Greedy generation by recomputing the whole sequence for every token; ties go
    to the lowest id (crates/vipera-sampler/src/lib.rs:135-156)."""
    tokens = list(prompt)
    produced = []
    for _ in range(steps):
        logits = forward(config, weights, tokens, **kwargs)[-1]
        token = _argmax_lowest(logits)
        produced.append(token)
        tokens.append(token)
    return produced


def _argmax_lowest(logits: torch.Tensor) -> int:
    best = logits.max()
    return int(torch.nonzero(logits == best)[0])
