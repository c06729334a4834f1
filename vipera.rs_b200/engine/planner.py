"""Memory plan of a model from its description: weights, cache, workspace against the device.

The reference plans before it loads (crates/vipera-core/src/planner.rs:224-263 for the sums,
:276-430 for ``feasible`` and ``violations``; bins/vipera/src/main.rs:186-251 prints the plan
and exits with 3 when it is infeasible).  Here the sums are asked of the architecture-neutral
description and of the parts' classes, so that a plan for another architecture needs no change:
weights from the tensor schema, cache bytes from what every scheduled layer says it keeps
between steps, workspace from what every part says it asks for in a step.
"""
from __future__ import annotations

from typing import Dict, Optional

from ..cache.pools import plan_groups
from ..config.registry import BLOCKS
from ..config.spec import ModelSpec
from ..parts.model import model_schema

DEVICE_RESERVE_BYTES = 16 << 20  # kept free on the device (crates/vipera-core/src/planner.rs:23)
PLANNED_STEP_TOKENS = 2048       # the step the workspace is sized for
PRODUCT_SCRATCH_BYTES = 32 << 20  # partial sums of split products (the buffer starts at this size)


def _element_bytes(dtype: str) -> int:
    return 4 if str(dtype).replace("torch.", "") in ("float32", "fp32", "f32") else 2


def spec_cache_requests(spec: ModelSpec) -> Dict[int, object]:
    """What every cache slot of the schedule has to hold, from the description alone."""
    requests = {}
    for entry in spec.schedule:
        if entry.writes_cache:
            layer = spec.layers[entry.layer]
            requests[entry.cache] = BLOCKS.find(layer.block).cache_request_for(layer)
    return requests


def weight_bytes(spec: ModelSpec, element_bytes: int) -> int:
    """Bytes of all tensors of the schema as the engine keeps them: tensors that follow the
    run's type in `element_bytes`, 32-bit tensors and integer tables in 4."""
    total = 0
    for tensor in model_schema(spec).values():
        count = 1
        for extent in tensor.shape:
            count *= int(extent)
        total += count * (element_bytes if tensor.store == "model" else 4)
    return total


def parameter_count(spec: ModelSpec) -> int:
    total = 0
    for tensor in model_schema(spec).values():
        count = 1
        for extent in tensor.shape:
            count *= int(extent)
        total += count
    return total


def cache_bytes(spec: ModelSpec, ctx: int, batch: int, element_bytes: int, page_size: int = 16) -> int:
    """Pages for `batch` requests of `ctx` tokens in every group of layers (a windowed group
    holds a window and a page's slack per request), and the fixed-size states."""
    groups, states = plan_groups(spec_cache_requests(spec))
    total = 0
    for group in groups:
        tokens = ctx if not group.window else min(ctx, group.window + page_size)
        pages = -(-tokens // page_size)
        total += batch * pages * page_size * group.bytes_per_token(element_bytes)
    for state in states.values():
        count = 1
        for extent in state.shape:
            count *= int(extent)
        total += batch * count * state.dtype.itemsize
    return total


def kv_bytes_per_token(spec: ModelSpec, element_bytes: int) -> int:
    groups, _ = plan_groups(spec_cache_requests(spec))
    return sum(group.bytes_per_token(element_bytes) for group in groups)


def workspace_bytes(spec: ModelSpec, batch: int, element_bytes: int, tokens: int = PLANNED_STEP_TOKENS) -> int:
    """The 32-bit residual stream, the normalised input, the most any layer asks for (layers
    share their buffers), the products' scratch for partial sums, and the 32-bit logits rows of
    a batch."""
    layers = max(BLOCKS.find(layer.block).workspace_bytes(layer, tokens, element_bytes) for layer in spec.layers)
    return (tokens * spec.hidden_size * (4 + element_bytes) + layers + PRODUCT_SCRATCH_BYTES
            + batch * spec.vocab_size * 4)


def plan_memory(spec: ModelSpec, ctx: int, batch: int, dtype: str, device_bytes: Optional[int] = None,
                page_size: int = 16) -> dict:
    """Weights + cache + workspace against the device's memory; what does not fit is listed in
    ``violations``, and ``feasible`` says whether the list is empty."""
    element = _element_bytes(dtype)
    weights = weight_bytes(spec, element)
    kv = cache_bytes(spec, ctx, batch, element, page_size)
    workspace = workspace_bytes(spec, batch, element)
    if device_bytes is None:
        try:
            import torch

            device_bytes = torch.cuda.get_device_properties(0).total_memory if torch.cuda.is_available() else None
        except Exception:
            device_bytes = None
    if device_bytes is None:
        device_bytes = 180 * 10**9  # one B200
    required = weights + kv + workspace + DEVICE_RESERVE_BYTES
    violations = []
    if ctx > spec.max_position_embeddings:
        violations.append({"constraint": "context_limit", "required": ctx,
                           "available": spec.max_position_embeddings,
                           "message": f"ctx {ctx} exceeds the model's limit of {spec.max_position_embeddings}"})
    if required > device_bytes:
        violations.append({"constraint": "device_memory", "required_bytes": required,
                           "available_bytes": device_bytes,
                           "message": f"{required} bytes needed, {device_bytes} on the device"})
    return {"architecture": spec.architecture, "ctx": ctx, "batch_size": batch, "dtype": dtype,
            "weight_bytes": weights, "kv_bytes": kv, "kv_bytes_per_token": kv_bytes_per_token(spec, element),
            "workspace_bytes": workspace, "reserve_bytes": DEVICE_RESERVE_BYTES,
            "predicted_device_bytes": required, "device_bytes": int(device_bytes),
            "feasible": not violations, "violations": violations}
