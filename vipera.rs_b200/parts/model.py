"""The decoder as a whole: embedding, blocks in schedule order, final norm, output matrix.

Order of a forward pass as in crates/vipera-backend-cpu/src/model.rs:883-1252: embedding
rows into a 32-bit residual stream, the layers, then the final norm and the output product
only for the rows whose logits are wanted (model.rs:1201-1250); the output matrix is the
embedding matrix when the model has none of its own (model.rs:425).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..config.registry import BLOCKS, NORMS
from ..config.spec import ModelSpec
from ..errors import InternalError, InvalidArgumentError
from ..kernels import ops
from ..weights import Schema, TensorSpec, WeightSource, check_source, to_run_dtype
from .base import StepContext
from .linear import Linear, NormedInput


def model_schema(spec: ModelSpec) -> Schema:
    """Every tensor the model reads, by name."""
    schema: Schema = {spec.embedding_name: TensorSpec((spec.vocab_size, spec.hidden_size), init="embedding")}
    for layer in spec.layers:
        schema.update(BLOCKS.find(layer.block).schema(layer))
    schema.update(NORMS.find(spec.final_norm.kind).schema(spec.final_norm.params, spec.final_norm_name))
    if spec.head_name is not None:
        schema[spec.head_name] = TensorSpec((spec.vocab_size, spec.hidden_size))
    return schema


class DecoderModel:
    def __init__(self, spec: ModelSpec, source: WeightSource, dtype: torch.dtype, device):
        spec.validate()
        if dtype not in (torch.float32, torch.bfloat16):
            raise InvalidArgumentError(f"the engine runs in float32 or bfloat16, not {dtype}")
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        if self.device.type != "cuda" or not torch.cuda.is_available():
            raise InternalError(f"no CUDA device for {device!r}: this engine has no CPU path")
        schema = model_schema(spec)
        check_source(schema, source)

        def fetch(names):
            return {name: to_run_dtype(source.get(name), dtype) for name in names}

        embedding = fetch([spec.embedding_name])[spec.embedding_name]
        self.embedding = embedding.to(device=self.device, dtype=dtype).contiguous()
        self.blocks = []
        for layer in spec.layers:
            block_cls = BLOCKS.find(layer.block)
            tensors = fetch(block_cls.schema(layer))
            self.blocks.append(block_cls(layer, tensors, dtype, self.device))
        norm_cls = NORMS.find(spec.final_norm.kind)
        self.final_norm = norm_cls(spec.final_norm.params, spec.final_norm_name,
                                   fetch(norm_cls.schema(spec.final_norm.params, spec.final_norm_name)),
                                   dtype, self.device)
        if spec.head_name is None:
            self.head = Linear(self.embedding, dtype, self.device)
        else:
            self.head = Linear(fetch([spec.head_name])[spec.head_name], dtype, self.device)
        # What each cache slot has to hold, asked of the mixer that writes it.
        self.cache_requests: Dict[int, object] = {}
        for entry in spec.schedule:
            if entry.writes_cache:
                self.cache_requests[entry.cache] = self.blocks[entry.layer].cache_request()

    def prepare(self, max_positions: int) -> None:
        """Tell every part that sizes something by position (tables of a position encoding)
        how far the engine goes: positions below `max_positions`."""
        for block in self.blocks:
            for part in block.parts():
                prepare = getattr(part, "prepare", None)
                if prepare is not None:
                    prepare(max_positions)

    @property
    def graph_safe(self) -> bool:
        """Whether decode steps of this model may be captured in CUDA graphs: every part must
        launch device work only, and no mixer may keep per-request state (padding a graph's
        batch with copies of an entry would update such a state twice)."""
        from .base import FixedState

        for block in self.blocks:
            for part in block.parts():
                if not getattr(part, "graph_safe", True):
                    return False
        return not any(isinstance(request, FixedState) for request in self.cache_requests.values())

    def kernel_families(self) -> List[str]:
        names = ["rowwise", *self.head.kernel_families()]
        for block in self.blocks:
            for part in block.parts():
                names.extend(part.kernel_families())
        names.extend(self.final_norm.kernel_families())
        return list(dict.fromkeys(names))

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        tensors = [self.embedding, self.head.weight]
        for block in self.blocks:
            for part in block.parts():
                for value in vars(part).values():
                    if isinstance(value, Linear):
                        tensors.append(value.weight)
        for tensor in tensors:
            if tensor.data_ptr() not in seen:
                seen.add(tensor.data_ptr())
                total += tensor.numel() * tensor.element_size()
        return total

    def forward(self, ctx: StepContext, caches: Dict[int, object]) -> Optional[torch.Tensor]:
        """Run the step's tokens through every scheduled layer; float32 logits
        [wanted rows, vocab], or None when no row is wanted."""
        ws = ctx.workspace
        residual = ws.get("model.residual", (ctx.num_tokens, self.spec.hidden_size), torch.float32)
        ops.embed(self.embedding, ctx.tokens, residual, self.spec.embedding_scale)
        for entry in self.spec.schedule:
            self.blocks[entry.layer].forward(ctx, residual, caches.get(entry.cache), entry.writes_cache)
        if ctx.num_logit_rows == 0:
            return None
        h = NormedInput(ctx, self.final_norm, residual, rows=ctx.logit_rows, num_rows=ctx.num_logit_rows,
                        name="model.final")
        logits = ws.get("model.logits", (ctx.num_logit_rows, self.spec.vocab_size), torch.float32)
        self.head(ctx, h, epilogue=ops.EPI_STORE, out=logits)
        if self.spec.logit_scale != 1.0:
            logits.mul_(self.spec.logit_scale)
        return logits
