"""Architecture-neutral description of a decoder: what the builder turns into parts.

An architecture's typed configuration (for instance ``Qwen2Config``) is turned
into a ``ModelSpec`` by that architecture's own function.  From there on nothing
knows the architecture's name: the builder looks up each ``PartSpec.kind`` in the
part registries and hands it ``PartSpec.params``.

The reference keeps one ``Layer`` struct with optional members
(crates/vipera-backend-cpu/src/model.rs:303-318); here the same idea is data, so
that layers of one model may differ and the order of execution is a list.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional


@dataclass(frozen=True)
class PartSpec:
    """One part: its registered kind and every size and constant it needs."""

    kind: str
    params: Dict[str, Any] = field(default_factory=dict)


@dataclass(frozen=True)
class LayerSpec:
    """One block of the decoder: an arrangement and the parts it arranges, by role.

    ``block`` names the arrangement (a key of the block registry).  ``parts`` maps a role to
    a part; which roles there are, and which kind of part fills each, is the arrangement's
    business: ``prenorm`` reads ``mixer_norm``, ``mixer``, ``ffn_norm`` and ``ffn``; an
    arrangement with four norms, or with a mixer beside the feed-forward, reads others.
    ``params`` holds constants of the arrangement itself (a residual scale, say).
    ``prefix`` is the tensor-name prefix of this layer in the weight file
    (``model.layers.3``) and ``names`` the sub-prefix of each role under it
    (``input_layernorm``, ``self_attn``, ...; a role not listed uses its own name); each
    part appends its own tensor names.
    """

    block: str
    prefix: str
    parts: Dict[str, PartSpec]
    names: Dict[str, str] = field(default_factory=dict)
    params: Dict[str, Any] = field(default_factory=dict)

    def part_prefix(self, role: str) -> str:
        return f"{self.prefix}.{self.names.get(role, role)}"

    def with_parts(self, **changes: PartSpec) -> "LayerSpec":
        """This layer with some roles filled by other parts."""
        return LayerSpec(self.block, self.prefix, {**self.parts, **changes}, dict(self.names), dict(self.params))


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.

    ``layer`` indexes ``ModelSpec.layers`` (the weights that run).  ``cache``
    names the cache slot the mixer uses: entries with the same ``cache`` share
    keys and values.  ``writes_cache`` is false for an entry that only reads a
    slot another entry filled earlier in the same step.
    """

    layer: int
    cache: int
    writes_cache: bool = True


@dataclass(frozen=True)
class ModelSpec:
    """Everything the builder needs; no size is implied by code."""

    architecture: str
    vocab_size: int
    hidden_size: int
    max_position_embeddings: int
    embedding_name: str
    layers: List[LayerSpec]
    schedule: List[ScheduleEntry]
    final_norm: PartSpec
    final_norm_name: str
    head_name: Optional[str]  # None: the embedding matrix is the output matrix
    logit_scale: float = 1.0      # logits are multiplied by this
    embedding_scale: float = 1.0  # embedding rows are multiplied by this on their way into the residual stream

    def validate(self) -> None:
        from ..errors import InvalidArgumentError

        if not self.layers:
            raise InvalidArgumentError("a model needs at least one layer")
        slots_written = set()
        for position, entry in enumerate(self.schedule):
            if not 0 <= entry.layer < len(self.layers):
                raise InvalidArgumentError(
                    f"schedule entry {position} names layer {entry.layer}, "
                    f"but the model has {len(self.layers)} layers"
                )
            if entry.writes_cache:
                if entry.cache in slots_written:
                    raise InvalidArgumentError(
                        f"schedule entry {position} writes cache slot {entry.cache}, "
                        "which an earlier entry already writes"
                    )
                slots_written.add(entry.cache)
            elif entry.cache not in slots_written:
                raise InvalidArgumentError(
                    f"schedule entry {position} reads cache slot {entry.cache} "
                    "before any entry has written it"
                )
