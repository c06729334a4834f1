"""Arrangements of a layer's parts.

An arrangement declares its roles: which named parts it reads from the layer's description
and which registry each comes from.  ``Block`` builds them, so a new arrangement (four norms
around the two sub-layers, a mixer beside the feed-forward, one norm only) is a subclass
that names its roles and writes ``forward``; nothing else changes.

``prenorm``: ``x += mixer(norm(x))``, then ``x += ffn(norm(x))`` — the order of
crates/vipera-backend-cpu/src/model.rs:977-1198.  The residual stream is 32-bit; mixers
and feed-forwards add into it themselves, so that the addition can be the ending of their
last product.
"""
from __future__ import annotations

from typing import Dict

from ..config.registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS, Registry
from .linear import NormedInput


class Block:
    """Base of all arrangements.  ``roles`` maps a role's name to the registry its part is
    looked up in; the built parts are attributes of the same names.  ``cache_role`` names the
    role whose part says what the layer keeps between steps (``cache_request()``); the layer's
    cache slot is handed to ``forward`` and the arrangement passes it on to that part."""

    roles: Dict[str, Registry] = {}
    cache_role = "mixer"

    def __init__(self, layer_spec, tensors, dtype, device):
        self.spec = layer_spec
        self.params = layer_spec.params
        self._parts = {}
        for role, registry in self.roles.items():
            part_spec = self._role_spec(layer_spec, role)
            part = registry.find(part_spec.kind)(part_spec.params, layer_spec.part_prefix(role), tensors, dtype, device)
            setattr(self, role, part)
            self._parts[role] = part

    @classmethod
    def _role_spec(cls, layer_spec, role):
        from ..errors import InvalidArgumentError

        try:
            return layer_spec.parts[role]
        except KeyError:
            raise InvalidArgumentError(
                f"the {layer_spec.block!r} arrangement needs a part for the role {role!r}; "
                f"layer {layer_spec.prefix} gives {sorted(layer_spec.parts)}") from None

    @classmethod
    def schema(cls, layer_spec):
        schema = {}
        for role, registry in cls.roles.items():
            part_spec = cls._role_spec(layer_spec, role)
            schema.update(registry.find(part_spec.kind).schema(part_spec.params, layer_spec.part_prefix(role)))
        return schema

    def parts(self):
        return tuple(self._parts.values())

    def cache_request(self):
        """What this layer keeps between steps: PagedKV, FixedState or None."""
        part = self._parts.get(self.cache_role)
        return None if part is None else part.cache_request()

    @classmethod
    def cache_request_for(cls, layer_spec):
        """The same from the description alone (no weights): for memory plans."""
        if cls.cache_role not in cls.roles:
            return None
        part_spec = cls._role_spec(layer_spec, cls.cache_role)
        return cls.roles[cls.cache_role].find(part_spec.kind).cache_request_for(part_spec.params)

    @classmethod
    def workspace_bytes(cls, layer_spec, tokens, element_bytes):
        """Workspace of one execution of the layer in a step of `tokens` tokens: what its parts
        ask for, together (their buffers have names of their own and live side by side)."""
        total = 0
        for role, registry in cls.roles.items():
            part_spec = cls._role_spec(layer_spec, role)
            total += registry.find(part_spec.kind).workspace_bytes(part_spec.params, tokens, element_bytes)
        return total

    def forward(self, ctx, residual, cache, writes_cache):
        raise NotImplementedError

    @staticmethod
    def _input(part, normed: NormedInput):
        """A part that sets ``takes_lazy_input`` receives the normalised input as a NormedInput
        and may fuse the norm into its first product; any other part receives a tensor."""
        return normed if getattr(part, "takes_lazy_input", False) else normed.tensor()


class PreNormBlock(Block):
    roles = {"mixer_norm": NORMS, "mixer": MIXERS, "ffn_norm": NORMS, "ffn": FEED_FORWARDS}

    def forward(self, ctx, residual, cache, writes_cache):
        h = NormedInput(ctx, self.mixer_norm, residual)
        self.mixer.forward(ctx, self._input(self.mixer, h), residual, cache, writes_cache)
        h = NormedInput(ctx, self.ffn_norm, residual)
        self.ffn.forward(ctx, self._input(self.ffn, h), residual)


BLOCKS.register("prenorm", PreNormBlock)
