"""Arrangements of a layer's four parts.

``prenorm``: ``x += mixer(norm(x))``, then ``x += ffn(norm(x))`` — the order of
crates/vipera-backend-cpu/src/model.rs:977-1198.  The residual stream is 32-bit; mixers
and feed-forwards add into it themselves, so that the addition can be the ending of their
last product.
"""
from __future__ import annotations

from ..config.registry import BLOCKS, FEED_FORWARDS, MIXERS, NORMS
from .linear import NormedInput


class PreNormBlock:
    def __init__(self, layer_spec, tensors, dtype, device):
        self.spec = layer_spec
        build = lambda registry, part, name: registry.find(part.kind)(  # noqa: E731
            part.params, layer_spec.part_prefix(name), tensors, dtype, device)
        self.mixer_norm = build(NORMS, layer_spec.mixer_norm, "mixer_norm")
        self.mixer = build(MIXERS, layer_spec.mixer, "mixer")
        self.ffn_norm = build(NORMS, layer_spec.ffn_norm, "ffn_norm")
        self.ffn = build(FEED_FORWARDS, layer_spec.ffn, "ffn")
        self.hidden = None

    @classmethod
    def schema(cls, layer_spec):
        schema = {}
        for registry, part, name in (
            (NORMS, layer_spec.mixer_norm, "mixer_norm"),
            (MIXERS, layer_spec.mixer, "mixer"),
            (NORMS, layer_spec.ffn_norm, "ffn_norm"),
            (FEED_FORWARDS, layer_spec.ffn, "ffn"),
        ):
            schema.update(registry.find(part.kind).schema(part.params, layer_spec.part_prefix(name)))
        return schema

    def parts(self):
        return (self.mixer_norm, self.mixer, self.ffn_norm, self.ffn)

    def forward(self, ctx, residual, cache, writes_cache):
        # A part that sets ``takes_lazy_input`` receives the normalised input as a NormedInput
        # and may fuse the norm into its first product; any other part receives a tensor.
        h = NormedInput(ctx, self.mixer_norm, residual)
        self.mixer.forward(ctx, h if getattr(self.mixer, "takes_lazy_input", False) else h.tensor(),
                           residual, cache, writes_cache)
        h = NormedInput(ctx, self.ffn_norm, residual)
        self.ffn.forward(ctx, h if getattr(self.ffn, "takes_lazy_input", False) else h.tensor(), residual)


BLOCKS.register("prenorm", PreNormBlock)
