"""Decode steps of few tokens as one persistent kernel.

A model qualifies when every scheduled layer is the pre-norm arrangement of RMSNorm,
grouped-query attention with rotary pairs (or no encoding) over paged keys and values, and
SwiGLU, in bfloat16, with sizes the kernel takes.  Anything else (a mixer with state of its
own, another feed-forward, a position encoding the kernel does not know, 32-bit runs, more
than 16 tokens) runs part by part as before; the parts themselves know nothing of this file.

The description handed to the kernel holds device addresses (weights, cache pools, block
tables, workspace buffers), so one is built per distinct set of addresses and kept: a
captured CUDA graph always sees the same one.
"""
from __future__ import annotations

import os
from typing import Dict, Optional

import torch

from ..kernels import ops
from ..parts.attention import GQAttention
from ..parts.base import PagedKVView
from ..parts.block import PreNormBlock
from ..parts.mlp import SwiGLU
from ..parts.norm import RMSNorm


def _enabled() -> bool:
    return os.environ.get("VIPERA_FUSED_DECODE", "0") == "1"


class FusedDecode:
    MAX_KEPT = 32

    def __init__(self, model):
        self.model = model
        self._kept: Dict[tuple, tuple] = {}
        self._barrier = None
        self._maps = None
        self.trace = None  # profiling: an int64 tensor [blocks, 2 + 12 * layers] that receives timestamps
        layers = [model.blocks[entry.layer] for entry in model.spec.schedule]
        self.head_dim = layers[0].mixer.head_dim
        self.max_heads = max(block.mixer.num_heads for block in layers)
        self.max_kv_heads = max(block.mixer.num_kv_heads for block in layers)
        self.max_inter = max(block.ffn.inter for block in layers)

    # ------------------------------------------------------------------------------
    @staticmethod
    def qualifies(model) -> bool:
        """Whether the model's parts are the ones the kernel computes (no kernel is asked)."""
        if not _enabled() or model.dtype != torch.bfloat16 or not model.spec.schedule:
            return False
        if type(model.final_norm) is not RMSNorm:
            return False
        hidden = model.spec.hidden_size
        if hidden % 64:
            return False
        head_dim = None
        for entry in model.spec.schedule:
            block = model.blocks[entry.layer]
            if type(block) is not PreNormBlock:
                return False
            if not (type(block.mixer_norm) is RMSNorm and type(block.ffn_norm) is RMSNorm):
                return False
            mixer, ffn = block.mixer, block.ffn
            if type(mixer) is not GQAttention or type(ffn) is not SwiGLU:
                return False
            if mixer.position.style not in (ops.ROPE_NONE, ops.ROPE_NEOX):
                return False
            if head_dim is None:
                head_dim = mixer.head_dim
            if mixer.head_dim != head_dim or head_dim not in ops.FUSED_HEAD_DIMS:
                return False
            if mixer.num_heads // mixer.num_kv_heads > 16 or mixer.hidden != hidden or ffn.hidden != hidden:
                return False
            if ffn.inter % 64 or (mixer.num_heads * head_dim) % 64:
                return False
        return True

    @classmethod
    def plan_for(cls, model) -> Optional["FusedDecode"]:
        """A plan when the model qualifies and the kernel takes its sizes, else None."""
        if not cls.qualifies(model):
            return None
        plan = cls(model)
        if not ops.decode_fused_takes(1, model.spec.hidden_size, plan.head_dim, plan.max_inter,
                                      plan.max_heads * plan.head_dim):
            return None
        return plan

    def takes(self, ctx, caches) -> bool:
        if not (ctx.all_single and ctx.dtype == torch.bfloat16 and ctx.logits_all_rows):
            return False
        if ctx.num_tokens > ops.FUSED_MAX_TOKENS or ctx.max_kv_len > ops.decode_fused_max_keys():
            return False
        model = self.model
        if not ops.decode_fused_takes(ctx.num_tokens, model.spec.hidden_size, self.head_dim, self.max_inter,
                                      self.max_heads * self.head_dim):
            return False
        return all(isinstance(caches.get(entry.cache), PagedKVView) for entry in model.spec.schedule)

    # ------------------------------------------------------------------------------
    def _describe(self, ctx, caches):
        model, ws = self.model, ctx.workspace
        tokens = ctx.num_tokens
        hidden, vocab, d = model.spec.hidden_size, model.spec.vocab_size, self.head_dim
        device = model.device
        chunk_keys = ops.decode_fused_chunk_keys()
        max_chunks = 1
        while max_chunks * chunk_keys < max(ctx.max_kv_len, 1):
            max_chunks *= 2
        x = ws.get("model.residual", (tokens, hidden), torch.float32)
        q = ws.get("attention.q", (tokens, self.max_heads * d), torch.bfloat16)
        attn = ws.get("attention.out", (tokens, self.max_heads * d), torch.bfloat16)
        act = ws.get("swiglu.act", (tokens, self.max_inter), torch.bfloat16)
        logits = ws.get("model.logits", (tokens, vocab), torch.float32)
        rows = tokens * self.max_heads * max_chunks
        partial_ml = ws.get("fused.partial_ml", (rows, 2), torch.float32)
        partial_out = ws.get("fused.partial_out", (rows, d), torch.float32)
        if self._barrier is None:
            self._barrier = torch.zeros(1, dtype=torch.int32, device=device)
        key = (tokens, max_chunks, ctx.tokens.data_ptr(), ctx.positions.data_ptr(), ws.generation,
               tuple((t.data_ptr(), t.shape[1]) for t in ctx.block_tables))
        kept = self._kept.get(key)
        if kept is not None:
            return kept[0], logits

        layers = (ops.FusedLayer * len(model.spec.schedule))()
        for index, entry in enumerate(model.spec.schedule):
            block = model.blocks[entry.layer]
            mixer, ffn, cache = block.mixer, block.ffn, caches[entry.cache]
            table = ctx.block_tables[cache.group]
            item = layers[index]
            item.w_qkv = mixer.qkv.weight.data_ptr()
            item.b_qkv = None if mixer.qkv.bias is None else mixer.qkv.bias.data_ptr()
            item.norm1 = block.mixer_norm.weight.data_ptr()
            item.w_o = mixer.out.weight.data_ptr()
            item.norm2 = block.ffn_norm.weight.data_ptr()
            item.w_gate_up = ffn.gate_up.weight.data_ptr()
            item.w_down = ffn.down.weight.data_ptr()
            item.k_pool = cache.k.data_ptr()
            item.v_pool = cache.v.data_ptr()
            item.block_table = table.data_ptr()
            if mixer.position.style == ops.ROPE_NEOX:
                cos, sin = mixer.position.tables()
                item.cos_table, item.sin_table = cos.data_ptr(), sin.data_ptr()
            item.eps1, item.eps2, item.scale = block.mixer_norm.eps, block.ffn_norm.eps, mixer.scale
            item.table_width, item.page_size = int(table.shape[1]), int(cache.page_size)
            item.window = int(mixer.window or 0)
            item.writes_cache = 1 if entry.writes_cache else 0
            item.num_heads, item.num_kv_heads, item.inter = mixer.num_heads, mixer.num_kv_heads, ffn.inter
            item.rope_style = int(mixer.position.style)
        raw = torch.frombuffer(bytearray(bytes(layers)), dtype=torch.uint8)
        device_layers = raw.to(device)

        if self._maps is None:
            weights = []
            for entry in model.spec.schedule:
                block = model.blocks[entry.layer]
                weights += [block.mixer.qkv.weight, block.mixer.out.weight, block.ffn.gate_up.weight,
                            block.ffn.down.weight]
            weights.append(model.head.weight)
            self._maps = ops.decode_fused_weight_maps(weights)
        m = ops.FusedModel()
        m.layers = device_layers.data_ptr()
        m.maps = self._maps.data_ptr()
        m.tokens, m.positions = ctx.tokens.data_ptr(), ctx.positions.data_ptr()
        m.embedding = model.embedding.data_ptr()
        m.x, m.q, m.attn, m.act = x.data_ptr(), q.data_ptr(), attn.data_ptr(), act.data_ptr()
        m.partial_ml, m.partial_out = partial_ml.data_ptr(), partial_out.data_ptr()
        m.barrier = self._barrier.data_ptr()
        m.final_norm, m.final_eps = model.final_norm.weight.data_ptr(), model.final_norm.eps
        m.head = model.head.weight.data_ptr()
        m.logits = logits.data_ptr()
        m.status = ops.kernel_status_word(device).data_ptr()
        if self.trace is not None:
            m.trace = self.trace.data_ptr()
        m.logit_scale = float(model.spec.logit_scale)
        m.T, m.hidden, m.vocab, m.num_layers = tokens, hidden, vocab, len(model.spec.schedule)
        m.max_chunks, m.head_dim = max_chunks, d
        if len(self._kept) >= self.MAX_KEPT:
            self._kept.clear()
        self._kept[key] = (m, device_layers)
        return m, logits

    def run(self, ctx, caches) -> torch.Tensor:
        description, logits = self._describe(ctx, caches)
        ops.decode_fused(description)
        return logits
