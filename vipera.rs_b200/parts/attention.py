"""Grouped-query attention over the paged cache.

In the reference's order (crates/vipera-backend-cpu/src/model.rs:1005-1126): q, k, v products
from the normalised input, bias added after the product and before the rotation, rotation
of q and k, keys and values written to their pages, attention of every new token over its
request's keys, output product added to the residual stream.  Query head h reads KV head
h // group (model.rs:1813-1826).

Here q, k and v come from one product with the concatenated matrix (the reference keeps
three products, model.rs:1005-1025); the rotation and the cache write are one kernel; the
output product adds into the 32-bit residual stream in its own ending.
"""
from __future__ import annotations

import torch

from ..config.registry import MIXERS, POSITION_ENCODINGS
from ..errors import UnsupportedError
from ..kernels import ops
from ..weights import TensorSpec
from .base import Mixer, PagedKV
from .linear import Linear, NormedInput


class GQAttention(Mixer):
    """params: hidden_size, num_heads, num_kv_heads, head_dim, qkv_bias, window (None or a
    count of keys), softmax_scale, position (a PartSpec of a position encoding) and,
    optionally, ``projection_names`` (defaults q_proj, k_proj, v_proj, o_proj)."""

    kernels = ("rope_cache", "attention", "attention_mma", "attention_tc")
    takes_lazy_input = True

    @staticmethod
    def _names(params):
        return params.get("projection_names", ("q_proj", "k_proj", "v_proj", "o_proj"))

    @classmethod
    def schema(cls, params, prefix):
        hidden, d = params["hidden_size"], params["head_dim"]
        q_width, kv_width = params["num_heads"] * d, params["num_kv_heads"] * d
        qn, kn, vn, on = cls._names(params)
        schema = {
            f"{prefix}.{qn}.weight": TensorSpec((q_width, hidden)),
            f"{prefix}.{kn}.weight": TensorSpec((kv_width, hidden)),
            f"{prefix}.{vn}.weight": TensorSpec((kv_width, hidden)),
            f"{prefix}.{on}.weight": TensorSpec((hidden, q_width)),
        }
        if params.get("qkv_bias", False):
            schema[f"{prefix}.{qn}.bias"] = TensorSpec((q_width,), init="bias")
            schema[f"{prefix}.{kn}.bias"] = TensorSpec((kv_width,), init="bias")
            schema[f"{prefix}.{vn}.bias"] = TensorSpec((kv_width,), init="bias")
        return schema

    def __init__(self, params, prefix, tensors, dtype, device):
        super().__init__(params, prefix, tensors, dtype, device)
        self.hidden = int(params["hidden_size"])
        self.num_heads = int(params["num_heads"])
        self.num_kv_heads = int(params["num_kv_heads"])
        self.head_dim = int(params["head_dim"])
        self.window = params.get("window")
        self.scale = float(params["softmax_scale"])
        if self.head_dim % 16 or self.head_dim > 256:
            raise UnsupportedError(
                f"head size {self.head_dim}: the attention kernels take multiples of 16 up to 256")
        if self.num_heads % self.num_kv_heads:
            raise UnsupportedError("the number of heads must be a multiple of the number of KV heads")
        qn, kn, vn, on = self._names(params)
        fused = torch.cat([tensors[f"{prefix}.{n}.weight"] for n in (qn, kn, vn)], dim=0)
        bias = None
        if params.get("qkv_bias", False):
            bias = torch.cat([tensors[f"{prefix}.{n}.bias"].to(torch.float32) for n in (qn, kn, vn)], dim=0)
        self.qkv = Linear(fused, dtype, device, bias=bias)
        self.out = Linear(tensors[f"{prefix}.{on}.weight"], dtype, device)
        position = params["position"]
        self.position = POSITION_ENCODINGS.find(position.kind)(position.params, prefix, tensors, dtype, device)

    def kernel_families(self):
        # the tensor-core attention kernels serve bfloat16 with head sizes 64 and 128; everything
        # else runs through the general kernel
        own = ["rope_cache", "attention"]
        if self.dtype == torch.bfloat16 and self.head_dim in (64, 128):
            own.append("attention_mma")
            if self.head_dim in ops.TC_ATTENTION_HEAD_DIMS:
                own.append("attention_tc")
        return tuple(dict.fromkeys(tuple(own) + self.qkv.kernel_families() + self.out.kernel_families()
                                   + self.position.kernel_families()))

    def prepare(self, max_positions: int) -> None:
        prepare = getattr(self.position, "prepare", None)
        if prepare is not None:
            prepare(max_positions)

    @classmethod
    def cache_request_for(cls, params):
        return PagedKV(int(params["num_kv_heads"]), int(params["head_dim"]), params.get("window"))

    @classmethod
    def workspace_bytes(cls, params, tokens, element_bytes):
        q_width = params["num_heads"] * params["head_dim"]
        qkv_width = q_width + 2 * params["num_kv_heads"] * params["head_dim"]
        # q and the attention's output in the run's type, and the 32-bit q/k/v product of the unfused route
        return tokens * (2 * q_width * element_bytes + qkv_width * 4)

    def forward(self, ctx, h, residual, cache, writes_cache):
        count = ctx.num_tokens
        heads, kv_heads, d = self.num_heads, self.num_kv_heads, self.head_dim
        ws = ctx.workspace
        q = ws.get("attention.q", (count, heads * d), ctx.dtype)
        table = ctx.block_tables[cache.group]
        style = self.position.style
        if self.qkv.takes_small(count) and style in (ops.ROPE_NONE, ops.ROPE_NEOX):
            # few tokens: one kernel for norm, q/k/v product, bias, rotation and cache write
            cos, sin = self.position.tables()
            rope = dict(num_heads=heads, num_kv_heads=kv_heads, head_dim=d, style=style, positions=ctx.positions,
                        cos=cos, sin=sin, q_out=q, write_cache=writes_cache, k_pool=cache.k, v_pool=cache.v,
                        token_entry=ctx.token_entry, block_table=table, page_size=cache.page_size)
            if isinstance(h, NormedInput) and h.fusable:
                ops.gemv_small(self.qkv.weight, x=h.residual, norm_weight=h.norm.weight, eps=h.norm.eps,
                               tokens=count, epilogue=ops.GEMV_ROPE_CACHE, bias=self.qkv.bias, rope=rope)
            else:
                ops.gemv_small(self.qkv.weight, a=h.tensor() if isinstance(h, NormedInput) else h,
                               epilogue=ops.GEMV_ROPE_CACHE, bias=self.qkv.bias, rope=rope)
            mixed = ws.get("attention.out", (count, heads * d), ctx.dtype)
            self._attend(ctx, q, mixed, cache, table)
            self.out(ctx, mixed, epilogue=ops.EPI_RESIDUAL, resid=residual)
            return
        if (ctx.dtype == torch.bfloat16 and style in (ops.ROPE_NONE, ops.ROPE_NEOX)
                and self.qkv.tensor_core
                and ops.gemm_tc_rope_takes(count, self.qkv.out_features, self.qkv.in_features, d)):
            # many tokens: the tensor-core product ends with bias, rotation and cache write
            cos, sin = self.position.tables()
            a = h.tensor() if isinstance(h, NormedInput) else h
            ops.gemm_tc_rope(a, self.qkv.weight, bias=self.qkv.bias, q_out=q, num_heads=heads, num_kv_heads=kv_heads,
                             head_dim=d, positions=ctx.positions, cos=cos, sin=sin, style=style, k_pool=cache.k,
                             v_pool=cache.v, token_entry=ctx.token_entry, block_table=table,
                             page_size=cache.page_size, write_cache=writes_cache)
            mixed = ws.get("attention.out", (count, heads * d), ctx.dtype)
            self._attend(ctx, q, mixed, cache, table)
            self.out(ctx, mixed, epilogue=ops.EPI_RESIDUAL, resid=residual)
            return
        qkv = ws.get("attention.qkv", (count, (heads + 2 * kv_heads) * d), torch.float32)
        self.qkv(ctx, h, epilogue=ops.EPI_STORE, out=qkv)
        if style is None:
            # An encoding the fused kernel does not know: the part applies it to the 32-bit
            # product itself, then the kernel only converts and stores.
            q_view = qkv[:, : heads * d].unflatten(1, (heads, d))
            k_view = qkv[:, heads * d : (heads + kv_heads) * d].unflatten(1, (kv_heads, d))
            self.position.apply(ctx, q_view, k_view)
            style, cos, sin = ops.ROPE_NONE, None, None
        else:
            cos, sin = self.position.tables()
        ops.rope_cache(qkv, q, num_heads=heads, num_kv_heads=kv_heads, head_dim=d,
                       positions=ctx.positions, cos=cos, sin=sin, style=style,
                       k_pool=cache.k, v_pool=cache.v, token_seq=ctx.token_entry, block_table=table,
                       page_size=cache.page_size, write_cache=writes_cache)
        mixed = ws.get("attention.out", (count, heads * d), ctx.dtype)
        self._attend(ctx, q, mixed, cache, table)
        self.out(ctx, mixed, epilogue=ops.EPI_RESIDUAL, resid=residual)

    def _attend(self, ctx, q, mixed, cache, table):
        """Choose the attention kernel: on the bfloat16 path with a head size the tensor-core
        kernels are built for, the split-key kernel for steps of single tokens and the flash
        kernel otherwise; in every other case the general kernel."""
        heads, kv_heads, d = self.num_heads, self.num_kv_heads, self.head_dim
        window = self.window or 0
        if ctx.dtype == torch.bfloat16 and d in ops.MMA_HEAD_DIMS:
            if ctx.all_single:
                chunk, splits = ops.decode_splits(ctx.num_entries, kv_heads, max(ctx.max_kv_len, 1),
                                                  ops.sm_count(q.device))
                scratch = ctx.workspace.get(
                    "attention.partials",
                    (ops.attention_decode_scratch_floats(ctx.num_entries, heads, d, splits),), torch.float32)
                ops.attention_decode(q, mixed, cache.k, cache.v, positions=ctx.positions, block_table=table,
                                     num_heads=heads, num_kv_heads=kv_heads, head_dim=d, scale=self.scale,
                                     window=window, chunk=chunk, num_splits=splits, scratch=scratch)
            else:
                # portions through the flash kernel; the single tokens beside them (the running
                # decodes of a mixed step) through the split-key kernel, which streams their
                # history once per KV head instead of once per head and tile of 128 queries
                ops.attention_prefill(q, mixed, cache.k, cache.v, entry_starts=ctx.entry_starts,
                                      entry_pos0=ctx.entry_pos0, block_table=table, num_entries=ctx.num_entries,
                                      num_heads=heads, num_kv_heads=kv_heads, head_dim=d, scale=self.scale,
                                      window=window, skip_single=ctx.any_single)
                if ctx.any_single:
                    chunk, splits = ops.decode_splits(ctx.num_entries, kv_heads, max(ctx.max_kv_len, 1),
                                                      ops.sm_count(q.device))
                    scratch = ctx.workspace.get(
                        "attention.partials",
                        (ops.attention_decode_scratch_floats(ctx.num_entries, heads, d, splits),), torch.float32)
                    ops.attention_decode(q, mixed, cache.k, cache.v, positions=ctx.entry_pos0, block_table=table,
                                         num_heads=heads, num_kv_heads=kv_heads, head_dim=d, scale=self.scale,
                                         window=window, chunk=chunk, num_splits=splits, scratch=scratch,
                                         entry_starts=ctx.entry_starts)
            return
        ops.attention(q, mixed, cache.k, cache.v, token_seq=ctx.token_entry, positions=ctx.positions,
                      block_table=table, num_heads=heads, num_kv_heads=kv_heads, head_dim=d,
                      scale=self.scale, window=window)


MIXERS.register("gqa_attention", GQAttention)
