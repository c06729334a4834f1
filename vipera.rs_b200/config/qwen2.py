"""Typed configuration of the Qwen2 / Qwen2.5 dense decoder, read from the keys of
its own config.json, and its description in terms of parts.

The reference reads the same nine quantities from GGUF metadata into
``ModelConfig{layers,hidden,heads,kv_heads,head_dim,ffn,vocab,rms_eps,rope_base}``
(crates/vipera-backend-cpu/src/model.rs:34-53) and validates them at
model.rs:1315-1401: required keys, ``hidden % heads``, an even head size,
``heads % kv_heads``, defaults 1e-6 for eps and 10000 for the rope base.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Any, Dict, List, Optional, Tuple

from ..errors import InvalidArgumentError, UnsupportedError
from .registry import register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

_REQUIRED = (
    "num_hidden_layers",
    "hidden_size",
    "num_attention_heads",
    "intermediate_size",
    "vocab_size",
)


@dataclass(frozen=True)
class Qwen2Config:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    attention_bias: bool
    use_sliding_window: bool
    sliding_window: Optional[int]
    max_window_layers: int
    hidden_act: str
    eos_token_ids: Tuple[int, ...] = ()
    architecture: str = "Qwen2ForCausalLM"
    extra: Dict[str, Any] = field(default_factory=dict, compare=False, hash=False)

    # ---- reading -----------------------------------------------------------------
    @classmethod
    def from_dict(cls, data: Dict[str, Any]) -> "Qwen2Config":
        for key in _REQUIRED:
            if key not in data:
                raise UnsupportedError(f"config.json has no {key!r}")

        def integer(key, value, least=1):
            if isinstance(value, bool) or not isinstance(value, int) or value < least:
                raise InvalidArgumentError(f"{key} must be an integer of at least {least}, got {value!r}")
            return value

        layers = integer("num_hidden_layers", data["num_hidden_layers"])
        hidden = integer("hidden_size", data["hidden_size"])
        heads = integer("num_attention_heads", data["num_attention_heads"])
        kv_heads = integer("num_key_value_heads", data.get("num_key_value_heads", heads))
        if data.get("head_dim") is not None:
            head_dim = integer("head_dim", data["head_dim"])
        else:
            if hidden % heads:
                raise InvalidArgumentError(
                    f"hidden_size {hidden} is not a multiple of num_attention_heads {heads} "
                    "and config.json gives no head_dim"
                )
            head_dim = hidden // heads
        if head_dim % 2:
            raise InvalidArgumentError(f"head_dim {head_dim} must be even for rotary pairs")
        if heads % kv_heads:
            raise InvalidArgumentError(
                f"num_attention_heads {heads} is not a multiple of num_key_value_heads {kv_heads}"
            )
        eps = float(data.get("rms_norm_eps", 1e-6))
        theta = float(data.get("rope_theta", 10000.0))
        if not (eps > 0 and math.isfinite(eps)):
            raise InvalidArgumentError(f"rms_norm_eps must be positive, got {eps}")
        if not (theta > 0 and math.isfinite(theta)):
            raise InvalidArgumentError(f"rope_theta must be positive, got {theta}")
        if data.get("rope_scaling") not in (None, {}):
            raise UnsupportedError("rope_scaling is not supported (the reference applies none)")
        act = data.get("hidden_act", "silu")
        if act != "silu":
            raise UnsupportedError(f"hidden_act {act!r} is not supported; Qwen2 uses 'silu'")
        use_window = bool(data.get("use_sliding_window", False))
        window = data.get("sliding_window")
        if use_window:
            if window is None:
                raise InvalidArgumentError("use_sliding_window is true but sliding_window is missing")
            window = integer("sliding_window", window)
        elif window is not None:
            window = integer("sliding_window", window)
        max_window_layers = integer("max_window_layers", data.get("max_window_layers", layers), least=0)
        eos = data.get("eos_token_id")
        if eos is None:
            eos_ids: Tuple[int, ...] = ()
        elif isinstance(eos, int):
            eos_ids = (eos,)
        else:
            eos_ids = tuple(int(x) for x in eos)
        archs = data.get("architectures") or ["Qwen2ForCausalLM"]
        known = set(_REQUIRED) | {
            "num_key_value_heads", "head_dim", "rms_norm_eps", "rope_theta", "rope_scaling",
            "hidden_act", "use_sliding_window", "sliding_window", "max_window_layers",
            "eos_token_id", "architectures", "tie_word_embeddings", "max_position_embeddings",
            "attention_bias",
        }
        return cls(
            num_hidden_layers=layers,
            hidden_size=hidden,
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            intermediate_size=integer("intermediate_size", data["intermediate_size"]),
            vocab_size=integer("vocab_size", data["vocab_size"]),
            rms_norm_eps=eps,
            rope_theta=theta,
            tie_word_embeddings=bool(data.get("tie_word_embeddings", False)),
            max_position_embeddings=integer(
                "max_position_embeddings", data.get("max_position_embeddings", 32768)
            ),
            attention_bias=bool(data.get("attention_bias", True)),
            use_sliding_window=use_window,
            sliding_window=window,
            max_window_layers=max_window_layers,
            hidden_act=act,
            eos_token_ids=eos_ids,
            architecture=str(archs[0]),
            extra={k: v for k, v in data.items() if k not in known},
        )

    def to_dict(self) -> Dict[str, Any]:
        """The config.json that reads back as this configuration."""
        out: Dict[str, Any] = {
            "architectures": [self.architecture],
            "model_type": "qwen2",
            "num_hidden_layers": self.num_hidden_layers,
            "hidden_size": self.hidden_size,
            "num_attention_heads": self.num_attention_heads,
            "num_key_value_heads": self.num_key_value_heads,
            "head_dim": self.head_dim,
            "intermediate_size": self.intermediate_size,
            "vocab_size": self.vocab_size,
            "rms_norm_eps": self.rms_norm_eps,
            "rope_theta": self.rope_theta,
            "tie_word_embeddings": self.tie_word_embeddings,
            "max_position_embeddings": self.max_position_embeddings,
            "attention_bias": self.attention_bias,
            "use_sliding_window": self.use_sliding_window,
            "sliding_window": self.sliding_window,
            "max_window_layers": self.max_window_layers,
            "hidden_act": self.hidden_act,
        }
        if self.eos_token_ids:
            out["eos_token_id"] = list(self.eos_token_ids)
        return out

    # ---- derived -----------------------------------------------------------------
    def layer_window(self, layer: int) -> Optional[int]:
        """The attention window of a layer, or None where it sees every key.

        config.json's ``use_sliding_window`` switches windows on; layers from
        ``max_window_layers`` upward then see the last ``sliding_window`` keys
        (their own position included).  The reference ignores these keys and has
        only a process-wide window switch (crates/vipera-core/src/window.rs:15-55).
        """
        if self.use_sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None

    def kv_bytes_per_token(self, element_bytes: int) -> int:
        """Keys and values of all layers for one token
        (crates/vipera-backend-cpu/src/model.rs:63-70)."""
        return 2 * self.num_hidden_layers * self.num_key_value_heads * self.head_dim * element_bytes

    def parameter_count(self) -> int:
        h, d = self.hidden_size, self.head_dim
        q = self.num_attention_heads * d
        kv = self.num_key_value_heads * d
        per_layer = h * q + 2 * h * kv + q * h + 3 * h * self.intermediate_size + 2 * h
        if self.attention_bias:
            per_layer += q + 2 * kv
        total = self.num_hidden_layers * per_layer + self.vocab_size * h + h
        if not self.tie_word_embeddings:
            total += self.vocab_size * h
        return total


def qwen2_model_spec(config: Qwen2Config) -> ModelSpec:
    """Qwen2 in parts: pre-norm blocks of grouped-query attention with q/k/v bias
    and NeoX rotary positions, and a SwiGLU feed-forward, in file order
    (crates/vipera-backend-cpu/src/model.rs:521-689 runs them in this order)."""
    layers: List[LayerSpec] = []
    norm = PartSpec("rmsnorm", {"size": config.hidden_size, "eps": config.rms_norm_eps})
    for index in range(config.num_hidden_layers):
        mixer = PartSpec(
            "gqa_attention",
            {
                "hidden_size": config.hidden_size,
                "num_heads": config.num_attention_heads,
                "num_kv_heads": config.num_key_value_heads,
                "head_dim": config.head_dim,
                "qkv_bias": config.attention_bias,
                "window": config.layer_window(index),
                "softmax_scale": 1.0 / math.sqrt(config.head_dim),
                "position": PartSpec(
                    "rope_neox",
                    {
                        "head_dim": config.head_dim,
                        "theta": config.rope_theta,
                        "max_positions": config.max_position_embeddings,
                    },
                ),
            },
        )
        ffn = PartSpec(
            "swiglu",
            {"hidden_size": config.hidden_size, "intermediate_size": config.intermediate_size},
        )
        layers.append(
            LayerSpec(
                block="prenorm",
                prefix=f"model.layers.{index}",
                parts={"mixer_norm": norm, "mixer": mixer, "ffn_norm": norm, "ffn": ffn},
                names={"mixer_norm": "input_layernorm", "mixer": "self_attn",
                       "ffn_norm": "post_attention_layernorm", "ffn": "mlp"},
            )
        )
    spec = ModelSpec(
        architecture=config.architecture,
        vocab_size=config.vocab_size,
        hidden_size=config.hidden_size,
        max_position_embeddings=config.max_position_embeddings,
        embedding_name="model.embed_tokens.weight",
        layers=layers,
        schedule=[ScheduleEntry(layer=i, cache=i) for i in range(config.num_hidden_layers)],
        final_norm=norm,
        final_norm_name="model.norm",
        head_name=None if config.tie_word_embeddings else "lm_head.weight",
    )
    spec.validate()
    return spec


# The names the reference's files use for the same tensors (GGUF names; same memory layout:
# a GGUF [cols, rows] matrix is a row-major [out, in] matrix).
_GGUF_GLOBAL = {
    "token_embd.weight": "model.embed_tokens.weight",
    "output_norm.weight": "model.norm.weight",
    "output.weight": "lm_head.weight",
}
_GGUF_LAYER = {
    "attn_norm.weight": "input_layernorm.weight",
    "attn_q.weight": "self_attn.q_proj.weight", "attn_q.bias": "self_attn.q_proj.bias",
    "attn_k.weight": "self_attn.k_proj.weight", "attn_k.bias": "self_attn.k_proj.bias",
    "attn_v.weight": "self_attn.v_proj.weight", "attn_v.bias": "self_attn.v_proj.bias",
    "attn_output.weight": "self_attn.o_proj.weight",
    "ffn_norm.weight": "post_attention_layernorm.weight",
    "ffn_gate.weight": "mlp.gate_proj.weight",
    "ffn_up.weight": "mlp.up_proj.weight",
    "ffn_down.weight": "mlp.down_proj.weight",
}


def qwen2_tensor_alias(name: str):
    """``blk.{i}.attn_q.weight`` -> ``model.layers.{i}.self_attn.q_proj.weight`` and so on."""
    if name in _GGUF_GLOBAL:
        return _GGUF_GLOBAL[name]
    if name.startswith("blk."):
        _, _, rest = name.partition(".")
        index, _, tail = rest.partition(".")
        if index.isdigit() and tail in _GGUF_LAYER:
            return f"model.layers.{int(index)}.{_GGUF_LAYER[tail]}"
    return None


register_architecture("Qwen2ForCausalLM", Qwen2Config.from_dict, qwen2_model_spec,
                      tensor_alias=qwen2_tensor_alias)
