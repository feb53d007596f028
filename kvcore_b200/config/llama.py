"""Typed configuration of the Llama 3 dense decoder, read from config.json keys.

Keys and their defaults follow how the reference reads them
(kvcore/model/models/llama3.py:28-33, 56-74, 121-122, 161-176, 219-225;
kvcore/model/layer/rotary_embedding.py:38-49; kvcore/engine/engine_core.py:162-173,
209-217).  Added here: the ``llama3`` (and ``linear``) frequency scaling of
``rope_scaling`` / ``rope_parameters``, which the reference's rotary layer does not read.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Mapping

from .config_json import ConfigError, read_config_json
from .model_spec import LayerSpec, ModelSpec, PartSpec, default_schedule

_REQUIRED_KEYS = (
    "vocab_size",
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
)


@dataclass(frozen=True)
class RopeScaling:
    """Frequency scaling of the rotary table.  ``rope_type`` is "default", "linear" or "llama3"."""

    rope_type: str = "default"
    factor: float = 1.0
    low_freq_factor: float = 1.0
    high_freq_factor: float = 4.0
    original_max_position_embeddings: int = 8192


@dataclass(frozen=True)
class LlamaConfig:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    rope_scaling: RopeScaling
    max_position_embeddings: int
    tie_word_embeddings: bool
    attention_bias: bool
    mlp_bias: bool
    hidden_act: str
    logit_scale: float
    eos_token_ids: tuple[int, ...]
    stored_dtype: str | None

    @classmethod
    def from_dict(cls, raw: Mapping[str, Any]) -> "LlamaConfig":
        missing = [key for key in _REQUIRED_KEYS if key not in raw]
        if missing:
            raise ConfigError(f"config.json is missing required key(s): {', '.join(missing)}")

        hidden = _positive_int(raw, "hidden_size")
        heads = _positive_int(raw, "num_attention_heads")
        kv_heads = int(raw.get("num_key_value_heads") or heads)
        head_dim = raw.get("head_dim")
        if head_dim is None:
            if hidden % heads:
                raise ConfigError(
                    f"hidden_size {hidden} is not divisible by num_attention_heads {heads} "
                    "and config.json gives no head_dim"
                )
            head_dim = hidden // heads
        head_dim = int(head_dim)
        if kv_heads <= 0 or heads % kv_heads:
            raise ConfigError(
                f"num_attention_heads {heads} must be a positive multiple of "
                f"num_key_value_heads {kv_heads}"
            )
        if head_dim <= 0 or head_dim % 2:
            raise ConfigError(f"head_dim must be positive and even for rotary encoding, got {head_dim}")

        hidden_act = str(raw.get("hidden_act", "silu"))
        if hidden_act != "silu":
            # the reference refuses other activations too (llama3.py:28-31)
            raise ConfigError(f"unsupported hidden_act {hidden_act!r}: only 'silu' is supported")

        theta, scaling = _parse_rope(raw)
        eos = raw.get("eos_token_id")
        if eos is None:
            eos_ids: tuple[int, ...] = ()
        elif isinstance(eos, (list, tuple)):
            eos_ids = tuple(int(x) for x in eos)
        else:
            eos_ids = (int(eos),)

        return cls(
            vocab_size=_positive_int(raw, "vocab_size"),
            hidden_size=hidden,
            intermediate_size=_positive_int(raw, "intermediate_size"),
            num_hidden_layers=_positive_int(raw, "num_hidden_layers"),
            num_attention_heads=heads,
            num_key_value_heads=kv_heads,
            head_dim=head_dim,
            rms_norm_eps=float(raw.get("rms_norm_eps", 1e-6)),
            rope_theta=theta,
            rope_scaling=scaling,
            max_position_embeddings=int(raw.get("max_position_embeddings", 2048)),
            tie_word_embeddings=bool(raw.get("tie_word_embeddings", False)),
            attention_bias=bool(raw.get("attention_bias", False)),
            mlp_bias=bool(raw.get("mlp_bias", False)),
            hidden_act=hidden_act,
            logit_scale=float(raw.get("logit_scale", 1.0)),
            eos_token_ids=eos_ids,
            stored_dtype=raw.get("dtype") or raw.get("torch_dtype"),
        )

    @classmethod
    def from_folder(cls, folder: str | Path) -> "LlamaConfig":
        return cls.from_dict(read_config_json(folder))

    def to_model_spec(self) -> ModelSpec:
        """Describe the decoder as parts: every layer the same here, but stated layer by layer."""
        position = PartSpec(
            "rope",
            dict(
                head_dim=self.head_dim,
                theta=self.rope_theta,
                rope_type=self.rope_scaling.rope_type,
                factor=self.rope_scaling.factor,
                low_freq_factor=self.rope_scaling.low_freq_factor,
                high_freq_factor=self.rope_scaling.high_freq_factor,
                original_max_position_embeddings=self.rope_scaling.original_max_position_embeddings,
            ),
        )
        mixer = PartSpec(
            "paged_attention",
            dict(
                hidden_size=self.hidden_size,
                num_heads=self.num_attention_heads,
                num_kv_heads=self.num_key_value_heads,
                head_dim=self.head_dim,
                scale=float(self.head_dim) ** -0.5,  # llama3.py:60
                bias=self.attention_bias,
                sliding_window=None,
                position=position,
            ),
        )
        feed_forward = PartSpec(
            "swiglu",
            dict(
                hidden_size=self.hidden_size,
                intermediate_size=self.intermediate_size,
                bias=self.mlp_bias,
            ),
        )
        norm = PartSpec("rmsnorm", dict(size=self.hidden_size, eps=self.rms_norm_eps))
        layers = tuple(
            LayerSpec(
                prefix=f"model.layers.{index}",
                block=PartSpec("prenorm_residual"),
                mixer=mixer.with_params(
                    name=f"model.layers.{index}.self_attn",
                    # checkpoints saved from modules that keep the frequency table as a buffer carry
                    # it under this name; the rotary part names it as ignorable
                    position=position.with_params(name=f"model.layers.{index}.self_attn.rotary_emb"),
                ),
                feed_forward=feed_forward.with_params(name=f"model.layers.{index}.mlp"),
                norms={
                    "mixer_norm": norm.with_params(name=f"model.layers.{index}.input_layernorm"),
                    "feed_forward_norm": norm.with_params(
                        name=f"model.layers.{index}.post_attention_layernorm"
                    ),
                },
            )
            for index in range(self.num_hidden_layers)
        )
        return ModelSpec(
            architecture="LlamaForCausalLM",
            vocab_size=self.vocab_size,
            hidden_size=self.hidden_size,
            layers=layers,
            schedule=default_schedule(self.num_hidden_layers),
            embedding=PartSpec(
                "token_embedding",
                dict(vocab_size=self.vocab_size, hidden_size=self.hidden_size, name="model.embed_tokens"),
            ),
            final_norm=norm.with_params(name="model.norm"),
            lm_head=PartSpec(
                "lm_head",
                dict(
                    vocab_size=self.vocab_size,
                    hidden_size=self.hidden_size,
                    name="lm_head",
                    tied_to="model.embed_tokens" if self.tie_word_embeddings else None,
                    logit_scale=self.logit_scale,
                ),
            ),
            max_position_embeddings=self.max_position_embeddings,
            eos_token_ids=self.eos_token_ids,
            stored_dtype=self.stored_dtype,
        )


def _positive_int(raw: Mapping[str, Any], key: str) -> int:
    value = raw[key]
    if not isinstance(value, int) or isinstance(value, bool) or value <= 0:
        raise ConfigError(f"config.json key {key!r} must be a positive integer, got {value!r}")
    return value


def _parse_rope(raw: Mapping[str, Any]) -> tuple[float, RopeScaling]:
    """Base and scaling from either ``rope_parameters`` or ``rope_theta`` + ``rope_scaling``."""
    params = raw.get("rope_parameters")
    legacy = raw.get("rope_scaling")
    theta = None
    source: Mapping[str, Any] | None = None
    if isinstance(params, Mapping):
        theta = params.get("rope_theta", params.get("theta"))
        source = params
    if theta is None:
        theta = raw.get("rope_theta")
    if theta is None:
        theta = 10000.0  # rotary_embedding.py:49
    if isinstance(legacy, Mapping):
        source = legacy
    if source is None:
        return float(theta), RopeScaling()
    rope_type = source.get("rope_type", source.get("type", "default")) or "default"
    if rope_type == "default":
        return float(theta), RopeScaling()
    if rope_type == "linear":
        return float(theta), RopeScaling(rope_type="linear", factor=float(source["factor"]))
    if rope_type == "llama3":
        needed = ("factor", "low_freq_factor", "high_freq_factor", "original_max_position_embeddings")
        absent = [key for key in needed if key not in source]
        if absent:
            raise ConfigError(f"llama3 rope scaling is missing key(s): {', '.join(absent)}")
        return float(theta), RopeScaling(
            rope_type="llama3",
            factor=float(source["factor"]),
            low_freq_factor=float(source["low_freq_factor"]),
            high_freq_factor=float(source["high_freq_factor"]),
            original_max_position_embeddings=int(source["original_max_position_embeddings"]),
        )
    raise ConfigError(
        f"unsupported rope_type {rope_type!r}: supported are 'default', 'linear' and 'llama3'"
    )


__all__ = ["ConfigError", "LlamaConfig", "RopeScaling", "read_config_json"]
