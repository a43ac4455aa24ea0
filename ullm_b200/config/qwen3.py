"""Typed configuration of the Qwen3 dense decoder, read from the keys of its
config.json, and its translation into a ModelSpec.

Keys and defaults follow ullm/models/qwen3.py:136-157 and :207-224 and
ullm/core/model_runner.py:38-63: head_dim defaults to hidden_size //
num_attention_heads, rope_theta to 1000000, attention_bias to False.  Three
things differ from the reference on purpose: tie_word_embeddings is honoured
(the reference never reads it), the sliding-window keys are honoured (the
reference ignores them; layers from max_window_layers on are windowed when
use_sliding_window is true), and a rope scaling other than the default is an
error instead of being ignored.
"""

from __future__ import annotations

from dataclasses import dataclass, fields
from typing import Any

from .specs import (
    FeedForwardSpec,
    LayerSpec,
    MixerSpec,
    ModelSpec,
    NormSpec,
    PositionSpec,
    ScheduleEntry,
)


class ConfigError(ValueError):
    pass


_REQUIRED = (
    "num_hidden_layers",
    "hidden_size",
    "num_attention_heads",
    "num_key_value_heads",
    "intermediate_size",
    "vocab_size",
)


@dataclass(frozen=True)
class Qwen3Config:
    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    intermediate_size: int
    vocab_size: int
    head_dim: int
    rope_theta: float = 1000000.0
    rms_norm_eps: float = 1e-6
    attention_bias: bool = False
    tie_word_embeddings: bool = False
    max_position_embeddings: int = 32768
    use_sliding_window: bool = False
    sliding_window: int | None = None
    max_window_layers: int = 0
    hidden_act: str = "silu"
    dtype: str = "float16"  # ullm/core/model_runner.py:38-51: "dtype" or "torch_dtype", float16 when neither is there
    eos_token_id: int | None = None

    @staticmethod
    def from_dict(d: dict[str, Any]) -> "Qwen3Config":
        missing = [k for k in _REQUIRED if k not in d]
        if missing:
            raise ConfigError(f"config.json lacks the keys {missing}")
        for k in _REQUIRED:
            if not isinstance(d[k], int) or isinstance(d[k], bool) or d[k] <= 0:
                raise ConfigError(f"config.json: {k} must be a positive integer, got {d[k]!r}")
        kw: dict[str, Any] = {k: d[k] for k in _REQUIRED}
        head_dim = d.get("head_dim")
        if head_dim is None:
            if d["hidden_size"] % d["num_attention_heads"]:
                raise ConfigError("head_dim is absent and hidden_size is no multiple of num_attention_heads")
            head_dim = d["hidden_size"] // d["num_attention_heads"]
        kw["head_dim"] = int(head_dim)
        rope = d.get("rope_parameters") or {}
        theta = d.get("rope_theta", rope.get("rope_theta"))
        if theta is not None:
            kw["rope_theta"] = float(theta)
        scaling = d.get("rope_scaling")
        rtype = (scaling or {}).get("rope_type", (scaling or {}).get("type")) if scaling else rope.get("rope_type")
        if rtype not in (None, "default"):
            raise ConfigError(f"rope scaling of type {rtype!r} is not supported (only the default rotary encoding)")
        for k in ("rms_norm_eps",):
            if k in d:
                kw[k] = float(d[k])
        for k in ("attention_bias", "tie_word_embeddings", "use_sliding_window"):
            if k in d and d[k] is not None:
                kw[k] = bool(d[k])
        for k in ("max_position_embeddings", "max_window_layers"):
            if k in d and d[k] is not None:
                kw[k] = int(d[k])
        if d.get("sliding_window") is not None:
            kw["sliding_window"] = int(d["sliding_window"])
        if "hidden_act" in d:
            kw["hidden_act"] = str(d["hidden_act"])
        dt = d.get("dtype", d.get("torch_dtype"))
        if dt is not None:
            dt = str(dt).replace("torch.", "")
            if dt not in ("bfloat16", "float32", "float16"):
                raise ConfigError(f"Unsupported dtype {dt!r}")
            kw["dtype"] = dt
        eos = d.get("eos_token_id")
        if isinstance(eos, list):
            eos = eos[0] if eos else None
        if eos is not None:
            kw["eos_token_id"] = int(eos)
        cfg = Qwen3Config(**kw)
        cfg.check()
        return cfg

    def check(self) -> None:
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads={self.num_attention_heads} is no multiple of "
                f"num_key_value_heads={self.num_key_value_heads}"
            )
        if self.head_dim <= 0 or self.head_dim % 2:
            raise ConfigError(f"head_dim={self.head_dim} must be even (rotary halves)")
        if self.hidden_act != "silu":
            raise ConfigError(f"hidden_act={self.hidden_act!r}: this architecture's feed-forward is SiLU-gated")
        if self.use_sliding_window and (self.sliding_window is None or self.sliding_window <= 0):
            raise ConfigError("use_sliding_window is true but sliding_window is not a positive integer")
        if self.rms_norm_eps <= 0:
            raise ConfigError("rms_norm_eps must be positive")

    def to_dict(self) -> dict[str, Any]:
        d = {f.name: getattr(self, f.name) for f in fields(self)}
        d["torch_dtype"] = d.pop("dtype")
        d["architectures"] = ["Qwen3ForCausalLM"]
        d["model_type"] = "qwen3"
        return d

    def layer_window(self, layer: int) -> int | None:
        if self.use_sliding_window and self.sliding_window and layer >= self.max_window_layers:
            return self.sliding_window
        return None


def qwen3_model_spec(cfg: Qwen3Config) -> ModelSpec:
    """Qwen3 dense as parts: every layer a pre-norm block of grouped-query
    attention (per-head q/k RMSNorm, rotary positions) and a SiLU-gated MLP."""
    position = PositionSpec(
        kind="rope", rotary_dim=cfg.head_dim, theta=cfg.rope_theta, max_positions=cfg.max_position_embeddings
    )
    layers = []
    for l in range(cfg.num_hidden_layers):
        mixer = MixerSpec(
            kind="paged_attention",
            args=dict(
                hidden_size=cfg.hidden_size,
                num_heads=cfg.num_attention_heads,
                num_kv_heads=cfg.num_key_value_heads,
                head_dim=cfg.head_dim,
                qkv_bias=cfg.attention_bias,
                qk_norm=NormSpec("rmsnorm", cfg.head_dim, cfg.rms_norm_eps),
                position=position,
                window=cfg.layer_window(l),
                scale=cfg.head_dim ** -0.5,
            ),
        )
        ff = FeedForwardSpec(
            kind="gated_mlp",
            args=dict(hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size, activation="silu"),
        )
        norm = NormSpec("rmsnorm", cfg.hidden_size, cfg.rms_norm_eps)
        layers.append(
            LayerSpec(
                block="prenorm_residual",
                mixer=mixer,
                feed_forward=ff,
                mixer_norm=norm,
                feed_forward_norm=norm,
                names=dict(
                    mixer="self_attn.",
                    feed_forward="mlp.",
                    mixer_norm="input_layernorm.",
                    feed_forward_norm="post_attention_layernorm.",
                ),
            )
        )
    return ModelSpec(
        architecture="Qwen3ForCausalLM",
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        layers=layers,
        schedule=[ScheduleEntry(l) for l in range(cfg.num_hidden_layers)],
        final_norm=NormSpec("rmsnorm", cfg.hidden_size, cfg.rms_norm_eps),
        tie_embeddings=cfg.tie_word_embeddings,
        max_positions=cfg.max_position_embeddings,
        dtype=cfg.dtype,
        eos_token_id=cfg.eos_token_id,
    )
