"""Architecture-neutral description of a decoder: what each layer is made of
and in which order layers run.  An architecture's config (see qwen3.py) is
translated into these; the parts are built from these and never see the
architecture's own config.

Every size and constant of a part is a field here.  Layers may differ from one
another: `ModelSpec.layers` is a list, not a count.
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class NormSpec:
    kind: str  # key in parts.registry.NORMS
    size: int
    eps: float


@dataclass(frozen=True)
class PositionSpec:
    """`args`: further keyword arguments of the encoding's constructor (a scaling factor, say), for kinds
    that need more than the three constants every rotary table has."""

    kind: str  # key in parts.registry.POSITION_ENCODINGS ("rope", "none", ...)
    rotary_dim: int = 0
    theta: float = 10000.0
    max_positions: int = 0
    args: dict[str, Any] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class MixerSpec:
    """`kind` chooses the class from parts.registry.MIXERS; `args` are its
    constructor's keyword arguments (sizes, constants, nested specs)."""

    kind: str
    args: dict[str, Any] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class FeedForwardSpec:
    kind: str  # key in parts.registry.FEED_FORWARDS
    args: dict[str, Any] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class LayerSpec:
    """One block: which arrangement (`block`, key in parts.registry.BLOCKS)
    of which mixer, feed-forward and norms.  `names` maps the block's sub-part
    roles to the tensor-name prefixes the checkpoint uses for them."""

    block: str
    mixer: MixerSpec
    feed_forward: FeedForwardSpec
    mixer_norm: NormSpec
    feed_forward_norm: NormSpec
    names: dict[str, str] = field(default_factory=dict, hash=False, compare=False)


@dataclass(frozen=True)
class ScheduleEntry:
    """One execution of a layer.  `layer` indexes ModelSpec.layers (a layer may
    be named by several entries: its weights are shared, each execution has a
    cache of its own).  `cache_of`, if set, is the index of an EARLIER schedule
    entry whose cache this execution reads instead of writing one of its own."""

    layer: int
    cache_of: int | None = None


@dataclass
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: list[LayerSpec]
    schedule: list[ScheduleEntry]
    final_norm: NormSpec
    tie_embeddings: bool
    max_positions: int
    dtype: str  # the checkpoint's own dtype ("bfloat16", "float32", "float16")
    embedding_name: str = "model.embed_tokens."
    layer_name: str = "model.layers.{}."
    final_norm_name: str = "model.norm."
    head_name: str = "lm_head."
    eos_token_id: int | None = None

    def validate(self) -> None:
        if not self.layers:
            raise ValueError("a model needs at least one layer")
        if not self.schedule:
            raise ValueError("the schedule names no layer")
        for i, e in enumerate(self.schedule):
            if not 0 <= e.layer < len(self.layers):
                raise ValueError(f"schedule entry {i} names layer {e.layer}, the model has {len(self.layers)}")
            if e.cache_of is not None:
                if not 0 <= e.cache_of < i:
                    raise ValueError(f"schedule entry {i}: cache_of={e.cache_of} must name an earlier entry")
                if self.schedule[e.cache_of].cache_of is not None:
                    raise ValueError(f"schedule entry {i}: entry {e.cache_of} has no cache of its own")
