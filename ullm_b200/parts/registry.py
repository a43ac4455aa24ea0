"""Registries of part kinds.  A spec's `kind` string picks the class; the
spec's fields are its constructor arguments.  Registering a new kind needs no
change to any file of the framework:

    from ullm_b200.parts import register_mixer
    @register_mixer("my_mixer")
    class MyMixer(Mixer): ...
"""

from __future__ import annotations

MIXERS: dict[str, type] = {}
FEED_FORWARDS: dict[str, type] = {}
NORMS: dict[str, type] = {}
POSITION_ENCODINGS: dict[str, type] = {}
BLOCKS: dict[str, type] = {}


def _register(table: dict[str, type], what: str):
    def outer(kind: str):
        def inner(cls):
            table[kind] = cls
            return cls

        return inner

    return outer


register_mixer = _register(MIXERS, "mixer")
register_feed_forward = _register(FEED_FORWARDS, "feed-forward")
register_norm = _register(NORMS, "norm")
register_position_encoding = _register(POSITION_ENCODINGS, "position encoding")
register_block = _register(BLOCKS, "block")


def _lookup(table: dict[str, type], what: str, kind: str) -> type:
    if kind not in table:
        raise KeyError(f"no {what} of kind {kind!r} is registered (known: {sorted(table)})")
    return table[kind]


def build_norm(spec):
    return _lookup(NORMS, "norm", spec.kind)(size=spec.size, eps=spec.eps)


def build_position_encoding(spec):
    return _lookup(POSITION_ENCODINGS, "position encoding", spec.kind)(
        rotary_dim=spec.rotary_dim, theta=spec.theta, max_positions=spec.max_positions, **spec.args
    )


def build_mixer(spec):
    return _lookup(MIXERS, "mixer", spec.kind)(**spec.args)


def build_feed_forward(spec):
    return _lookup(FEED_FORWARDS, "feed-forward", spec.kind)(**spec.args)


def build_block(layer_spec):
    cls = _lookup(BLOCKS, "block", layer_spec.block)
    return cls(
        mixer=build_mixer(layer_spec.mixer),
        feed_forward=build_feed_forward(layer_spec.feed_forward),
        mixer_norm=build_norm(layer_spec.mixer_norm),
        feed_forward_norm=build_norm(layer_spec.feed_forward_norm),
        names=layer_spec.names,
    )
