"""Plain data that describes a model to the engine.

An architecture's configuration turns itself into a `ModelPlan`: which parts
each layer is made of (by registered kind name and parameters), in which order
the layers run, and which cache each run of a layer uses.  The engine builds
and runs a plan without knowing which architecture produced it.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Optional


class ConfigError(ValueError):
    """A configuration that cannot describe a runnable model."""


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: the registered kind and the constructor's parameters."""
    kind: str
    params: dict[str, Any] = field(default_factory=dict)

    def __hash__(self):
        return hash((self.kind, repr(sorted(self.params.items()))))


@dataclass(frozen=True)
class BlockSpec:
    """A layer: how its parts are arranged (`arrangement` is a registered block kind) and the
    parts themselves by the names the arrangement gives its places (`prenorm_residual`:
    mixer_norm, mixer, ffn_norm, ffn).  Another arrangement has other places: more norms, no
    feed-forward, two mixers."""
    arrangement: str
    parts: dict[str, PartSpec] = field(default_factory=dict)
    params: dict[str, Any] = field(default_factory=dict)      # constants of the arrangement itself (its constructor's)

    def __hash__(self):
        return hash((self.arrangement, tuple(sorted((k, hash(v)) for k, v in self.parts.items())),
                     repr(sorted(self.params.items()))))

    def __getattr__(self, place):
        """`spec.mixer` reads the part at the place `mixer`."""
        parts = self.__dict__.get("parts", {})
        if place in parts:
            return parts[place]
        raise AttributeError(f"block {self.__dict__.get('arrangement')!r} has no place {place!r}; it has {sorted(parts)}")


@dataclass(frozen=True)
class WeightBinding:
    """A parameter of the plan and the checkpoint tensor that fills it.  `source` may be a tuple of names:
    tensors of one shape that are stacked along a new first axis (experts stored one by one)."""
    target: str                 # e.g. "layers.3.ffn.experts_down"
    source: object              # checkpoint tensor name, or a tuple of names to stack
    source_shape: tuple         # exact shape expected in the file (of each, if several)
    transform: Optional[str] = None   # a registered weight transform (spite_b200.weights.register_weight_transform)
    init: str = "normal"        # how the random-weights mode fills it: "normal" | "ones"

    @property
    def sources(self) -> tuple:
        return (self.source,) if isinstance(self.source, str) else tuple(self.source)


@dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    `layer` indexes `ModelPlan.blocks` (a layer may be named more than once: its
    weights are then shared).  `cache` names the cache this run uses; two runs
    with the same `cache` read the same keys and values, and only the runs with
    `write_cache` append to it.
    """
    layer: int
    cache: int
    write_cache: bool = True


@dataclass(frozen=True)
class JunctionCall:
    """An entry of the run order that is not a layer: the junction `junction` (an index into
    `ModelPlan.junctions`) rewrites the residual stream between two layers.  `step` counts the
    times the same junction has run before in the order (a loop's pass number)."""
    junction: int
    step: int = 0


@dataclass(frozen=True)
class ModelPlan:
    hidden_size: int
    vocab_size: int
    blocks: tuple[BlockSpec, ...]
    order: tuple                          # of LayerCall and JunctionCall
    final_norm: PartSpec
    tie_word_embeddings: bool
    max_positions: int
    embedding_scale: float = 1.0          # the embedding row is multiplied by this as it enters the residual stream
    logit_scale: float = 1.0              # logits are multiplied by this,
    logit_softcap: float | None = None    # then squashed to cap * tanh(logit / cap)
    position_table: int | None = None     # learned position vectors [this many, hidden], added (unscaled) to the embedding
    junctions: tuple[PartSpec, ...] = ()  # parts of the family "junction" that `JunctionCall`s of the order name

    def layer_calls(self):
        """The runs of layers in the order (without the junctions between them)."""
        return [c for c in self.order if isinstance(c, LayerCall)]

    def validate(self):
        if self.hidden_size <= 0 or self.vocab_size <= 0:
            raise ConfigError("hidden_size and vocab_size must be positive")
        if not self.blocks:
            raise ConfigError("a model needs at least one layer")
        if self.logit_softcap is not None and not self.logit_softcap > 0:
            raise ConfigError("logit_softcap must be positive")
        if self.position_table is not None and self.position_table < self.max_positions:
            raise ConfigError(f"{self.position_table} learned position vectors cannot serve {self.max_positions} positions")
        for call in self.order:
            if isinstance(call, JunctionCall) and not 0 <= call.junction < len(self.junctions):
                raise ConfigError(f"run order names junction {call.junction}, model has {len(self.junctions)}")
        writers = {}
        for call in self.layer_calls():
            if not 0 <= call.layer < len(self.blocks):
                raise ConfigError(f"run order names layer {call.layer}, model has {len(self.blocks)}")
            if call.write_cache:
                if call.cache in writers:
                    raise ConfigError(f"cache {call.cache} is written by two runs of the order")
                writers[call.cache] = call.layer
        seen = set()
        for call in self.layer_calls():
            if not call.write_cache and call.cache not in seen:
                raise ConfigError(f"cache {call.cache} is read before any run writes it")
            if call.write_cache:
                seen.add(call.cache)
        return self
