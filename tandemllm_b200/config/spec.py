"""The architecture-neutral description of a decoder: what the engine builds a model from.

An architecture's own configuration (its config.json keys, read by a module beside this one) is
translated into a `ModelSpec`. Nothing below this point reads config.json or knows a model's name:
the parts (mixers, feed-forwards, norms, position encodings, block arrangements) are chosen layer
by layer from the `kind` strings here and receive every size and constant as a parameter.

The order in which layers run is data too: `ModelSpec.schedule` is a list of `Site`s. A site names
the layer whose weights it runs and the site whose cache it reads, so a layer can run twice (two
sites naming one layer, each with a cache of its own) and a layer can attend over the keys another
site wrote (a site whose `cache_of` names an earlier site).

The reference keeps the same split between a family's config and what shared code is told as data
(engine/models/adapter.py:19-118, engine/models/lfm2_moe/config.py:58-123).
"""

from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Mapping


@dataclass(frozen=True)
class PartSpec:
    """One part of a layer: its registered `kind` and its parameters (sizes and constants)."""
    kind: str
    params: Mapping[str, Any] = field(default_factory=dict)

    def __getitem__(self, key: str) -> Any:
        return self.params[key]

    def get(self, key: str, default: Any = None) -> Any:
        return self.params.get(key, default)


@dataclass(frozen=True)
class LayerSpec:
    """A layer: a mixer and a feed-forward, the norms in front of each, and how they are arranged.

    `prefix` is the layer's part of its tensors' names ("layers.3."); each part adds its own suffixes.
    """
    prefix: str
    mixer: PartSpec
    feed_forward: PartSpec
    mixer_norm: PartSpec
    feed_forward_norm: PartSpec
    arrangement: str = "prenorm_residual"


@dataclass(frozen=True)
class Site:
    """One entry of the run order: run `layer`'s weights; read and write the cache of site `cache_of`
    (None: this site's own cache)."""
    layer: int
    cache_of: int | None = None


@dataclass(frozen=True)
class ModelSpec:
    architecture: str
    hidden_size: int
    vocab_size: int
    layers: tuple[LayerSpec, ...]
    schedule: tuple[Site, ...]
    final_norm: PartSpec
    embedding_name: str = field(kw_only=True)       # the embedding table's tensor name; an architecture says its own
    final_norm_prefix: str = field(kw_only=True)    # the last norm's part of its tensors' names
    head_name: str | None = None           # None: the head is the embedding (tied)
    ignored_names: tuple[str, ...] = ()    # stored tensors that are neither read nor an error (a tied model's copy
                                           # of its head, for one)
    max_positions: int = 1 << 17
    stop_token_ids: tuple[int, ...] = ()
    name_prefixes: tuple[str, ...] = ("model.",)   # stored names may carry one of these in front

    def __post_init__(self) -> None:
        for i, s in enumerate(self.schedule):
            if not 0 <= s.layer < len(self.layers):
                raise ValueError(f"schedule[{i}] names layer {s.layer}, the model has {len(self.layers)}")
            if s.cache_of is not None:
                if not 0 <= s.cache_of < i:
                    raise ValueError(f"schedule[{i}] reads the cache of site {s.cache_of}, which is not before it")
                if self.schedule[s.cache_of].cache_of is not None:
                    raise ValueError(f"schedule[{i}] reads the cache of site {s.cache_of}, which has none of its own")


def plain_schedule(n_layers: int) -> tuple[Site, ...]:
    """Every layer once, in order, each with its own cache."""
    return tuple(Site(i) for i in range(n_layers))
