"""Descriptions of parts: what a model is made of, as data.

An architecture turns its typed configuration into a `ModelBlueprint`: the
embedding, a list of layers (each naming its mixer, feed-forward, norms and
block arrangement by *kind* with their sizes and constants as parameters), the
order in which layers run, the final norm and the output head.  The generic
model builder looks each kind up in the part registries, so a part never knows
which model it is in, and one model may hold different mixers and feed-forwards
in different layers.
"""
from __future__ import annotations

import dataclasses
from typing import Any, Optional


@dataclasses.dataclass(frozen=True)
class TensorSpec:
    """One tensor a part wants from the checkpoint."""
    name: str                 # full tensor name in the safetensors file
    shape: tuple[int, ...]
    init: str = "matrix"      # random-weights mode: "matrix" | "bias" | "norm" | "table" | "around_zero" | "fraction"
    keep_f32: bool = False    # kept in 32-bit even in a bfloat16 engine


@dataclasses.dataclass(frozen=True)
class PartSpec:
    """A part chosen by kind, with its sizes and constants."""
    kind: str
    params: dict[str, Any]
    prefix: str = ""          # tensor-name prefix of this part's weights

    def __getitem__(self, key):
        return self.params[key]

    def get(self, key, default=None):
        return self.params.get(key, default)


@dataclasses.dataclass(frozen=True)
class LayerSpec:
    """One layer: a block arrangement around a mixer and a feed-forward."""
    block: str                     # arrangement kind, e.g. "prenorm"
    mixer: PartSpec
    ffn: Optional[PartSpec]        # None: a layer without a feed-forward (arrangements that allow it)
    norms: tuple[PartSpec, ...]    # as many as the arrangement wants
    hidden: int = 0
    block_spec: Optional[PartSpec] = None   # constants and tensors of the arrangement itself, if it has any


@dataclasses.dataclass(frozen=True)
class LayerCall:
    """One entry of the run order.

    ``layer`` indexes `ModelBlueprint.layers` (a layer may be named twice);
    ``cache`` names the cache this call uses (calls that give the same number
    share one cache); ``write`` is False for a call that only reads a cache
    another call has filled.
    """
    layer: int
    cache: int
    write: bool = True


@dataclasses.dataclass(frozen=True)
class Reentry:
    """Something done to the residual stream right before the layer call ``before`` of the run order
    (e.g. mixing the embedding output back in at the start of a pass over looped layers)."""
    before: int
    part: PartSpec


@dataclasses.dataclass(frozen=True)
class ModelBlueprint:
    hidden: int
    vocab: int
    embedding: PartSpec
    layers: tuple[LayerSpec, ...]
    order: tuple[LayerCall, ...]
    final_norm: PartSpec
    head: PartSpec
    max_positions: int
    eos_token_ids: tuple[int, ...] = ()
    reentries: tuple[Reentry, ...] = ()
    # True: the residual stream is kept in 32-bit floats whatever the engine's storage type; the
    # embedding then hands out a 32-bit stream and the blocks add to it in 32-bit.
    stream_f32: bool = False


# ----------------------------------------------------------------------------------------
# What a mixer keeps per request between steps.
# ----------------------------------------------------------------------------------------

@dataclasses.dataclass(frozen=True)
class PagedKV:
    """Keys and values for every position (window == 0) or for the last ``window`` ones; with a window,
    ``keep_first`` > 0 keeps the first that many positions readable for the request's whole life."""
    n_kv_heads: int
    head_dim: int
    window: int = 0
    keep_first: int = 0

    def group_key(self):
        # Layers whose pages live and die together share a block table.
        return ("paged_kv", self.window, self.keep_first if self.window else 0)


@dataclasses.dataclass(frozen=True)
class PagedLatent:
    """One vector of ``width`` numbers per position, shared by all heads (a compressed key/value),
    for every position (window == 0) or for the last ``window`` ones.  Lives in pages like `PagedKV`
    and shares its block tables with every other paged cache of the same window."""
    width: int
    window: int = 0

    def group_key(self):
        return ("paged_kv", self.window, 0)


@dataclasses.dataclass(frozen=True)
class FixedState:
    """A state of fixed size per request (recurrent mixers), kept in 32-bit."""
    shape: tuple[int, ...]

    def group_key(self):
        return ("fixed_state",)


@dataclasses.dataclass(frozen=True)
class CacheParts:
    """Several needs of one layer call, in a fixed order: a mixer made of mixers that each keep a cache
    of their own, or one that keeps state of several shapes.  Each part is a need of the other kinds (or
    None); the layer call's `CacheView.parts` holds one view per part."""
    parts: tuple

    def group_key(self):
        return ("parts",)


CacheNeed = Optional[PagedKV | PagedLatent | FixedState | CacheParts]
