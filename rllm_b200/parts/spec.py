"""What a model is made of, as data.

A model is a ``ModelSpec``: an embedding, a list of layers, the order in which
the layers run, a final norm and an output head.  A layer is a ``LayerSpec``:
an arrangement (``block``) of a mixer, a feed-forward and norms, each a
``PartSpec`` = (kind, parameters).  ``kind`` is a key of the part registries in
``rllm_b200.parts.registry``; the parameters hold every size and constant the
part needs, so a part never looks at a model configuration and does not know
which model it is in.  Layers of one model may have different kinds.

The order is data too: ``ModelSpec.order`` is a list of ``Run(layer, cache)``.
A layer index may appear twice (the same weights run twice); ``cache`` names
the cache slot that the run's mixer uses.  A run whose ``cache`` is its own
index in the order owns that slot and writes it; a run that names an earlier
run's slot reads what that run wrote and writes nothing.

The reference has one hard-wired stack instead
(crates/rllm-model/src/llama.rs:186-249).
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Any, Dict, Mapping, Optional, Tuple


def _freeze(v: Any) -> Any:
    if isinstance(v, Mapping):
        return tuple(sorted((k, _freeze(x)) for k, x in v.items()))
    if isinstance(v, (list, tuple)):
        return tuple(_freeze(x) for x in v)
    return v


@dataclass(frozen=True)
class PartSpec:
    kind: str
    params: Tuple[Tuple[str, Any], ...] = ()

    @staticmethod
    def of(kind: str, **params: Any) -> "PartSpec":
        return PartSpec(kind, _freeze(params))

    def get(self) -> Dict[str, Any]:
        return dict(self.params)

    def __getitem__(self, key: str) -> Any:
        for k, v in self.params:
            if k == key:
                return v
        raise KeyError(key)


@dataclass(frozen=True)
class TensorSpec:
    """One tensor a part takes from the weight file.

    role: "matrix": held in the run's dtype (bfloat16 or float32);
          "vector": like a matrix, but a tensor that the file stores in 32-bit
                    stays 32-bit in a bfloat16 run;
          "int":    an integer table, held as int32.
    init: how the random-weights mode draws it: ("normal", std),
          ("one_plus_normal", std), ("zeros",), ("ones",) or ("randint", high).
    An optional tensor is used when the file has it and is not drawn by the
    random-weights mode.
    """

    name: str
    shape: Tuple[int, ...]
    role: str = "matrix"
    init: Tuple[Any, ...] = ("normal", 0.02)
    optional: bool = False           # absent from the file is not an error


@dataclass(frozen=True)
class LayerSpec:
    block: str                       # arrangement kind, e.g. "pre_norm"
    mixer: PartSpec
    ffn: Optional[PartSpec]          # None: the layer has no feed-forward (arrangements that allow it)
    norms: Tuple[PartSpec, ...]      # in the order the arrangement uses them
    prefix: str                      # tensor-name prefix, e.g. "model.layers.3."
    block_params: Optional[PartSpec] = None   # sizes, constants and tensor names of the arrangement itself


@dataclass(frozen=True)
class Run:
    layer: int
    cache: int


@dataclass(frozen=True)
class ModelSpec:
    hidden_size: int
    vocab_size: int
    embedding: PartSpec
    layers: Tuple[LayerSpec, ...]
    order: Tuple[Run, ...]
    final_norm: PartSpec
    head: PartSpec
    max_positions: int
    eos_token_ids: Tuple[int, ...] = ()
    streams: int = 0                 # > 0: the residual is that many parallel streams [S, T, H] (blocks that read
                                     # and write them all); 0: the one residual [T, H]

    def validate(self) -> None:
        for i, run in enumerate(self.order):
            if not 0 <= run.layer < len(self.layers):
                raise ValueError(f"order[{i}] names layer {run.layer}, the model has {len(self.layers)}")
            if not 0 <= run.cache <= i:
                raise ValueError(f"order[{i}] names cache slot {run.cache}; a run may use its own slot "
                                 f"({i}) or an earlier run's")
            if self.order[run.cache].cache != run.cache:
                raise ValueError(f"order[{i}] reads slot {run.cache}, which is not owned by run {run.cache}")


# ---------------------------------------------------------------------------
# what a mixer needs from the cache manager
# ---------------------------------------------------------------------------
@dataclass(frozen=True)
class KVPagesNeed:
    """Keys and values of every token (``window`` None) or of the last
    ``window`` tokens, in pages.  ``values`` False: a token keeps ONE row of
    ``head_dim`` values per kv head that serves as key and as value (a latent);
    the storage then has no second buffer.  ``v_dim``: the size of a value row
    where it is not a key row's (None: ``head_dim``).  ``keep_first``: beside
    the window, the first that many tokens of a sequence stay (their pages are
    never given back).  ``chunk``: a query needs only the keys of its own chunk
    of that many positions, counted from position 0 (None: no such limit)."""

    num_kv_heads: int
    head_dim: int
    window: Optional[int] = None
    values: bool = True
    v_dim: Optional[int] = None
    keep_first: int = 0
    chunk: Optional[int] = None

    @property
    def value_dim(self) -> int:
        return self.head_dim if self.v_dim is None else self.v_dim

    @property
    def span(self) -> Optional[int]:
        """The most keys behind a query (itself included) that it can still need, the kept first tokens
        aside; None: all of them.  Pages behind that are given back."""
        spans = [int(x) for x in (self.window, self.chunk) if x is not None]
        return min(spans) if spans else None

    def widened(self, other: "KVPagesNeed") -> Optional["KVPagesNeed"]:
        """The need that keeps what both keep, if the rows are the same and only what is visible differs."""
        if (self.num_kv_heads, self.head_dim, self.values, self.value_dim) != \
                (other.num_kv_heads, other.head_dim, other.values, other.value_dim):
            return None
        if (self.keep_first, self.chunk) != (other.keep_first, other.chunk):
            return KVPagesNeed(self.num_kv_heads, self.head_dim, None, self.values, self.v_dim)   # every key
        w = None if self.window is None or other.window is None else max(self.window, other.window)
        return KVPagesNeed(self.num_kv_heads, self.head_dim, w, self.values, self.v_dim, self.keep_first, self.chunk)


@dataclass(frozen=True)
class StateNeed:
    """Per-request state of fixed size: one slot of ``shape`` float32 values."""

    shape: Tuple[int, ...]
