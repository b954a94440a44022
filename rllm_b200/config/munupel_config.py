"""Typed configuration of the Munupel decoder, read from ``config.json``.

A Munupel model is a list of layers with a parallel residual: one layer norm
(weight and bias) whose output both the mixer and the feed-forward read.  A
layer's mixer is one of two kinds of grouped-query attention with partial
rotary positions and a sigmoid gate on the heads' outputs; a layer may use the
tensors of another layer (``weights_of``) with a cache of its own.  Keys:

    architecture: "Munupel"      vocab, width      norm: {eps}
    layers: [{type, mixer: {...}, mlp: {kind: "dense", ff} | null, weights_of: j (optional)}, ...]
      mixer: heads, kv_heads, dim, vdim, scale,
             rot: {base, dims, scaling: {factor, original, fast, slow} (optional)},
             mask: {size, keep_first (optional)}, softcap (optional)
      type "attention":   projections with biases, scores capped by softcap * tanh(s / softcap),
                          a query sees the keys of its own chunk of mask.size positions,
                          ordinary softmax, a gate per output element
      type "attention_2": no biases, a sliding window of mask.size keys beside the first
                          mask.keep_first tokens, a softmax with one learned term per head in the
                          denominator, a gate per head

Every size and constant is taken from these keys; optional ``max_positions``
(default 131,072) bounds a request's length for the engine, which sizes its
cache pools by it (the design itself has no bound).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple

from .model_config import ConfigError

MIXER_KINDS = ("attention", "attention_2")


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class MunupelAttention:
    kind: str                         # "attention": chunked; "attention_2": window with kept first tokens and a sink
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[RotaryScaling]
    mask_size: int
    keep_first: int = 0
    softcap: Optional[float] = None


@dataclass(frozen=True)
class MunupelLayer:
    mixer: MunupelAttention
    ff: Optional[int]                 # inner size of the dense feed-forward; None: the layer has none
    weights_of: Optional[int] = None  # the layer whose tensors this one uses (resolved to a layer with its own)


@dataclass(frozen=True)
class MunupelConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[MunupelLayer, ...]
    max_positions: int = 1 << 17
    torch_dtype: str = "bfloat16"

    @staticmethod
    def from_json(raw: Mapping[str, Any]) -> "MunupelConfig":
        def need(d: Mapping[str, Any], key: str, where: str):
            if not isinstance(d, Mapping) or key not in d:
                raise ConfigError(f"config.json: {where} lacks {key!r}")
            return d[key]

        def positive(d, key, where) -> int:
            v = int(need(d, key, where))
            if v < 1:
                raise ConfigError(f"config.json: {where}.{key} must be positive")
            return v

        raw_layers = need(raw, "layers", "the configuration")
        if not isinstance(raw_layers, (list, tuple)) or not raw_layers:
            raise ConfigError("config.json: layers must be a non-empty list")
        layers = []
        for i, L in enumerate(raw_layers):
            where = f"layers[{i}]"
            kind = str(need(L, "type", where))
            if kind not in MIXER_KINDS:
                raise ConfigError(f"config.json: {where} has mixer type {kind!r}; known: {list(MIXER_KINDS)}")
            m, mw = need(L, "mixer", where), where + ".mixer"
            rot, rw = need(m, "rot", mw), mw + ".rot"
            sc = rot.get("scaling") if isinstance(rot, Mapping) else None
            scaling = None
            if sc is not None:
                sw = rw + ".scaling"
                scaling = RotaryScaling(float(need(sc, "factor", sw)), float(need(sc, "original", sw)),
                                        float(need(sc, "fast", sw)), float(need(sc, "slow", sw)))
                if scaling.factor <= 0 or scaling.original <= 0 or scaling.fast <= 0 or scaling.slow <= 0:
                    raise ConfigError(f"config.json: {sw}: factor, original, fast and slow must be positive")
            mask, kw = need(m, "mask", mw), mw + ".mask"
            keep = int(mask.get("keep_first", 0) or 0) if kind == "attention_2" else 0
            if keep < 0:
                raise ConfigError(f"config.json: {kw}.keep_first must not be negative")
            cap = m.get("softcap") if kind == "attention" else None
            if cap is not None and not float(cap) > 0:
                raise ConfigError(f"config.json: {mw}.softcap must be positive")
            mixer = MunupelAttention(kind, positive(m, "heads", mw), positive(m, "kv_heads", mw),
                                     positive(m, "dim", mw), positive(m, "vdim", mw), float(need(m, "scale", mw)),
                                     positive(rot, "dims", rw), float(need(rot, "base", rw)), scaling,
                                     positive(mask, "size", kw), keep, float(cap) if cap is not None else None)
            if mixer.heads % mixer.kv_heads:
                raise ConfigError(f"config.json: {mw}: heads {mixer.heads} is no multiple of kv_heads {mixer.kv_heads}")
            if mixer.rot_dims % 2 or mixer.rot_dims > mixer.dim:
                raise ConfigError(f"config.json: {rw}.dims {mixer.rot_dims} must be even and at most dim {mixer.dim}")
            if not mixer.rot_base > 1:
                raise ConfigError(f"config.json: {rw}.base must be greater than 1")
            mlp, ff = L.get("mlp"), None
            if mlp is not None:
                fw = where + ".mlp"
                mk = str(need(mlp, "kind", fw))
                if mk != "dense":
                    raise ConfigError(f"config.json: {fw}.kind {mk!r}; known: ['dense']")
                ff = positive(mlp, "ff", fw)
            src = L.get("weights_of")
            if src is not None:
                src = int(src)
                if not 0 <= src < len(raw_layers) or src == i:
                    raise ConfigError(f"config.json: {where}.weights_of {src} names no other layer")
            layers.append(MunupelLayer(mixer, ff, src))
        # a layer may name one that itself uses another's tensors: follow to the one that has them
        resolved = []
        for i, L in enumerate(layers):
            src, seen = L.weights_of, {i}
            while src is not None and layers[src].weights_of is not None:
                if src in seen:
                    raise ConfigError(f"config.json: layers[{i}].weights_of runs in a circle")
                seen.add(src)
                src = layers[src].weights_of
            if src is not None and (layers[src].mixer, layers[src].ff) != (L.mixer, L.ff):
                raise ConfigError(f"config.json: layers[{i}] uses the tensors of layers[{src}] but has other sizes")
            resolved.append(MunupelLayer(L.mixer, L.ff, src))
        return MunupelConfig(vocab=positive(raw, "vocab", "the configuration"),
                             width=positive(raw, "width", "the configuration"),
                             eps=float(need(need(raw, "norm", "the configuration"), "eps", "norm")),
                             layers=tuple(resolved), max_positions=int(raw.get("max_positions", 1 << 17)),
                             torch_dtype=str(raw.get("torch_dtype", "bfloat16")))
