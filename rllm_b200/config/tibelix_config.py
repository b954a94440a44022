"""Typed configuration of the Tibelix decoder, read from ``config.json``.

A Tibelix model is a list of layers, each a mixer and an optional feed-forward with an
RMS norm (weight stored as its distance from one) before and after each of the two.
Three kinds of mixer and two kinds of feed-forward, chosen per layer.  Keys:

    architecture: "Tibelix"      vocab, width      norm: {eps}
    layers: [{type, mixer: {...}, mlp: {...} | null}, ...]
      type "attention":        heads, kv_heads, dim, vdim, scale, q_temp: {coef, every} (optional),
                               kv_from: j (optional: the layer reads layer j's keys and values)
      type "latent_attention": heads, dim, rot_dim, vdim, q_rank, kv_rank, scale,
                               rot: {base, dims, scaling: {factor, original, fast, slow} (optional)}
      type "mlstm":            heads, dim, vdim, gate_cap
      mlp "dense":             ff
      mlp "moe":               expert: {ff}, router: {experts, top, groups: {count, keep} (optional)},
                               shared: {ff} (optional)

Every size and constant is taken from these keys; optional ``max_positions`` (default
131,072) bounds a request's length for the engine, which sizes its cache pools by it (the
design itself has no bound).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping, Optional, Tuple, Union

from .model_config import ConfigError

MIXER_KINDS = ("attention", "latent_attention", "mlstm")
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class RotaryScaling:
    factor: float
    original: float
    fast: float
    slow: float


@dataclass(frozen=True)
class TibelixAttention:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    q_temp: Optional[Tuple[float, int]]      # (coef, every)
    kv_from: Optional[int]                   # the layer whose keys and values this one reads


@dataclass(frozen=True)
class TibelixLatentAttention:
    heads: int
    dim: int
    rot_dim: int
    vdim: int
    q_rank: int
    kv_rank: int
    scale: float
    rot_dims: int
    rot_base: float
    rot_scaling: Optional[RotaryScaling]


@dataclass(frozen=True)
class TibelixMatrixLSTM:
    heads: int
    dim: int
    vdim: int
    gate_cap: float


@dataclass(frozen=True)
class TibelixDense:
    ff: int


@dataclass(frozen=True)
class TibelixExperts:
    ff: int
    experts: int
    top: int
    groups: Optional[Tuple[int, int]]        # (count, keep)
    shared_ff: Optional[int]


@dataclass(frozen=True)
class TibelixLayer:
    kind: str
    mixer: Union[TibelixAttention, TibelixLatentAttention, TibelixMatrixLSTM]
    mlp: Union[None, TibelixDense, TibelixExperts]


@dataclass(frozen=True)
class TibelixConfig:
    vocab: int
    width: int
    eps: float
    layers: Tuple[TibelixLayer, ...]
    max_positions: int = 1 << 17
    torch_dtype: str = "bfloat16"

    @staticmethod
    def from_json(raw: Mapping[str, Any]) -> "TibelixConfig":
        def need(d, key: str, where: str):
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
            if kind == "attention":
                qt, q_temp = m.get("q_temp"), None
                if qt is not None:
                    q_temp = (float(need(qt, "coef", mw + ".q_temp")), positive(qt, "every", mw + ".q_temp"))
                src = m.get("kv_from")
                mixer = TibelixAttention(positive(m, "heads", mw), positive(m, "kv_heads", mw), positive(m, "dim", mw),
                                         positive(m, "vdim", mw), float(need(m, "scale", mw)), q_temp,
                                         None if src is None else int(src))
                if mixer.heads % mixer.kv_heads:
                    raise ConfigError(f"config.json: {mw}: heads {mixer.heads} is no multiple of kv_heads "
                                      f"{mixer.kv_heads}")
            elif kind == "latent_attention":
                rot, rw = need(m, "rot", mw), mw + ".rot"
                sc, scaling = (rot.get("scaling") if isinstance(rot, Mapping) else None), None
                if sc is not None:
                    sw = rw + ".scaling"
                    scaling = RotaryScaling(float(need(sc, "factor", sw)), float(need(sc, "original", sw)),
                                            float(need(sc, "fast", sw)), float(need(sc, "slow", sw)))
                    if min(scaling.factor, scaling.original, scaling.fast, scaling.slow) <= 0:
                        raise ConfigError(f"config.json: {sw}: factor, original, fast and slow must be positive")
                mixer = TibelixLatentAttention(positive(m, "heads", mw), positive(m, "dim", mw),
                                               positive(m, "rot_dim", mw), positive(m, "vdim", mw),
                                               positive(m, "q_rank", mw), positive(m, "kv_rank", mw),
                                               float(need(m, "scale", mw)), positive(rot, "dims", rw),
                                               float(need(rot, "base", rw)), scaling)
                if mixer.rot_dim % 2 or mixer.rot_dims % 2 or mixer.rot_dims > mixer.rot_dim:
                    raise ConfigError(f"config.json: {mw}: rot_dim {mixer.rot_dim} and rot.dims {mixer.rot_dims} must "
                                      f"be even, and rot.dims at most rot_dim")
                if not mixer.rot_base > 1:
                    raise ConfigError(f"config.json: {rw}.base must be greater than 1")
            else:
                mixer = TibelixMatrixLSTM(positive(m, "heads", mw), positive(m, "dim", mw), positive(m, "vdim", mw),
                                          float(m.get("gate_cap") or 0.0))
                if mixer.gate_cap < 0:
                    raise ConfigError(f"config.json: {mw}.gate_cap must not be negative")
            f, mlp = L.get("mlp"), None
            if f is not None:
                fw = where + ".mlp"
                fk = str(need(f, "kind", fw))
                if fk not in MLP_KINDS:
                    raise ConfigError(f"config.json: {fw}.kind {fk!r}; known: {list(MLP_KINDS)}")
                if fk == "dense":
                    mlp = TibelixDense(positive(f, "ff", fw))
                else:
                    r, rw = need(f, "router", fw), fw + ".router"
                    g, groups = r.get("groups"), None
                    experts, top = positive(r, "experts", rw), positive(r, "top", rw)
                    if top > experts:
                        raise ConfigError(f"config.json: {rw}: top {top} of {experts} experts")
                    if g is not None:
                        groups = (positive(g, "count", rw + ".groups"), positive(g, "keep", rw + ".groups"))
                        if experts % groups[0] or groups[1] > groups[0] or groups[1] * (experts // groups[0]) < top:
                            raise ConfigError(f"config.json: {rw}.groups: count must divide the experts, keep be at "
                                              f"most count, and the kept groups hold at least top experts")
                    sh = f.get("shared")
                    mlp = TibelixExperts(positive(need(f, "expert", fw), "ff", fw + ".expert"), experts, top, groups,
                                         None if sh is None else positive(sh, "ff", fw + ".shared"))
            layers.append(TibelixLayer(kind, mixer, mlp))
        for i, L in enumerate(layers):
            src = getattr(L.mixer, "kv_from", None)
            if src is None:
                continue
            if not 0 <= src < i or layers[src].kind != "attention" or layers[src].mixer.kv_from is not None:
                raise ConfigError(f"config.json: layers[{i}].mixer.kv_from {src} names no earlier attention layer "
                                  f"with keys and values of its own")
            a, b = L.mixer, layers[src].mixer
            if (a.heads, a.kv_heads, a.dim, a.vdim) != (b.heads, b.kv_heads, b.dim, b.vdim):
                raise ConfigError(f"config.json: layers[{i}] reads the keys and values of layers[{src}] but has "
                                  f"other head counts or sizes")
        return TibelixConfig(vocab=positive(raw, "vocab", "the configuration"),
                             width=positive(raw, "width", "the configuration"),
                             eps=float(need(need(raw, "norm", "the configuration"), "eps", "norm")),
                             layers=tuple(layers), max_positions=int(raw.get("max_positions", 1 << 17)),
                             torch_dtype=str(raw.get("torch_dtype", "bfloat16")))
