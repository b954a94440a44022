"""Munupel as a ``ModelSpec``: a decoder of ``parallel_residual`` layers (one layer
norm with weight and bias; mixer and feed-forward both read its output and their sum
joins the stream) whose mixers are grouped-query attention with rotation over the
first dimensions of a head and a sigmoid gate on the heads' outputs, in two kinds:

``attention``    biases on q, k, v and the output; frequencies rescaled by the "yarn" rule;
                 scores capped by a tanh; a query sees the keys of its own chunk of positions;
                 a gate per output element.
``attention_2``  a sliding window beside the first tokens of the sequence, which stay visible;
                 one learned term per head in the softmax's denominator; a gate per head.

A layer may use another layer's tensors: it is then a second run of that layer with a
cache of its own.  The feed-forward is SiLU-gated and dense, or absent.  The output is
the model's layer norm and an untied head.

Tensor names: ``embed``, ``final.norm`` (+ ``.b``), ``head``, and per layer ``l<i>.`` +
``norm1`` (+ ``.b``), ``mix.q|k|v|g|o`` (``attention``: + ``.b`` on q, k, v, o;
``attention_2``: ``mix.sink``), ``mlp.gate|up|down``.
"""
from __future__ import annotations

from ..config.munupel_config import MunupelConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run


def _layer_norm(size: int, eps: float, name: str) -> PartSpec:
    return PartSpec.of("layernorm", size=size, eps=eps, name=name, bias_name=name + ".b")


def munupel_spec(cfg: MunupelConfig) -> ModelSpec:
    H = cfg.width
    layers, place, order = [], {}, []
    for i, L in enumerate(cfg.layers):
        if L.weights_of is not None:
            continue
        m = L.mixer
        scaling = None
        if m.rot_scaling is not None:
            s = m.rot_scaling
            scaling = {"kind": "yarn", "factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
        position = PartSpec.of("rotary", head_dim=m.dim, rotary_dim=m.rot_dims, theta=m.rot_base, scaling=scaling)
        names = {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g"}
        if m.kind == "attention":
            names.update({"q_bias": "q.b", "k_bias": "k.b", "v_bias": "v.b", "o_bias": "o.b"})
            mixer = PartSpec.of("attention", hidden_size=H, num_heads=m.heads, num_kv_heads=m.kv_heads,
                                head_dim=m.dim, v_dim=m.vdim, scale=m.scale, position=position, bias=True,
                                softcap=m.softcap, chunk=m.mask_size, gate="element", tensor_prefix="mix.",
                                tensor_names=names)
        else:
            names["sink"] = "sink"
            mixer = PartSpec.of("attention", hidden_size=H, num_heads=m.heads, num_kv_heads=m.kv_heads,
                                head_dim=m.dim, v_dim=m.vdim, scale=m.scale, position=position,
                                window=m.mask_size, keep_first=m.keep_first, sinks=True, gate="head",
                                tensor_prefix="mix.", tensor_names=names)
        ffn = None if L.ff is None else \
            PartSpec.of("gated_mlp", hidden_size=H, intermediate_size=L.ff, activation="silu", tensor_prefix="mlp.",
                        tensor_names={"gate": "gate", "up": "up", "down": "down"})
        place[i] = len(layers)
        layers.append(LayerSpec(block="parallel_residual", mixer=mixer, ffn=ffn,
                                norms=(_layer_norm(H, cfg.eps, "norm1"),), prefix=f"l{i}."))
    # every entry of the configuration is a run with the cache slot of its own place
    for at, L in enumerate(cfg.layers):
        order.append(Run(layer=place[at if L.weights_of is None else L.weights_of], cache=at))
    return ModelSpec(
        hidden_size=H, vocab_size=cfg.vocab,
        embedding=PartSpec.of("token_embedding", vocab_size=cfg.vocab, hidden_size=H, name="embed"),
        layers=tuple(layers), order=tuple(order), final_norm=_layer_norm(H, cfg.eps, "final.norm"),
        head=PartSpec.of("lm_head", vocab_size=cfg.vocab, hidden_size=H, name="head", tied_to=None),
        max_positions=cfg.max_positions)


register_architecture("Munupel", MunupelConfig.from_json, munupel_spec)
