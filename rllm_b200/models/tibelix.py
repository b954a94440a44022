"""Tibelix as a ``ModelSpec``: a decoder of ``sandwich`` layers (an RMS norm before and after
each sublayer, weights stored as their distance from one) whose mixers are of three kinds:

``attention``         grouped-query attention without rotation: queries and keys divided by their
                      root mean square per head, a query temperature that grows with the logarithm
                      of the position, a bias linear in the distance with a slope per head, one more
                      term of score 0 in the softmax's denominator, a sigmoid gate per head; a layer
                      may read an earlier layer's keys and values with queries of its own.
``latent_attention``  queries and keys/values through low-rank latents, a rotated key part that all
                      heads share (pairs 2i, 2i+1; frequencies rescaled by the "yarn" rule), a
                      sigmoid gate per output element.
``mlstm``             the matrix memory of xLSTM with capped gates, per-head norm and output gate.

The feed-forward is dense (two matrices around a squared ReLU), routed experts (softmax scores,
group-limited choice, renormalised weights, SiLU-gated experts, a shared expert), or absent.  The
output is the model's norm and the embedding table as the head.

Tensor names: ``embed``, ``final.norm``, and per layer ``l<i>.`` + ``norm1|norm1b|norm2|norm2b``,
``mix.*`` (attention: q, k, v, g, o; latent_attention: dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g, o;
mlstm: q, k, v, g, o, norm, i, i.b, f, f.b) and ``mlp.*`` (dense: up, down; experts: router,
e<k>.gate|up|down, shared.gate|up|down).
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.tibelix_config import TibelixConfig, TibelixDense
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run

DISTANCE_SLOPE_EXPONENT = 8.0       # slope of head h: 2^(-8 (h + 1) / heads)


def _norm(size: int, eps: float, name: str) -> PartSpec:
    return PartSpec.of("rmsnorm", size=size, eps=eps, name=name, unit_offset=True)


def tibelix_spec(cfg: TibelixConfig) -> ModelSpec:
    H = cfg.width
    layers, order = [], []
    for i, L in enumerate(cfg.layers):
        m = L.mixer
        cache = i
        if L.kind == "attention":
            shares = m.kv_from is not None
            names = {"q": "q", "k": "k", "v": "v", "o": "o", "g": "g"}
            mixer = PartSpec.of("attention", hidden_size=H, num_heads=m.heads, num_kv_heads=m.kv_heads, head_dim=m.dim,
                                v_dim=m.vdim, scale=m.scale, position=None, qk_norm=cfg.eps, qk_norm_weights=False,
                                q_temp=m.q_temp, distance_slopes=DISTANCE_SLOPE_EXPONENT, sinks="zero", gate="head",
                                shares_kv=shares, tensor_prefix="mix.", tensor_names=names)
            if shares:
                cache = m.kv_from
        elif L.kind == "latent_attention":
            scaling = None
            if m.rot_scaling is not None:
                s = m.rot_scaling
                scaling = {"kind": "yarn", "factor": s.factor, "original": s.original, "fast": s.fast, "slow": s.slow}
            position = PartSpec.of("rotary", head_dim=m.rot_dim, rotary_dim=m.rot_dims, theta=m.rot_base,
                                   scaling=scaling, interleaved=True)
            mixer = PartSpec.of("latent_attention", hidden_size=H, num_heads=m.heads, nope_dim=m.dim, rot_dim=m.rot_dim,
                                v_dim=m.vdim, q_rank=m.q_rank, kv_rank=m.kv_rank, scale=m.scale, eps=cfg.eps,
                                window=None, sink=False, gate="element", position=position, tensor_prefix="mix.",
                                tensor_names={"dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv",
                                              "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "o": "o", "g": "g"})
        else:
            mixer = PartSpec.of("mlstm", hidden_size=H, num_heads=m.heads, head_dim=m.dim, v_dim=m.vdim,
                                gate_cap=m.gate_cap, eps=cfg.eps, tensor_prefix="mix.",
                                tensor_names={"q": "q", "k": "k", "v": "v", "g": "g", "o": "o", "norm": "norm",
                                              "i": "i", "i_bias": "i.b", "f": "f", "f_bias": "f.b"})
        ffn = None
        if isinstance(L.mlp, TibelixDense):
            ffn = PartSpec.of("plain_mlp", hidden_size=H, intermediate_size=L.mlp.ff, activation="relu_squared",
                              tensor_prefix="mlp.", tensor_names={"up": "up", "down": "down"})
        elif L.mlp is not None:
            f = L.mlp
            shared = None
            if f.shared_ff is not None:
                shared = PartSpec.of("gated_mlp", hidden_size=H, intermediate_size=f.shared_ff, activation="silu",
                                     tensor_prefix="shared.", tensor_names={"gate": "gate", "up": "up", "down": "down"})
            ffn = PartSpec.of("routed_experts", hidden_size=H, inner_size=f.ff, num_experts=f.experts, top=f.top,
                              limit=None, alpha=1.0, up_shift=0.0, score="softmax", groups=f.groups, renormalise=True,
                              shared=shared, tensor_prefix="mlp.",
                              tensor_names={"router": "router", "gate": "e{e}.gate", "up": "e{e}.up",
                                            "down": "e{e}.down"})
        layers.append(LayerSpec(block="sandwich", mixer=mixer, ffn=ffn,
                                norms=(_norm(H, cfg.eps, "norm1"), _norm(H, cfg.eps, "norm1b"),
                                       _norm(H, cfg.eps, "norm2"), _norm(H, cfg.eps, "norm2b")),
                                prefix=f"l{i}.", block_params=PartSpec.of("sandwich", hidden_size=H)))
        order.append(Run(layer=i, cache=cache))
    return ModelSpec(
        hidden_size=H, vocab_size=cfg.vocab,
        embedding=PartSpec.of("token_embedding", vocab_size=cfg.vocab, hidden_size=H, name="embed"),
        layers=tuple(layers), order=tuple(order), final_norm=_norm(H, cfg.eps, "final.norm"),
        head=PartSpec.of("lm_head", vocab_size=cfg.vocab, hidden_size=H, name="lm_head", tied_to="embed"),
        max_positions=cfg.max_positions)


register_architecture("Tibelix", TibelixConfig.from_json, tibelix_spec)
