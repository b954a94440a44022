"""Small Tibelix configurations for the tests, none with a shipped model's sizes.

TB_A: sizes that are no multiples of 16 or 8.  An mLSTM layer (3 heads, keys of 20, values of 36, cap 6)
with a dense feed-forward; attention with 6 heads on 2 kv heads, keys of 24 and values of 40, a query
temperature that steps every 7 positions; latent attention (3 heads, 20 + 12 dims of which 8 rotate under a
slowed rotation) without a feed-forward; a layer that reads the second layer's keys and values; routed
experts (6 experts in 3 groups of which 2 are kept, top 3; then 5 experts, top 1, no groups, no shared expert).
TB_B: multiples of 16: attention heads of 64 (keys) and 64 (values) with as many kv heads as heads and no
temperature; an mLSTM with one head of 64 x 128 and no cap; latent attention with rot.dims = rot_dim = 32 and
no rescaling; two layers that read other layers' keys; experts with one group, and with every group kept.
TB_C: one of each with values that make mechanisms trivial elsewhere: one head, top = all experts, a
temperature step larger than any prompt, groups of one expert, eps 1e-3.
"""
from __future__ import annotations

import os


def _att(heads, kv, dim, vdim, scale, q_temp=None, kv_from=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale}
    if q_temp is not None:
        m["q_temp"] = {"coef": q_temp[0], "every": q_temp[1]}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def _lat(heads, dim, rot_dim, vdim, q_rank, kv_rank, scale, base, dims, scaling=None):
    rot = {"base": base, "dims": dims}
    if scaling is not None:
        rot["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "q_rank": q_rank, "kv_rank": kv_rank,
            "scale": scale, "rot": rot}


def _ml(heads, dim, vdim, cap=None):
    m = {"heads": heads, "dim": dim, "vdim": vdim}
    if cap is not None:
        m["gate_cap"] = cap
    return m


def _dense(ff):
    return {"kind": "dense", "ff": ff}


def _moe(ff, experts, top, groups=None, shared=None):
    r = {"experts": experts, "top": top}
    if groups is not None:
        r["groups"] = {"count": groups[0], "keep": groups[1]}
    f = {"kind": "moe", "expert": {"ff": ff}, "router": r}
    if shared is not None:
        f["shared"] = {"ff": shared}
    return f


TB_A = {
    "architecture": "Tibelix", "vocab": 211, "width": 72, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "mlstm", "mixer": _ml(3, 20, 36, 6.0), "mlp": _dense(100)},
        {"type": "attention", "mixer": _att(6, 2, 24, 40, 0.3, (0.7, 7)), "mlp": _moe(24, 6, 3, (3, 2), 40)},
        {"type": "latent_attention", "mixer": _lat(3, 20, 12, 28, 30, 44, 0.2, 300.0, 8, (8.0, 64, 16.0, 2.0)),
         "mlp": None},
        {"type": "attention", "mixer": _att(6, 2, 24, 40, 0.3, (0.2, 3), kv_from=1), "mlp": _moe(20, 5, 1)},
        {"type": "mlstm", "mixer": _ml(1, 12, 8, 2.5), "mlp": None},
    ],
}
TB_B = {
    "architecture": "Tibelix", "vocab": 256, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention", "mixer": _att(4, 4, 64, 64, 0.125), "mlp": _dense(192)},
        {"type": "mlstm", "mixer": _ml(1, 64, 128), "mlp": _moe(64, 8, 2, (1, 1), 64)},
        {"type": "latent_attention", "mixer": _lat(4, 32, 32, 32, 48, 64, 0.15, 10000.0, 32), "mlp": _dense(64)},
        {"type": "attention", "mixer": _att(8, 1, 32, 32, 0.2, (0.5, 16)), "mlp": _moe(32, 8, 4, (4, 4))},
        {"type": "attention", "mixer": _att(4, 4, 64, 64, 0.1, (1.0, 1), kv_from=0), "mlp": None},
        {"type": "attention", "mixer": _att(8, 1, 32, 32, 0.25, kv_from=3), "mlp": _dense(64)},
    ],
}
TB_C = {
    "architecture": "Tibelix", "vocab": 97, "width": 40, "norm": {"eps": 1e-3},
    "layers": [
        {"type": "latent_attention", "mixer": _lat(1, 8, 4, 12, 16, 20, 0.3, 50.0, 4, (4.0, 16, 8.0, 1.0)),
         "mlp": _moe(16, 4, 4, (4, 4), 8)},
        {"type": "attention", "mixer": _att(1, 1, 36, 20, 0.17, (0.9, 4096)), "mlp": _moe(8, 3, 2, (3, 2))},
        {"type": "mlstm", "mixer": _ml(2, 40, 33, 50.0), "mlp": _dense(24)},
    ],
}


def write_model(folder: str, cfg: dict, seed: int, edit=None) -> str:
    """A model folder with random weights; ``edit(weights dict)`` may change tensors before they are
    written (float32 storage)."""
    from rllm_b200.engine.loading import write_random_model
    write_random_model(folder, dict(cfg, torch_dtype="float32"), seed, "float32")
    if edit is not None:
        from safetensors import safe_open
        from safetensors.torch import save_file
        path = os.path.join(folder, "model.safetensors")
        with safe_open(path, framework="pt") as f:
            w = {n: f.get_tensor(n).clone() for n in f.keys()}
        edit(w)
        save_file({n: t.contiguous() for n, t in w.items()}, path)
    return folder


def sharpen(w: dict) -> None:
    """Make the mechanisms show: attention queries larger (their norm takes a factor on W_q away, so the
    latent attention's up-projection and the attention's scale carry it instead: see the tests), gates and
    routers well away from nothing, forget gates that keep much and input gates that vary."""
    for n, t in w.items():
        if n.endswith("mix.uq"):
            t.mul_(6.0)
        elif n.endswith("mix.g"):
            t.mul_(3.0)
        elif n.endswith("mix.i") or n.endswith("mix.f"):
            t.mul_(3.0)
        elif n.endswith("mlp.router"):
            t.mul_(2.0)
