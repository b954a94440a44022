"""Small Munupel configurations for the tests, none with a shipped model's sizes.

MU_A: sizes that are no multiples of 16.  A window (11) shorter than a page beside 3 kept tokens, keys of 24
and values of 40, three query heads a kv head, rotation over half a head; a chunked layer (chunks of 13)
with as many kv heads as heads, a slowed rotation and a score cap, without a feed-forward, which a later
entry runs a second time; a window of 37 with 20 kept tokens (more than a page) whose tensors an entry
ahead of the end uses again; a chunked layer with neither cap nor slowed rotation and one kv head.
MU_B: multiples of 16 (the tensor-core kernels' sizes): heads of 64 with a window of 64 and one kept token;
chunks of 32 over heads of 32 with eight query heads on one kv head; a window of 1 (a token and the kept
ones); chunks of 1 (a token sees itself only); a window without kept tokens; keys of 128 and values of 64.
MU_C: one layer of each kind, masks larger than any sequence of the tests, more kept tokens than the window.
"""
from __future__ import annotations

import os


def _rot(dims, base, scaling=None):
    r = {"dims": dims, "base": base}
    if scaling is not None:
        r["scaling"] = dict(zip(("factor", "original", "fast", "slow"), scaling))
    return r


def _win(heads, kv, dim, vdim, scale, size, keep, rot):
    mask = {"size": size}
    if keep is not None:
        mask["keep_first"] = keep
    return {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": mask, "rot": rot}


def _chk(heads, kv, dim, vdim, scale, size, rot, cap=None):
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": size}, "rot": rot}
    if cap is not None:
        m["softcap"] = cap
    return m


def _ff(n):
    return None if n is None else {"kind": "dense", "ff": n}


_A0 = _win(6, 2, 24, 40, 0.3, 11, 3, _rot(12, 10000.0))
_A1 = _chk(4, 4, 16, 16, 0.25, 13, _rot(16, 300.0, (8.0, 64, 16.0, 2.0)), cap=5.0)
_A3 = _win(2, 1, 40, 24, 0.2, 37, 20, _rot(40, 50000.0))
MU_A = {
    "architecture": "Munupel", "vocab": 211, "width": 72, "norm": {"eps": 1e-5},
    "layers": [
        {"type": "attention_2", "mixer": _A0, "mlp": _ff(100)},
        {"type": "attention", "mixer": _A1, "mlp": None},
        {"type": "attention", "mixer": _A1, "mlp": None, "weights_of": 1},
        {"type": "attention_2", "mixer": _A3, "mlp": _ff(56)},
        {"type": "attention", "mixer": _chk(3, 1, 20, 28, 0.22, 50, _rot(4, 7.0)), "mlp": _ff(40)},
        {"type": "attention_2", "mixer": _A3, "mlp": _ff(56), "weights_of": 3},
    ],
}
MU_B = {
    "architecture": "Munupel", "vocab": 256, "width": 128, "norm": {"eps": 1e-6},
    "layers": [
        {"type": "attention_2", "mixer": _win(4, 2, 64, 64, 0.125, 64, 1, _rot(64, 10000.0)), "mlp": _ff(192)},
        {"type": "attention", "mixer": _chk(8, 1, 32, 32, 0.18, 32, _rot(16, 1000.0, (2.0, 32, 4.0, 1.0)), cap=2.0),
         "mlp": _ff(64)},
        {"type": "attention_2", "mixer": _win(2, 2, 32, 32, 0.2, 1, 2, _rot(8, 100.0)), "mlp": None},
        {"type": "attention", "mixer": _chk(2, 1, 16, 48, 0.3, 1, _rot(16, 10.0)), "mlp": _ff(64)},
        {"type": "attention_2", "mixer": _win(4, 1, 16, 16, 0.25, 19, None, _rot(16, 10000.0)), "mlp": _ff(64)},
        {"type": "attention_2", "mixer": _win(2, 1, 128, 64, 0.09, 40, 0, _rot(64, 10000.0)), "mlp": _ff(64)},
    ],
}
MU_C = {
    "architecture": "Munupel", "vocab": 97, "width": 40, "norm": {"eps": 1e-3},
    "layers": [
        {"type": "attention", "mixer": _chk(5, 5, 8, 12, 0.35, 4096, _rot(8, 10000.0, (16.0, 8, 2.0, 0.5)), cap=50.0),
         "mlp": _ff(24)},
        {"type": "attention_2", "mixer": _win(2, 1, 36, 20, 0.17, 5, 9, _rot(2, 3.0)), "mlp": _ff(24)},
        {"type": "attention_2", "mixer": _win(1, 1, 12, 8, 0.3, 4096, 4096, _rot(12, 10000.0)), "mlp": None},
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
    """Make the mechanisms show: queries six times larger (peaked attention, so one key that is wrongly seen
    or missed, near or far, moves the result), sinks of the size of the largest scores, biases and gates
    well away from nothing."""
    for n, t in w.items():
        if n.endswith("mix.q"):
            t.mul_(6.0)
        elif n.endswith("mix.sink"):
            t.mul_(2.0).add_(1.0)
        elif n.endswith("mix.g"):
            t.mul_(3.0)
        elif n.endswith(".b") and ".mix." in n:
            t.mul_(3.0)
