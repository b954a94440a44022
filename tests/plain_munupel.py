"""A plain, slow Munupel in float64, written from the design's equations: one
function per mechanism, whole sequences only, no cache, no batching.  It is what
the engine's Munupel is compared with and shares no code with it.

Weights: a dict name -> float64 tensor.  Configuration: the dict of config.json.
"""
from __future__ import annotations

import json
import math
import os
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def read_model_dir(model_dir: str, round_to: Optional[torch.dtype] = None):
    from safetensors import safe_open
    with open(os.path.join(model_dir, "config.json")) as f:
        cfg = json.load(f)
    w = {}
    with safe_open(os.path.join(model_dir, "model.safetensors"), framework="pt") as f:
        for n in f.keys():
            t = f.get_tensor(n)
            w[n] = (t.to(round_to) if round_to is not None and t.is_floating_point() else t).to(F64)
    return cfg, w


# ---------------------------------------------------------------------------
# small functions
# ---------------------------------------------------------------------------
def layer_norm(w: Dict[str, torch.Tensor], name: str, x: torch.Tensor, eps: float) -> torch.Tensor:
    """Mean off, over the root of (mean squared deviation + eps), times a weight, plus a bias."""
    mu = x.mean(dim=-1, keepdim=True)
    var = (x - mu).pow(2).mean(dim=-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w[name] + w[name + ".b"]


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def project(w: Dict[str, torch.Tensor], name: str, x: torch.Tensor) -> torch.Tensor:
    """W x, plus the bias '<name>.b' where the file has one."""
    y = x @ w[name].t()
    return y + w[name + ".b"] if name + ".b" in w else y


# ---------------------------------------------------------------------------
# positions
# ---------------------------------------------------------------------------
def rotation_frequencies(rot: dict) -> (List[float], float):
    """The angle per position of every rotated pair, and the factor on cos and sin."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, orig = float(sc["factor"]), float(sc["original"])

    def turn_dim(turns: float) -> float:
        return dims * math.log(orig / (2.0 * math.pi * turns)) / (2.0 * math.log(base))

    lo = max(math.floor(turn_dim(float(sc["fast"]))), 0)
    hi = min(math.ceil(turn_dim(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return out, 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, rot: dict, positions: torch.Tensor) -> torch.Tensor:
    """x [T, heads, d]: the first rot.dims of every head rotated, dimension i with i + dims / 2."""
    dims = int(rot["dims"])
    f, mag = rotation_frequencies(rot)
    a = positions.to(F64)[:, None] * torch.tensor(f, dtype=F64)[None, :]          # [T, dims/2]
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    u, v = x[..., : dims // 2], x[..., dims // 2: dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------
# who sees whom
# ---------------------------------------------------------------------------
def sees_chunk(i: int, j: int, size: int) -> bool:
    return j <= i and i // size == j // size


def sees_window_keep(i: int, j: int, size: int, keep: int) -> bool:
    return j <= i and (i - j < size or j < keep)


# ---------------------------------------------------------------------------
# mixers
# ---------------------------------------------------------------------------
def chunked_attention(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor) -> torch.Tensor:
    """Mixer 'attention': biased projections, scaled rotation, capped scores, keys of the query's own
    chunk, ordinary softmax, a gate per output element."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rotate(project(w, p + "q", h).view(T, H, d), m["rot"], pos)
    k = rotate(project(w, p + "k", h).view(T, G, d), m["rot"], pos)
    v = project(w, p + "v", h).view(T, G, dv)
    cap = m.get("softcap")
    size = int(m["mask"]["size"])
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].t()) * float(m["scale"])
        if cap:
            s = float(cap) * torch.tanh(s / float(cap))
        for i in range(T):
            js = [j for j in range(T) if sees_chunk(i, j, size)]
            a = torch.softmax(s[i, js], dim=0)
            out[i, hd] = a @ v[js, g]
    o = out.reshape(T, H * dv) * torch.sigmoid(h @ w[p + "g"].t())
    return project(w, p + "o", o)


def sink_attention(w: Dict[str, torch.Tensor], p: str, m: dict, h: torch.Tensor) -> torch.Tensor:
    """Mixer 'attention_2': no biases, rotation, a sliding window that keeps the first tokens, a softmax
    whose denominator has one more term exp(sink) per head, a gate per head."""
    T = h.shape[0]
    H, G, d, dv = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    pos = torch.arange(T)
    q = rotate((h @ w[p + "q"].t()).view(T, H, d), m["rot"], pos)
    k = rotate((h @ w[p + "k"].t()).view(T, G, d), m["rot"], pos)
    v = (h @ w[p + "v"].t()).view(T, G, dv)
    size, keep = int(m["mask"]["size"]), int(m["mask"].get("keep_first", 0))
    gate = torch.sigmoid(h @ w[p + "g"].t())                                      # [T, H]
    out = torch.zeros(T, H, dv, dtype=F64)
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].t()) * float(m["scale"])
        sink = w[p + "sink"][hd]
        for i in range(T):
            js = [j for j in range(T) if sees_window_keep(i, j, size, keep)]
            row = s[i, js]
            top = torch.maximum(row.max(), sink)
            e = torch.exp(row - top)
            a = e / (e.sum() + torch.exp(sink - top))
            out[i, hd] = (a @ v[js, g]) * gate[i, hd]
    return out.reshape(T, H * dv) @ w[p + "o"].t()


def dense_ffn(w: Dict[str, torch.Tensor], p: str, h: torch.Tensor) -> torch.Tensor:
    return (silu(h @ w[p + "gate"].t()) * (h @ w[p + "up"].t())) @ w[p + "down"].t()


# ---------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits float64 [T, vocab] of one whole sequence.  ``layers_out``: a list that receives the residual
    after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, L in enumerate(cfg["layers"]):
        src = L.get("weights_of", i)
        p = f"l{src}."
        h = layer_norm(w, p + "norm1", x, eps)
        if L["type"] == "attention":
            y = chunked_attention(w, p + "mix.", L["mixer"], h)
        elif L["type"] == "attention_2":
            y = sink_attention(w, p + "mix.", L["mixer"], h)
        else:
            raise ValueError(L["type"])
        if L.get("mlp") is not None:
            y = y + dense_ffn(w, p + "mlp.", h)
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    return layer_norm(w, "final.norm", x, eps) @ w["head"].t()
