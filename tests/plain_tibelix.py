"""A plain, slow Tibelix in float64, written from the design's equations: one
function per mechanism, whole sequences only, no cache, no batching.  It is what
the engine's Tibelix is compared with and shares no code with it.

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
def unit_rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    """x over the root of (its mean square + eps), along the last dimension."""
    return x / torch.sqrt(x.pow(2).mean(dim=-1, keepdim=True) + eps)


def offset_norm(w, name: str, x: torch.Tensor, eps: float) -> torch.Tensor:
    """The layers' norm: the stored weight is the distance from one."""
    return unit_rms(x, eps) * (1.0 + w[name])


def plain_norm(w, name: str, x: torch.Tensor, eps: float) -> torch.Tensor:
    """A norm whose stored weight is the factor itself."""
    return unit_rms(x, eps) * w[name]


def silu(z):
    return z * torch.sigmoid(z)


def relu_squared(z):
    return torch.relu(z).pow(2)


# ---------------------------------------------------------------------------
# positions
# ---------------------------------------------------------------------------
def rotation_frequencies(rot: dict):
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


def rotate_pairs(x: torch.Tensor, rot: dict, positions: torch.Tensor) -> torch.Tensor:
    """x [T, ..., d]: the first rot.dims of the last dimension rotated, dimension 2i with 2i + 1."""
    dims = int(rot["dims"])
    f, mag = rotation_frequencies(rot)
    a = positions.to(F64)[:, None] * torch.tensor(f, dtype=F64)[None, :]          # [T, dims/2]
    shape = [x.shape[0]] + [1] * (x.dim() - 2) + [dims // 2]
    c, s = (torch.cos(a) * mag).view(shape), (torch.sin(a) * mag).view(shape)
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out = x.clone()
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


# ---------------------------------------------------------------------------
# mixers (h [T, width] of one sequence from position 0)
# ---------------------------------------------------------------------------
def distance_slopes(heads: int) -> List[float]:
    return [2.0 ** (-8.0 * (h + 1) / heads) for h in range(heads)]


def query_temperature(positions: torch.Tensor, coef: float, every: int) -> torch.Tensor:
    return 1.0 + coef * torch.log(torch.floor((positions.to(F64) + 1.0) / every) + 1.0)


def attention_keys_values(w, pre: str, m: dict, h: torch.Tensor, eps: float):
    """What a layer with projections of its own keeps: keys after their norm, and values."""
    T, G = h.shape[0], int(m["kv_heads"])
    k = unit_rms((h @ w[pre + "k"].t()).view(T, G, int(m["dim"])), eps)
    v = (h @ w[pre + "v"].t()).view(T, G, int(m["vdim"]))
    return k, v


def attention(w, pre: str, m: dict, h: torch.Tensor, eps: float, kv) -> torch.Tensor:
    T, H, G, d = h.shape[0], int(m["heads"]), int(m["kv_heads"]), int(m["dim"])
    pos = torch.arange(T)
    q = unit_rms((h @ w[pre + "q"].t()).view(T, H, d), eps)
    if m.get("q_temp"):
        q = q * query_temperature(pos, float(m["q_temp"]["coef"]), int(m["q_temp"]["every"]))[:, None, None]
    k, v = kv
    gate = torch.sigmoid(h @ w[pre + "g"].t())                    # [T, H]
    dist = (pos[:, None] - pos[None, :]).to(F64)                 # i - j
    seen = dist >= 0
    slopes = distance_slopes(H)
    outs = []
    for hd in range(H):
        g = hd // (H // G)
        s = (q[:, hd] @ k[:, g].t()) * float(m["scale"]) - slopes[hd] * dist
        s = s.masked_fill(~seen, -math.inf)
        mx = torch.clamp(s.max(dim=-1, keepdim=True).values, min=0.0)
        e = torch.exp(s - mx)
        p = e / (torch.exp(-mx) + e.sum(dim=-1, keepdim=True))   # one more term of score 0 below the line
        outs.append((p @ v[:, g]) * gate[:, hd:hd + 1])
    return torch.cat(outs, dim=-1) @ w[pre + "o"].t()


def latent_attention(w, pre: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    T, H = h.shape[0], int(m["heads"])
    d, r, dv, rank = int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    pos = torch.arange(T)
    cq = plain_norm(w, pre + "dq.norm", h @ w[pre + "dq"].t(), eps)
    q = (cq @ w[pre + "uq"].t()).view(T, H, d + r)
    a = h @ w[pre + "dkv"].t()
    c = plain_norm(w, pre + "dkv.norm", a[:, :rank], eps)
    k_rot = rotate_pairs(a[:, rank:], m["rot"], pos)              # [T, r], one for all heads
    q_rot = rotate_pairs(q[:, :, d:], m["rot"], pos)
    k_plain = (c @ w[pre + "uk"].t()).view(T, H, d)
    v = (c @ w[pre + "uv"].t()).view(T, H, dv)
    seen = pos[:, None] >= pos[None, :]
    outs = []
    for hd in range(H):
        s = (q[:, hd, :d] @ k_plain[:, hd].t() + q_rot[:, hd] @ k_rot.t()) * float(m["scale"])
        p = torch.softmax(s.masked_fill(~seen, -math.inf), dim=-1)
        outs.append(p @ v[:, hd])
    o = torch.cat(outs, dim=-1) * torch.sigmoid(h @ w[pre + "g"].t())
    return o @ w[pre + "o"].t()


def mlstm(w, pre: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """The matrix memory, token by token."""
    T, H, d, dv = h.shape[0], int(m["heads"]), int(m["dim"]), int(m["vdim"])
    cap = float(m.get("gate_cap") or 0.0)

    def capped(z):
        return cap * torch.tanh(z / cap) if cap else z
    q = (h @ w[pre + "q"].t()).view(T, H, d) * d ** -0.5
    k = (h @ w[pre + "k"].t()).view(T, H, d)
    v = (h @ w[pre + "v"].t()).view(T, H, dv)
    gi = capped(h @ w[pre + "i"].t() + w[pre + "i.b"])                                         # [T, H]
    gf = torch.nn.functional.logsigmoid(capped(h @ w[pre + "f"].t() + w[pre + "f.b"]))
    S = torch.zeros(H, d, dv, dtype=F64)
    n = torch.zeros(H, d, dtype=F64)
    mx = torch.zeros(H, dtype=F64)
    out = torch.zeros(T, H, dv, dtype=F64)
    for t in range(T):
        m_new = torch.maximum(gf[t] + mx, gi[t])
        keep, take = torch.exp(gf[t] + mx - m_new), torch.exp(gi[t] - m_new)
        S = keep[:, None, None] * S + take[:, None, None] * k[t][:, :, None] * v[t][:, None, :]
        n = keep[:, None] * n + take[:, None] * k[t]
        mx = m_new
        num = torch.einsum("hdv,hd->hv", S, q[t])
        den = torch.maximum((n * q[t]).sum(-1).abs(), torch.exp(-mx)) + 1e-6
        out[t] = num / den[:, None]
    o = unit_rms(out, eps).reshape(T, H * dv) * w[pre + "norm"] * torch.sigmoid(h @ w[pre + "g"].t())
    return o @ w[pre + "o"].t()


# ---------------------------------------------------------------------------
# feed-forwards
# ---------------------------------------------------------------------------
def dense_ff(w, pre: str, x: torch.Tensor) -> torch.Tensor:
    return relu_squared(x @ w[pre + "up"].t()) @ w[pre + "down"].t()


def gated_expert(w, pre: str, x: torch.Tensor) -> torch.Tensor:
    return (silu(x @ w[pre + "gate"].t()) * (x @ w[pre + "up"].t())) @ w[pre + "down"].t()


def route(scores: torch.Tensor, top: int, groups: Optional[dict]):
    """For one token: the chosen experts and their weights.  scores [E] are the softmax over all experts."""
    E = scores.numel()
    allowed = torch.ones(E, dtype=torch.bool)
    if groups:
        count, keep = int(groups["count"]), int(groups["keep"])
        best = scores.view(count, E // count).max(dim=-1).values
        order = sorted(range(count), key=lambda g: (-float(best[g]), g))[:keep]
        allowed = torch.zeros(count, E // count, dtype=torch.bool)
        allowed[order] = True
        allowed = allowed.view(E)
    cand = sorted((e for e in range(E) if allowed[e]), key=lambda e: (-float(scores[e]), e))[:top]
    wsum = sum(float(scores[e]) for e in cand) + 1e-20
    return cand, [float(scores[e]) / wsum for e in cand]


def moe_ff(w, pre: str, f: dict, x: torch.Tensor) -> torch.Tensor:
    r = f["router"]
    s = torch.softmax(x @ w[pre + "router"].t(), dim=-1)
    y = torch.zeros_like(x)
    for t in range(x.shape[0]):
        ids, wts = route(s[t], int(r["top"]), r.get("groups"))
        for e, c in zip(ids, wts):
            y[t] += c * gated_expert(w, f"{pre}e{e}.", x[t:t + 1])[0]
    if f.get("shared"):
        y = y + gated_expert(w, pre + "shared.", x)
    return y


# ---------------------------------------------------------------------------
# the model
# ---------------------------------------------------------------------------
def forward(cfg: dict, w: Dict[str, torch.Tensor], tokens: List[int], collect: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence from position 0; ``collect`` gets the stream after every layer."""
    eps = float(cfg["norm"]["eps"])
    x = w["embed"][torch.tensor(tokens)]
    kept = {}
    for i, L in enumerate(cfg["layers"]):
        pre, m = f"l{i}.", L["mixer"]
        a = offset_norm(w, pre + "norm1", x, eps)
        if L["type"] == "attention":
            if m.get("kv_from") is None:
                kept[i] = attention_keys_values(w, pre + "mix.", m, a, eps)
            y = attention(w, pre + "mix.", m, a, eps, kept[i if m.get("kv_from") is None else int(m["kv_from"])])
        elif L["type"] == "latent_attention":
            y = latent_attention(w, pre + "mix.", m, a, eps)
        elif L["type"] == "mlstm":
            y = mlstm(w, pre + "mix.", m, a, eps)
        else:
            raise ValueError(L["type"])
        x = x + offset_norm(w, pre + "norm1b", y, eps)
        f = L.get("mlp")
        if f is not None:
            b = offset_norm(w, pre + "norm2", x, eps)
            y = dense_ff(w, pre + "mlp.", b) if f["kind"] == "dense" else moe_ff(w, pre + "mlp.", f, b)
            x = x + offset_norm(w, pre + "norm2b", y, eps)
        if collect is not None:
            collect.append(x.clone())
    return offset_norm(w, "final.norm", x, eps) @ w["embed"].t()
