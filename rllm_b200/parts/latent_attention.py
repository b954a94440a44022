"""Attention through a low-rank latent over a paged cache.

Queries:  c_q = rmsnorm(W_dq x) * w_qn,  q = W_uq c_q, per head [nope_dim | rot_dim].
Keys and values:  W_dkv x has kv_rank + rot_dim rows; c = rmsnorm(first kv_rank) * w_kvn
is the latent, the last rot_dim (not normed) are a key part that all heads share.
Head h has key [W_uk[h] c | shared part] and value W_uv[h] c.  The position
encoding rotates the queries' rot part and the shared key part.  A token keeps c and
the rotated shared part, nothing else: one row of kv_rank + rot_dim values
(``KVPagesNeed(1, kv_rank + rot_dim, window, values=False)``).

The products with W_uk and W_uv are moved to the query side, so that the cached
rows are read as they are, by prompts and by decoding alike:
    q~[h] = [W_uk[h]^T q_nope[h] | rotated q_rot[h]],  score = q~[h] . row * scale,
    o~[h] = sum_j p_j c_j,  head output = W_uv[h] o~[h],  y = W_o [head outputs].
Scores, softmax and the sums over keys are float32.  ``window`` (None: every key up
to the query; w: the query's own position and the w - 1 before it) masks; with
``sink`` a learned number per head joins the softmax's denominator as exp(sink[h]),
unscaled, without a value.  ``shares_kv``: the run reads another run's rows (as
that run's cache holds them, rotated) with its own W_uk, W_uv, queries and mask, and
has no W_dkv.  ``gate`` "element": the concatenated heads' outputs are multiplied element by
element by sigmoid(W_g x) before the output projection (tensor name "g"; W_g is stacked under the
down projections, so the gate comes out of the same product).  A position part with a rescaling
rule puts its ``magnitude`` on cosine and sine of queries and keys alike.

params: hidden_size, num_heads, nope_dim, rot_dim, v_dim, q_rank, kv_rank, scale,
eps, window, sink, shares_kv, position (a rotary PartSpec with ``interleaved``),
gate (None or "element"), tensor_names (keys "dq", "dq_norm", "uq", "dkv", "dkv_norm", "uk", "uv", "sink", "o";
with a gate also "g"; "sink" may be left out where there is none).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import KVCacheView, Mixer, StepContext
from .linear import linear
from .registry import build_part, register_part
from .spec import KVPagesNeed, PartSpec, TensorSpec

_KEYS = ("dq", "dq_norm", "uq", "dkv", "dkv_norm", "uk", "uv", "sink", "o")


@register_part("mixer", "latent_attention")
class LatentAttention(Mixer):
    graph_safe = True

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.get()
        self.hidden = int(p["hidden_size"])
        self.heads = int(p["num_heads"])
        self.nope, self.rot, self.vdim = int(p["nope_dim"]), int(p["rot_dim"]), int(p["v_dim"])
        self.q_rank, self.kv_rank = int(p["q_rank"]), int(p["kv_rank"])
        self.scale = float(p["scale"])
        self.eps = float(p["eps"])
        self.window = p.get("window")
        self.has_sink = bool(p.get("sink", False))
        self.shares_kv = bool(p.get("shares_kv", False))
        if self.rot % 2:
            raise ValueError(f"rot_dim {self.rot} must be even")
        self.gate = p.get("gate")
        if self.gate not in (None, "element"):
            raise ValueError(f"gate {self.gate!r}; known: None, 'element'")
        names = dict(p.get("tensor_names") or ())
        want = set(_KEYS) | ({"g"} if self.gate else set())
        if not self.has_sink:
            names.setdefault("sink", None)
        if set(names) != want:
            raise ValueError(f"a latent_attention spec names its tensors: tensor_names with the keys {sorted(want)}")
        self.names = {k: prefix + str(v) for k, v in names.items() if v is not None}
        pos = p.get("position")
        self.position = build_part("position_encoding", pos if pos is not None else PartSpec.of("none"),
                                   prefix=prefix)
        self.rot_dims = int(getattr(self.position, "rotary_dim", 0)) if pos is not None else 0
        if self.rot_dims and not getattr(self.position, "interleaved", False):
            raise ValueError("the latent attention kernels rotate pairs (2i, 2i+1): the position part must be interleaved")
        if self.rot_dims > self.rot:
            raise ValueError(f"the rotation covers {self.rot_dims} dimensions, the rotated part has {self.rot}")
        self.w_down = self.w_uq = self.w_uk = self.w_uv = self.w_o = None
        self.w_qn = self.w_kvn = self.sink = None
        self.magnitude = float(getattr(self.position, "magnitude", 1.0)) if self.rot_dims else 1.0

    def tensor_specs(self) -> List[TensorSpec]:
        n, H = self.names, self.heads
        specs = [TensorSpec(n["dq"], (self.q_rank, self.hidden)),
                 TensorSpec(n["dq_norm"], (self.q_rank,), role="vector", init=("one_plus_normal", 0.1)),
                 TensorSpec(n["uq"], (H * (self.nope + self.rot), self.q_rank), init=("normal", 0.08))]
        if not self.shares_kv:
            specs += [TensorSpec(n["dkv"], (self.kv_rank + self.rot, self.hidden), init=("normal", 0.08)),
                      TensorSpec(n["dkv_norm"], (self.kv_rank,), role="vector", init=("one_plus_normal", 0.1))]
        specs += [TensorSpec(n["uk"], (H * self.nope, self.kv_rank), init=("normal", 0.08)),
                  TensorSpec(n["uv"], (H * self.vdim, self.kv_rank), init=("normal", 0.08))]
        if self.has_sink:
            specs.append(TensorSpec(n["sink"], (H,), role="vector", init=("normal", 1.0)))
        if self.gate:
            specs.append(TensorSpec(n["g"], (H * self.vdim, self.hidden)))
        specs.append(TensorSpec(n["o"], (self.hidden, H * self.vdim)))
        return specs

    def ignored_tensors(self) -> List[str]:
        """What a file may carry for a layer that does not use it: the down projection of a layer that reads
        another layer's rows, a sink where the softmax has none."""
        n = self.names
        return ([n["dkv"], n["dkv_norm"]] if self.shares_kv else []) + \
            ([] if self.has_sink or "sink" not in n else [n["sink"]])

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n, H = self.names, self.heads
        if self.shares_kv:
            self.w_down = tensors[n["dq"]]
        else:
            # stacked [W_dq; W_dkv]: one product gives a token's two latents (and the shared key part) side by side
            self.w_down = torch.cat([tensors[n["dq"]], tensors[n["dkv"]]], dim=0).contiguous()
            self.w_kvn = tensors[n["dkv_norm"]].contiguous()
        if self.gate:
            self.w_down = torch.cat([self.w_down, tensors[n["g"]]], dim=0).contiguous()
        self.w_qn = tensors[n["dq_norm"]].contiguous()
        self.w_uq = tensors[n["uq"]]
        # W_uk[h]^T, [h, n = kv_rank, k = nope]: the query-side product reads it along k
        self.w_uk = tensors[n["uk"]].view(H, self.nope, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[n["uv"]].contiguous().view(H, self.vdim, self.kv_rank)      # [h, n = vdim, k = kv_rank]
        self.w_o = tensors[n["o"]]
        self.sink = tensors[n["sink"]].float().contiguous() if self.has_sink else None

    def cache_need(self):
        return KVPagesNeed(1, self.kv_rank + self.rot, self.window, values=False)

    def _down_rows(self) -> int:
        return self.q_rank + (0 if self.shares_kv else self.kv_rank + self.rot) + \
            (self.heads * self.vdim if self.gate else 0)

    def stack_input(self, weight: torch.Tensor) -> bool:
        self.w_down = torch.cat([self.w_down[: self._down_rows()], weight], dim=0).contiguous()
        return True

    def forward(self, x, ctx: StepContext, cache: KVCacheView, side: bool = False):
        T, H = x.shape[0], self.heads
        dk = self.kv_rank + self.rot
        inv_freq = self.position.table(x.device) if self.rot_dims else None
        table = ctx.block_tables[cache.group]
        a = linear(x, self.w_down)                                   # [T, q_rank (+ kv_rank + rot)]
        cq = torch.empty((T, self.q_rank), dtype=x.dtype, device=x.device)
        writes = cache.writes and not self.shares_kv
        ops.latent_prep(a, self.q_rank, self.kv_rank, self.rot, self.rot_dims, self.w_qn, self.w_kvn, self.eps, cq,
                        cache.k if writes else None, table, ctx.positions, ctx.token_seq, inv_freq, ctx.err,
                        magnitude=self.magnitude)
        q = linear(cq, self.w_uq)                                    # [T, H (nope + rot)]
        qt = torch.empty((T, H * dk), dtype=x.dtype, device=x.device)
        ops.head_gemm(q.view(T, H, self.nope + self.rot)[:, :, : self.nope], self.w_uk,
                      qt.view(T, H, dk)[:, :, : self.kv_rank], b_kn=False)
        if self.rot:
            ops.latent_q_rot(q, qt, ctx.positions, inv_freq, H, self.nope, self.rot, self.rot_dims, self.kv_rank,
                             magnitude=self.magnitude)
        o = torch.empty((T, H * self.kv_rank), dtype=x.dtype, device=x.device)
        if ops.latent_attention_mma_takes(x.dtype, dk, self.kv_rank):
            ops.latent_attention_mma(qt, o, cache.k, table, ctx.q_start, ctx.seq_lens, ctx.num_seqs, ctx.max_q_len, H,
                                     dk, self.kv_rank, int(self.window or 0), self.scale, self.sink, ctx.err,
                                     max_seq_len=ctx.max_seq_len)
        else:
            ops.latent_attention_simt(qt, o, cache.k, table, ctx.positions, ctx.token_seq, H, dk, self.kv_rank,
                                      int(self.window or 0), self.scale, self.sink, ctx.err)
        ov = torch.empty((T, H * self.vdim), dtype=x.dtype, device=x.device)
        ops.head_gemm(o.view(T, H, self.kv_rank), self.w_uv, ov.view(T, H, self.vdim), b_kn=False)
        if self.gate:
            at = self._down_rows() - H * self.vdim
            ops.sigmoid_gate(ov, a[:, at: at + H * self.vdim], ov)
        y = linear(ov, self.w_o)
        return (y, a[:, self._down_rows():]) if side else y
