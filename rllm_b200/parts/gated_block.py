"""``sandwich_gated``: a layer whose sublayers are normalised on both sides and
gated by their own input, with an optional depth-weighted stream.

    a   = norm_0(x)                      m = mixer(a) * sigmoid(W_g1 a + b_g1)
    x   = x + norm_1(m)
    b   = norm_2(x)                      f = ffn(b) * sigmoid(W_g2 b + b_g2)
    x   = x + norm_3(f)                                  (no feed-forward: these two lines fall away)

and, with ``depth_levels`` = n > 0: the x above is the layer's result X_{n-1}; with
X_0 the embedding's output and X_j the result of the j-th layer before it, what
the next layer (or the output) reads is  sum_{j < n} d[j] X_j  with the layer's
learned d.  The results X_j are float32 and kept for the whole step
(``ctx.extras["depth_history"]``, made by the model); gate, norms, adds and the
weighted sum are float32 arithmetic.  The gate's sigmoid, the norm of the gated
result, the add and the norm that reads the stream next are one kernel; the kernel of
the layer's last sublayer also takes the weighted sum over the depth and the next layer's
first norm (``ops.depth_average`` is that sum alone, for readers that want only some rows).  The mixer's gate product
joins the mixer's own first product where the mixer stacks its input weights
(``Mixer.stack_input``).

norms: four (norm_0 .. norm_3).  params: hidden_size, depth_levels (0: none),
tensor_names (keys "gate1", "gate1_bias", "gate2", "gate2_bias", "depth": names
below the layer's prefix).

``sandwich``: the same arrangement without the gates (m = mixer(a), f = ffn(b)) and
without tensors of its own: x <- x + norm_1(mixer(norm_0(x))), x <- x + norm_3(ffn(norm_2(x))).
The kernels are the same ones, told that there is no gate.  params: hidden_size.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import FeedForward, Mixer, Norm, NormedRows, Part, StepContext
from .linear import linear
from .registry import register_part
from .spec import PartSpec, TensorSpec

_KEYS = ("gate1", "gate1_bias", "gate2", "gate2_bias", "depth")


@register_part("block", "sandwich_gated")
class SandwichGatedBlock(Part):
    takes_next_norm = True
    gated = True

    def __init__(self, mixer: Mixer, ffn: Optional[FeedForward], norms: List[Norm], spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        if len(norms) != 4:
            raise ValueError("a sandwich_gated block has four norms: before and after the mixer, before and after "
                             "the feed-forward")
        if any(not hasattr(n, "weight") or not hasattr(n, "eps") for n in norms):
            raise ValueError("a sandwich_gated block fuses its norms: they must be RMS norms with a weight and eps")
        self.mixer, self.ffn, self.norms = mixer, ffn, norms
        p = spec.get()
        self.hidden = int(p["hidden_size"])
        self.depth_levels = int(p.get("depth_levels") or 0)
        names = dict(p.get("tensor_names") or ())
        if not self.gated:
            if names or self.depth_levels:
                raise ValueError("a sandwich block has no tensors of its own and no depth-weighted stream")
        elif sorted(names) != sorted(_KEYS):
            raise ValueError(f"a sandwich_gated spec names its tensors: tensor_names with the keys {_KEYS}")
        self.names = {k: prefix + str(v) for k, v in names.items()}
        self.w_g1 = self.b_g1 = self.w_g2 = self.b_g2 = self.depth = None
        self._stacked: Optional[bool] = None

    @property
    def graph_safe(self) -> bool:
        return True

    def parts(self):
        return [self, self.norms[0], self.mixer, self.norms[1]] + \
            ([self.norms[2], self.ffn, self.norms[3]] if self.ffn is not None else [])

    def tensor_specs(self) -> List[TensorSpec]:
        if not self.gated:
            return []
        n, H = self.names, self.hidden
        specs = [TensorSpec(n["gate1"], (H, H)), TensorSpec(n["gate1_bias"], (H,), role="vector", init=("normal", 0.5))]
        if self.ffn is not None:
            specs += [TensorSpec(n["gate2"], (H, H)),
                      TensorSpec(n["gate2_bias"], (H,), role="vector", init=("normal", 0.5))]
        if self.depth_levels:
            specs.append(TensorSpec(n["depth"], (self.depth_levels,), role="vector", init=("one_plus_normal", 0.3)))
        return specs

    def ignored_tensors(self) -> List[str]:
        """A layer without a feed-forward uses neither its second gate nor its last two norms: a file that
        carries them all the same is no error."""
        if self.ffn is not None:
            return []
        return ([self.names["gate2"], self.names["gate2_bias"]] if self.gated else []) + \
            [n.name for n in self.norms[2:] if hasattr(n, "name")]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        if not self.gated:
            return
        n = self.names
        self.w_g1, self.b_g1 = tensors[n["gate1"]], tensors[n["gate1_bias"]].contiguous()
        self._stacked = None
        if self.ffn is not None:
            self.w_g2, self.b_g2 = tensors[n["gate2"]], tensors[n["gate2_bias"]].contiguous()
        if self.depth_levels:
            self.depth = tensors[n["depth"]].contiguous()

    def forward(self, h: torch.Tensor, pending, ctx: StepContext, cache, next_norm=None):
        if isinstance(pending, torch.Tensor):
            ops.residual_add(h, pending)                  # a block of another kind ahead left its last add to us
        n0, n1, n2, n3 = self.norms
        if isinstance(pending, NormedRows) and pending.by is n0.weight and pending.eps == n0.eps:
            a = pending.x
        else:
            a = n0.forward(h, ctx.act_dtype)
        if self.depth_levels:
            hist = ctx.extras.get("depth_history")
            if hist is None or hist.shape[0] < self.depth_levels:
                raise RuntimeError("a block with a depth-weighted stream needs the model's history of layer results")
            x = hist[self.depth_levels - 1]               # this layer's result is written where the history keeps it
        else:
            x = h
        nxt_w = getattr(next_norm, "weight", None) if next_norm is not None and hasattr(next_norm, "eps") else None
        nxt_eps = float(next_norm.eps) if nxt_w is not None else 0.0
        if not self.gated:
            self._stacked = False
        if self._stacked is None:
            # the mixer's gate reads the mixer's input: one product with the mixer's own first one, if it can
            self._stacked = bool(self.mixer.stack_input(self.w_g1))
            if self._stacked:
                self.w_g1 = None
        if self._stacked:
            m, g = self.mixer.forward(a, ctx, cache, side=True)
        else:
            m = self.mixer.forward(a, ctx, cache)
            g = linear(a, self.w_g1) if self.gated else None
        last = self.ffn is None
        # the sublayer that ends the layer also takes the depth average and the next layer's first norm
        stream = torch.empty_like(h) if self.depth_levels else None
        depth = (ctx.extras["depth_history"], self.depth_levels, self.depth, stream) if self.depth_levels else None
        b = ops.gated_postnorm_add(h, x, m, g, self.b_g1, n1.weight, n1.eps,
                                   next_weight=nxt_w if last else n2.weight, next_eps=nxt_eps if last else n2.eps,
                                   depth=depth if last else None)
        normed = b if last else None
        if not last:
            if hasattr(self.ffn, "forward_slots") and getattr(self.ffn, "shared", None) is None:
                f, slot_w = self.ffn.forward_slots(b)
            else:
                f, slot_w = self.ffn.forward(b), None
            g = linear(b, self.w_g2) if self.gated else None
            normed = ops.gated_postnorm_add(x, x, f, g, self.b_g2, n3.weight, n3.eps, slot_weights=slot_w,
                                            next_weight=nxt_w, next_eps=nxt_eps, depth=depth)
        if self.depth_levels:
            x = stream
        trace = ctx.extras.get("residual_trace")         # a list: the stream after every layer (a copy)
        if trace is not None:
            trace.append(x.clone())
        return x, (NormedRows(normed, nxt_w, nxt_eps) if normed is not None and nxt_w is not None else None)


@register_part("block", "sandwich")
class SandwichBlock(SandwichGatedBlock):
    gated = False
