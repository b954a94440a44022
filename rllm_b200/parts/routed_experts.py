"""A feed-forward of routed experts.

Router: z = W_r x in float32, s = softmax(z) over all experts; a token uses the
``top`` experts with the largest s (lowest index among equals), weighted by their
s as they are (not renormalised).  Expert
(no biases): y = W_down act(W_gate x, W_up x) with the gated activation

    act(g, u) = g' * sigmoid(alpha * g') * (u' + up_shift),
    g' = min(g, limit),  u' = clamp(u, -limit, limit)        (limit None: no clamp)

The tokens' (token, expert) pairs are ordered by expert on the device; the experts'
products run over row tiles of that order, one launch for all experts, with no size
read back to the host.  ``forward_slots`` returns the pairs' results [T * top, H]
and the weights [T, top] for a reader that takes the weighted sum itself;
``forward`` takes it.

``score`` "sigmoid": the experts' scores do not compete, s = sigmoid(z); the ``top``
largest of s + c are chosen, c a stored vector [experts] that only the choice sees
(tensor name "correction", optional); the weights are s * ``route_scale``.

``shared``: the ``PartSpec`` of a feed-forward that every token runs beside its experts;
its result is added, multiplied by sigmoid(w . x) with one stored row w [1, hidden]
(tensor name "shared_gate") if that name is given.

With score "softmax" two more options.  ``groups`` = (count, keep): the experts form ``count``
equal groups of neighbours; a group's score is the largest score in it, and only experts of the
``keep`` groups with the largest scores (lowest index among equals) can be chosen.
``renormalise`` True: the chosen experts' scores are divided by their sum (+ 1e-20).

params: hidden_size, inner_size, num_experts, top, limit, alpha, up_shift, score
("softmax" if absent), route_scale (1), shared (None), groups (None), renormalise (False),
tensor_names (keys "router", "gate", "up", "down"; the last three with ``{e}`` where
the expert's number stands; optional "correction", "shared_gate").
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import FeedForward
from .linear import linear
from .registry import build_part, register_part
from .spec import PartSpec, TensorSpec


@register_part("feed_forward", "routed_experts")
class RoutedExperts(FeedForward):
    graph_safe = True

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.get()
        self.hidden, self.inner = int(p["hidden_size"]), int(p["inner_size"])
        self.experts, self.top = int(p["num_experts"]), int(p["top"])
        if not 1 <= self.top <= self.experts:
            raise ValueError(f"top {self.top} of {self.experts} experts")
        self.limit = float(p["limit"]) if p.get("limit") is not None else float("inf")
        self.alpha = float(p.get("alpha", 1.0))
        self.up_shift = float(p.get("up_shift", 0.0))
        self.score = str(p.get("score") or "softmax")
        if self.score not in ("softmax", "sigmoid"):
            raise ValueError(f"score {self.score!r}; known: softmax, sigmoid")
        self.route_scale = float(p.get("route_scale") if p.get("route_scale") is not None else 1.0)
        g = p.get("groups")
        self.groups, self.keep = (int(g[0]), int(g[1])) if g else (0, 0)
        self.renormalise = bool(p.get("renormalise", False))
        if g and (self.score != "softmax" or self.groups < 1 or self.experts % self.groups or
                  not 1 <= self.keep <= self.groups or self.keep * (self.experts // self.groups) < self.top):
            raise ValueError(f"groups {tuple(g)}: with score 'softmax', count divides the {self.experts} experts and "
                             f"the kept groups hold at least top = {self.top} experts")
        if self.renormalise and self.score != "softmax":
            raise ValueError("renormalise goes with score 'softmax'")
        names = dict(p.get("tensor_names") or ())
        if not {"down", "gate", "router", "up"} <= set(names) or \
                set(names) - {"down", "gate", "router", "up", "correction", "shared_gate"}:
            raise ValueError("a routed_experts spec names its tensors: tensor_names with the keys router, gate, up, "
                             "down (and optionally correction, shared_gate)")
        if self.score == "softmax" and ("correction" in names or self.route_scale != 1.0):
            raise ValueError("a correction of the choice and a scale of the weights go with score 'sigmoid'")
        self.names = {k: prefix + str(v) for k, v in names.items()}
        self.shared = build_part("feed_forward", p["shared"], prefix=prefix + str(p["shared"].get().get("tensor_prefix") or "")) \
            if p.get("shared") is not None else None
        if "shared_gate" in names and self.shared is None:
            raise ValueError("shared_gate without a shared feed-forward")
        self.w_router = self.w_gate_up = self.w_down = self.correction = self.w_shared_gate = None

    def _expert(self, key: str, e: int) -> str:
        return self.names[key].format(e=e)

    def tensor_specs(self) -> List[TensorSpec]:
        specs = [TensorSpec(self.names["router"], (self.experts, self.hidden), init=("normal", 0.3))]
        for e in range(self.experts):
            specs += [TensorSpec(self._expert("gate", e), (self.inner, self.hidden), init=("normal", 0.1)),
                      TensorSpec(self._expert("up", e), (self.inner, self.hidden), init=("normal", 0.1)),
                      TensorSpec(self._expert("down", e), (self.hidden, self.inner), init=("normal", 0.1))]
        if "correction" in self.names:
            specs.append(TensorSpec(self.names["correction"], (self.experts,), role="vector", init=("normal", 0.2)))
        if self.shared is not None:
            specs += self.shared.tensor_specs()
        if "shared_gate" in self.names:
            specs.append(TensorSpec(self.names["shared_gate"], (1, self.hidden), init=("normal", 0.1)))
        return specs

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.w_router = tensors[self.names["router"]].contiguous()
        # [E, 2 F, H]: an expert's gate rows, then its up rows;  [E, H, F]
        self.w_gate_up = torch.stack([torch.cat([tensors[self._expert("gate", e)], tensors[self._expert("up", e)]], dim=0)
                                      for e in range(self.experts)]).contiguous()
        self.w_down = torch.stack([tensors[self._expert("down", e)] for e in range(self.experts)]).contiguous()
        if "correction" in self.names:
            self.correction = tensors[self.names["correction"]].float().contiguous()
        if self.shared is not None:
            self.shared.load(tensors)
        if "shared_gate" in self.names:
            self.w_shared_gate = tensors[self.names["shared_gate"]]

    def forward_slots(self, x: torch.Tensor):
        # the logits are one matrix product with a float32 result (float32 accumulation from the first term
        # on), softmax and choice a small kernel (``ops.moe_route`` is the same in one kernel, a warp a token:
        # the form the two are checked against)
        logits = linear(x, self.w_router, out_dtype=torch.float32)
        if self.score == "sigmoid":
            ids, scores = ops.moe_choose_sigmoid(logits, self.top, self.correction, self.route_scale)
        else:
            ids, scores = ops.moe_choose(logits, self.top, self.groups, self.keep, self.renormalise)
        return ops.moe_experts(x, ids, self.w_gate_up, self.w_down, self.limit, self.alpha, self.up_shift), scores

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        y, scores = self.forward_slots(x)
        out = torch.empty_like(x)
        if self.shared is None:
            ops.weighted_slot_sum(y, scores, out)
            return out
        gate = None
        if self.w_shared_gate is not None:
            gate = linear(x, self.w_shared_gate, out_dtype=torch.float32).reshape(-1)
        ops.weighted_slot_sum(y, scores, out, extra=self.shared.forward(x), extra_gate=gate)
        return out
