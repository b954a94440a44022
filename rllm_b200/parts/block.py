"""Arrangements of a mixer, a feed-forward and norms in a layer.

``pre_norm`` is the Llama decoder layer
(crates/rllm-model/src/layers.rs:677-699):
    h   = x + mixer(norm_0(x))
    out = h + ffn(norm_1(h))
The residual stream h is float32 and every add into it is a float32 add.  The
last add of a block is not done here: the block returns (h, pending) with
out = h + pending, and whichever norm reads the stream next adds ``pending``
in the same kernel that normalises.

With few rows (decoding) and parts that can do it, no norm kernel runs at all:
the product that ends the mixer (and the feed-forward) adds into h itself and
leaves what the next norm needs, and the product that follows the norm applies
it (see ``RowSumsq`` and ``ScaledRows`` in ``parts/base.py``).

``parallel_residual`` has one norm that both sublayers read:
    u   = norm_0(x)
    out = x + (mixer(u) + ffn(u))
(the feed-forward may be absent).  Neither add is done here where the norm that
reads the stream next can take both results at once (``PendingSum``): that
norm's kernel completes the stream, in float32, and normalises it.
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from .base import FeedForward, Mixer, Norm, PendingSum, RowSumsq, StepContext
from .registry import register_part


@register_part("block", "pre_norm")
class PreNormBlock:
    def __init__(self, mixer: Mixer, ffn: FeedForward, norms: List[Norm]):
        if len(norms) != 2:
            raise ValueError("a pre_norm block has two norms: before the mixer and before the feed-forward")
        self.mixer, self.ffn, self.norms = mixer, ffn, norms

    def parts(self):
        return [self.norms[0], self.mixer, self.norms[1], self.ffn]

    takes_next_norm = True

    def _fused(self, num_rows: int, ctx: StepContext) -> bool:
        import os
        return (all(getattr(p, "fused_residual", None) is not None and p.fused_residual(num_rows, ctx.act_dtype)
                    for p in (self.mixer, self.ffn))
                and all(hasattr(n, "scaled_input") for n in self.norms)
                and os.environ.get("RLLM_FUSED_NORM") != "0")

    def forward(self, h: torch.Tensor, pending, ctx: StepContext, cache, next_norm=None):
        """``next_norm``: the norm that reads the stream after this block, if the caller knows it."""
        if self._fused(h.shape[0], ctx):
            xn = self.norms[0].scaled_input(pending) if isinstance(pending, RowSumsq) else None
            if xn is None:
                if not isinstance(pending, torch.Tensor):
                    xn = self.norms[0].forward(h, ctx.act_dtype)
                else:
                    xn = self.norms[0].add_forward(h, pending)
            stats = self.mixer.forward(xn, ctx, cache, residual=(h, self.norms[1]))
            stats = self.ffn.forward(self.norms[1].scaled_input(stats), residual=(h, next_norm))
            return h, stats
        if not isinstance(pending, torch.Tensor):
            pending = None                      # h is complete (whatever a block ahead prepared beside it)
        if pending is None:
            xn = self.norms[0].forward(h, ctx.act_dtype)
        else:
            xn = self.norms[0].add_forward(h, pending)
        a = self.mixer.forward(xn, ctx, cache)
        xn = self.norms[1].add_forward(h, a)
        return h, self.ffn.forward(xn)


@register_part("block", "parallel_residual")
class ParallelResidualBlock:
    def __init__(self, mixer: Mixer, ffn: Optional[FeedForward], norms: List[Norm]):
        if len(norms) != 1:
            raise ValueError("a parallel_residual block has one norm, read by the mixer and the feed-forward")
        self.mixer, self.ffn, self.norms = mixer, ffn, norms

    def parts(self):
        return [self.norms[0], self.mixer] + ([self.ffn] if self.ffn is not None else [])

    takes_next_norm = True
    takes_final_norm = True      # the last block of a model is handed the model's own norm as the next one

    def forward(self, h: torch.Tensor, pending, ctx: StepContext, cache, next_norm=None):
        norm = self.norms[0]
        if isinstance(pending, PendingSum) and not getattr(norm, "takes_pending_sum", False):
            from ..kernels import ops
            ops.add_rows(h, pending.terms, pending.bias)
            pending = None
        if isinstance(pending, (torch.Tensor, PendingSum)):
            u = norm.add_forward(h, pending)
        else:
            u = norm.forward(h, ctx.act_dtype)           # h is complete
        # a mixer that ends in a bias on every row may leave it to whoever completes the stream
        defer = getattr(self.mixer, "deferred_output_bias", None)
        bias = defer() if defer is not None else None
        a = self.mixer.forward(u, ctx, cache, add_output_bias=False) if bias is not None else \
            self.mixer.forward(u, ctx, cache)
        terms = (a,) if self.ffn is None else (a, self.ffn.forward(u))
        trace = ctx.extras.get("residual_trace")         # a list: the stream after every layer (a copy)
        if trace is not None or not getattr(next_norm, "takes_pending_sum", False):
            from ..kernels import ops
            ops.add_rows(h, terms, bias)
            if trace is not None:
                trace.append(h.clone())
            return h, None
        return h, PendingSum(terms, bias)
