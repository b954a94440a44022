"""``mlstm``: the matrix memory of xLSTM (its mLSTM layer), with capped gates.

    q = W_q h * d^(-1/2),  k = W_k h  [heads, d],   v = W_v h  [heads, dv]
    per head:  a = cap * tanh((W_i h + b_i) / cap)                   (log input gate)
               b = logsigmoid(cap * tanh((W_f h + b_f) / cap))       (log forget gate)
    m_t = max(b_t + m_(t-1), a_t)                                    (m_0 = 0)
    S_t = exp(b_t + m_(t-1) - m_t) S_(t-1) + exp(a_t - m_t) k_t v_t^T,   n_t likewise with k_t alone
    o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
    y = W_o (rms_per_head(o) * w * sigmoid(W_g h))                   (eps inside the root)

S [heads, d, dv], n [heads, d] and m [heads] are float32 per request, start at zero and are
carried from step to step in the request's state slot.  q, k, v and the output gate are one matrix
product over the stacked weights; the two gates' pre-activations are a second one whose result stays
float32 (they enter the recurrence); caps, logarithms, exponentials, the recurrence and the norm are
float32 arithmetic in the kernels.  Portions of 129 tokens and more are scanned as chunks of 64 side by
side (``ops.mlstm_scan``).

params: hidden_size, num_heads, head_dim, v_dim, gate_cap (None or 0: no cap), eps,
tensor_names (keys "q", "k", "v", "g", "o", "norm", "i", "i_bias", "f", "f_bias").
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import Mixer, StateCacheView, StepContext
from .linear import linear
from .registry import register_part
from .spec import PartSpec, StateNeed, TensorSpec

_KEYS = ("q", "k", "v", "g", "o", "norm", "i", "i_bias", "f", "f_bias")


@register_part("mixer", "mlstm")
class MatrixLSTM(Mixer):
    graph_safe = True

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        p = spec.get()
        self.hidden, self.heads = int(p["hidden_size"]), int(p["num_heads"])
        self.d, self.dv, self.eps = int(p["head_dim"]), int(p["v_dim"]), float(p["eps"])
        self.cap = float(p.get("gate_cap") or 0.0)
        if self.cap < 0:
            raise ValueError("mlstm: gate_cap must not be negative")
        if self.d > 256:
            raise ValueError(f"mlstm: head_dim {self.d}; the scan kernel takes up to 256")
        names = dict(p.get("tensor_names") or ())
        if sorted(names) != sorted(_KEYS):
            raise ValueError(f"an mlstm spec names its tensors: tensor_names with the keys {_KEYS}")
        self.names = {k: prefix + str(v) for k, v in names.items()}
        self.w_in = self.w_gates = self.w_o = self.w_norm = self.b_i = self.b_f = None

    def tensor_specs(self) -> List[TensorSpec]:
        n, H, qk, vv = self.names, self.hidden, self.heads * self.d, self.heads * self.dv
        return [TensorSpec(n["q"], (qk, H)), TensorSpec(n["k"], (qk, H)), TensorSpec(n["v"], (vv, H)),
                TensorSpec(n["g"], (vv, H)), TensorSpec(n["o"], (H, vv)),
                TensorSpec(n["norm"], (vv,), role="vector", init=("one_plus_normal", 0.1)),
                TensorSpec(n["i"], (self.heads, H), init=("normal", 0.1)),
                TensorSpec(n["i_bias"], (self.heads,), role="vector", init=("normal", 1.0)),
                TensorSpec(n["f"], (self.heads, H), init=("normal", 0.1)),
                TensorSpec(n["f_bias"], (self.heads,), role="vector", init=("one_plus_normal", 1.0))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        n = self.names
        self.w_in = torch.cat([tensors[n["q"]], tensors[n["k"]], tensors[n["v"]], tensors[n["g"]]], dim=0).contiguous()
        self.w_gates = torch.cat([tensors[n["i"]], tensors[n["f"]]], dim=0).contiguous()
        self.w_o, self.w_norm = tensors[n["o"]], tensors[n["norm"]].contiguous()
        # the gates' biases enter float32 arithmetic: kept so, whatever the run's dtype
        self.b_i, self.b_f = tensors[n["i_bias"]].float().contiguous(), tensors[n["f_bias"]].float().contiguous()

    def cache_need(self):
        return StateNeed((self.heads, ops.mlstm_state_size(self.d, self.dv)))

    def forward(self, x: torch.Tensor, ctx: StepContext, cache: StateCacheView) -> torch.Tensor:
        qk, vv = self.heads * self.d, self.heads * self.dv
        a = linear(x, self.w_in)                                     # [T, 2 qk + 2 vv]: q | k | v | g
        gates = linear(x, self.w_gates, out_dtype=torch.float32)     # [T, 2 heads]: input gates | forget gates
        o = ops.mlstm_scan(a[:, :qk], a[:, qk:2 * qk], a[:, 2 * qk:2 * qk + vv], gates, self.b_i, self.b_f, self.cap,
                           float(self.d) ** -0.5, cache.state, ctx.q_start, ctx.state_slots, ctx.num_seqs,
                           self.heads, self.d, self.dv, ctx.err, q_lens=ctx.q_lens_host)
        y = ops.head_gated_rmsnorm(o, a[:, 2 * qk + vv:], self.w_norm, self.eps, self.heads, x.dtype)
        return linear(y, self.w_o)
