"""RMSNorm: y = x / sqrt(mean(x^2) + eps) * w, eps inside the root, the weight
as it is, all in float32 (crates/rllm-model/src/layers.rs:133-140).  ``eps``
is a parameter (the reference hard-codes 1e-6, crates/rllm-model/src/llama.rs:183).

The norm reads the float32 residual stream; ``add_forward`` first adds a
block's output to it in float32, in the same kernel.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..kernels import ops
from .base import Norm, PendingSum, RowSumsq, ScaledRows
from .registry import register_part
from .spec import PartSpec, TensorSpec


@register_part("norm", "rmsnorm")
class RMSNorm(Norm):
    """params: size, eps, name (tensor name below the prefix), unit_offset (True: the file stores the
    weight's distance from one, y = x / rms * (1 + w); the sum is taken once, in float32, when the
    weights are loaded, and the kernels see an ordinary weight)."""
    graph_safe = True

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.name = prefix + str(spec["name"])
        self.unit_offset = bool(spec.get().get("unit_offset", False))
        self.weight: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        init = ("normal", 0.1) if self.unit_offset else ("one_plus_normal", 0.1)
        return [TensorSpec(self.name, (self.size,), role="vector", init=init)]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        w = tensors[self.name]
        self.weight = (1.0 + w.float()).contiguous() if self.unit_offset else w

    def forward(self, x: torch.Tensor, act_dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty(x.shape, dtype=act_dtype, device=x.device)
        ops.rmsnorm(x, self.weight, self.eps, out)
        return out

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        out = torch.empty(x.shape, dtype=delta.dtype, device=x.device)
        ops.rmsnorm(x, self.weight, self.eps, out, delta=delta, writeback=True)
        return out

    def scaled_input(self, stats: RowSumsq) -> Optional[ScaledRows]:
        """The normalised stream for a product that applies the rows' factors itself, if
        ``stats`` was prepared with this norm's weight."""
        if stats.scaled is None or stats.scaled_by is not self.weight:
            return None
        return ScaledRows(stats.scaled, stats.parts, self.eps)

    def gather_forward(self, x, delta, rows, act_dtype):
        out = torch.empty((rows.numel(), x.shape[1]), dtype=act_dtype, device=x.device)
        ops.rmsnorm(x, self.weight, self.eps, out, delta=delta, rows=rows)
        return out


@register_part("norm", "dynamic_tanh")
class DynamicTanh(Norm):
    """y = tanh(alpha * x) * w + c: a norm without statistics (no mean, no variance, no eps), element by
    element in float32.  alpha is one learned number, w and c vectors.

    params: size, name, alpha_name, shift_name (tensor names below the prefix)."""
    graph_safe = True

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.size = int(spec["size"])
        self.name = prefix + str(spec["name"])
        self.alpha_name = prefix + str(spec["alpha_name"])
        self.shift_name = prefix + str(spec["shift_name"])
        self.weight: Optional[torch.Tensor] = None
        self.shift: Optional[torch.Tensor] = None
        self.alpha: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.size,), role="vector", init=("one_plus_normal", 0.1)),
                TensorSpec(self.shift_name, (self.size,), role="vector", init=("normal", 0.1)),
                TensorSpec(self.alpha_name, (), role="vector", init=("one_plus_normal", 0.1))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        self.weight = tensors[self.name].contiguous()
        self.shift = tensors[self.shift_name].to(self.weight.dtype).contiguous()
        self.alpha = tensors[self.alpha_name].float().reshape(1).contiguous()

    def elementwise(self):
        """(alpha float32 [1], weight, shift): what a kernel needs to apply this norm to a value it holds."""
        return self.alpha, self.weight, self.shift

    def forward(self, x: torch.Tensor, act_dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty(x.shape, dtype=act_dtype, device=x.device)
        ops.dyt(x, self.alpha, self.weight, self.shift, out)
        return out

    def add_forward(self, x: torch.Tensor, delta: torch.Tensor) -> torch.Tensor:
        out = torch.empty(x.shape, dtype=delta.dtype, device=x.device)
        ops.dyt(x, self.alpha, self.weight, self.shift, out, delta=delta, writeback=True)
        return out

    def gather_forward(self, x, delta, rows, act_dtype):
        out = torch.empty((rows.numel(), x.shape[1]), dtype=act_dtype, device=x.device)
        ops.dyt(x, self.alpha, self.weight, self.shift, out, delta=delta, rows=rows)
        return out


@register_part("norm", "layernorm")
class LayerNorm(Norm):
    """y = (x - mean(x)) / sqrt(mean((x - mean(x))^2) + eps) * w + b, row by row in float32: the norm with
    statistics of both orders, a weight and a bias.  It completes the stream in the same kernel from up to
    two sublayer results and a bias on every row (``PendingSum``), which is what a layer whose mixer and
    feed-forward read the same normalised input leaves behind.

    params: size, eps, name, bias_name (tensor names below the prefix)."""
    graph_safe = True
    takes_pending_sum = True

    def __init__(self, spec: PartSpec, prefix: str = ""):
        super().__init__(spec, prefix)
        self.size = int(spec["size"])
        self.eps = float(spec["eps"])
        self.name = prefix + str(spec["name"])
        self.bias_name = prefix + str(spec["bias_name"])
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None

    def tensor_specs(self) -> List[TensorSpec]:
        return [TensorSpec(self.name, (self.size,), role="vector", init=("one_plus_normal", 0.1)),
                TensorSpec(self.bias_name, (self.size,), role="vector", init=("normal", 0.1))]

    def load(self, tensors: Dict[str, torch.Tensor]) -> None:
        # two vectors of the model's width: kept in float32 whatever the run's dtype
        self.weight = tensors[self.name].float().contiguous()
        self.bias = tensors[self.bias_name].float().contiguous()

    @staticmethod
    def _terms(delta):
        if delta is None:
            return (), None
        if isinstance(delta, PendingSum):
            return tuple(delta.terms), delta.bias
        return (delta,), None

    def forward(self, x: torch.Tensor, act_dtype: torch.dtype) -> torch.Tensor:
        out = torch.empty(x.shape, dtype=act_dtype, device=x.device)
        ops.layernorm(x, self.weight, self.bias, self.eps, out)
        return out

    def add_forward(self, x: torch.Tensor, delta) -> torch.Tensor:
        terms, row_bias = self._terms(delta)
        out = torch.empty(x.shape, dtype=terms[0].dtype, device=x.device)
        ops.layernorm(x, self.weight, self.bias, self.eps, out, deltas=terms, row_bias=row_bias, writeback=True)
        return out

    def gather_forward(self, x, delta, rows, act_dtype):
        terms, row_bias = self._terms(delta)
        out = torch.empty((rows.numel(), x.shape[1]), dtype=act_dtype, device=x.device)
        ops.layernorm(x, self.weight, self.bias, self.eps, out, deltas=terms, row_bias=row_bias, rows=rows)
        return out
