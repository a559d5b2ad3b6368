"""RMSNorm, fused with the residual addition that precedes it.

y = (x * rsqrt(mean(x^2) + eps)) * w, statistics in float
(src/kernels/layernorm.cu:20-23,41,48).  ``eps`` is a parameter; the reference
passes the literal 1e-6 at every call (src/model/qwen.cpp:303,312,322).
"""
from __future__ import annotations

from typing import Dict, Optional

import torch

from ..csrc import ops
from .base import Norm, ParamSpec, register_norm


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """``tensor_name``: local name of the gain (""; the slot's prefix itself, for checkpoints that name the norm and
    not a tensor inside it).  ``unit_offset``: the tensor is stored around zero and the gain is 1 + tensor."""

    def __init__(self, size: int, eps: float, dtype, device, tensor_name: str = "weight", unit_offset: bool = False):
        if size <= 0 or not eps > 0:
            raise ValueError(f"rmsnorm: size {size} and eps {eps} must be positive")
        self.size, self.eps = size, float(eps)
        self.tensor_name, self.unit_offset = tensor_name, bool(unit_offset)
        self.weight: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.tensor_name: ParamSpec((self.size,), "offset_gain" if self.unit_offset else "gain")}

    def load_params(self, tensors):
        w = tensors[self.tensor_name]
        self.weight = (w + 1.0).contiguous() if self.unit_offset else w

    def folded(self, factor):
        return (self.weight if factor is None else (self.weight * factor).contiguous()), self.eps

    def split(self):
        return (self.weight, self.eps) if self.weight is not None and self.weight.dtype == torch.float32 else None

    def forward(self, residual, delta, out, row_index=None, mult=1.0):
        ops.add_rmsnorm(residual, delta, self.weight, out, self.eps, row_index, mult)

    def add_normed(self, y, gate, gate_bias, residual, plain, mult):
        ops.gated_norm_residual(y, gate, gate_bias, self.weight, residual, plain, mult, self.eps)


@register_norm("rmsnorm_scalar")
class ScalarRMSNorm(Norm):
    """RMSNorm whose gain is one number for all coordinates: y = x / sqrt(mean(x^2) + eps) * g.  The tensor
    has no dimensions and the slot's name itself (local name "").  ``out_scale`` is a constant that
    multiplies what ``forward`` returns (a model that scales its logits puts the factor here: the output
    product is linear)."""

    def __init__(self, size: int, eps: float, dtype, device, out_scale: float = 1.0):
        if size <= 0 or not eps > 0:
            raise ValueError(f"rmsnorm_scalar: size {size} and eps {eps} must be positive")
        self.size, self.eps, self.out_scale = size, float(eps), float(out_scale)
        self.gain: Optional[torch.Tensor] = None          # the number, float32 [1]
        self.weight: Optional[torch.Tensor] = None        # gain * out_scale on every coordinate, for the vector kernel

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {"": ParamSpec((), "gain")}

    def load_params(self, tensors):
        self.gain = tensors[""].reshape(1).to(torch.float32).contiguous()
        self.weight = (self.gain * self.out_scale).expand(self.size).contiguous()

    def forward(self, residual, delta, out, row_index=None, mult=1.0):
        ops.add_rmsnorm(residual, delta, self.weight, out, self.eps, row_index, mult)

    def add_normed(self, y, gate, gate_bias, residual, plain, mult):
        ops.gated_norm_residual(y, gate, gate_bias, self.gain, residual, plain, mult * self.out_scale, self.eps)


@register_norm("layernorm")
class LayerNorm(Norm):
    """y = (x - mean(x)) / sqrt(var(x) + eps) * w + b, the variance the mean of the squared deviations; statistics in
    float32.  ``tensor_name`` is the local name of the gain ("": the slot's prefix itself), the bias is that name plus
    ``bias_suffix``.  ``out_scale`` multiplies what the norm returns (a model that scales its logits puts the factor
    here: the output product is linear).  ``forward_streams`` reads a residual stream kept as several copies."""

    def __init__(self, size: int, eps: float, dtype, device, tensor_name: str = "weight", bias_suffix: str = ".b",
                 bias_name: str = "", out_scale: float = 1.0):
        if size <= 0 or not eps > 0:
            raise ValueError(f"layernorm: size {size} and eps {eps} must be positive")
        self.size, self.eps, self.out_scale = size, float(eps), float(out_scale)
        self.tensor_name = tensor_name
        self.bias_name = bias_name or tensor_name + bias_suffix
        self.weight: Optional[torch.Tensor] = None
        self.bias: Optional[torch.Tensor] = None
        self._one: Optional[torch.Tensor] = None

    def param_specs(self) -> Dict[str, ParamSpec]:
        return {self.tensor_name: ParamSpec((self.size,), "gain"), self.bias_name: ParamSpec((self.size,), "bias")}

    def load_params(self, tensors):
        self.weight, self.bias = tensors[self.tensor_name].contiguous(), tensors[self.bias_name].contiguous()
        self._one = torch.ones(1, dtype=torch.float32, device=self.weight.device)

    def forward_streams(self, streams, coef, out, row_index=None):
        """out = norm(sum_s coef[s] streams[s]); streams float32 [S, n, size]."""
        ops.stream_norm(streams, coef, self.weight, self.bias, out, self.eps, row_index, self.out_scale)

    def forward(self, residual, delta, out, row_index=None, mult=1.0):
        if mult != 1.0:
            raise ValueError("layernorm: a pending addition joins with factor 1 only")
        x = residual.unsqueeze(0)
        if delta is not None:
            if row_index is not None:
                raise ValueError("layernorm: a pending addition cannot be made on gathered rows")
            ops.stream_join(x, delta, self._one, self._one)
        ops.stream_norm(x, self._one, self.weight, self.bias, out, self.eps, row_index, self.out_scale)


@register_norm("none")
class NoNorm(Norm):
    """Fills the norm slot of a sublayer that a layer does not have."""

    def __init__(self, dtype=None, device=None):
        pass
