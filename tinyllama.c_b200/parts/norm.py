"""RMSNorm over the 32-bit residual stream.

o = x * 1/sqrt(mean(x^2) + eps) * w  (CodeClaper/tinyllama.c cpu_op.c:44-64, applied per
row at cpu_op.c:526-533).  The reference fixes eps at 1e-6 (def.h:10); here it is a
parameter.  Statistics are 32-bit; the output takes the activation type.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from .base import LayerCache, Part, StateRequest, StepInfo, WeightSpec, register_norm, to_vec


@register_norm("rmsnorm")
class RMSNorm(Part):
    def __init__(self, width: int, eps: float, weight_name: str, offset: float = 0.0):
        """offset: what is added to the stored weight (1.0 for a weight stored as its distance from one)."""
        self.width, self.eps, self.weight_name, self.offset = int(width), float(eps), weight_name, float(offset)
        self.weight: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return [WeightSpec(self.weight_name, (self.width,), "ones" if self.offset == 0.0 else "near_zero")]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.weight = to_vec(tensors[self.weight_name], device)
        if self.offset != 0.0:
            self.weight = (self.weight + self.offset).contiguous()        # in 32 bits

    def forward(self, x32: torch.Tensor, out: torch.Tensor, rows: Optional[torch.Tensor] = None) -> torch.Tensor:
        ops.rmsnorm(x32, self.weight, self.eps, out, rows)
        return out

    def add_normed(self, parts: Optional[torch.Tensor], residual: torch.Tensor, extra: Optional[torch.Tensor] = None,
                   gate: Optional[torch.Tensor] = None) -> None:
        """As a sublayer's output norm: residual += norm(y) with y = the sum of parts [T, (n,) D] (+ sigmoid(gate[t]) *
        extra[t], gate being a logit per row)."""
        ops.rmsnorm_add(parts, self.weight, self.eps, residual, extra, gate, gate_sigmoid=True)


@register_norm("rmsnorm_shift")
class RMSNormShift(RMSNorm):
    """RMSNorm followed by a token shift: with n[t] the normed row, the result is n[t] + (n[t-1] - n[t]) * mix, mix a
    learned vector [D] and n[t-1] the normed row of the sequence's previous token (zeros before the first).  The last
    normed row of a sequence is kept per sequence (32-bit) between steps."""

    def __init__(self, width: int, eps: float, weight_name: str, mix_name: str, offset: float = 0.0,
                 cache_key: str = "shift"):
        super().__init__(width, eps, weight_name, offset)
        self.mix_name, self.cache_key = mix_name, cache_key
        self.mix: Optional[torch.Tensor] = None

    def weight_specs(self) -> List[WeightSpec]:
        return super().weight_specs() + [WeightSpec(self.mix_name, (self.width,), "unit_interval")]

    def cache_requests(self) -> list:
        return [StateRequest(self.cache_key, (self.width,))]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        super().bind(tensors, dtype, device)
        self.mix = to_vec(tensors[self.mix_name], device)

    def forward(self, x32, out, rows=None):
        raise ValueError("rmsnorm_shift: a norm with a token shift needs the step and the cache (forward_step)")

    def forward_step(self, x32: torch.Tensor, out: torch.Tensor, step: StepInfo, cache: LayerCache) -> torch.Tensor:
        if not cache.writes:
            raise ValueError("rmsnorm_shift: the kept row would advance twice in a step on another entry's cache")
        ops.rmsnorm_shift(x32, self.weight, self.mix, self.eps, cache.state[self.cache_key], step, out)
        return out
