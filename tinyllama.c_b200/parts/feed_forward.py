"""Dense gated feed-forward.

d = W_down (act(W_gate x) * (W_up x)), act = SiLU (SwiGLU; CodeClaper/tinyllama.c
falcon_h1.c:382-395) or another registered activation.  The gate and up projections are
stacked into one product.  The multiplier on the gate's pre-activation, the one on the
output, the biases, the choice of activation and of tensor names have no counterpart in
the reference.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from .. import ops
from .base import Part, PartSpec, WeightSpec, act_empty, register_feed_forward, scratch_buf
from .linear import StackedLinear


@register_feed_forward("swiglu")
class SwiGLU(Part):
    def __init__(self, hidden: int, intermediate: int, prefix: str, bias: bool = False, gate_scale: float = 1.0,
                 down_scale: float = 1.0, act: str = "silu", names: Optional[Dict[str, str]] = None):
        """act: "silu" or "gelu_tanh".  names: tensor names of gate, up, down after the prefix (default: the
        gate_proj.weight / up_proj.weight / down_proj.weight of the architecture's checkpoints; biases, where asked
        for, are those names with .bias for .weight)."""
        self.hidden, self.F = int(hidden), int(intermediate)
        if act not in ops.GLU_ACTS:
            raise ValueError(f"feed-forward: unknown activation '{act}'; known: {sorted(ops.GLU_ACTS)}")
        self.act = act
        nm = dict(gate="gate_proj.weight", up="up_proj.weight", down="down_proj.weight")
        nm.update(names or {})
        w = lambda n: prefix + nm[n]
        b = (lambda n: prefix + (nm[n][:-len(".weight")] if nm[n].endswith(".weight") else nm[n]) + ".bias") if bias \
            else (lambda n: None)
        self.gate_up = StackedLinear(hidden)
        self.gate_up.add(w("gate"), self.F, b("gate"), 1.0, gate_scale)
        self.gate_up.add(w("up"), self.F, b("up"))
        self.down = StackedLinear(self.F)
        self.down.add(w("down"), hidden, b("down"), 1.0, down_scale)

    def weight_specs(self) -> List[WeightSpec]:
        return self.gate_up.weight_specs() + self.down.weight_specs()

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.gate_up.bind(tensors, dtype, device)
        self.down.bind(tensors, dtype, device)
        # Rows regrouped as 8 gate rows followed by their 8 up rows, so that the product's epilogue
        # has a feature's gate and up side by side and writes silu(gate) * up directly.
        self.interleaved = self.F % 8 == 0
        if self.interleaved:
            F = self.F
            idx = torch.arange(2 * F, device=self.gate_up.weight.device).reshape(2, F // 8, 8).permute(1, 0, 2).reshape(-1)
            self.gate_up.weight = self.gate_up.weight[idx].contiguous()
            if self.gate_up.colscale is not None:
                self.gate_up.colscale = self.gate_up.colscale[idx].contiguous()
            if self.gate_up.colbias is not None:
                self.gate_up.colbias = self.gate_up.colbias[idx].contiguous()

    def forward(self, normed: torch.Tensor, residual: torch.Tensor, accumulate: bool = True) -> None:
        """Adds the result into `residual` (float32 [T, D]), or overwrites it with accumulate False."""
        T = normed.shape[0]
        act = scratch_buf("swiglu.act", (T, self.F), normed.dtype, normed.device)
        if self.interleaved:
            ops.linear_swiglu(normed, self.gate_up.weight, act, self.gate_up.colscale, self.gate_up.colbias, self.act)
        else:
            gu = scratch_buf("swiglu.gate_up", (T, 2 * self.F), torch.float32, normed.device)
            self.gate_up.forward(normed, gu)
            ops.glu(gu, act, self.act, interleaved=self.interleaved)
        self.down.forward(act, residual, accumulate=accumulate)



@register_feed_forward("moe")
class MoEFeedForward(Part):
    """Mixture of experts.  By default, with a sigmoid router:

    Router scores s = sigmoid(W_router h), the logits as 32-bit sums; a token is routed to its `top` highest-scoring experts, and
    its weights are those scores unchanged (they need not sum to one).  An expert is fed the token scaled by its weight: the result
    is sum_e expert_e(s_e h), every expert a gated feed-forward W_down (silu(W_gate x) * (W_up x)) without biases.
    Gate and up are linear, so the weight is applied to their 32-bit results.  An optional shared expert (a
    feed-forward part of its own) runs on every token and is added times sigmoid(w_sg . h), one number per token; its
    gate is computed with the router, as one more row of the router's matrix.

    The experts' weights are stacked [E, 2F, D] and [E, D, F]; rows are sorted by expert on the device, and every
    (token, choice) pair's result gets a row of its own, which the norm that follows (or `forward`) adds in the order
    of the token's choices: a token's result does not depend on what else is in the batch.

    Other routers and experts, by constructor arguments: a bias on the router's logits (router_bias_name); weights that are
    a softmax restricted to the picked logits (weights="softmax"); the weight applied to what the expert returns instead of
    to what it is fed (weight_on="output": sum_e s_e expert_e(h); the down product is linear, so the weight multiplies the
    32-bit activation); the activation act="swish_clamped": with g = min(W_gate h, limit) and u = W_up h held within
    +-limit, g * sigmoid(alpha g) * (u + 1)."""

    def __init__(self, hidden: int, n_experts: int, top: int, expert_ff: int, router_name: str, expert_names: Dict[str, str],
                 shared: Optional[PartSpec] = None, shared_gate_name: Optional[str] = None, router_bias_name: Optional[str] = None,
                 weights: str = "sigmoid", weight_on: str = "input", act: str = "silu", limit: float = 0.0, alpha: float = 1.0):
        """expert_names: patterns of gate, up, down with {e} for the expert's index."""
        if weights not in ops.ROUTE_WEIGHTS or weight_on not in ("input", "output") or act not in ops.MOE_ACTS:
            raise ValueError(f"moe: unknown weighting '{weights}', weight placement '{weight_on}' or activation '{act}'")
        if act == "swish_clamped" and not limit > 0:
            raise ValueError(f"moe: the clamped activation needs a positive limit, got {limit!r}")
        self.router_bias_name, self.weights, self.weight_on, self.act = router_bias_name, weights, weight_on, act
        self.limit, self.alpha = float(limit), float(alpha)
        self.hidden, self.E, self.top, self.F = int(hidden), int(n_experts), int(top), int(expert_ff)
        if not (1 <= self.top <= self.E):
            raise ValueError(f"moe: {self.top} of {self.E} experts cannot be chosen")
        self.router_name, self.expert_names, self.shared_gate_name = router_name, dict(expert_names), shared_gate_name
        self.shared = shared.build() if shared is not None else None
        if (self.shared is None) != (shared_gate_name is None):
            raise ValueError("moe: a shared expert and its gate come together")
        self.dtype = None

    def weight_specs(self) -> List[WeightSpec]:
        specs = [WeightSpec(self.router_name, (self.E, self.hidden))]
        if self.router_bias_name:
            specs.append(WeightSpec(self.router_bias_name, (self.E,)))
        for e in range(self.E):
            n = {k: v.format(e=e) for k, v in self.expert_names.items()}
            specs += [WeightSpec(n["gate"], (self.F, self.hidden)), WeightSpec(n["up"], (self.F, self.hidden)),
                      WeightSpec(n["down"], (self.hidden, self.F))]
        if self.shared is not None:
            specs += self.shared.weight_specs() + [WeightSpec(self.shared_gate_name, (1, self.hidden))]
        return specs

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        from .linear import matrix_dtype
        self.dtype = dtype
        # The router's logits are 32-bit sums.  A weight stored in bfloat16 times an input rounded to bfloat16 has an exact
        # 32-bit product, so the bfloat16 product with 32-bit accumulation IS the 32-bit result and a bfloat16 run keeps
        # such a router in bfloat16 (the tensor cores); a router stored in 32-bit, and every 32-bit run, multiplies in 32-bit.
        rows = [tensors[self.router_name]] + ([tensors[self.shared_gate_name]] if self.shared is not None else [])
        rdt = torch.bfloat16 if all(matrix_dtype(r.dtype, dtype) == torch.bfloat16 for r in rows) else torch.float32
        self.router = torch.cat([r.to(device=device, dtype=rdt) for r in rows], dim=0).contiguous()
        self.router_bias = None
        if self.router_bias_name:                # added to the 32-bit logits in the product's epilogue (nothing on the shared gate's)
            self.router_bias = torch.zeros(self.router.shape[0], dtype=torch.float32, device=device)
            self.router_bias[:self.E] = tensors[self.router_bias_name].to(device=device, dtype=torch.float32)
        names = [{k: v.format(e=e) for k, v in self.expert_names.items()} for e in range(self.E)]
        mdt = torch.bfloat16
        for n in names:
            for k in ("gate", "up", "down"):
                if matrix_dtype(tensors[n[k]].dtype, dtype) == torch.float32:
                    mdt = torch.float32
        to = lambda t: t.to(device=device, dtype=mdt)
        self.w_gate_up = torch.stack([torch.cat([to(tensors[n["gate"]]), to(tensors[n["up"]])], dim=0) for n in names]).contiguous()
        self.w_down = torch.stack([to(tensors[n["down"]]) for n in names]).contiguous()
        if self.shared is not None:
            self.shared.bind(tensors, dtype, device)

    def forward_parts(self, normed: torch.Tensor):
        """(parts float32 [T, top, D], shared expert's output float32 [T, D] or None, its gate's logit float32 [T] or
        None): the result is sum_k parts[:, k] + sigmoid(logit) * shared."""
        T, dev = normed.shape[0], normed.device
        n_logits = self.router.shape[0]
        logits = scratch_buf("moe.logits", (T, n_logits), torch.float32, dev)
        ops.linear(normed, self.router, logits, None, self.router_bias)
        routing = ops.moe_route(logits, self.E, self.top, ops.moe_tile_rows(normed, self.w_gate_up, self.dtype, self.top),
                                self.weights)
        act = scratch_buf("moe.act", (T * self.top, self.F), self.dtype, dev)
        parts = scratch_buf("moe.parts", (T, self.top, self.hidden), torch.float32, dev)
        ops.moe_experts(normed, self.w_gate_up, self.w_down, routing, self.top, act, parts, self.act, self.weight_on, self.limit,
                        self.alpha)
        if self.shared is None:
            return parts, None, None
        shared_out = scratch_buf("moe.shared", (T, self.hidden), torch.float32, dev)
        self.shared.forward(normed, shared_out, accumulate=False)
        return parts, shared_out, logits[:, self.E]          # the gate's logit: whoever adds the terms takes its sigmoid

    def add_parts(self, terms, residual: torch.Tensor, accumulate: bool = True) -> None:
        """Adds what forward_parts returned into `residual` (a token's terms in the order of its choices).  A block that
        runs this feed-forward beside its mixers computes the terms on a stream of their own and adds them here."""
        parts, extra, gate = terms
        ops.rmsnorm_add(parts, None, 0.0, residual, extra, gate, gate_sigmoid=True, accumulate=accumulate)

    def forward(self, normed: torch.Tensor, residual: torch.Tensor, accumulate: bool = True) -> None:
        self.add_parts(self.forward_parts(normed), residual, accumulate)
