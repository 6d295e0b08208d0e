"""minGRU mixer: a recurrence over tokens whose update gate and candidate are functions of the token's input alone
(never of the previous state).

z = sigmoid(W_z h + b_z), u = W_x h + b_x, candidate = u + 1/2 where u >= 0 and sigmoid(u) where u < 0;
element by element S_t = (1 - z) S_(t-1) + z * candidate; output W_o (S_t * silu(W_g h)).  S starts at zero,
is 32-bit and is kept per sequence between steps.  Since the gates do not read S, the recurrence is linear in
S and a long prompt runs as chunks side by side (the step's chunk table).
"""
from __future__ import annotations

from typing import Dict, List

import torch

from ... import ops
from ..base import ChunkRequest, LayerCache, Part, StateRequest, StepInfo, WeightSpec, register_mixer, scratch_buf
from ..linear import StackedLinear


@register_mixer("mingru")
class MinGRUMixer(Part):
    CHUNK = 64                 # rows of a chunk of the scan
    CHUNKS_FROM_ROWS = 128     # a sequence that brings more rows than this is scanned in chunks

    def __init__(self, hidden: int, width: int, names: Dict[str, str], cache_key: str = "mingru"):
        """names: tensor names of z, z_bias, x, x_bias, g, o."""
        self.hidden, self.W, self.names, self.cache_key = int(hidden), int(width), dict(names), cache_key
        self.proj = StackedLinear(hidden)
        self.z_off = self.proj.add(names["z"], self.W, names["z_bias"])
        self.u_off = self.proj.add(names["x"], self.W, names["x_bias"])
        self.g_off = self.proj.add(names["g"], self.W)
        self.o = StackedLinear(self.W)
        self.o.add(names["o"], hidden)
        self.dtype = None

    def weight_specs(self) -> List[WeightSpec]:
        return self.proj.weight_specs() + self.o.weight_specs()

    def cache_requests(self) -> list:
        return [StateRequest(self.cache_key, (self.W,))]

    def step_requests(self) -> list:
        return [ChunkRequest(self.CHUNK, self.CHUNKS_FROM_ROWS)]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        self.dtype = dtype
        self.proj.bind(tensors, dtype, device)
        self.o.bind(tensors, dtype, device)

    def forward(self, normed: torch.Tensor, step: StepInfo, cache: LayerCache, residual: torch.Tensor,
                accumulate: bool = True) -> None:
        if not cache.writes:
            raise ValueError("mingru: a recurrent mixer cannot run on another layer's cache without storing "
                             "(its state would advance twice in one step)")
        T, dev = step.n_rows, normed.device
        proj = scratch_buf("mingru.proj", (T, 3 * self.W), torch.float32, dev)
        self.proj.forward(normed, proj)
        y = scratch_buf("mingru.y", (T, self.W), self.dtype, dev)
        ops.mingru_scan(proj, self.z_off, self.u_off, self.g_off, self.W, cache.state[self.cache_key], step, y,
                        step.chunks.get(self.CHUNK))
        self.o.forward(y, residual, accumulate=accumulate)
