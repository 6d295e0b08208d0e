"""Multi-head latent attention: all heads attend over one low-rank row per token, with a softmax sink.

A token's input h is projected down to R + r values: the first R, RMS-normed with a weight, are the
latent c; the last r, rotated, are a key part kr that every head shares.  Only [c | kr] is cached.
Head i has up-projections of its own: key_i = U_i c (dn values) and value_i = V_i c (dv values); its query
is (qn_i | qr_i) with qr_i rotated like kr; score = (qn_i . key_i + qr_i . kr) * scale; the softmax's
denominator gets one extra term exp(sink_i): sink_i is a per-head parameter, a logit that attracts probability mass
without contributing any value vector.

The keys are never built: qn_i . U_i c = (U_i^T qn_i) . c, so the query is carried into the latent space
(one product per head), every head attends over the same cached rows with the query [U_i^T qn_i | qr_i]
and collects sum_j p_j c_j, and V_i is applied to that sum afterwards.  A layer may attend over the rows
that ANOTHER layer cached (LayerRun.kv_cache) with its own queries, U, V and sink; it then has no
down-projection.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ... import ops
from ..base import KVRequest, LayerCache, Part, PartSpec, StepInfo, WeightSpec, register_mixer, scratch_buf, to_vec
from ..linear import StackedLinear, matrix_dtype


@register_mixer("latent_attention")
class LatentAttentionMixer(Part):
    def __init__(self, hidden: int, n_heads: int, head_dim: int, rot_dim: int, v_dim: int, kv_rank: int, scale: float,
                 eps: float, position: PartSpec, names: Dict[str, str], own_latent: bool = True, cache_key: str = "latent"):
        """names: tensor names of q, dkv, dkv_norm, uk, uv, sink, o.  own_latent False: the layer has no down-projection
        and reads the rows of the entry that its run-order entry names."""
        self.hidden, self.H, self.dn, self.r, self.dv, self.R = (int(hidden), int(n_heads), int(head_dim), int(rot_dim),
                                                                 int(v_dim), int(kv_rank))
        if not (1 <= self.R <= ops.MAX_LATENT):
            raise ValueError(f"latent_attention: a latent of {self.R} values is outside what the kernels are built for "
                             f"(1..{ops.MAX_LATENT})")
        if self.H > ops.MAX_HEADS:
            raise ValueError(f"latent_attention: {self.H} heads exceed the kernels' limit of {ops.MAX_HEADS}")
        self.scale, self.eps, self.names, self.own_latent, self.cache_key = float(scale), float(eps), dict(names), bool(own_latent), cache_key
        self.position = position.build()
        if getattr(self.position, "layout", None) != "interleaved" and position.name != "none":
            raise ValueError(f"latent_attention: the kernels of this mixer rotate interleaved pairs; position part "
                             f"'{position.name}' does not")
        self.proj = StackedLinear(hidden)
        self.q_off = self.proj.add(names["q"], self.H * (self.dn + self.r))
        self.dkv_off = self.proj.add(names["dkv"], self.R + self.r) if self.own_latent else None
        self.o = StackedLinear(self.H * self.dv)
        self.o.add(names["o"], hidden)
        self.dtype = None

    def weight_specs(self) -> List[WeightSpec]:
        n = self.names
        specs = self.proj.weight_specs() + self.o.weight_specs()
        specs += [WeightSpec(n["uk"], (self.H * self.dn, self.R)), WeightSpec(n["uv"], (self.H * self.dv, self.R)),
                  WeightSpec(n["sink"], (self.H,))]
        if self.own_latent:
            specs.append(WeightSpec(n["dkv_norm"], (self.R,), "ones"))
        return specs

    def cache_requests(self) -> list:
        return [KVRequest(self.cache_key, 1, self.R + self.r, None, values=False)]

    def bind(self, tensors: Dict[str, torch.Tensor], dtype, device) -> None:
        n = self.names
        self.dtype = dtype
        self.proj.bind(tensors, dtype, device)
        self.o.bind(tensors, dtype, device)
        self.position.bind(tensors, dtype, device)
        uk, uv = tensors[n["uk"]], tensors[n["uv"]]
        mdt = matrix_dtype(uk.dtype, dtype)
        # U_i^T as the weight [R, dn] of head i's product into the latent space; V_i [dv, R] as it is stored
        self.uk_t = uk.to(device=device, dtype=mdt).reshape(self.H, self.dn, self.R).transpose(1, 2).contiguous()
        self.uv = uv.to(device=device, dtype=matrix_dtype(uv.dtype, dtype)).reshape(self.H, self.dv, self.R).contiguous()
        self.sink = to_vec(tensors[n["sink"]], device)
        self.c_norm = to_vec(tensors[n["dkv_norm"]], device) if self.own_latent else None

    def forward(self, normed: torch.Tensor, step: StepInfo, cache: LayerCache, residual: torch.Tensor,
                accumulate: bool = True) -> None:
        T, dev = step.n_rows, normed.device
        H, dn, r, dv, R = self.H, self.dn, self.r, self.dv, self.R
        kv = cache.kv[self.cache_key]
        if self.own_latent and not (cache.writes and cache.kv_writes):
            raise ValueError("latent_attention: a layer with a down-projection of its own stores its rows; it cannot run on "
                             "another entry's keys")
        new = lambda tag, shape, dt: scratch_buf(f"latent.{tag}", shape, dt, dev)
        proj = new("proj", (T, self.proj.out_features), torch.float32)
        self.proj.forward(normed, proj)
        qn = new("qn", (T, H * dn), self.dtype)
        qa = new("qa", (T, H * (R + r)), self.dtype)
        pages = kv.k_pages.view(kv.k_pages.shape[0], ops.PAGE, R + r)        # one key/value head
        ops.latent_prepare(proj, self.q_off, self.dkv_off, self.c_norm, self.eps, self.position.rotation_table(), step,
                           kv.block_table, pages, qn, qa, H, dn, r, R)
        ops.linear_heads(qn, dn, self.uk_t, qa, R + r)                       # qa[:, i, :R] = U_i^T qn_i
        lat = new("lat", (T, H * R), self.dtype)
        ops.latent_attention(qa, pages, self.sink, kv.block_table, step, lat, H, R, r, self.scale)
        att = new("att", (T, H * dv), self.dtype)
        ops.linear_heads(lat, R, self.uv, att, dv)                           # att[:, i] = V_i (sum_j p_j c_j)
        self.o.forward(att, residual, accumulate=accumulate)
