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

Options: no rotated part at all (rot_dim 0 with the position part "none": attention without positions); no sink
(names without 'sink'); queries through a latent of their own (q_rank: c_q = RMSnorm(W_dq h) * w, q = W_uq c_q, names
dq, dq_norm, uq instead of q); a sliding window (a row sees itself and the window - 1 rows before it).
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
                 eps: float, position: PartSpec, names: Dict[str, str], own_latent: bool = True, cache_key: str = "latent",
                 q_rank: Optional[int] = None, window: Optional[int] = None, cache_window: Optional[int] = None):
        """names: tensor names of q (or, with q_rank, of dq, dq_norm, uq), dkv, dkv_norm, uk, uv, o and optionally sink.
        own_latent False: the layer has no down-projection and reads the rows of the entry that its run-order entry names.
        window: how many keys a row sees, itself included (None: all).  cache_window: how many rows back the cache must
        keep (None: all); a layer whose rows other layers read with windows of their own is given the widest."""
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
        self.window = int(window) if window else None
        self.cache_window = int(cache_window) if cache_window else None
        if self.window and self.cache_window and self.cache_window < self.window:
            raise ValueError(f"latent_attention: a cache that keeps {self.cache_window} rows cannot serve a window of {self.window}")
        self.q_rank = int(q_rank) if q_rank else None
        self.proj = StackedLinear(hidden)
        if self.q_rank:
            # queries through a latent: the first product gives c_q's pre-norm values (and the down-projection), a second
            # one the queries
            self.q_off = self.proj.add(names["dq"], self.q_rank)
            self.uq = StackedLinear(self.q_rank)
            self.uq.add(names["uq"], self.H * (self.dn + self.r))
        else:
            self.q_off = self.proj.add(names["q"], self.H * (self.dn + self.r))
            self.uq = None
        self.dkv_off = self.proj.add(names["dkv"], self.R + self.r) if self.own_latent else None
        self.o = StackedLinear(self.H * self.dv)
        self.o.add(names["o"], hidden)
        self.dtype = None

    def weight_specs(self) -> List[WeightSpec]:
        n = self.names
        specs = self.proj.weight_specs() + self.o.weight_specs()
        specs += [WeightSpec(n["uk"], (self.H * self.dn, self.R)), WeightSpec(n["uv"], (self.H * self.dv, self.R))]
        if n.get("sink"):
            specs.append(WeightSpec(n["sink"], (self.H,)))
        if self.q_rank:
            specs += self.uq.weight_specs() + [WeightSpec(n["dq_norm"], (self.q_rank,), "ones")]
        if self.own_latent:
            specs.append(WeightSpec(n["dkv_norm"], (self.R,), "ones"))
        return specs

    def cache_requests(self) -> list:
        return [KVRequest(self.cache_key, 1, self.R + self.r, self.cache_window, values=False)]

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
        self.sink = to_vec(tensors[n["sink"]], device) if n.get("sink") else None
        if self.q_rank:
            self.uq.bind(tensors, dtype, device)
            self.q_norm = to_vec(tensors[n["dq_norm"]], device)
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
        q_proj, q_off = None, self.q_off
        if self.q_rank:
            cq = new("cq", (T, self.q_rank), self.dtype)
            ops.rmsnorm(proj[:, self.q_off:self.q_off + self.q_rank], self.q_norm, self.eps, cq)
            q_proj, q_off = new("q", (T, self.uq.out_features), torch.float32), 0
            self.uq.forward(cq, q_proj)
        ops.latent_prepare(proj, q_off, self.dkv_off, self.c_norm, self.eps, self.position.rotation_table(), step,
                           kv.block_table, pages, qn, qa, H, dn, r, R, q_proj)
        ops.linear_heads(qn, dn, self.uk_t, qa, R + r)                       # qa[:, i, :R] = U_i^T qn_i
        lat = new("lat", (T, H * R), self.dtype)
        ops.latent_attention(qa, pages, self.sink, kv.block_table, step, lat, H, R, r, self.scale, window=self.window or 0)
        att = new("att", (T, H * dv), self.dtype)
        ops.linear_heads(lat, R, self.uv, att, dv)                           # att[:, i] = V_i (sum_j p_j c_j)
        self.o.forward(att, residual, accumulate=accumulate)
