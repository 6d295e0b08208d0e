"""Turevik: per layer a latent-attention or minGRU mixer and a dense or mixture-of-experts feed-forward, each sublayer
between two norms, with a token shift applied to the mixer's input.

    x <- x + norm1b(mixer(shift(norm1(x))))        x <- x + norm2b(ff(norm2(x)))

All norms are RMS norms whose weight is stored as its distance from one.  shift(h)[t] = h[t] + (h[t-1] - h[t]) * mu
with a learned vector mu per layer.  A latent-attention layer with 'kv_from' has no down-projection and attends over the
rows another layer cached.  The head is the embedding table.  This file only turns a TurevikConfig into data: one
LayerSpec per layer, the run order (which entry reads whose cached rows), and the tensor names ('l<i>.' + norm1, norm2,
norm1b, norm2b, shift, mix.*, mlp.*; 'embed'; 'final.norm').
"""
from __future__ import annotations

from typing import List

from ..config.base import register_architecture
from ..config.turevik import TurevikConfig
from ..parts.base import LayerRun, LayerSpec, PartSpec
from .model import Model


def _norm(cfg: TurevikConfig, name: str) -> PartSpec:
    return PartSpec("norm", "rmsnorm", dict(width=cfg.width, eps=cfg.eps, weight_name=name, offset=1.0))


def _mixer(cfg: TurevikConfig, i: int) -> PartSpec:
    layer, p = cfg.layers[i], f"l{i}.mix."
    m = layer["mixer"]
    if layer["type"] == "latent_attention":
        names = {k: p + v for k, v in dict(q="q", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv", sink="sink", o="o").items()}
        position = PartSpec("position", "rope_interleaved", dict(head_dim=m["rot_dim"], theta=m["rot"]["base"],
                                                                rope_dim=m["rot"]["dims"]))
        return PartSpec("mixer", "latent_attention", dict(
            hidden=cfg.width, n_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], v_dim=m["vdim"],
            kv_rank=m["kv_rank"], scale=m["scale"], eps=cfg.eps, position=position, names=names,
            own_latent=m.get("kv_from") is None))
    names = {k: p + v for k, v in dict(z="z", z_bias="z.b", x="x", x_bias="x.b", g="g", o="o").items()}
    return PartSpec("mixer", "mingru", dict(hidden=cfg.width, width=m["width"], names=names))


def _feed_forward(cfg: TurevikConfig, i: int):
    mlp, p = cfg.layers[i].get("mlp"), f"l{i}.mlp."
    if mlp is None:
        return None
    plain = dict(gate="gate", up="up", down="down")
    if mlp["kind"] == "dense":
        return PartSpec("feed_forward", "swiglu", dict(hidden=cfg.width, intermediate=mlp["ff"], prefix=p, act="gelu_tanh",
                                                       names=plain))
    shared = mlp.get("shared")
    return PartSpec("feed_forward", "moe", dict(
        hidden=cfg.width, n_experts=mlp["router"]["experts"], top=mlp["router"]["top"], expert_ff=mlp["expert"]["ff"],
        router_name=p + "router", expert_names={k: p + "e{e}." + k for k in plain},
        shared=None if shared is None else PartSpec("feed_forward", "swiglu", dict(
            hidden=cfg.width, intermediate=shared["ff"], prefix=p + "shared.", act="silu", names=plain)),
        shared_gate_name=None if shared is None else p + "shared.sg"))


def layer_specs(cfg: TurevikConfig) -> List[LayerSpec]:
    specs = []
    for i in range(len(cfg.layers)):
        L = f"l{i}."
        pre = PartSpec("norm", "rmsnorm_shift", dict(width=cfg.width, eps=cfg.eps, weight_name=L + "norm1", offset=1.0,
                                                     mix_name=L + "shift"))
        ffn = _feed_forward(cfg, i)
        specs.append(LayerSpec(pre, (_mixer(cfg, i),), _norm(cfg, L + "norm2") if ffn is not None else None, ffn,
                               mixer_out_norm=_norm(cfg, L + "norm1b"),
                               ffn_out_norm=_norm(cfg, L + "norm2b") if ffn is not None else None))
    return specs


def build(cfg: TurevikConfig) -> Model:
    schedule = [LayerRun(i, kv_cache=layer["mixer"].get("kv_from")) for i, layer in enumerate(cfg.layers)]
    return Model(cfg, layer_specs(cfg), schedule, _norm(cfg, "final.norm"), embed_name="embed", head_name=None,
                 vocab=cfg.vocab, hidden=cfg.width)


register_architecture("Turevik", TurevikConfig, build)
