"""Porarax: per layer one norm, then a mixer and a mixture-of-experts feed-forward side by side on the normed input,

    h = norm1(x);    x <- mixer(h) + ff(h) + x

with three kinds of mixer: latent attention without positions over a sliding window (queries through a latent of their
own; a layer may attend over the latents ANOTHER layer cached), grouped-query attention with a partial rotation of
neighbouring pairs, unit-RMS queries and keys and a sigmoid output gate, and the gated delta rule.  The experts' router
adds a bias to its logits and weighs the picked experts by a softmax restricted to their own logits; an expert is
W_down ((u + 1) * g / (1 + exp(-1.702 g))) with g = min(W_gate h, limit) and u = W_up h held within +-limit.  The head is the
embedding table.  This file only turns a PoraraxConfig into data: one LayerSpec per layer, the run order (which entry
reads whose cached latents), and the tensor names ('l<i>.' + norm1, mix.*, mlp.*; 'embed'; 'final.norm').
"""
from __future__ import annotations

from typing import List, Optional

from ..config.base import register_architecture
from ..config.porarax import PoraraxConfig
from ..parts.base import LayerRun, LayerSpec, PartSpec
from .model import Model

SWISH_ALPHA = 1.702        # the experts' activation: g * sigmoid(SWISH_ALPHA * g)
UNIT_EPS = 1e-6            # under the root when the delta rule's queries and keys are made unit vectors


def _norm(cfg: PoraraxConfig, name: str) -> PartSpec:
    return PartSpec("norm", "rmsnorm", dict(width=cfg.width, eps=cfg.eps, weight_name=name))


def _cache_window(cfg: PoraraxConfig, i: int) -> int:
    """How many rows back layer i's cached latents are read: the widest window among the layer and its readers."""
    sizes = [cfg.layers[i]["mixer"]["mask"]["size"]]
    sizes += [l["mixer"]["mask"]["size"] for l in cfg.layers if l["type"] == "latent_attention" and l["mixer"].get("kv_from") == i]
    return max(sizes)


def _mixer(cfg: PoraraxConfig, i: int) -> PartSpec:
    layer, p = cfg.layers[i], f"l{i}.mix."
    m, kind = layer["mixer"], layer["type"]
    if kind == "latent_attention":
        names = {k: p + v for k, v in dict(dq="dq", dq_norm="dq.norm", uq="uq", dkv="dkv", dkv_norm="dkv.norm", uk="uk", uv="uv",
                                           o="o").items()}
        own = m.get("kv_from") is None
        return PartSpec("mixer", "latent_attention", dict(
            hidden=cfg.width, n_heads=m["heads"], head_dim=m["dim"], rot_dim=0, v_dim=m["vdim"], kv_rank=m["kv_rank"],
            scale=m["scale"], eps=cfg.eps, position=PartSpec("position", "none", dict(head_dim=0)), names=names,
            own_latent=own, q_rank=m["q_rank"], window=m["mask"]["size"],
            cache_window=_cache_window(cfg, i) if own else None))
    if kind == "attention":
        position = PartSpec("position", "rope_interleaved", dict(head_dim=m["dim"], theta=m["rot"]["base"], rope_dim=m["rot"]["dims"])) \
            if m["rot"]["dims"] > 0 else PartSpec("position", "none", dict(head_dim=m["dim"]))
        return PartSpec("mixer", "attention", dict(
            hidden=cfg.width, n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"], v_dim=m["vdim"], prefix=p,
            position=position, names=dict(q="q", k="k", v="v", g="g", o="o"), scale=m["scale"], qk_norm_eps=cfg.eps,
            gate="sigmoid"))
    names = {k: p + v for k, v in dict(q="q", k="k", v="v", b="b", a="a", A_log="A_log", dt_bias="dt_bias", norm="norm", g="g",
                                       o="o").items()}
    return PartSpec("mixer", "delta", dict(hidden=cfg.width, n_heads=m["heads"], n_qk_heads=m["kv_heads"], key_dim=m["dim"],
                                           v_dim=m["vdim"], conv_taps=m["conv"], eps=cfg.eps, names=names, l2_eps=UNIT_EPS))


def _feed_forward(cfg: PoraraxConfig, i: int) -> Optional[PartSpec]:
    mlp, p = cfg.layers[i].get("mlp"), f"l{i}.mlp."
    if mlp is None:
        return None
    return PartSpec("feed_forward", "moe", dict(
        hidden=cfg.width, n_experts=mlp["router"]["experts"], top=mlp["router"]["top"], expert_ff=mlp["expert"]["ff"],
        router_name=p + "router", router_bias_name=p + "router.b",
        expert_names={k: p + "e{e}." + k for k in ("gate", "up", "down")}, weights="softmax", weight_on="output",
        act="swish_clamped", limit=mlp["expert"]["limit"], alpha=SWISH_ALPHA))


def layer_specs(cfg: PoraraxConfig) -> List[LayerSpec]:
    # no norm before the feed-forward: it reads the mixer's normed input and runs beside the mixer
    return [LayerSpec(_norm(cfg, f"l{i}.norm1"), (_mixer(cfg, i),), None, _feed_forward(cfg, i)) for i in range(len(cfg.layers))]


def build(cfg: PoraraxConfig) -> Model:
    schedule = [LayerRun(i, kv_cache=layer["mixer"].get("kv_from")) for i, layer in enumerate(cfg.layers)]
    return Model(cfg, layer_specs(cfg), schedule, _norm(cfg, "final.norm"), embed_name="embed", head_name=None,
                 vocab=cfg.vocab, hidden=cfg.width)


register_architecture("Porarax", PoraraxConfig, build)
