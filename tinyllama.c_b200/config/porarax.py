"""Porarax configuration: a list of layers, each with its own mixer and an optional mixture-of-experts feed-forward that
runs in parallel with the mixer.

config.json names the architecture in 'architecture' and gives 'vocab', 'width', 'norm' ({'eps'}) and 'layers': one
object per layer with 'type' (the mixer), 'mixer' (its sizes and constants) and 'mlp' (the feed-forward, or null).

  latent_attention mixer: heads, dim (query/key values per head), vdim, kv_rank, q_rank, scale, mask {size}, and
                          optionally kv_from (the layer whose cached latents this one attends over)
  attention mixer:        heads, kv_heads, dim, vdim, scale, rot {base, dims}
  delta mixer:            heads, kv_heads (query/key heads), dim, vdim, conv (taps)
  mlp kind 'moe':         router {experts, top}, expert {ff, limit}
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Tuple

from .base import ConfigError, ModelConfig


def _pos_int(v: Any) -> bool:
    return isinstance(v, int) and not isinstance(v, bool) and v > 0


def _num(v: Any) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


@dataclass(frozen=True)
class PoraraxConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[Dict[str, Any], ...]
    norm: Dict[str, Any]
    initializer_range: float = 0.02

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": dict(self.norm),
                "layers": [dict(l) for l in self.layers]}

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    def validate(self) -> None:
        bad = []
        for k in ("vocab", "width"):
            if not _pos_int(getattr(self, k)):
                bad.append(f"'{k}' must be a positive integer, got {getattr(self, k)!r}")
        if not (isinstance(self.norm, dict) and _num(self.norm.get("eps")) and self.norm["eps"] > 0):
            bad.append("'norm' must be an object with a positive 'eps'")
        if not (isinstance(self.layers, (list, tuple)) and len(self.layers) > 0):
            bad.append("'layers' must be a non-empty list")
            raise ConfigError("config.json: " + "; ".join(bad))
        object.__setattr__(self, "layers", tuple(self.layers))
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
                bad.append(f"{where} must be an object with a 'mixer' object")
                continue
            m, kind = layer["mixer"], layer.get("type")

            def ints(*keys):
                for k in keys:
                    if not _pos_int(m.get(k)):
                        bad.append(f"{where}.mixer.{k} must be a positive integer, got {m.get(k)!r}")

            if kind == "latent_attention":
                ints("heads", "dim", "vdim", "kv_rank", "q_rank")
                if not _num(m.get("scale")):
                    bad.append(f"{where}.mixer.scale must be a number")
                if not (isinstance(m.get("mask"), dict) and _pos_int(m["mask"].get("size"))):
                    bad.append(f"{where}.mixer.mask must give a positive 'size'")
                src = m.get("kv_from")
                if src is not None:
                    ok = isinstance(src, int) and not isinstance(src, bool) and 0 <= src < i \
                        and isinstance(self.layers[src], dict) and self.layers[src].get("type") == "latent_attention" \
                        and isinstance(self.layers[src].get("mixer"), dict) and self.layers[src]["mixer"].get("kv_from") is None
                    if not ok:
                        bad.append(f"{where}.mixer.kv_from must name an earlier latent_attention layer with a down-projection "
                                   f"of its own, got {src!r}")
                    elif self.layers[src]["mixer"].get("kv_rank") != m.get("kv_rank"):
                        bad.append(f"{where}.mixer.kv_rank must equal that of layer {src}, whose latents it reads")
            elif kind == "attention":
                ints("heads", "kv_heads", "dim", "vdim")
                if _pos_int(m.get("heads")) and _pos_int(m.get("kv_heads")) and m["heads"] % m["kv_heads"]:
                    bad.append(f"{where}.mixer.heads must be a multiple of kv_heads")
                if not _num(m.get("scale")):
                    bad.append(f"{where}.mixer.scale must be a number")
                rot = m.get("rot")
                if not (isinstance(rot, dict) and _num(rot.get("base")) and rot["base"] > 0 and isinstance(rot.get("dims"), int)
                        and not isinstance(rot["dims"], bool) and rot["dims"] >= 0 and rot["dims"] % 2 == 0
                        and _pos_int(m.get("dim")) and rot["dims"] <= m["dim"]):
                    bad.append(f"{where}.mixer.rot must give a positive 'base' and an even 'dims' of at most dim")
            elif kind == "delta":
                ints("heads", "kv_heads", "dim", "vdim", "conv")
                if _pos_int(m.get("heads")) and _pos_int(m.get("kv_heads")) and m["heads"] % m["kv_heads"]:
                    bad.append(f"{where}.mixer.heads must be a multiple of kv_heads")
            else:
                bad.append(f"{where}.type must be 'latent_attention', 'attention' or 'delta', got {kind!r}")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") != "moe":
                bad.append(f"{where}.mlp must be null or an object of kind 'moe'")
                continue
            router, expert = mlp.get("router"), mlp.get("expert")
            if not (isinstance(router, dict) and _pos_int(router.get("experts")) and _pos_int(router.get("top"))
                    and router["top"] <= router["experts"]):
                bad.append(f"{where}.mlp.router must give 'experts' and 'top' <= experts")
            if not (isinstance(expert, dict) and _pos_int(expert.get("ff")) and _num(expert.get("limit")) and expert["limit"] > 0):
                bad.append(f"{where}.mlp.expert must give 'ff' and a positive 'limit'")
        if bad:
            raise ConfigError("config.json: " + "; ".join(bad))
