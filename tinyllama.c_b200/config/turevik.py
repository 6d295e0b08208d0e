"""Turevik configuration: a list of layers, each with its own mixer and feed-forward.

config.json names the architecture in 'architecture' and gives 'vocab', 'width', 'norm' ({'eps'}) and 'layers': one
object per layer with 'type' (the mixer: 'latent_attention' or 'mingru'), 'mixer' (its sizes) and 'mlp' (the
feed-forward, or null).  Every size and every constant that may differ between models is read from there.

  latent_attention mixer: heads, dim (unrotated query/key values per head), rot_dim (rotated), vdim, kv_rank, scale,
                          rot {base, dims}, and optionally kv_from (the layer whose cached rows this one attends over)
  mingru mixer:           width
  mlp kind 'dense':       ff
  mlp kind 'moe':         router {experts, top}, expert {ff}, and optionally shared {ff}
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
class TurevikConfig(ModelConfig):
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
            if kind == "latent_attention":
                for k in ("heads", "dim", "rot_dim", "vdim", "kv_rank"):
                    if not _pos_int(m.get(k)):
                        bad.append(f"{where}.mixer.{k} must be a positive integer, got {m.get(k)!r}")
                if not _num(m.get("scale")):
                    bad.append(f"{where}.mixer.scale must be a number")
                rot = m.get("rot")
                if not (isinstance(rot, dict) and _num(rot.get("base")) and rot["base"] > 0 and _pos_int(rot.get("dims"))
                        and rot["dims"] % 2 == 0 and _pos_int(m.get("rot_dim")) and rot["dims"] <= m["rot_dim"]):
                    bad.append(f"{where}.mixer.rot must give a positive 'base' and an even 'dims' of at most rot_dim")
                src = m.get("kv_from")
                if src is not None:
                    ok = isinstance(src, int) and not isinstance(src, bool) and 0 <= src < i \
                        and isinstance(self.layers[src], dict) and self.layers[src].get("type") == "latent_attention" \
                        and isinstance(self.layers[src].get("mixer"), dict) and self.layers[src]["mixer"].get("kv_from") is None
                    if not ok:
                        bad.append(f"{where}.mixer.kv_from must name an earlier latent_attention layer with a down-projection "
                                   f"of its own, got {src!r}")
                    elif any(self.layers[src]["mixer"].get(k) != m.get(k) for k in ("kv_rank", "rot_dim", "rot")):
                        bad.append(f"{where}.mixer: kv_rank, rot_dim and rot must equal those of layer {src}, whose rows it reads")
            elif kind == "mingru":
                if not _pos_int(m.get("width")):
                    bad.append(f"{where}.mixer.width must be a positive integer, got {m.get('width')!r}")
            else:
                bad.append(f"{where}.type must be 'latent_attention' or 'mingru', got {kind!r}")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict):
                bad.append(f"{where}.mlp must be an object or null")
            elif mlp.get("kind") == "dense":
                if not _pos_int(mlp.get("ff")):
                    bad.append(f"{where}.mlp.ff must be a positive integer")
            elif mlp.get("kind") == "moe":
                router, expert, shared = mlp.get("router"), mlp.get("expert"), mlp.get("shared")
                if not (isinstance(router, dict) and _pos_int(router.get("experts")) and _pos_int(router.get("top"))
                        and router["top"] <= router["experts"]):
                    bad.append(f"{where}.mlp.router must give 'experts' and 'top' <= experts")
                if not (isinstance(expert, dict) and _pos_int(expert.get("ff"))):
                    bad.append(f"{where}.mlp.expert must give 'ff'")
                if shared is not None and not (isinstance(shared, dict) and _pos_int(shared.get("ff"))):
                    bad.append(f"{where}.mlp.shared must give 'ff' (or be null)")
            else:
                bad.append(f"{where}.mlp.kind must be 'dense' or 'moe', got {mlp.get('kind')!r}")
        if bad:
            raise ConfigError("config.json: " + "; ".join(bad))
