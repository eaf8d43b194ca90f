"""Sogazen configuration: a list of layers, each a mixer and an optional feed-forward that read the residual stream itself
and whose results are normed before they are added.

config.json names the architecture in 'architecture' and gives 'vocab', 'width', 'norm' ({'eps'}), 'logit_softcap' and
'layers': one object per layer with 'type' (the mixer), 'mixer' (its sizes and constants) and 'mlp' (the feed-forward, or
null).

  parallel mixer:  'left'  {heads, kv_heads, dim, vdim (= dim: the values are the keys), scale, softcap, rot {base, dims}}
                   'right' {heads, vdim, state, groups, norm_groups, conv (taps)}
  wkv mixer:       heads, dim   (the width of the decay's hidden layer is the stored tensor's; 'decay_rank' may give it
                   for a model written with random weights)
  mlp kind 'dense': ff, limit
  mlp kind 'moe':   router {experts, top, identity}, expert {ff}
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
class SogazenConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[Dict[str, Any], ...]
    norm: Dict[str, Any]
    logit_softcap: float
    initializer_range: float = 0.02

    def to_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": dict(self.norm),
                "logit_softcap": self.logit_softcap, "layers": [dict(l) for l in self.layers]}

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
        if not (_num(self.logit_softcap) and self.logit_softcap > 0):
            bad.append(f"'logit_softcap' must be a positive number, got {self.logit_softcap!r}")
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

            def ints(obj, path, *keys):
                ok = True
                for k in keys:
                    if not _pos_int(obj.get(k)):
                        bad.append(f"{where}.{path}.{k} must be a positive integer, got {obj.get(k)!r}")
                        ok = False
                return ok

            if kind == "parallel":
                left, right = m.get("left"), m.get("right")
                if not isinstance(left, dict) or not isinstance(right, dict):
                    bad.append(f"{where}.mixer must give 'left' and 'right' objects")
                    continue
                if ints(left, "mixer.left", "heads", "kv_heads", "dim", "vdim"):
                    if left["heads"] % left["kv_heads"]:
                        bad.append(f"{where}.mixer.left.heads must be a multiple of kv_heads")
                    if left["vdim"] != left["dim"]:
                        bad.append(f"{where}.mixer.left.vdim must equal dim (the values are the keys)")
                    rot = left.get("rot")
                    if not (isinstance(rot, dict) and _num(rot.get("base")) and rot["base"] > 0 and isinstance(rot.get("dims"), int)
                            and not isinstance(rot["dims"], bool) and rot["dims"] >= 0 and rot["dims"] % 2 == 0
                            and rot["dims"] <= left["dim"]):
                        bad.append(f"{where}.mixer.left.rot must give a positive 'base' and an even 'dims' of at most dim")
                if not _num(left.get("scale")):
                    bad.append(f"{where}.mixer.left.scale must be a number")
                if not (_num(left.get("softcap")) and left["softcap"] > 0):
                    bad.append(f"{where}.mixer.left.softcap must be a positive number")
                if ints(right, "mixer.right", "heads", "vdim", "state", "groups", "norm_groups", "conv"):
                    if right["heads"] % right["groups"]:
                        bad.append(f"{where}.mixer.right.heads must be a multiple of groups")
                    if (right["heads"] * right["vdim"]) % right["norm_groups"]:
                        bad.append(f"{where}.mixer.right: heads * vdim must be a multiple of norm_groups")
            elif kind == "wkv":
                ints(m, "mixer", "heads", "dim")
                if m.get("decay_rank") is not None and not _pos_int(m["decay_rank"]):
                    bad.append(f"{where}.mixer.decay_rank must be a positive integer where it is given")
            else:
                bad.append(f"{where}.type must be 'parallel' or 'wkv', got {kind!r}")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                bad.append(f"{where}.mlp must be null or an object of kind 'dense' or 'moe'")
                continue
            if mlp["kind"] == "dense":
                if not (_pos_int(mlp.get("ff")) and _num(mlp.get("limit")) and mlp["limit"] > 0):
                    bad.append(f"{where}.mlp must give 'ff' and a positive 'limit'")
                continue
            router, expert = mlp.get("router"), mlp.get("expert")
            ident = router.get("identity", 0) if isinstance(router, dict) else None
            if not (isinstance(router, dict) and _pos_int(router.get("experts")) and _pos_int(router.get("top"))
                    and isinstance(ident, int) and not isinstance(ident, bool) and ident >= 0
                    and router["top"] <= router["experts"] + ident):
                bad.append(f"{where}.mlp.router must give 'experts', 'identity' >= 0 and 'top' <= experts + identity")
            if not (isinstance(expert, dict) and _pos_int(expert.get("ff"))):
                bad.append(f"{where}.mlp.expert must give 'ff'")
        if bad:
            raise ConfigError("config.json: " + "; ".join(bad))
