"""Kimutar configuration: a list of layers, each a mixer and an optional feed-forward that both read a layer norm of
the layer's input, and a range of layers that repeats.

config.json names the architecture in 'architecture' and gives 'vocab', 'width', 'norm' ({'eps'}), 'layers' (one object
per layer with 'type' (the mixer), 'mixer' (its sizes and constants) and 'mlp' (the feed-forward, or null)) and optionally
'loop' ({'start', 'stop', 'times'}: layers start .. stop - 1 run `times` times in a row).

  attention mixer:      heads, kv_heads, dim, vdim, scale, diff, rot {base, dims, scaling {factor, original, fast, slow}}
                        (two score maps a head; their difference)
  attention_2 mixer:    heads, kv_heads, dim, vdim, scale, rot {base, dims, scaling {factor, original, low, high}},
                        mask {size, keep_first} (biases, a sliding window that keeps the first tokens, a sink per head)
  channel_delta mixer:  heads, kv_heads (query/key heads), dim, vdim, conv (taps); the hidden widths of the decay's and the
                        gate's low-rank pairs are the stored tensors' ('decay_rank' and 'gate_rank' may give them for a
                        model written with random weights)
  mlp kind 'dense':     ff
  mlp kind 'moe':       router {experts, top, scale}, expert {ff}, and optionally shared {ff}

'rot.scaling' and 'mask' may be absent (plain frequencies; no window).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional, Tuple

from .base import ConfigError, ModelConfig


def _int(v: Any, least: int = 1) -> bool:
    return isinstance(v, int) and not isinstance(v, bool) and v >= least


def _num(v: Any) -> bool:
    return isinstance(v, (int, float)) and not isinstance(v, bool)


SCALING_KEYS = {"attention": ("factor", "original", "fast", "slow"), "attention_2": ("factor", "original", "low", "high")}


@dataclass(frozen=True)
class KimutarConfig(ModelConfig):
    vocab: int
    width: int
    layers: Tuple[Dict[str, Any], ...]
    norm: Dict[str, Any]
    loop: Optional[Dict[str, Any]] = None
    initializer_range: float = 0.02

    def to_dict(self) -> Dict[str, Any]:
        out = {"architecture": self.architecture, "vocab": self.vocab, "width": self.width, "norm": dict(self.norm),
               "layers": [dict(l) for l in self.layers]}
        if self.loop is not None:
            out["loop"] = dict(self.loop)
        return out

    @property
    def eps(self) -> float:
        return float(self.norm["eps"])

    def validate(self) -> None:
        bad = []
        for k in ("vocab", "width"):
            if not _int(getattr(self, k)):
                bad.append(f"'{k}' must be a positive integer, got {getattr(self, k)!r}")
        if not (isinstance(self.norm, dict) and _num(self.norm.get("eps")) and self.norm["eps"] > 0):
            bad.append("'norm' must be an object with a positive 'eps'")
        if not (isinstance(self.layers, (list, tuple)) and len(self.layers) > 0):
            bad.append("'layers' must be a non-empty list")
            raise ConfigError("config.json: " + "; ".join(bad))
        object.__setattr__(self, "layers", tuple(self.layers))
        n = len(self.layers)
        if self.loop is not None:
            lp = self.loop
            if not (isinstance(lp, dict) and _int(lp.get("start"), 0) and _int(lp.get("stop"), 0) and _int(lp.get("times"))
                    and lp["start"] < lp["stop"] <= n):
                bad.append(f"'loop' must give 0 <= start < stop <= {n} and times >= 1, got {lp!r}")
        for i, layer in enumerate(self.layers):
            where = f"layers[{i}]"
            if not isinstance(layer, dict) or not isinstance(layer.get("mixer"), dict):
                bad.append(f"{where} must be an object with a 'mixer' object")
                continue
            m, kind = layer["mixer"], layer.get("type")

            def ints(*keys):
                for k in keys:
                    if not _int(m.get(k)):
                        bad.append(f"{where}.mixer.{k} must be a positive integer, got {m.get(k)!r}")

            if kind in ("attention", "attention_2"):
                ints("heads", "kv_heads", "dim", "vdim")
                if _int(m.get("heads")) and _int(m.get("kv_heads")) and m["heads"] % m["kv_heads"]:
                    bad.append(f"{where}.mixer.heads must be a multiple of kv_heads")
                if not _num(m.get("scale")):
                    bad.append(f"{where}.mixer.scale must be a number")
                rot = m.get("rot")
                if not (isinstance(rot, dict) and _num(rot.get("base")) and rot["base"] > 1 and _int(rot.get("dims"), 0)
                        and rot["dims"] % 2 == 0 and _int(m.get("dim")) and rot["dims"] <= m["dim"]):
                    bad.append(f"{where}.mixer.rot must give a 'base' above 1 and an even 'dims' of at most dim")
                elif rot.get("scaling") is not None:
                    sc = rot["scaling"]
                    if not (isinstance(sc, dict) and all(_num(sc.get(k)) for k in SCALING_KEYS[kind]) and sc["factor"] > 0
                            and sc["original"] > 0):
                        bad.append(f"{where}.mixer.rot.scaling must give the numbers {SCALING_KEYS[kind]}, factor and original positive")
                    elif kind == "attention_2" and sc["high"] == sc["low"]:
                        bad.append(f"{where}.mixer.rot.scaling: high and low must differ")
                    elif kind == "attention" and not (sc["fast"] > 0 and sc["slow"] > 0):
                        bad.append(f"{where}.mixer.rot.scaling: fast and slow must be positive")
                if kind == "attention":
                    if not _num(m.get("diff")):
                        bad.append(f"{where}.mixer.diff must be a number")
                elif m.get("mask") is not None:
                    mask = m["mask"]
                    if not (isinstance(mask, dict) and _int(mask.get("size")) and _int(mask.get("keep_first", 0), 0)):
                        bad.append(f"{where}.mixer.mask must give a positive 'size' and a 'keep_first' of 0 or more")
            elif kind == "channel_delta":
                ints("heads", "kv_heads", "dim", "vdim", "conv")
                if _int(m.get("heads")) and _int(m.get("kv_heads")) and m["heads"] % m["kv_heads"]:
                    bad.append(f"{where}.mixer.heads must be a multiple of kv_heads")
                for k in ("decay_rank", "gate_rank"):
                    if m.get(k) is not None and not _int(m[k]):
                        bad.append(f"{where}.mixer.{k} must be a positive integer where it is given")
            else:
                bad.append(f"{where}.type must be 'attention', 'attention_2' or 'channel_delta', got {kind!r}")
            mlp = layer.get("mlp")
            if mlp is None:
                continue
            if not isinstance(mlp, dict) or mlp.get("kind") not in ("dense", "moe"):
                bad.append(f"{where}.mlp must be null or an object of kind 'dense' or 'moe'")
                continue
            if mlp["kind"] == "dense":
                if not _int(mlp.get("ff")):
                    bad.append(f"{where}.mlp.ff must be a positive integer")
                continue
            router, expert, shared = mlp.get("router"), mlp.get("expert"), mlp.get("shared")
            if not (isinstance(router, dict) and _int(router.get("experts")) and _int(router.get("top"))
                    and router["top"] <= router["experts"] and _num(router.get("scale")) and router["scale"] > 0):
                bad.append(f"{where}.mlp.router must give 'experts', 'top' <= experts and a positive 'scale'")
            if not (isinstance(expert, dict) and _int(expert.get("ff"))):
                bad.append(f"{where}.mlp.expert must give 'ff'")
            if shared is not None and not (isinstance(shared, dict) and _int(shared.get("ff"))):
                bad.append(f"{where}.mlp.shared must give 'ff' where it is given")
        if bad:
            raise ConfigError("config.json: " + "; ".join(bad))
