"""Configuration of the Lupusun design: a decoder whose ``config.json`` lists its layers one by one, some of which may
run several times in a row.

    {"architecture": "Lupusun", "vocab": V, "width": d, "norm": {"eps": e}, "residual_mult": m,
     "layers": [{"type": "attention" | "delta", "mixer": {...}, "mlp": {"kind": "dense", "ff": F} | null}, ...],
     "loop": {"start": a, "stop": b, "times": n}}

An ``attention`` mixer gives heads, kv_heads, dim, vdim, scale, ``mask`` {size} (chunks of that many positions;
absent: plain causal) and ``rot`` {base, dims, scaling {factor, original, fast, slow} or nothing}.  A ``delta`` mixer
gives heads, kv_heads, dim, vdim and conv (taps of its short convolutions).  ``loop``: layers a .. b-1 run n times in
a row with the same weights.  Every size and constant is read from here; keys this reader does not know are listed in
``unread_keys``."""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, List, Tuple

from .model_config import ConfigError, _take, register_config_class

_TOP = {"architecture", "architectures", "vocab", "width", "norm", "residual_mult", "layers", "loop"}
_ATTENTION = {"heads", "kv_heads", "dim", "vdim", "scale", "mask", "rot"}
_DELTA = {"heads", "kv_heads", "dim", "vdim", "conv"}
_ROT = {"base", "dims", "scaling"}
_SCALING = {"factor", "original", "fast", "slow"}


def _unknown(d: Dict[str, Any], known, where: str, out: List[str]) -> None:
    out.extend(f"{where}{k}" for k in sorted(set(d) - set(known)))


@dataclass(frozen=True)
class LupusunConfig:
    architecture: str
    vocab_size: int
    width: int
    norm_eps: float
    residual_mult: float
    layers: Tuple[Dict[str, Any], ...]
    loop_start: int
    loop_stop: int
    loop_times: int
    unread_keys: Tuple[str, ...] = ()

    @classmethod
    def from_json_dict(cls, d: Dict[str, Any]) -> "LupusunConfig":
        unread: List[str] = []
        _unknown(d, _TOP, "", unread)
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        norm = d.get("norm") or {}
        _unknown(norm, {"eps"}, "norm.", unread)
        out = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            _unknown(layer, {"type", "mixer", "mlp"}, where + ".", unread)
            kind, m = layer.get("type"), layer.get("mixer") or {}
            if kind not in ("attention", "delta"):
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design "
                                  f"(known: 'attention', 'delta')")
            _unknown(m, _ATTENTION if kind == "attention" else _DELTA, where + ".mixer.", unread)
            for key in ("heads", "kv_heads", "dim", "vdim"):
                if _take(m, key, int) <= 0:
                    raise ConfigError(f"config.json: {where}.mixer.{key} must be positive")
            if m["heads"] % m["kv_heads"]:
                raise ConfigError(f"config.json: {where}.mixer.heads must be a multiple of kv_heads")
            if kind == "attention":
                _take(m, "scale", float)
                mask = m.get("mask")
                if mask is not None:
                    _unknown(mask, {"size"}, where + ".mixer.mask.", unread)
                    if _take(mask, "size", int) <= 0:
                        raise ConfigError(f"config.json: {where}.mixer.mask.size must be positive")
                rot = m.get("rot")
                if rot is not None:
                    _unknown(rot, _ROT, where + ".mixer.rot.", unread)
                    _take(rot, "base", float)
                    dims = _take(rot, "dims", int)
                    if dims < 0 or dims % 2 or dims > m["dim"]:
                        raise ConfigError(f"config.json: {where}.mixer.rot.dims must be even and at most dim")
                    if rot.get("scaling"):
                        _unknown(rot["scaling"], _SCALING, where + ".mixer.rot.scaling.", unread)
                        for key in sorted(_SCALING):
                            _take(rot["scaling"], key, float)
            elif _take(m, "conv", int) < 1:
                raise ConfigError(f"config.json: {where}.mixer.conv must be at least 1")
            f = layer.get("mlp")
            if f is not None:
                if f.get("kind", "dense") != "dense":
                    raise ConfigError(f"config.json: {where}.mlp.kind {f.get('kind')!r} is not known ('dense' or null)")
                _unknown(f, {"kind", "ff"}, where + ".mlp.", unread)
                if _take(f, "ff", int) <= 0:
                    raise ConfigError(f"config.json: {where}.mlp.ff must be positive")
            out.append(copy.deepcopy(layer))
        loop = d.get("loop") or {}
        _unknown(loop, {"start", "stop", "times"}, "loop.", unread)
        start, stop, times = _take(loop, "start", int, 0), _take(loop, "stop", int, 0), _take(loop, "times", int, 1)
        if not (0 <= start <= stop <= len(out)) or times < 1:
            raise ConfigError(f"config.json: loop {loop} does not fit {len(out)} layers")
        cfg = cls(architecture=d.get("architecture") or (d.get("architectures") or [None])[0],
                  vocab_size=_take(d, "vocab", int), width=_take(d, "width", int), norm_eps=_take(norm, "eps", float),
                  residual_mult=_take(d, "residual_mult", float, 1.0), layers=tuple(out), loop_start=start,
                  loop_stop=stop, loop_times=times, unread_keys=tuple(unread))
        if cfg.vocab_size <= 0 or cfg.width <= 0 or not cfg.norm_eps > 0:
            raise ConfigError("config.json: vocab and width must be positive and norm.eps > 0")
        return cfg

    def run_order(self) -> List[Tuple[int, bool]]:
        """(layer, whether it opens a pass after the first) for every layer run: layers before the loop, the looped
        layers ``loop_times`` times in a row, the layers after it."""
        n, a, b, times = len(self.layers), self.loop_start, self.loop_stop, self.loop_times
        if b <= a or times <= 1:
            return [(i, False) for i in range(n)]
        runs = [(i, False) for i in range(a)]
        for t in range(times):
            runs += [(i, t > 0 and i == a) for i in range(a, b)]
        return runs + [(i, False) for i in range(b, n)]

    def to_json_dict(self) -> Dict[str, Any]:
        return {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.width,
                "norm": {"eps": self.norm_eps}, "residual_mult": self.residual_mult,
                "layers": copy.deepcopy(list(self.layers)),
                "loop": {"start": self.loop_start, "stop": self.loop_stop, "times": self.loop_times}}


register_config_class("Lupusun", LupusunConfig)
