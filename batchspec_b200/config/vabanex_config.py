"""Configuration of the Vabanex design: a decoder whose ``config.json`` lists its layers one by one.

    {"architecture": "Vabanex", "vocab": V, "width": d, "embedding": {"scale": a}, "norm": {"eps": e},
     "logit_softcap": c, "layers": [{"type": "latent_attention", "mixer": {...}, "mlp": {...} | null}, ...]}

A layer's ``mixer`` gives heads, dim (unrotated numbers per head), rot_dim, vdim, q_rank, kv_rank, scale and
``rot`` {base, dims, scaling {factor, original, fast, slow} or nothing}.  ``mlp`` is {"kind": "dense", ff, limit},
{"kind": "moe", "expert": {ff}, "router": {experts, top, scale, groups {count, keep}}}, or null for a layer
without a feed-forward.  Every size and constant is read from here; a key this reader does not know is an error,
since it would stand for arithmetic the engine does not do."""
from __future__ import annotations

import copy
from dataclasses import dataclass
from typing import Any, Dict, Tuple

from .model_config import ConfigError, _take, register_config_class

_TOP = {"architecture", "architectures", "vocab", "width", "embedding", "norm", "logit_softcap", "layers"}
_MIXER = {"heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank", "scale", "rot"}
_ROT = {"base", "dims", "scaling"}
_SCALING = {"factor", "original", "fast", "slow"}


def _only(d: Dict[str, Any], known, where: str) -> None:
    extra = sorted(set(d) - set(known))
    if extra:
        raise ConfigError(f"config.json: {where} has keys this engine does not apply: {', '.join(extra)}")


@dataclass(frozen=True)
class VabanexConfig:
    architecture: str
    vocab_size: int
    width: int
    embedding_scale: float
    norm_eps: float
    logit_softcap: float            # 0: none
    layers: Tuple[Dict[str, Any], ...]
    unread_keys: Tuple[str, ...] = ()

    @classmethod
    def from_json_dict(cls, d: Dict[str, Any]) -> "VabanexConfig":
        _only(d, _TOP, "the model")
        layers = d.get("layers")
        if not isinstance(layers, list) or not layers:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        emb = d.get("embedding") or {}
        _only(emb, {"scale"}, "'embedding'")
        norm = d.get("norm") or {}
        _only(norm, {"eps"}, "'norm'")
        out = []
        for i, layer in enumerate(layers):
            where = f"layers[{i}]"
            _only(layer, {"type", "mixer", "mlp"}, where)
            if layer.get("type") != "latent_attention":
                raise ConfigError(f"config.json: {where}.type {layer.get('type')!r} is not a mixer of this design "
                                  f"(known: 'latent_attention')")
            m = layer.get("mixer") or {}
            _only(m, _MIXER, where + ".mixer")
            for key in ("heads", "dim", "rot_dim", "vdim", "q_rank", "kv_rank"):
                if _take(m, key, int) <= 0:
                    raise ConfigError(f"config.json: {where}.mixer.{key} must be positive")
            _take(m, "scale", float)
            rot = m.get("rot") or {}
            _only(rot, _ROT, where + ".mixer.rot")
            _take(rot, "base", float)
            if _take(rot, "dims", int) != m["rot_dim"] or m["rot_dim"] % 2:
                raise ConfigError(f"config.json: {where}.mixer.rot.dims must equal rot_dim and be even")
            if rot.get("scaling"):
                _only(rot["scaling"], _SCALING, where + ".mixer.rot.scaling")
                for key in _SCALING:
                    _take(rot["scaling"], key, float)
            f = layer.get("mlp")
            if f is not None:
                kind = f.get("kind")
                if kind == "dense":
                    _only(f, {"kind", "ff", "limit"}, where + ".mlp")
                    _take(f, "ff", int)
                    _take(f, "limit", float)
                elif kind == "moe":
                    _only(f, {"kind", "expert", "router"}, where + ".mlp")
                    _only(f.get("expert") or {}, {"ff"}, where + ".mlp.expert")
                    _take(f.get("expert") or {}, "ff", int)
                    r = f.get("router") or {}
                    _only(r, {"experts", "top", "scale", "groups"}, where + ".mlp.router")
                    E, top = _take(r, "experts", int), _take(r, "top", int)
                    _take(r, "scale", float, 1.0)
                    g = r.get("groups") or {}
                    _only(g, {"count", "keep"}, where + ".mlp.router.groups")
                    G, keep = _take(g, "count", int, 1), _take(g, "keep", int, 1)
                    if not (0 < top <= E and G > 0 and E % G == 0 and 0 < keep <= G and keep * (E // G) >= top):
                        raise ConfigError(f"config.json: {where}.mlp.router cannot choose {top} of {E} experts in {G} "
                                          f"groups keeping {keep}")
                else:
                    raise ConfigError(f"config.json: {where}.mlp.kind {kind!r} is not known ('dense', 'moe' or null)")
            out.append(copy.deepcopy(layer))
        cfg = cls(architecture=d.get("architecture") or (d.get("architectures") or [None])[0],
                  vocab_size=_take(d, "vocab", int), width=_take(d, "width", int),
                  embedding_scale=_take(emb, "scale", float, 1.0), norm_eps=_take(norm, "eps", float),
                  logit_softcap=_take(d, "logit_softcap", float, 0.0), layers=tuple(out))
        if cfg.vocab_size <= 0 or cfg.width <= 0 or not cfg.norm_eps > 0 or cfg.logit_softcap < 0:
            raise ConfigError("config.json: vocab and width must be positive, norm.eps > 0, logit_softcap >= 0")
        return cfg

    def to_json_dict(self) -> Dict[str, Any]:
        d: Dict[str, Any] = {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.width,
                             "embedding": {"scale": self.embedding_scale}, "norm": {"eps": self.norm_eps},
                             "layers": copy.deepcopy(list(self.layers))}
        if self.logit_softcap:
            d["logit_softcap"] = self.logit_softcap
        return d


register_config_class("Vabanex", VabanexConfig)
