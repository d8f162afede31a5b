"""The Lupusun design as a model description: an RMS-normed embedding; pre-norm layers whose branches are added with a
common factor, each with either a chunk-masked grouped-query attention (biases, partial YaRN rotation, q/k norm after
the rotation, a sink per head) or a gated delta rule mixer, and a ReLU-gated feed-forward or none; a span of layers
that runs several times in a row with shared weights, separate caches and state, and the embedding output added
before every pass but the first; a final RMS norm and an untied head.

Checkpoint names: ``embed``, ``embed.norm``, ``l<i>.norm1``, ``l<i>.norm2``, ``l<i>.mix.{q, k, v, o}`` with
``.b`` added for the attention's biases and ``.conv`` for the delta mixer's convolutions, ``l<i>.mix.sink``,
``l<i>.mix.{b, a, A_log, dt_bias, g, norm}``, ``l<i>.mlp.{gate, up, down}``, ``final.norm``, ``head``."""
from __future__ import annotations

from ..config.lupusun_config import LupusunConfig
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, RunEntry


def build_lupusun(cfg: LupusunConfig) -> ModelSpec:
    norm = PartSpec("rmsnorm", dict(dim=cfg.width, eps=cfg.norm_eps, single_rounding=True))
    block_params = dict(residual_mult=cfg.residual_mult)
    layers, ignore = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        names = {"norm1.weight": p + "norm1"}
        if layer["type"] == "attention":
            rot = m.get("rot")
            if rot and rot["dims"]:
                scaling = dict(rope_type="yarn", **rot["scaling"]) if rot.get("scaling") else None
                position = PartSpec("rope", dict(head_dim=m["dim"], theta=rot["base"], scaling=scaling,
                                                 rotary_dim=rot["dims"], interleaved=False))
            else:
                position = PartSpec("none")
            mixer = PartSpec("sink_attention", dict(
                dim=cfg.width, n_heads=m["heads"], n_kv_heads=m["kv_heads"], head_dim=m["dim"], v_dim=m["vdim"],
                scale=m["scale"], position=position, bias=True, qk_norm_eps=cfg.norm_eps,
                chunk=(m.get("mask") or {}).get("size"), sink=True))
            names.update({f"mixer.{k}": p + "mix." + k for k in ("q", "k", "v", "o", "sink")})
            names.update({f"mixer.{k}_bias": f"{p}mix.{k}.b" for k in ("q", "k", "v")})
        else:
            mixer = PartSpec("gated_delta", dict(dim=cfg.width, n_heads=m["heads"], n_kv_heads=m["kv_heads"],
                                                 head_dim=m["dim"], v_dim=m["vdim"], taps=m["conv"], eps=cfg.norm_eps))
            names.update({f"mixer.{k}": p + "mix." + k for k in ("q", "k", "v", "o", "b", "a", "A_log", "dt_bias", "g",
                                                                "norm")})
            names.update({f"mixer.{k}_conv": f"{p}mix.{k}.conv" for k in ("q", "k", "v")})
        f = layer.get("mlp")
        if f is None:
            layers.append(LayerSpec({"norm1": norm, "mixer": mixer}, names, "prenorm_mixer", block_params))
            ignore.append(p + "norm2")                   # a second norm without a feed-forward is never applied
            continue
        names["norm2.weight"] = p + "norm2"
        names.update({f"ffn.{k}": p + "mlp." + k for k in ("gate", "up", "down")})
        ffn = PartSpec("swiglu", dict(dim=cfg.width, intermediate=f["ff"], activation="relu"))
        layers.append(LayerSpec({"norm1": norm, "mixer": mixer, "norm2": norm, "ffn": ffn}, names, "prenorm",
                                block_params))
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden_size=cfg.width, layers=layers,
        order=[RunEntry(i, add_input=again) for i, again in cfg.run_order()], final_norm=norm, embed_name="embed",
        final_norm_names={"weight": "final.norm"}, lm_head_name="head", ignore_names=tuple(ignore),
        input_part=PartSpec("rmsnorm", dict(dim=cfg.width, eps=cfg.norm_eps)), input_names={"weight": "embed.norm"})
