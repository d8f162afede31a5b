"""The Vabanex design as a model description: an embedding times a constant; pre-norm layers with layer norms
(weight and bias), a latent-attention mixer with an output gate per head, and a feed-forward that is a clamped
GLU, a routed set of GELU experts, or absent; a final layer norm, an untied head and a tanh soft cap on the
logits.  Layers are listed one by one in the configuration and may all differ.

Checkpoint names: ``embed``, ``l<i>.norm1`` (bias: ``.b``), ``l<i>.mix.{dq, dq.norm, uq, dkv, dkv.norm, uk, uv, g,
o}``, ``l<i>.norm2``, ``l<i>.mlp.{gate, up, down}`` or ``l<i>.mlp.{router, correction, e<j>.up, e<j>.down}``,
``final.norm``, ``head``."""
from __future__ import annotations

from ..config.vabanex_config import VabanexConfig
from ..parts.base import PartSpec
from .spec import LayerSpec, ModelSpec, RunEntry


def build_vabanex(cfg: VabanexConfig) -> ModelSpec:
    norm = PartSpec("layernorm", dict(dim=cfg.width, eps=cfg.norm_eps))
    layers, ignore = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer["mixer"]
        rot = m["rot"]
        scaling = dict(rope_type="yarn", **rot["scaling"]) if rot.get("scaling") else None
        position = PartSpec("rope", dict(head_dim=m["rot_dim"], theta=rot["base"], scaling=scaling,
                                         rotary_dim=rot["dims"], interleaved=True))
        mixer = PartSpec("latent_attention", dict(
            dim=cfg.width, n_heads=m["heads"], head_dim=m["dim"], rot_dim=m["rot_dim"], v_dim=m["vdim"],
            q_rank=m["q_rank"], kv_rank=m["kv_rank"], scale=m["scale"], eps=cfg.norm_eps, position=position))
        names = {"norm1.weight": p + "norm1", "norm1.bias": p + "norm1.b", "mixer.dq_norm": p + "mix.dq.norm",
                 "mixer.dkv_norm": p + "mix.dkv.norm"}
        names.update({f"mixer.{k}": p + "mix." + k for k in ("dq", "uq", "dkv", "uk", "uv", "g", "o")})
        f = layer.get("mlp")
        if f is None:
            layers.append(LayerSpec({"norm1": norm, "mixer": mixer}, names, "prenorm_mixer"))
            ignore += [p + "norm2", p + "norm2.b"]       # a second norm without a feed-forward is never applied
            continue
        names.update({"norm2.weight": p + "norm2", "norm2.bias": p + "norm2.b"})
        if f["kind"] == "dense":
            ffn = PartSpec("clamped_glu", dict(dim=cfg.width, intermediate=f["ff"], limit=f["limit"]))
            names.update({f"ffn.{k}": p + "mlp." + k for k in ("gate", "up", "down")})
        else:
            r = f["router"]
            g = r.get("groups") or {}
            E = r["experts"]
            ffn = PartSpec("routed_gelu", dict(dim=cfg.width, intermediate=f["expert"]["ff"], n_experts=E, top=r["top"],
                                               scale=r.get("scale", 1.0), n_groups=g.get("count", 1),
                                               keep_groups=g.get("keep", 1)))
            names.update({"ffn.router": p + "mlp.router", "ffn.correction": p + "mlp.correction"})
            for e in range(E):
                names[f"ffn.up{e}"] = f"{p}mlp.e{e}.up"
                names[f"ffn.down{e}"] = f"{p}mlp.e{e}.down"
        layers.append(LayerSpec({"norm1": norm, "mixer": mixer, "norm2": norm, "ffn": ffn}, names, "prenorm"))
    return ModelSpec(
        vocab_size=cfg.vocab_size, hidden_size=cfg.width, layers=layers,
        order=[RunEntry(i) for i in range(len(layers))], final_norm=norm, embed_name="embed",
        final_norm_names={"weight": "final.norm", "bias": "final.norm.b"}, lm_head_name="head",
        ignore_names=tuple(ignore), embed_scale=cfg.embedding_scale,
        logits_part=PartSpec("tanh_softcap", dict(cap=cfg.logit_softcap)) if cfg.logit_softcap else None)
