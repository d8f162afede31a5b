"""The Vabanex configuration reader, the model description's tensor names, and the plain implementation's router
on a case worked by hand (CPU)."""
import copy
import json

import pytest
import torch

import plain_vabanex as P
from batchspec_b200.config import ConfigError, config_from_json_dict, load_config
from batchspec_b200.models import get_model
from batchspec_b200.parts.base import Runtime

MIXER = dict(heads=3, dim=16, rot_dim=8, vdim=24, q_rank=40, kv_rank=48, scale=0.2,
             rot=dict(base=10000.0, dims=8, scaling=dict(factor=8.0, original=64, fast=16.0, slow=2.0)))
CFG = dict(architecture="Vabanex", vocab=300, width=64, embedding=dict(scale=2.5), norm=dict(eps=1e-5), logit_softcap=20.0,
           layers=[dict(type="latent_attention", mixer=MIXER, mlp=dict(kind="dense", ff=80, limit=0.7)),
                   dict(type="latent_attention", mixer=MIXER,
                        mlp=dict(kind="moe", expert=dict(ff=24),
                                 router=dict(experts=6, top=3, scale=1.5, groups=dict(count=3, keep=2)))),
                   dict(type="latent_attention", mixer=MIXER, mlp=None)])


def test_reads_every_size_and_round_trips(tmp_path):
    cfg = config_from_json_dict(CFG)
    assert (cfg.architecture, cfg.vocab_size, cfg.width, cfg.embedding_scale, cfg.logit_softcap) == ("Vabanex", 300, 64, 2.5, 20.0)
    assert config_from_json_dict(cfg.to_json_dict()) == cfg
    (tmp_path / "config.json").write_text(json.dumps(CFG))
    assert load_config(tmp_path) == cfg


@pytest.mark.parametrize("path,value", [(("layers", 0, "type"), "other_mixer"), (("layers", 0, "mixer", "window"), 5),
                                        (("layers", 1, "mlp", "kind"), "glu"), (("layers", 0, "mixer", "rot", "dims"), 6),
                                        (("layers", 1, "mlp", "router", "top"), 5), (("pool",), 2),
                                        (("layers", 1, "mlp", "router", "groups", "count"), 4)])
def test_refuses_what_it_does_not_compute(path, value):
    bad = copy.deepcopy(CFG)
    node = bad
    for k in path[:-1]:
        node = node[k]
    node[path[-1]] = value
    with pytest.raises(ConfigError):
        config_from_json_dict(bad)


def test_tensor_names_and_shapes():
    model = get_model(config_from_json_dict(CFG), Runtime(torch.float32, torch.device("cpu")))
    specs = model.param_specs()
    assert specs["embed"].shape == (300, 64) and specs["head"].shape == (300, 64)
    assert specs["l0.mix.dkv"].shape == (48 + 8, 64) and specs["l0.mix.uq"].shape == (3 * (16 + 8), 40)
    assert specs["l0.mix.uk"].shape == (3 * 16, 48) and specs["l0.mix.uv"].shape == (3 * 24, 48)
    assert specs["l0.mix.g"].shape == (3, 64) and specs["l0.mix.o"].shape == (64, 72)
    assert specs["l0.mix.dq.norm"].shape == (40,) and specs["l0.norm1.b"].shape == (64,)
    assert specs["l1.mlp.e5.down"].shape == (64, 24) and specs["l1.mlp.correction"].shape == (6,)
    assert "l2.norm2" not in specs and "l2.mlp.gate" not in specs and "final.norm.b" in specs
    assert len(model.cache_needs()) == 3 and model.cache_needs()[0].cache.entry_shape == (56,)
    assert model.cache_needs()[0].cache.tensors == 1 and model.graph_safe


def test_router_by_hand():
    """Six experts in three pairs, keep two groups, take three.  The scores make the middle pair's sum the
    smallest although it holds the second largest single score, and the correction moves one choice."""
    s = torch.tensor([[0.9, 0.1, 0.85, 0.05, 0.5, 0.45]], dtype=torch.float64)
    z = torch.log(s / (1 - s))
    w = {"router": torch.eye(6, dtype=torch.float64), "correction": torch.tensor([0, 0, 0, 0, 0, 0.1], dtype=torch.float64)}
    ids, wt = P.route(z, w, "", dict(experts=6, top=3, scale=2.0, groups=dict(count=3, keep=2)))
    # group sums: 1.0, 0.9, 1.05 -> the middle pair is dropped; choices left: 0.9, 0.1, 0.5, 0.55
    assert sorted(ids[0].tolist()) == [0, 4, 5]
    got = dict(zip(ids[0].tolist(), wt[0].tolist()))
    assert got[5] == pytest.approx(0.9) and got[4] == pytest.approx(1.0) and got[0] == pytest.approx(1.8)


def _tiny_model(seed=3):
    g = torch.Generator().manual_seed(seed)
    cfg = copy.deepcopy(CFG)
    model = get_model(config_from_json_dict(cfg), Runtime(torch.float32, torch.device("cpu")))
    w = {}
    for name, spec in model.param_specs().items():
        t = torch.randn(spec.shape, generator=g, dtype=torch.float64) * (0.2 if len(spec.shape) > 1 else 0.1)
        w[name] = t + 1.0 if spec.init == "ones_normal" else t
    return cfg, w


def test_plain_implementation_is_causal_and_position_aware():
    """Properties the oracle must have whatever its weights: a later token changes no earlier logits; the same
    token at another position gives other logits (the rotation acts); the soft cap bounds the logits."""
    cfg, w = _tiny_model()
    toks = [5, 17, 3, 250, 99, 17, 8, 64, 1, 2, 33]
    base = P.forward(cfg, w, toks)
    other = P.forward(cfg, w, toks[:6] + [77] + toks[7:])
    assert torch.equal(base[:6], other[:6]) and not torch.allclose(base[6:], other[6:])
    assert not torch.allclose(base[1], base[5])                  # token 17 at positions 1 and 5
    assert base.abs().max() < cfg["logit_softcap"]
    layers = []
    P.forward(cfg, w, toks, layers)
    assert len(layers) == 3 and layers[0].shape == (len(toks), cfg["width"])


def test_rotation_keeps_pairs_lengths_times_the_magnitude():
    f, mag = P.yarn_frequencies(MIXER["rot"])
    assert mag == pytest.approx(0.1 * torch.log(torch.tensor(8.0)).item() + 1.0)
    x = torch.randn(7, 8, dtype=torch.float64)
    y = P.rotate_pairs(x, torch.arange(7) * 13, f, mag)
    assert torch.allclose((y[:, 0::2] ** 2 + y[:, 1::2] ** 2), mag ** 2 * (x[:, 0::2] ** 2 + x[:, 1::2] ** 2))
    assert torch.allclose(y[0], x[0] * mag)                      # position 0 rotates by nothing
