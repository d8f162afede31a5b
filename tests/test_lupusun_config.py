"""The Lupusun design without a GPU: its configuration reader, the order of its layer runs, its model description
against the tensors a folder holds, the cache manager's chunk policy, and the plain implementation's own mechanisms
against closed forms."""
import math

import pytest
import torch

import plain_lupusun as P
from batchspec_b200.cache.manager import CacheManager
from batchspec_b200.config import ConfigError, config_from_json_dict
from batchspec_b200.models import get_model
from batchspec_b200.models.decoder import CacheNeed
from batchspec_b200.parts.base import CacheSpec, Runtime


def attention(heads=3, kv_heads=3, dim=16, vdim=24, scale=0.3, size=10, dims=8, scaling=True):
    rot = dict(base=5000.0, dims=dims)
    if scaling:
        rot["scaling"] = dict(factor=3.0, original=32, fast=8.0, slow=1.0)
    return dict(type="attention", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, scale=scale,
                                             mask=dict(size=size), rot=rot), mlp=dict(kind="dense", ff=40))


def delta(heads=4, kv_heads=2, dim=8, vdim=12, conv=3, mlp=None):
    return dict(type="delta", mixer=dict(heads=heads, kv_heads=kv_heads, dim=dim, vdim=vdim, conv=conv), mlp=mlp)


def config(layers, loop=None, **kw):
    d = dict(architecture="Lupusun", vocab=200, width=48, norm=dict(eps=1e-5), residual_mult=0.5, layers=layers)
    if loop:
        d["loop"] = dict(zip(("start", "stop", "times"), loop))
    d.update(kw)
    return d


def test_reader_takes_every_size_from_the_file_and_round_trips():
    d = config([attention(), delta(), attention(heads=4, kv_heads=1, dim=12, vdim=12, size=7)], loop=(0, 2, 3))
    cfg = config_from_json_dict(d)
    assert (cfg.vocab_size, cfg.width, cfg.norm_eps, cfg.residual_mult) == (200, 48, 1e-5, 0.5)
    assert (cfg.loop_start, cfg.loop_stop, cfg.loop_times) == (0, 2, 3) and not cfg.unread_keys
    assert config_from_json_dict(cfg.to_json_dict()) == cfg
    d2 = config([attention()], foo=1)
    d2["layers"][0]["mixer"]["bar"] = 2
    assert set(config_from_json_dict(d2).unread_keys) == {"foo", "layers[0].mixer.bar"}


@pytest.mark.parametrize("break_it", [
    lambda d: d["layers"][0].update(type="conv"), lambda d: d["layers"][0]["mixer"].update(heads=4, kv_heads=3),
    lambda d: d["layers"][0]["mixer"]["rot"].update(dims=7), lambda d: d["layers"][0]["mixer"]["mask"].update(size=0),
    lambda d: d["layers"][1]["mixer"].update(conv=0), lambda d: d.update(loop=dict(start=1, stop=5, times=2)),
    lambda d: d["layers"][0]["mlp"].update(kind="moe"), lambda d: d["norm"].update(eps=0.0),
    lambda d: d["layers"][0]["mixer"].pop("scale")])
def test_reader_refuses_what_the_engine_cannot_run(break_it):
    d = config([attention(), delta()])
    break_it(d)
    with pytest.raises(ConfigError):
        config_from_json_dict(d)


@pytest.mark.parametrize("n,loop,want", [
    (4, (1, 4, 2), [0, 1, 2, 3, (1,), 2, 3]), (3, (0, 1, 3), [0, (0,), (0,), 1, 2]), (3, None, [0, 1, 2]),
    (3, (1, 2, 1), [0, 1, 2]), (2, (0, 2, 2), [0, 1, (0,), 1]), (3, (2, 2, 5), [0, 1, 2])])
def test_run_order(n, loop, want):
    cfg = config_from_json_dict(config([delta(mlp=dict(kind="dense", ff=8)) for _ in range(n)], loop=loop))
    got = [(i,) if again else i for i, again in cfg.run_order()]
    assert got == want
    assert [(i,) if again else i for i, again in P.layer_order(cfg.to_json_dict())] == want
    spec = get_model(cfg, Runtime(torch.float32, torch.device("cpu"))).spec
    assert [(r.layer,) if r.add_input else r.layer for r in spec.order] == want
    assert all(r.cache_from is None for r in spec.order)          # every run has a cache or state of its own


def test_model_description_names_the_folders_tensors():
    cfg = config_from_json_dict(config([attention(), delta(), delta(mlp=dict(kind="dense", ff=20))], loop=(1, 3, 2)))
    model = get_model(cfg, Runtime(torch.float32, torch.device("cpu")))
    specs = {k: tuple(v.shape) for k, v in model.param_specs().items()}
    assert specs["embed"] == specs["head"] == (200, 48) and specs["embed.norm"] == specs["final.norm"] == (48,)
    assert specs["l0.mix.q"] == (48, 48) and specs["l0.mix.q.b"] == (48,) and specs["l0.mix.v"] == (72, 48)
    assert specs["l0.mix.v.b"] == (72,) and specs["l0.mix.o"] == (48, 72) and specs["l0.mix.sink"] == (3,)
    assert specs["l1.mix.q"] == (16, 48) and specs["l1.mix.q.conv"] == (16, 3) and specs["l1.mix.v.conv"] == (48, 3)
    assert specs["l1.mix.b"] == specs["l1.mix.a"] == (4, 48) and specs["l1.mix.A_log"] == specs["l1.mix.dt_bias"] == (4,)
    assert specs["l1.mix.g"] == (48, 48) and specs["l1.mix.norm"] == (12,) and specs["l1.mix.o"] == (48, 48)
    assert "l1.norm2" not in specs and specs["l2.norm2"] == (48,) and specs["l2.mlp.gate"] == (20, 48)
    needs = model.cache_needs()
    assert len(needs) == 5 and needs[0].cache.policy == "chunk" and needs[0].cache.window == 10
    assert needs[0].cache.tensors == 1 and needs[0].cache.entry_shape == (3 * (16 + 24),)       # values of another size
    assert needs[1].cache is None and needs[1].state.shape[0] >= 4 * 8 * 12 + 2 * (2 * 2 * 8 + 4 * 12)
    assert needs[1].state.shape[0] % 4 == 0 and needs[1].state.dtype == torch.float32


def test_chunk_policy_gives_back_the_pages_before_the_next_positions_chunk():
    need = [CacheNeed(CacheSpec("chunk", (2, 8), 10), None, None), CacheNeed(CacheSpec("full", (2, 8)), None, None)]
    cm = CacheManager(need, page_size=4, num_pages=[5, 12], max_requests=2, dtype=torch.float32, device="cpu",
                      allocate=False)
    cm.admit("a")
    held = lambda: [sum(p >= 0 for p in t) for t in cm.requests["a"].tables]
    for n_new, length, chunk_pages in [(9, 9, 3), (1, 10, 1), (7, 17, 3), (3, 20, 0), (1, 21, 1), (9, 30, 1), (2, 32, 1)]:
        cm.reserve("a", n_new)
        cm.commit("a", n_new)
        cm.check_invariants()
        assert cm.length("a") == length
        # the chunk of the next position starts at (length // 10) * 10; pages wholly before it are gone
        first = (length // 10) * 10 // 4
        assert held() == [-(-length // 4) - first, -(-length // 4)], (length, held())
        assert held()[0] == chunk_pages
        assert all((p < 0) == (i < first) for i, p in enumerate(cm.requests["a"].tables[0]))
    cm.release("a")
    assert cm.free_pages() == [5, 12]


# ------------------------------------------------------------------------ the plain implementation's own mechanisms
def test_plain_attention_mask_sink_and_groups():
    torch.manual_seed(0)
    T, H, G, dim, vdim, size = 23, 4, 2, 6, 5, 7
    q, k, v = torch.randn(T, H, dim).double(), torch.randn(T, G, dim).double(), torch.randn(T, G, vdim).double()
    sink = torch.tensor([-1.0, 0.0, 2.0, 30.0]).double()
    pos = torch.arange(T)
    out = P.chunked_sink_attention(q, k, v, sink, 0.4, size, pos)
    for i in (0, 6, 7, 13, 14, 22):
        for h in range(H):
            js = [j for j in range(T) if j <= i and j // size == i // size]
            s = torch.stack([(q[i, h] @ k[j, h // 2]) * 0.4 for j in js])
            w = torch.exp(s) / (torch.exp(s).sum() + torch.exp(sink[h]))
            assert torch.allclose(out[i, h], sum(w[n] * v[j, h // 2] for n, j in enumerate(js)), atol=1e-12)
    assert out[:, 3].abs().max() < 1e-9                 # a huge sink takes all the weight and gives nothing back
    # shifting all positions by a multiple of the chunk changes nothing; by another amount it does
    assert torch.allclose(P.chunked_sink_attention(q, k, v, sink, 0.4, size, pos + 3 * size), out)
    assert not torch.allclose(P.chunked_sink_attention(q, k, v, sink, 0.4, size, pos + 2), out)


def test_plain_rotation_pairs_halves_and_leaves_the_rest():
    rot = dict(base=100.0, dims=4, scaling=dict(factor=2.0, original=16, fast=4.0, slow=0.5))
    f, mag = P.yarn_frequencies(rot)
    assert mag == pytest.approx(0.1 * math.log(2.0) + 1.0)
    x = torch.tensor([[[1.0, 2.0, 3.0, 4.0, 5.0, 6.0]]], dtype=torch.float64)
    y = P.rotate(x, torch.tensor([3]), rot)
    for i in range(2):
        a = 3 * float(f[i])
        u, v = x[0, 0, i], x[0, 0, i + 2]
        assert y[0, 0, i] == pytest.approx(float(u * math.cos(a) - v * math.sin(a)) * mag)
        assert y[0, 0, i + 2] == pytest.approx(float(v * math.cos(a) + u * math.sin(a)) * mag)
    assert torch.equal(y[..., 4:], x[..., 4:])
    plain, one = P.yarn_frequencies(dict(base=100.0, dims=4))
    assert one == 1.0 and torch.allclose(plain, torch.tensor([1.0, 0.1], dtype=torch.float64))


def test_plain_delta_rule_and_convolution():
    torch.manual_seed(1)
    T, H, dim, vdim = 9, 2, 4, 3
    k = torch.randn(T, H, dim).double()
    k = k / k.norm(dim=-1, keepdim=True)
    q, v = torch.randn(T, H, dim).double(), torch.randn(T, H, vdim).double()
    # beta = 1 and no decay: the state answers the key it has just been given with exactly that value
    o = P.gated_delta_rule(k, k, v, torch.ones(T, H).double(), torch.ones(T, H).double())
    assert torch.allclose(o, v, atol=1e-12)
    # beta = 0 writes nothing
    assert P.gated_delta_rule(q, k, v, torch.zeros(T, H).double(), torch.ones(T, H).double()).abs().max() == 0
    # decay 0 forgets everything before the token: o = beta (q . k) v
    o = P.gated_delta_rule(q, k, v, torch.full((T, H), 0.5).double(), torch.zeros(T, H).double())
    assert torch.allclose(o, 0.5 * (q * k).sum(-1, keepdim=True) * v, atol=1e-12)
    x, w = torch.randn(6, 2).double(), torch.tensor([[1.0, 10.0, 100.0], [0.0, 0.0, 1.0]]).double()
    y = P.short_conv(x, w)
    assert y[0, 0] == pytest.approx(100 * float(x[0, 0])) and torch.allclose(y[:, 1], x[:, 1])
    assert y[4, 0] == pytest.approx(float(x[2, 0] + 10 * x[3, 0] + 100 * x[4, 0]))


def test_kernel_library_features_leave_out_only_what_they_name():
    from batchspec_b200.csrc import build
    every = {p.name for p in build.sources()}
    core = {p.name for p in build.sources(())}
    assert {"delta.cu", "attention_generic.cu", "attention_bf16.cu", "elementwise.cu", "gemm_tcgen05.cu"} <= core
    assert every - core == {n for names in build.FEATURES.values() for n in names}
    assert {p.name for p in build.sources(("moe",))} == core | set(build.FEATURES["moe"])
    assert build.lib_name(None) == build.lib_name(tuple(build.FEATURES)) == build.LIB_NAME
    assert build.lib_name(()) != build.lib_name(("moe",)) != build.LIB_NAME
    with pytest.raises(KeyError):
        build.sources(("nothing",))
