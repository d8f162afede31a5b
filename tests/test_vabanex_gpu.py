"""The Vabanex design on the GPU against its plain implementation (tests/plain_vabanex.py): every mechanism alone,
then the engine on whole prompts, decoded tails, portions down to two tokens, mixed batches on a pool so small
that pages are used again, and greedy generation through the scheduler.  The configurations are made here; their
sizes all differ from each other (heads, unrotated / rotated / value sizes, ranks, groups), one has layers of
different mixers (two cache groups), a layer without a feed-forward, groups of a single expert, no frequency
blend, no soft cap, and a width that is no multiple of 8."""
import math
from types import SimpleNamespace

import numpy as np
import pytest
import torch

import helpers as H
import plain_vabanex as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
DTYPES = ["float32", "bfloat16"]


def _mixer(heads, dim, rot, vdim, q_rank, kv_rank, scale, base, scaling):
    return dict(heads=heads, dim=dim, rot_dim=rot, vdim=vdim, q_rank=q_rank, kv_rank=kv_rank, scale=scale,
                rot=dict(base=base, dims=rot, **({"scaling": scaling} if scaling else {})))


def _moe(ff, experts, top, scale, count, keep):
    return dict(kind="moe", expert=dict(ff=ff), router=dict(experts=experts, top=top, scale=scale,
                                                           groups=dict(count=count, keep=keep)))


MIX_A = _mixer(3, 16, 8, 24, 40, 48, 0.2, 10000.0, dict(factor=8.0, original=64, fast=16.0, slow=2.0))
CFG_A = dict(architecture="Vabanex", vocab=300, width=64, embedding=dict(scale=2.5), norm=dict(eps=1e-5),
             logit_softcap=20.0,
             layers=[dict(type="latent_attention", mixer=MIX_A, mlp=dict(kind="dense", ff=80, limit=0.7)),
                     dict(type="latent_attention", mixer=MIX_A, mlp=_moe(24, 6, 3, 1.5, 3, 2)),
                     dict(type="latent_attention", mixer=MIX_A, mlp=None)])
MIX_B1 = _mixer(5, 24, 16, 8, 24, 72, 0.15, 50000.0, None)
MIX_B2 = _mixer(2, 8, 4, 40, 56, 20, 0.3, 777.0, dict(factor=2.0, original=16, fast=8.0, slow=0.5))
CFG_B = dict(architecture="Vabanex", vocab=513, width=100, embedding=dict(scale=1.0), norm=dict(eps=1e-6),
             layers=[dict(type="latent_attention", mixer=MIX_B1, mlp=_moe(36, 4, 2, 0.8, 4, 2)),
                     dict(type="latent_attention", mixer=MIX_B2, mlp=dict(kind="dense", ff=52, limit=3.0)),
                     dict(type="latent_attention", mixer=MIX_B1, mlp=_moe(20, 8, 1, 2.0, 1, 1))])
# sizes at which the tensor-core attention kernel runs in bfloat16 (ranks and rotated part multiples of 16)
MIX_C = _mixer(16, 32, 32, 48, 64, 128, 0.09, 100000.0, dict(factor=4.0, original=128, fast=32.0, slow=1.0))
CFG_C = dict(architecture="Vabanex", vocab=640, width=256, embedding=dict(scale=4.0), norm=dict(eps=1e-5),
             logit_softcap=25.0,
             layers=[dict(type="latent_attention", mixer=MIX_C, mlp=_moe(64, 16, 4, 2.5, 4, 2)),
                     dict(type="latent_attention", mixer=MIX_C, mlp=dict(kind="dense", ff=192, limit=1.5))])
CONFIGS = {"A": (CFG_A, 11, 4), "B": (CFG_B, 12, 8), "C": (CFG_C, 13, 16)}       # config, seed, page size
LENGTHS = {"A": [1, 6, 23, 70], "B": [2, 9, 41, 130], "C": [3, 64, 150, 333]}


def _folder(tmp_path, name, dtype):
    cfg, seed, _ = CONFIGS[name]
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    return H.make_folder(tmp_path / f"v{name}_{dtype}", cfg, seed, dtype=stored)


def _engine(folder, dtype, page_size, num_pages, max_requests=8):
    from batchspec_b200.engine import Engine
    eng = Engine(dtype=dtype, device=DEV)
    eng.load_model(model_dir=folder)
    eng.setup_caches(max_batch_size=max_requests, page_size=page_size, num_pages=num_pages)
    return eng


def _oracle(folder, tokens):
    cfg, w = P.read_model_folder(folder)
    return P.forward(cfg, w, tokens).numpy()


def _requests(name):
    cfg, seed, _ = CONFIGS[name]
    return {f"r{i}": H.random_tokens(n, cfg["vocab"], 100 * seed + i) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def ops():
    from batchspec_b200.kernels import ops as o
    o.load_library()
    return o


def _flips(dtype):
    """Share of rows that may miss the tolerance: in bfloat16 a router's choice between two experts whose scores
    differ by less than the rounding of its input falls either way, and the row (not its neighbours) moves."""
    return 0.05 if dtype == "bfloat16" else 0.0


def _rows_agree(a, b, dtype):
    far = sum(np.abs(a[k] - b[k]).max() > H.TOL[dtype] * np.abs(a[k]).max() for k in a)
    assert far <= _flips(dtype) * len(a), f"{far} of {len(a)} rows differ between two ways of cutting"


def _tol(dtype):
    return 2e-5 if dtype == torch.float32 else 2e-2


# ------------------------------------------------------------------------------------------- mechanisms alone

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,d,eps", [(3, 96, 1e-6), (17, 1000, 1e-5), (2, 4096, 1e-2), (5, 50, 1e-5), (1, 18000, 1e-5)])
def test_add_layernorm(ops, dtype, n, d, eps):
    g = torch.Generator(device=DEV).manual_seed(d)
    resid = torch.randn(n, d, device=DEV, generator=g) * 3 + 5.0          # a mean far from 0: var is not E[x^2]
    delta = torch.randn(n, d, device=DEV, generator=g).to(dtype)
    w = (1 + 0.3 * torch.randn(d, device=DEV, generator=g)).to(dtype)
    b = torch.randn(d, device=DEV, generator=g).to(dtype)
    for dl in (None, delta):
        r = resid.clone()
        out = torch.full((n, d), float("nan"), device=DEV, dtype=dtype)
        ops.add_layernorm(r, dl, w, b, eps, out)
        x = resid.double() + (dl.double() if dl is not None else 0)
        want = P.layer_norm(x.cpu(), w.double().cpu(), b.double().cpu(), eps)
        assert torch.allclose(r.double().cpu(), x.cpu(), atol=1e-6)
        err = (out.double().cpu() - want).abs().max() / want.abs().max()
        assert err <= _tol(dtype), err


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_clamped_glu_and_gelu_and_softcap(ops, dtype):
    g = torch.Generator(device=DEV).manual_seed(1)
    n, inter, L = 7, 52, 0.9
    u = (2.5 * torch.randn(n, 2 * inter, device=DEV, generator=g)).to(dtype)
    m = torch.empty(n, inter, device=DEV, dtype=dtype)
    ops.clamped_glu(u, m, 1.702, L)
    gate, up = u[:, :inter].double().clamp(max=L), u[:, inter:].double().clamp(-L, L)
    want = gate * torch.sigmoid(1.702 * gate) * (up + 1)
    assert (gate == L).any() and (up == -L).any() and (gate < -L).any()       # the clamps act, and only one on the gate
    assert (m.double() - want).abs().max() <= _tol(dtype) * want.abs().max() * 2
    x = (3 * torch.randn(1000, device=DEV, generator=g)).to(dtype)
    want = 0.5 * x.double() * (1 + torch.erf(x.double() / math.sqrt(2)))
    assert (ops.gelu_erf_(x.clone()).double() - want).abs().max() <= _tol(dtype) * 3
    z = 40 * torch.randn(5, 33, device=DEV, generator=g)
    want = 12.5 * torch.tanh(z.double() / 12.5)
    assert (ops.tanh_softcap_(z.clone(), 12.5).double() - want).abs().max() <= 1e-5


@pytest.mark.parametrize("M,I,K", [(1, 80, 64), (8, 8448, 2048), (5, 176, 72), (40, 256, 96), (3, 52, 64)])
def test_clamped_glu_in_the_products_epilogue(ops, M, I, K):
    """bfloat16 gate/up product with the clamped activation: decode-sized steps apply it in the product's epilogue
    (weights interleaved in groups of 8), larger ones in a kernel of its own; both against float64."""
    g = torch.Generator(device=DEV).manual_seed(M + I)
    x = torch.randn(M, K, device=DEV, generator=g).bfloat16()
    wg = (2.0 * torch.randn(I, K, device=DEV, generator=g) / K ** 0.5).bfloat16()
    wu = (2.0 * torch.randn(I, K, device=DEV, generator=g) / K ** 0.5).bfloat16()
    L, alpha = 1.1, 1.702
    gate = (x.double() @ wg.double().T).clamp(max=L)
    up = (x.double() @ wu.double().T).clamp(-L, L)
    want = gate * torch.sigmoid(alpha * gate) * (up + 1)
    if I % ops.GLU_GROUP == 0:
        got = ops.linear_clamped_glu(x, ops.interleave_gate_up(wg, wu), alpha, L)
    else:
        got = torch.empty(M, I, device=DEV, dtype=torch.bfloat16)
        ops.clamped_glu(ops.linear(x, torch.cat([wg, wu])), got, alpha, L)
    torch.cuda.synchronize()
    ops.check_status()
    assert (got.double() - want).abs().max() <= 3e-2 * max(1.0, want.abs().max().item())


def test_yarn_frequencies_and_rotation_of_strided_heads(ops):
    from batchspec_b200.parts.rope import rope_inv_freq, yarn_magnitude
    for rot in (dict(base=250.0, dims=16, scaling=dict(factor=6.0, original=40, fast=10.0, slow=1.5)),
                dict(base=1e6, dims=64, scaling=dict(factor=40.0, original=4096, fast=32.0, slow=1.0)),
                dict(base=10.0, dims=4, scaling=dict(factor=3.0, original=8, fast=1.0, slow=1.0)),      # a ramp of no width
                dict(base=5000.0, dims=8)):
        sc = rot.get("scaling")
        f = rope_inv_freq(rot["dims"], rot["base"], dict(rope_type="yarn", **sc) if sc else None)
        want, mag = P.yarn_frequencies(rot)
        assert torch.allclose(f, want, rtol=1e-12, atol=0)
        assert (yarn_magnitude(sc["factor"]) if sc else 1.0) == pytest.approx(mag, rel=1e-12)
        if sc:
            assert not torch.allclose(f, P.yarn_frequencies(dict(base=rot["base"], dims=rot["dims"]))[0])
    # the rotated part sits at the end of wider heads: a view with a head stride larger than its width
    rot = dict(base=250.0, dims=16, scaling=dict(factor=6.0, original=40, fast=10.0, slow=1.5))
    f, mag = P.yarn_frequencies(rot)
    n, Hh, wide = 9, 3, 40
    g = torch.Generator(device=DEV).manual_seed(3)
    pos = torch.tensor([0, 1, 2, 39, 40, 41, 1000, 5003, 70001], dtype=torch.int32, device=DEV)
    for dtype in (torch.float32, torch.bfloat16):
        q = torch.randn(n, Hh, wide, device=DEV, generator=g).to(dtype)
        before = q.clone()
        ops.rope_inplace(q[:, :, wide - 16:], pos, ops.rope_frequency_table(f, DEV), 16, True, mag)
        want = P.rotate_pairs(before[:, :, wide - 16:].double().cpu().transpose(0, 1), pos.cpu().long(), f, mag).transpose(0, 1)
        assert torch.equal(q[:, :, :wide - 16], before[:, :, :wide - 16])
        assert (q[:, :, wide - 16:].double().cpu() - want).abs().max() <= (1e-5 if dtype == torch.float32 else 2e-2)


def _latent_case(ops, dtype, H_, R, Pd, ps, q_lens, kv_lens, spike=None, seed=0, generic=False):
    """Random queries and entries, pages in scrambled order; returns (got, want) [n, H, R]."""
    g = torch.Generator(device=DEV).manual_seed(seed)
    n = sum(q_lens)
    ql = torch.randn(H_, n, R, device=DEV, generator=g)
    qr = torch.randn(n, H_, Pd, device=DEV, generator=g)
    ents = [torch.randn(L, R + Pd, device=DEV, generator=g) for L in kv_lens]
    if spike is not None:                      # one far key that must take all of one query's softmax
        e, key, head = spike
        t = sum(q_lens[:e]) + q_lens[e] - 1
        ql[head, t] = 0
        qr[t, head] = 0
        qr[t, head, Pd - 1] = 40.0             # the LAST number of the entry: the rotated part counts
        ents[e][:, R + Pd - 1].clamp_(-1, 1)
        ents[e][key, R + Pd - 1] = 30.0
    ql, qr, ents = ql.to(dtype), qr.to(dtype), [x.to(dtype) for x in ents]
    pages_per = [-(-L // ps) for L in kv_lens]
    n_pages = sum(pages_per) + 3
    perm = torch.randperm(n_pages - 1, generator=torch.Generator().manual_seed(seed + 1))[:sum(pages_per)]
    cache = torch.randn(n_pages, 1, ps * (R + Pd), device=DEV, generator=g).to(dtype)
    indptr = [0] + list(np.cumsum(pages_per))
    for e, L in enumerate(kv_lens):
        for p in range(L):
            cache[int(perm[indptr[e] + p // ps]), 0].view(ps, R + Pd)[p % ps] = ents[e][p]
    qo = [0] + list(np.cumsum(q_lens))
    pos = torch.cat([torch.arange(L - q, L) for q, L in zip(q_lens, kv_lens)]).to(DEV, torch.int32)
    ent = torch.cat([torch.full((q,), i) for i, q in enumerate(q_lens)]).to(DEV, torch.int32)
    ctx = SimpleNamespace(qo_indptr=torch.tensor(qo, dtype=torch.int32, device=DEV), positions=pos, tok_entry=ent,
                          n_entries=len(q_lens), n_tokens=n, max_q_len=max(q_lens), max_kv_len=max(kv_lens),
                          kv_len=torch.tensor(kv_lens, dtype=torch.int32, device=DEV),
                          extras={"min_q_len": min(q_lens)})
    tables = SimpleNamespace(kv_indptr=torch.tensor(indptr, dtype=torch.int32, device=DEV),
                             kv_indices=perm.to(DEV, torch.int32), page_size=ps)
    out = torch.full((H_, n, R), float("nan"), device=DEV, dtype=dtype)
    scale = 0.5 / math.sqrt(R + Pd)
    ops.FORCE_GENERIC_LATENT = generic
    try:
        ops.latent_attention(ql, qr, out, cache, ctx, tables, H_, R, Pd, scale)
        torch.cuda.synchronize()
        ops.check_status()
    finally:
        ops.FORCE_GENERIC_LATENT = False
    want = torch.empty(n, H_, R, device=DEV)
    for e, (q, L) in enumerate(zip(q_lens, kv_lens)):
        x = ents[e].float()
        for i in range(q):
            p, t = L - q + i, qo[e] + i
            for h in range(H_):
                s = (x[:p + 1] @ torch.cat([ql[h, t].float(), qr[t, h].float()])) * scale
                want[t, h] = torch.softmax(s, 0) @ x[:p + 1, :R]
    return out.float().transpose(0, 1), want


LATENT_SHAPES = [
    # heads, latent, rotated, page, q_lens, kv_lens
    (3, 48, 8, 4, [5, 1, 2], [5, 9, 30]),
    (1, 20, 4, 1, [1, 1, 7], [40, 1, 7]),
    (5, 72, 16, 5, [3, 11], [17, 11]),
    (16, 128, 32, 16, [1, 1, 1, 1], [300, 17, 64, 129]),
    (16, 128, 32, 16, [70, 2, 1], [200, 5, 333]),
    (6, 112, 16, 16, [130, 1, 3, 64], [130, 555, 40, 600]),
    (128, 512, 64, 64, [1, 2], [700, 65]),
    (20, 256, 64, 32, [129], [385]),
    (7, 64, 16, 8, [33, 1], [33, 2049]),
    (5, 48, 16, 8, [9, 1], [40, 200]),                 # a latent of 3 x 16: an odd number of output tiles per warp
    (3, 80, 48, 16, [70], [70]),
    (2, 96, 16, 16, [1, 1, 1], [5, 130, 64]),          # decode with a latent of 3 x 32
    (32, 160, 32, 16, [1, 1], [300, 31]),
]


@pytest.mark.parametrize("generic", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", LATENT_SHAPES, ids=lambda s: f"H{s[0]}r{s[1]}p{s[2]}ps{s[3]}")
def test_latent_attention(ops, dtype, shape, generic):
    if generic and dtype == torch.float32:
        pytest.skip("float32 always runs the generic kernel")
    got, want = _latent_case(ops, dtype, *shape, generic=generic)
    assert not torch.isnan(got).any()
    assert (got - want).abs().max() <= (2e-5 if dtype == torch.float32 else 2.5e-2)


@pytest.mark.parametrize("generic", [False, True])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_attention_rotates_the_queries_on_the_way(ops, dtype, generic):
    """Given a frequency table, the kernels take the queries' rotated parts unrotated (a view inside wider heads)
    and give what rotating them first and attending then gives."""
    Hh, R, Pd, ps, dh = 16, 64, 32, 16, 24
    f, mag = P.yarn_frequencies(dict(base=5000.0, dims=Pd, scaling=dict(factor=4.0, original=64, fast=16.0, slow=1.0)))
    table = ops.rope_frequency_table(f, DEV)
    q_lens, kv_lens = [40, 1, 3], [300, 77, 3]
    n = sum(q_lens)
    g = torch.Generator(device=DEV).manual_seed(17)
    ql = torch.randn(Hh, n, R, device=DEV, generator=g).to(dtype)
    q = torch.randn(n, Hh, dh + Pd, device=DEV, generator=g).to(dtype)
    pages_per = [-(-L // ps) for L in kv_lens]
    cache = torch.randn(sum(pages_per), 1, ps * (R + Pd), device=DEV, generator=g).to(dtype)
    qo = [0] + list(np.cumsum(q_lens))
    pos = torch.cat([torch.arange(L - x, L) for x, L in zip(q_lens, kv_lens)]).to(DEV, torch.int32)
    ent = torch.cat([torch.full((x,), i) for i, x in enumerate(q_lens)]).to(DEV, torch.int32)
    ctx = SimpleNamespace(qo_indptr=torch.tensor(qo, dtype=torch.int32, device=DEV), positions=pos, tok_entry=ent,
                          n_entries=3, n_tokens=n, max_q_len=max(q_lens), max_kv_len=max(kv_lens), extras={})
    tables = SimpleNamespace(kv_indptr=torch.tensor([0] + list(np.cumsum(pages_per)), dtype=torch.int32, device=DEV),
                             kv_indices=torch.arange(sum(pages_per), dtype=torch.int32, device=DEV), page_size=ps)
    first = q.clone()
    ops.rope_inplace(first[:, :, dh:], pos, table, Pd, True, mag)
    want = torch.empty(Hh, n, R, device=DEV, dtype=dtype)
    got = torch.empty(Hh, n, R, device=DEV, dtype=dtype)
    ops.FORCE_GENERIC_LATENT = generic
    try:
        ops.latent_attention(ql, first[:, :, dh:], want, cache, ctx, tables, Hh, R, Pd, 0.1)
        ops.latent_attention(ql, q.clone()[:, :, dh:], got, cache, ctx, tables, Hh, R, Pd, 0.1, rotate=(table, mag))
    finally:
        ops.FORCE_GENERIC_LATENT = False
    assert torch.equal(got, want)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("key", [0, 15, 16, 511, 512, 1023, 1500])
def test_one_far_entry_among_hundreds_is_found(ops, dtype, key):
    """A query whose score with one far entry (first of the request, page borders, deep inside) stands out returns
    that entry's latent, from a decoded token and from the last token of a portion."""
    for q_lens in ([1, 1], [3, 40]):
        got, want = _latent_case(ops, dtype, 16, 64, 16, 16, q_lens, [90, 1501], spike=(1, key, 5), seed=key)
        t = sum(q_lens) - 1
        assert (got[t, 5] - want[t, 5]).abs().max() <= (1e-4 if dtype == torch.float32 else 2e-2)
        assert (got - want).abs().max() <= (2e-5 if dtype == torch.float32 else 2.5e-2) * 5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_latent_prepare_norms_rotation_and_append(ops, dtype):
    Rq, R, Pd, ps, eps = 24, 40, 12, 4, 1e-3
    rot = dict(base=300.0, dims=Pd, scaling=dict(factor=5.0, original=32, fast=6.0, slow=1.0))
    f, mag = P.yarn_frequencies(rot)
    lens = [3, 1, 9]
    starts = [0, 6, 2]                               # positions the portions begin at
    n = sum(lens)
    g = torch.Generator(device=DEV).manual_seed(5)
    down = torch.randn(n, 5 + Rq + R + Pd + 3, device=DEV, generator=g) * 2
    wq = (1 + 0.2 * torch.randn(Rq, device=DEV, generator=g)).to(dtype)
    wkv = (1 + 0.2 * torch.randn(R, device=DEV, generator=g)).to(dtype)
    pages_per = [-(-(s + L) // ps) for s, L in zip(starts, lens)]
    indptr = [0] + list(np.cumsum(pages_per))
    n_pages = sum(pages_per) + 2
    perm = torch.randperm(n_pages, generator=torch.Generator().manual_seed(2))[:sum(pages_per)]
    cache = torch.zeros(n_pages, 1, ps * (R + Pd), device=DEV, dtype=dtype)
    pos = torch.cat([torch.arange(s, s + L) for s, L in zip(starts, lens)]).to(DEV, torch.int32)
    ent = torch.cat([torch.full((L,), i) for i, L in enumerate(lens)]).to(DEV, torch.int32)
    cq = ops.latent_prepare(down, 5, Rq, 5 + Rq, R, Pd, wq, wkv, eps, ops.rope_frequency_table(f, DEV), mag, pos, ent,
                            torch.tensor(indptr, dtype=torch.int32, device=DEV), perm.to(DEV, torch.int32), cache, ps)
    tol = 1e-5 if dtype == torch.float32 else 2e-2
    d64 = down.double().cpu()
    want_q = P.rms_norm(d64[:, 5:5 + Rq], wq.double().cpu(), eps)
    assert (cq.double().cpu() - want_q).abs().max() <= tol * want_q.abs().max()
    want_c = P.rms_norm(d64[:, 5 + Rq:5 + Rq + R], wkv.double().cpu(), eps)
    want_k = P.rotate_pairs(d64[:, 5 + Rq + R:5 + Rq + R + Pd], pos.cpu().long(), f, mag)
    written = torch.zeros(n_pages, ps, dtype=torch.bool)
    for t in range(n):
        e, p = int(ent[t]), int(pos[t])
        page = int(perm[indptr[e] + p // ps])
        got = cache[page, 0].view(ps, R + Pd)[p % ps].double().cpu()
        assert (got[:R] - want_c[t]).abs().max() <= tol * want_c.abs().max()
        assert (got[R:] - want_k[t]).abs().max() <= tol * want_k.abs().max()
        written[page, p % ps] = True
    assert not cache.view(n_pages, ps, R + Pd)[~written.to(DEV)].any()         # nothing else was touched


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("E,G,keep,top", [(8, 2, 1, 3), (6, 3, 2, 3), (4, 4, 2, 2), (8, 1, 1, 1), (16, 4, 3, 5), (64, 8, 4, 6)])
def test_router_groups_and_negative_choices(ops, dtype, E, G, keep, top):
    """Choice scores made negative by the correction: a dropped group counts as minus infinity, not as 0."""
    d, n = 40, 50
    g = torch.Generator(device=DEV).manual_seed(E * 10 + G)
    h = torch.randn(n, d, device=DEV, generator=g).to(dtype)
    wr = (0.3 * torch.randn(E, d, device=DEV, generator=g)).to(dtype)
    corr = (-3.0 + 0.3 * torch.randn(E, device=DEV, generator=g)).to(dtype)
    w = {"router": wr.double().cpu(), "correction": corr.double().cpu()}
    for fused_max in (0, 1 << 30):                 # logits by a matrix product; logits inside the kernel
        was = ops.MOE_ROUTE_FUSED_MAX
        ops.MOE_ROUTE_FUSED_MAX = fused_max
        try:
            ids, wts = ops.moe_route(h, wr, corr, G, keep, top, 1.7)
        finally:
            ops.MOE_ROUTE_FUSED_MAX = was
        _check_routing(h, w, ids, wts, E, G, keep, top, n, dtype)


def _check_routing(h, w, ids, wts, E, G, keep, top, n, dtype):
    want_ids, want_w = P.route(h.double().cpu(), w, "", dict(experts=E, top=top, scale=1.7, groups=dict(count=G, keep=keep)))
    s = torch.sigmoid(h.double().cpu() @ w["router"].T)
    assert ((s + w["correction"]) < 0).all()
    same = 0
    for t in range(n):
        a, b = sorted(ids[t].tolist()), sorted(want_ids[t].tolist())
        if a == b:
            same += 1
            got = dict(zip(ids[t].tolist(), wts[t].tolist()))
            for e, x in zip(want_ids[t].tolist(), want_w[t].tolist()):
                assert got[e] == pytest.approx(x, rel=1e-5 if dtype == torch.float32 else 1e-2)
    assert same >= (n if dtype == torch.float32 else n - 3)            # bfloat16 may flip a close call


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n,E,top,d,ff", [(1, 4, 2, 32, 24), (9, 6, 3, 100, 36), (300, 8, 4, 64, 40), (40, 16, 1, 72, 8),
                                          (8, 64, 6, 512, 136), (64, 32, 4, 264, 1032), (8, 64, 6, 512, 160),
                                          (64, 16, 4, 288, 1056), (3, 8, 2, 2048, 96), (700, 8, 4, 64, 40)])
def test_routed_experts(ops, dtype, n, E, top, d, ff):
    g = torch.Generator(device=DEV).manual_seed(n)
    h = torch.randn(n, d, device=DEV, generator=g).to(dtype)
    w_up = (0.2 * torch.randn(E, ff, d, device=DEV, generator=g)).to(dtype)
    w_down = (0.2 * torch.randn(E, d, ff, device=DEV, generator=g)).to(dtype)
    ids = torch.stack([torch.randperm(E, generator=torch.Generator().manual_seed(t))[:top] for t in range(n)]).to(DEV, torch.int32)
    if n > 8:
        ids[3:8] = ids[3]                          # some experts with many rows, some perhaps with none
    wts = torch.rand(n, top, device=DEV, generator=g) + 0.1
    # the kinds of grouped product: weight-streaming on the tensor cores, the same with plain arithmetic, tiled, library
    for library, skinny, mma in ((False, True, True), (False, True, False), (False, False, False), (True, True, True)):
        was = ops.MOE_LIBRARY_MIN_ROWS, ops.MOE_SKINNY, ops.MOE_SKINNY_MMA
        ops.MOE_LIBRARY_MIN_ROWS, ops.MOE_SKINNY, ops.MOE_SKINNY_MMA = (0 if library else 1 << 30), skinny, mma
        try:
            out = ops.moe_experts(h, ids, wts, w_up, w_down, dtype)
        finally:
            ops.MOE_LIBRARY_MIN_ROWS, ops.MOE_SKINNY, ops.MOE_SKINNY_MMA = was
        want = torch.zeros(n, d, dtype=torch.float64)
        for t in range(n):
            for k in range(top):
                e = int(ids[t, k])
                up = w_up[e].double().cpu() @ h[t].double().cpu()
                want[t] += float(wts[t, k]) * (w_down[e].double().cpu() @ (0.5 * up * (1 + torch.erf(up / math.sqrt(2)))))
        assert (out.double().cpu() - want).abs().max() <= _tol(dtype) * want.abs().max() * 2


def test_gate_heads_and_batched_products(ops):
    g = torch.Generator(device=DEV).manual_seed(9)
    for dtype in (torch.float32, torch.bfloat16):
        Hh, n, V = 5, 13, 24
        v = torch.randn(Hh, n, V, device=DEV, generator=g).to(dtype)
        rows = torch.randn(n, 7 + Hh, device=DEV, generator=g)
        out = torch.empty(n, Hh * V, device=DEV, dtype=dtype)
        ops.gate_heads(v, rows[:, 7:], out)
        want = (v.double() * torch.sigmoid(rows[:, 7:].double()).T[:, :, None]).transpose(0, 1).reshape(n, Hh * V)
        assert (out.double() - want).abs().max() <= _tol(dtype) * 4
        x = torch.randn(n, Hh, 40, device=DEV, generator=g).to(dtype)            # heads strided inside rows
        w = torch.randn(Hh, 9, 16, device=DEV, generator=g).to(dtype)
        got = ops.linear_batched(x[:, :, 8:24].transpose(0, 1), w)
        want = torch.einsum("nhk,hmk->hnm", x[:, :, 8:24].double(), w.double())
        assert (got.double() - want).abs().max() <= _tol(dtype) * want.abs().max() * 2


# ------------------------------------------------------------------------------------------- the engine

@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_whole_tail_portions(tmp_path, name, dtype):
    cfg, seed, page = CONFIGS[name]
    folder = _folder(tmp_path, name, dtype)
    reqs = _requests(name)
    longest = max(len(t) for t in reqs.values())
    eng = _engine(folder, dtype, page, -(-longest // page) + 1)
    for rid, toks in reqs.items():
        one = {rid: toks}
        got = H.run_steps_in_process(eng, H.whole(rid, toks))
        H.compare_with_oracle(got, folder, one, dtype, oracle=_oracle, allow_over=_flips(dtype))
        got_tail = H.run_steps_in_process(eng, H.tail_decoded(rid, toks, tail=40))
        H.compare_with_oracle(got_tail, folder, one, dtype, oracle=_oracle, allow_over=_flips(dtype))
        got_port = H.run_steps_in_process(eng, H.portions(rid, toks, [7, 2, 16, 3, 2, 5, 2, 31]))
        H.compare_with_oracle(got_port, folder, one, dtype, oracle=_oracle, allow_over=_flips(dtype))
        _rows_agree(got, got_tail, dtype)
        _rows_agree(got, got_port, dtype)
    assert all(g.pool.num_held == 0 for g in eng.cache.groups)


@pytest.mark.parametrize("dtype", DTYPES)
def test_token_by_token_from_the_first_token(tmp_path, dtype):
    """A whole request decoded one token at a time (the first tokens of a sequence, every page border, long
    decoding) against the whole prompt in one step."""
    cfg, seed, page = CONFIGS["A"]
    folder = _folder(tmp_path, "A", dtype)
    toks = H.random_tokens(150, cfg["vocab"], 4)
    eng = _engine(folder, dtype, page, 40)
    got = H.run_steps_in_process(eng, H.portions("t", toks, [1]))
    H.compare_with_oracle(got, folder, {"t": toks}, dtype, oracle=_oracle, allow_over=_flips(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_mixed_requests_reuse_pages_and_slots(tmp_path, name, dtype):
    cfg, seed, page = CONFIGS[name]
    folder = _folder(tmp_path, name, dtype)
    base = _requests(name)
    reqs = dict(base)
    for i, (rid, toks) in enumerate(base.items()):          # twice as many requests as fit at once
        reqs[f"s{i}"] = H.random_tokens(max(2, len(toks) // 2 + 3), cfg["vocab"], 999 + i)
    steps = H.mixed(reqs, seed=seed + 7, max_live=4)
    max_tokens = H.max_live_tokens(steps, round_to=page)
    eng = _engine(folder, dtype, page, max_tokens // page, max_requests=4)
    got = H.run_steps_in_process(eng, steps)
    assert sum(-(-len(t) // page) for t in reqs.values()) > eng.cache.groups[0].pool.num_pages
    H.compare_with_oracle(got, folder, reqs, dtype, oracle=_oracle, allow_over=_flips(dtype))
    # every request alone gives the same rows as in the batch, up to rounding
    alone = _engine(folder, dtype, page, -(-max(len(t) for t in reqs.values()) // page) + 1)
    for rid in ("r2", "r3"):
        one = H.run_steps_in_process(alone, H.whole(rid, reqs[rid]))
        _rows_agree(one, {k: got[k] for k in one}, dtype)


@pytest.mark.parametrize("dtype", DTYPES)
def test_trace_run_program(tmp_path, dtype):
    cfg, seed, page = CONFIGS["B"]
    folder = _folder(tmp_path, "B", dtype)
    reqs = _requests("B")
    steps = H.mixed(reqs, seed=3, max_live=4)
    got = H.run_trace_subprocess(folder, dtype, steps, tmp_path / "out", H.max_live_tokens(steps, round_to=64))
    H.compare_with_oracle(got, folder, reqs, dtype, oracle=_oracle, allow_over=_flips(dtype))


@pytest.mark.parametrize("dtype", DTYPES)
def test_a_far_token_decides_the_logits(tmp_path, dtype):
    """Weights made so that attention matters: with the output projection scaled up, changing ONE token far back
    (the first, one at a page border, one deep inside) changes the last position's logits in the oracle, and the
    engine follows it, decoded alone and as the end of a portion."""
    cfg, seed, page = CONFIGS["A"]
    stored = torch.float32 if dtype == "float32" else torch.bfloat16
    folder = H.make_folder(tmp_path / "far", cfg, 21, dtype=stored, std=0.15)
    base = H.random_tokens(260, cfg["vocab"], 8)
    eng = _engine(folder, dtype, page, 70)
    ref0 = _oracle(folder, base)[-1]
    moved = []
    for where in (0, 3, 4, 127, 128, 200):
        toks = list(base)
        toks[where] = (toks[where] + 17) % cfg["vocab"]
        ref = _oracle(folder, toks)
        moved.append(np.abs(ref[-1] - ref0).max() / np.abs(ref0).max())
        for steps in (H.tail_decoded("f", toks, tail=3), H.portions("f", toks, [250, 10])):
            got = H.run_steps_in_process(eng, steps)
            err = np.abs(got[("f", len(toks) - 1)] - ref[-1]).max() / np.abs(ref).max()
            assert err <= H.TOL[dtype], (where, err)
    assert max(moved) > 1e-3, "no far token moved the last logits: the weights hide what this test is for"


def test_generation_through_the_scheduler(tmp_path):
    """Greedy generation through Engine.generate (scheduler, portions, captured decode steps) gives the tokens that
    the oracle's argmax gives, token by token, for requests of unequal length under page pressure."""
    from batchspec_b200.engine.sequence import Sequence
    cfg, seed, page = CONFIGS["A"]
    folder = H.make_folder(tmp_path / "gen", cfg, 31, dtype=torch.float32, std=0.2)
    prompts = [H.random_tokens(n, cfg["vocab"], 50 + n) for n in (3, 19, 42, 7, 64)]
    from batchspec_b200.engine import Engine
    for graphs in (True, False):
        eng = Engine(dtype="float32", device=DEV)
        eng.load_model(model_dir=folder)
        eng.use_cuda_graphs = graphs
        eng.setup_caches(max_batch_size=3, max_seq_length=96, page_size=page, prefill_chunk_size=16, num_pages=50)
        eng.setup_sampling_params(temperature=0.0)
        seqs = [Sequence(i, list(p), max_new_tokens=12) for i, p in enumerate(prompts)]
        done = {s.seq_id: s for s in eng.generate(seqs)}
        for i, p in enumerate(prompts):
            toks = list(p)
            for k in range(12):
                ref = _oracle(folder, toks)[-1]
                top2 = np.sort(ref)[-2:]
                nxt = done[i].output_ids[k]
                if top2[1] - top2[0] > 1e-3 * np.abs(ref).max():
                    assert nxt == int(ref.argmax()), (graphs, i, k)
                toks.append(nxt)
