"""Plain, slow Vabanex decoder: the oracle the engine tests of that design compare against.

Whole sequences, no cache, no batching, float64 on the CPU, one function per
mechanism.  It shares no code with ``batchspec_b200``: it reads ``config.json`` as a
plain dict, has its own safetensors reader, and forms keys and values per head
from the latent (the product attends in the latent space instead).

The design in this file's notation (h: a layer's normed input, one row per token):

  layer        x <- x + mixer(LN1(x));  x <- x + ff(LN2(x)) when the layer has a feed-forward
  LN           (x - mean) / sqrt(var + eps) * w + b, var the mean squared deviation
  mixer        cq = RMS(Wdq h) * n_q;  q = Wuq cq, per head [dim plain | rot_dim rotated]
               [c' | kr] = Wdkv h;  c = RMS(c') * n_kv;  kr is one rotated key part for all heads
               k_h = Wuk_h c,  v_h = Wuv_h c
               score_h(i, j) = (q_plain . k_h + rot(q_rot, i) . rot(kr, j)) * scale,  j <= i, softmax
               out = Wo concat_h(sigmoid(Wg h)_h * sum_j p_h(i, j) v_h(j))
  rotation     adjacent pairs (2i, 2i+1), angle p * f_i, f_i = base^(-2i/dims), with the YaRN blend of
               f_i / factor and f_i and the magnitude 0.1 ln(factor) + 1 on cosine and sine
  dense ff     g = min(Wgate h, L), u = clamp(Wup h, -L, L), y = g sigmoid(1.702 g) (u + 1), out = Wdown y
  routed ff    s = sigmoid(Wr h); choice = s + correction; experts in equal groups of neighbours, a group's
               score the sum of its two largest choices, only the best `keep` groups stay; the `top` largest
               choices among them are used with weights s * scale; expert = Wdown gelu_erf(Wup h)
  output       LN_final, head, cap * tanh(logits / cap)
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np
import torch

F64 = torch.float64
_ST = {"F32": np.float32, "F16": np.float16, "BF16": np.uint16, "I32": np.int32, "I64": np.int64, "F64": np.float64}


def read_tensors(path) -> dict:
    raw = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", raw[:8])
    header = json.loads(raw[8:8 + hlen])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        arr = np.frombuffer(raw[8 + hlen + b:8 + hlen + e], dtype=_ST[meta["dtype"]]).copy()
        if meta["dtype"] == "BF16":
            arr = (arr.astype(np.uint32) << 16).view(np.float32)
        out[name] = torch.from_numpy(arr.astype(np.float64)).reshape(meta["shape"])
    return out


def read_model_folder(folder):
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_tensors(folder / "model.safetensors")


# --------------------------------------------------------------------------- mechanisms

def layer_norm(x, w, b, eps):
    mu = x.mean(-1, keepdim=True)
    var = ((x - mu) ** 2).mean(-1, keepdim=True)
    return (x - mu) / torch.sqrt(var + eps) * w + b


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def yarn_frequencies(rot):
    """(frequencies [dims/2], magnitude) of a rotation description {base, dims, scaling or nothing}."""
    dims, base = int(rot["dims"]), float(rot["base"])
    f = [base ** (-2.0 * i / dims) for i in range(dims // 2)]
    sc = rot.get("scaling")
    if not sc:
        return torch.tensor(f, dtype=F64), 1.0
    factor = float(sc["factor"])

    def dim_of(turns):
        return dims * math.log(float(sc["original"]) / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(dim_of(float(sc["fast"]))), 0)
    hi = min(math.ceil(dim_of(float(sc["slow"]))), dims - 1)
    out = []
    for i, fi in enumerate(f):
        ramp = min(1.0, max(0.0, (i - lo) / max(hi - lo, 0.001)))
        out.append(fi / factor * ramp + fi * (1.0 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(factor) + 1.0


def rotate_pairs(x, positions, freqs, magnitude):
    """x [..., T, dims] with T the token axis at -2; adjacent pairs."""
    ang = positions.to(F64)[:, None] * freqs[None, :]
    cos, sin = torch.cos(ang) * magnitude, torch.sin(ang) * magnitude
    u, v = x[..., 0::2], x[..., 1::2]
    out = torch.empty_like(x)
    out[..., 0::2] = u * cos - v * sin
    out[..., 1::2] = v * cos + u * sin
    return out


def latent_attention(h, w, p, m, eps, positions):
    """h [T, width]; w: the model's tensors; p: the layer's tensor prefix; m: the mixer's sizes."""
    H, dim, rd, vd, r = int(m["heads"]), int(m["dim"]), int(m["rot_dim"]), int(m["vdim"]), int(m["kv_rank"])
    T = h.shape[0]
    cq = rms_norm(h @ w[p + "dq"].T, w[p + "dq.norm"], eps)
    q = (cq @ w[p + "uq"].T).view(T, H, dim + rd).transpose(0, 1)             # [H, T, dim + rd]
    down = h @ w[p + "dkv"].T
    c = rms_norm(down[:, :r], w[p + "dkv.norm"], eps)
    freqs, mag = yarn_frequencies(m["rot"])
    assert int(m["rot"]["dims"]) == rd
    kr = rotate_pairs(down[:, r:], positions, freqs, mag)                       # [T, rd]
    qr = rotate_pairs(q[:, :, dim:], positions, freqs, mag)                     # [H, T, rd]
    k = (c @ w[p + "uk"].T).view(T, H, dim).transpose(0, 1)                     # [H, T, dim]
    v = (c @ w[p + "uv"].T).view(T, H, vd).transpose(0, 1)
    s = (q[:, :, :dim] @ k.transpose(1, 2) + qr @ kr.T[None]) * float(m["scale"])
    i = torch.arange(T)
    s = s.masked_fill(i[None, :] > i[:, None], float("-inf"))
    o = torch.softmax(s, dim=-1) @ v                                            # [H, T, vd]
    gate = torch.sigmoid(h @ w[p + "g"].T)                                      # [T, H]
    o = o * gate.T[:, :, None]
    return o.transpose(0, 1).reshape(T, H * vd) @ w[p + "o"].T


def dense_ff(h, w, p, f):
    L = float(f["limit"])
    g = torch.clamp(h @ w[p + "gate"].T, max=L)
    u = torch.clamp(h @ w[p + "up"].T, -L, L)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ w[p + "down"].T


def route(h, w, p, r):
    """(chosen expert ids [T, top], their weights [T, top])."""
    E, top = int(r["experts"]), int(r["top"])
    s = torch.sigmoid(h @ w[p + "router"].T)
    choice = s + w[p + "correction"]
    groups = r.get("groups")
    if groups:
        G, keep = int(groups["count"]), int(groups["keep"])
        per = choice.view(-1, G, E // G)
        gs = per.topk(min(2, E // G), dim=-1).values.sum(-1)
        kept = torch.zeros_like(gs, dtype=torch.bool).scatter_(1, gs.topk(keep, dim=-1).indices, True)
        choice = choice.masked_fill(~kept[:, :, None].expand(-1, -1, E // G).reshape(-1, E), float("-inf"))
    ids = choice.topk(top, dim=-1).indices
    return ids, s.gather(1, ids) * float(r["scale"])


def routed_ff(h, w, p, f):
    ids, wt = route(h, w, p, f["router"])
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for e, a in zip(ids[t].tolist(), wt[t]):
            up = w[f"{p}e{e}.up"] @ h[t]
            out[t] += a * (w[f"{p}e{e}.down"] @ (0.5 * up * (1.0 + torch.erf(up / math.sqrt(2.0)))))
    return out


def forward(cfg, w, tokens, layers_out=None):
    """float64 logits [T, vocab] of one sequence; ``layers_out`` (a list) receives the residual after every layer."""
    eps = float(cfg["norm"]["eps"])
    T = len(tokens)
    positions = torch.arange(T)
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)] * float(cfg["embedding"]["scale"])
    for i, layer in enumerate(cfg["layers"]):
        p = f"l{i}."
        assert layer["type"] == "latent_attention"
        x = x + latent_attention(layer_norm(x, w[p + "norm1"], w[p + "norm1.b"], eps), w, p + "mix.", layer["mixer"],
                                 eps, positions)
        f = layer.get("mlp")
        if f:
            h = layer_norm(x, w[p + "norm2"], w[p + "norm2.b"], eps)
            x = x + (dense_ff(h, w, p + "mlp.", f) if f["kind"] == "dense" else routed_ff(h, w, p + "mlp.", f))
        if layers_out is not None:
            layers_out.append(x.clone())
    z = layer_norm(x, w["final.norm"], w["final.norm.b"], eps) @ w["head"].T
    cap = cfg.get("logit_softcap")
    return cap * torch.tanh(z / cap) if cap else z
