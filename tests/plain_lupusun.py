"""Plain, slow oracle of the Lupusun design: one function per mechanism, whole sequences at once, no cache, no
batching, torch on the CPU.  It shares no code with the package: configuration dicts and tensors come in as
they are stored ([out, in] weights applied as W x), and every equation is written out here.

    x0 = rms(embed[token]) * embed.norm
    per layer:  x += m * mixer(rms(x) * norm1);  x += m * ff(rms(x) * norm2)   (the second only with a feed-forward)
    layers loop.start .. loop.stop-1 run loop.times times in a row (weights shared); x0 is added to x before
    every pass but the first
    logits = head (rms(x) * final.norm)
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def rms(x: torch.Tensor, eps: float) -> torch.Tensor:
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps)


def silu(x):
    return x / (1.0 + torch.exp(-x))


def softplus(x):
    return torch.where(x > 30.0, x, torch.log1p(torch.exp(torch.clamp(x, max=30.0))))


# ---------------------------------------------------------------------------------------------- rotary positions
def yarn_frequencies(rot: dict, dtype=torch.float64):
    """(frequency per pair [dims/2], what cosine and sine are multiplied by)."""
    dims, base = int(rot["dims"]), float(rot["base"])
    i = torch.arange(dims // 2, dtype=dtype)
    f = base ** (-2.0 * i / dims)
    sc = rot.get("scaling")
    if not sc:
        return f, 1.0
    factor, original = float(sc["factor"]), float(sc["original"])

    def where(turns):
        return dims * math.log(original / (2.0 * math.pi * turns)) / (2.0 * math.log(base))
    lo = max(math.floor(where(float(sc["fast"]))), 0)
    hi = min(math.ceil(where(float(sc["slow"]))), dims - 1)
    ramp = torch.clamp((i - lo) / max(hi - lo, 0.001), 0.0, 1.0)
    return f / factor * ramp + f * (1.0 - ramp), 0.1 * math.log(factor) + 1.0


def rotate(x: torch.Tensor, positions: torch.Tensor, rot: dict) -> torch.Tensor:
    """x [T, heads, dim]: dimension i of the first rot.dims is paired with i + dims/2; the rest pass."""
    dims = int(rot["dims"])
    f, mag = yarn_frequencies(rot, x.dtype)
    a = positions.to(x.dtype)[:, None] * f[None, :]                     # [T, dims/2]
    c, s = (torch.cos(a) * mag)[:, None, :], (torch.sin(a) * mag)[:, None, :]
    u, v = x[..., :dims // 2], x[..., dims // 2:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], dim=-1)


# ---------------------------------------------------------------------------------------------- attention mixer
def chunked_sink_attention(q, k, v, sink, scale: float, size: int, positions: torch.Tensor) -> torch.Tensor:
    """q [T, H, dim], k [T, G, dim], v [T, G, vdim], sink [H].  Position i sees j <= i of its own chunk
    (floor(i / size) == floor(j / size)); the softmax denominator also holds exp(sink_h)."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros((T, H, v.shape[2]), dtype=q.dtype)
    pi, pj = positions[:, None], positions[None, :]
    seen = (pj <= pi) & (torch.div(pi, size, rounding_mode="floor") == torch.div(pj, size, rounding_mode="floor"))
    for h in range(H):
        g = h // (H // G)
        s = (q[:, h, :] @ k[:, g, :].T) * scale
        s = torch.where(seen, s, torch.full_like(s, -float("inf")))
        top = torch.maximum(s.max(dim=-1, keepdim=True).values, sink[h].expand(T, 1))
        w = torch.exp(s - top)
        den = w.sum(dim=-1, keepdim=True) + torch.exp(sink[h] - top)
        out[:, h, :] = (w / den) @ v[:, g, :]
    return out


def attention_mixer(h: torch.Tensor, p: Dict[str, torch.Tensor], m: dict, eps: float, positions) -> torch.Tensor:
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = (h @ p["q"].T + p["q.b"]).view(T, H, dim)
    k = (h @ p["k"].T + p["k.b"]).view(T, G, dim)
    v = (h @ p["v"].T + p["v.b"]).view(T, G, vdim)
    if m.get("rot") and m["rot"]["dims"]:
        q, k = rotate(q, positions, m["rot"]), rotate(k, positions, m["rot"])
    q, k = rms(q, eps), rms(k, eps)
    size = int(m["mask"]["size"]) if m.get("mask") else 1 << 40              # no mask: one chunk for all positions
    o = chunked_sink_attention(q, k, v, p["sink"], float(m["scale"]), size, positions)
    return o.reshape(T, H * vdim) @ p["o"].T


# ---------------------------------------------------------------------------------------------- delta mixer
def short_conv(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """x [T, C], w [C, taps]: y[t, c] = sum_j w[c, taps-1-j] x[t-j, c], zeros before the start."""
    T, C = x.shape
    taps = w.shape[1]
    y = torch.zeros_like(x)
    for j in range(taps):
        if j < T:
            y[j:] += x[:T - j] * w[:, taps - 1 - j][None, :]
    return y


def unit(x: torch.Tensor) -> torch.Tensor:
    return x / torch.sqrt((x * x).sum(dim=-1, keepdim=True) + 1e-6)


def gated_delta_rule(q, k, v, beta, g) -> torch.Tensor:
    """q, k [T, H, dim], v [T, H, vdim], beta, g [T, H].  Per head, token by token:
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q."""
    T, H, dim = q.shape
    vdim = v.shape[2]
    S = torch.zeros((H, dim, vdim), dtype=q.dtype)
    out = torch.zeros((T, H, vdim), dtype=q.dtype)
    for t in range(T):
        S = S * g[t][:, None, None]
        u = beta[t][:, None] * (v[t] - torch.einsum("hdv,hd->hv", S, k[t]))
        S = S + torch.einsum("hd,hv->hdv", k[t], u)
        out[t] = torch.einsum("hdv,hd->hv", S, q[t])
    return out


def delta_mixer(h: torch.Tensor, p: Dict[str, torch.Tensor], m: dict, eps: float) -> torch.Tensor:
    T = h.shape[0]
    H, G, dim, vdim = m["heads"], m["kv_heads"], m["dim"], m["vdim"]
    q = silu(short_conv(h @ p["q"].T, p["q.conv"])).view(T, G, dim)
    k = silu(short_conv(h @ p["k"].T, p["k.conv"])).view(T, G, dim)
    v = silu(short_conv(h @ p["v"].T, p["v.conv"])).view(T, H, vdim)
    q, k = unit(q) * dim ** -0.5, unit(k)
    rep = H // G
    q, k = q.repeat_interleave(rep, dim=1), k.repeat_interleave(rep, dim=1)        # head h uses q/k head h // rep
    beta = torch.sigmoid(h @ p["b"].T)
    g = torch.exp(-torch.exp(p["A_log"]) * softplus(h @ p["a"].T + p["dt_bias"]))
    o = gated_delta_rule(q, k, v, beta, g)
    o = rms(o, eps) * p["norm"] * silu(h @ p["g"].T).view(T, H, vdim)
    return o.reshape(T, H * vdim) @ p["o"].T


# ---------------------------------------------------------------------------------------------- feed-forward
def relu_glu(h, p):
    return (torch.relu(h @ p["gate"].T) * (h @ p["up"].T)) @ p["down"].T


# ---------------------------------------------------------------------------------------------- the model
def layer_order(config: dict) -> List[tuple]:
    """(layer index, is the first layer of a pass after the first) for every layer run."""
    n = len(config["layers"])
    loop = config.get("loop") or {"start": 0, "stop": 0, "times": 1}
    start, stop, times = loop["start"], loop["stop"], loop["times"]
    if stop <= start or times <= 1:
        return [(i, False) for i in range(n)]
    runs = [(i, False) for i in range(start)]
    for t in range(times):
        runs += [(i, t > 0 and i == start) for i in range(start, stop)]
    return runs + [(i, False) for i in range(stop, n)]


def forward(config: dict, tensors: Dict[str, torch.Tensor], tokens, dtype=torch.float32,
            layers_out: Optional[list] = None) -> torch.Tensor:
    """Logits [T, vocab] of one sequence fed whole.  ``layers_out``: receives x after every layer run."""
    W = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in tensors.items()}
    eps, m = float(config["norm"]["eps"]), float(config.get("residual_mult", 1.0))
    tokens = torch.as_tensor(tokens, dtype=torch.long)
    positions = torch.arange(tokens.numel())
    x0 = rms(W["embed"][tokens], eps) * W["embed.norm"]
    x = x0.clone()
    for i, again in layer_order(config):
        layer, pre = config["layers"][i], f"l{i}."
        if again:
            x = x + x0
        p = {k[len(pre) + 4:]: v for k, v in W.items() if k.startswith(pre + "mix.")}
        hin = rms(x, eps) * W[pre + "norm1"]
        if layer["type"] == "attention":
            y = attention_mixer(hin, p, layer["mixer"], eps, positions)
        elif layer["type"] == "delta":
            y = delta_mixer(hin, p, layer["mixer"], eps)
        else:
            raise ValueError(layer["type"])
        x = x + m * y
        if layer.get("mlp") is not None:
            f = {k[len(pre) + 4:]: v for k, v in W.items() if k.startswith(pre + "mlp.")}
            x = x + m * relu_glu(rms(x, eps) * W[pre + "norm2"], f)
        if layers_out is not None:
            layers_out.append(x.clone())
    return (rms(x, eps) * W["final.norm"]) @ W["head"].T


# ---------------------------------------------------------------------------------------------- a model folder
def read_tensors(path) -> Dict[str, torch.Tensor]:
    """A safetensors file: 8-byte little-endian header length, a JSON header, the data."""
    import json
    import struct
    import numpy as np
    kinds = {"F32": np.float32, "BF16": np.uint16, "I32": np.int32, "F64": np.float64}
    raw = open(path, "rb").read()
    (hlen,) = struct.unpack("<Q", raw[:8])
    out = {}
    for name, meta in json.loads(raw[8:8 + hlen]).items():
        if name == "__metadata__":
            continue
        b, e = meta["data_offsets"]
        arr = np.frombuffer(raw[8 + hlen + b:8 + hlen + e], dtype=kinds[meta["dtype"]]).copy()
        if meta["dtype"] == "BF16":
            arr = (arr.astype(np.uint32) << 16).view(np.float32)
        out[name] = torch.from_numpy(arr).reshape(meta["shape"])
    return out


def read_model_folder(folder):
    import json
    from pathlib import Path
    folder = Path(folder)
    return json.loads((folder / "config.json").read_text()), read_tensors(folder / "model.safetensors")
