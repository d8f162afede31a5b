"""Gated delta rule: a recurrent mixer whose state per request and head is a [key dim x value dim] matrix S.

With h the token's normed input, H value heads, G query/key heads (value head j reads q/k head j // (H / G)):

    q, k, v = silu(conv(Wq h)), silu(conv(Wk h)), silu(conv(Wv h))      conv: causal, per channel, ``taps`` long
    q <- q / |q| * dim^-1/2,  k <- k / |k|                               per head, |x| = sqrt(sum x^2 + unit_eps)
    beta = sigmoid(Wb h),  g = exp(-exp(A_log) softplus(Wa h + dt_bias)) per value head
    S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q         the read-out sees the token's own write
    out = Wo concat_heads(o / rms(o) * w * silu(Wg h))

Everything after the projections is float32: the convolutions, the unit lengths, beta, the decay, the state and the
output norm.  The state of a request is one float32 row [S of every head | the last taps-1 projection rows], zero at
admission.  Launch sequence: one product for [Wq; Wk; Wv; Wg; Wb; Wa] with float32 output -> delta_prepare ->
delta_recurrence -> gated_rmsnorm -> output projection."""
from __future__ import annotations

from typing import Dict

import torch

from ..kernels import ops
from ..profiler import bucket
from .base import MIXERS, Mixer, ParamSpec, Runtime, StateSpec, register_part


@register_part(MIXERS, "gated_delta")
class GatedDeltaRule(Mixer):
    graph_safe = True

    def __init__(self, runtime: Runtime, dim: int, n_heads: int, n_kv_heads: int, head_dim: int, v_dim: int, taps: int,
                 eps: float, unit_eps: float = 1e-6):
        if n_heads <= 0 or n_kv_heads <= 0 or n_heads % n_kv_heads:
            raise ValueError(f"n_heads {n_heads} must be a positive multiple of n_kv_heads {n_kv_heads}")
        if not 0 < head_dim <= 256 or v_dim <= 0 or taps < 1:
            raise ValueError(f"the delta rule kernels take key sizes up to 256, got {head_dim}")
        self.runtime = runtime
        self.dim, self.n_heads, self.n_kv_heads = int(dim), int(n_heads), int(n_kv_heads)
        self.head_dim, self.v_dim, self.taps = int(head_dim), int(v_dim), int(taps)
        self.eps, self.unit_eps = float(eps), float(unit_eps)
        self.channels = 2 * self.n_kv_heads * self.head_dim + self.n_heads * self.v_dim
        self.tail_off = self.n_heads * self.v_dim * (-(-self.head_dim // 4) * 4)      # columns padded to float4s

    def param_specs(self) -> Dict[str, ParamSpec]:
        qk, v, H = self.n_kv_heads * self.head_dim, self.n_heads * self.v_dim, self.n_heads
        return {"q": ParamSpec((qk, self.dim)), "k": ParamSpec((qk, self.dim)), "v": ParamSpec((v, self.dim)),
                "q_conv": ParamSpec((qk, self.taps)), "k_conv": ParamSpec((qk, self.taps)),
                "v_conv": ParamSpec((v, self.taps)), "b": ParamSpec((H, self.dim)), "a": ParamSpec((H, self.dim)),
                "A_log": ParamSpec((H,), role="vector"), "dt_bias": ParamSpec((H,), role="vector"),
                "g": ParamSpec((v, self.dim)), "norm": ParamSpec((self.v_dim,), role="vector", init="ones_normal"),
                "o": ParamSpec((self.dim, v))}

    def bind(self, params):
        self.w_in = torch.cat([params[n] for n in ("q", "k", "v", "g", "b", "a")], dim=0).contiguous()
        f32 = lambda t: t.to(torch.float32).contiguous()
        self.conv = f32(torch.cat([params["q_conv"], params["k_conv"], params["v_conv"]], dim=0))
        self.a_log, self.dt_bias, self.norm = f32(params["A_log"]), f32(params["dt_bias"]), f32(params["norm"])
        self.w_o = params["o"].contiguous()
        self.g_off = self.channels
        self.b_off = self.g_off + self.n_heads * self.v_dim
        self.a_off = self.b_off + self.n_heads

    def state_spec(self) -> StateSpec:
        size = self.tail_off + (self.taps - 1) * self.channels
        return StateSpec((-(-size // 4) * 4,), torch.float32)        # rows start on 16-byte boundaries

    def forward(self, x, ctx, cache):
        H, G, dk, dv = self.n_heads, self.n_kv_heads, self.head_dim, self.v_dim
        state = cache.state
        with bucket("delta.in_proj"):
            proj = ops.linear(x, self.w_in, out_dtype=torch.float32)
        with bucket("delta.prepare"):
            mix, gates = ops.delta_prepare(proj, self.b_off, self.a_off, self.conv, self.a_log, self.dt_bias, state,
                                           self.tail_off, ctx, H, G, dk, dv, self.taps, dk ** -0.5, self.unit_eps)
        with bucket("delta.recurrence"):
            o = ops.delta_recurrence(mix, gates, proj, state, self.tail_off, ctx, H, G, dk, dv, self.taps)
        with bucket("delta.out_norm"):
            y = ops.gated_rmsnorm(o, proj[:, self.g_off:self.g_off + H * dv], self.norm, self.eps, H, dv, x.dtype)
        with bucket("delta.o_proj"):
            return ops.linear(y, self.w_o)
