from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..cache.manager import StateNeed
from ..weights.loader import TensorDecl
from .base import Mixer, register_mixer


@register_mixer("gated_linear_attention")
class GatedLinearAttention(Mixer):
    """Linear attention with a decay that is made from the input, one per token and key channel.

    q = Wq x * key_dim^-1/2, k = Wk x [heads, key_dim], v = Wv x [heads, value_dim]; z = Wa2 (Wa1 x) + b (a low-rank
    projection, float32 from the second product on), alpha = sigmoid(z)^(1 / tau) [heads, key_dim].  Per head and request a
    float32 state S [key_dim, value_dim] that starts at zero: S <- diag(alpha) S + k v^T, o = S^T q, token by token.  Every
    head's o gets an RMS norm with one weight [value_dim] for all heads; the heads side by side times silu(Wg x); output
    projection.  Decays, their logarithms and exponentials, the state, the norm and the gate's product are float32.

    params: hidden_size, num_heads, key_dim, value_dim, tau, norm_eps, decay_rank (for random weights only: the checkpoint's
            tensors give the rank), names.
    """

    graph_safe = True

    def __init__(self, spec, prefix, env, position=None):
        super().__init__(spec, prefix, env)
        s = spec
        self.E, self.heads, self.dk, self.dv = int(s["hidden_size"]), int(s["num_heads"]), int(s["key_dim"]), int(s["value_dim"])
        self.tau = float(s["tau"])
        if not self.tau > 0:
            raise ValueError("tau must be positive")
        if self.dk > ops.DECAY_ATTENTION_MAX_KEY_DIM:
            raise ValueError(f"key size {self.dk}: the kernel takes key sizes up to {ops.DECAY_ATTENTION_MAX_KEY_DIM}")
        self.eps = float(s["norm_eps"])
        self.rank_hint = int(s.get("decay_rank", 16))
        names = {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "norm": "norm", "a1": "a1", "a2": "a2", "a2_bias": "a2.b"}
        names.update(s.get("names") or {})
        self.names = {k: self.name(v) for k, v in names.items()}
        self.Nk, self.Nv = self.heads * self.dk, self.heads * self.dv
        self.w_in = self.w_a2 = self.a2_bias = self.w_out = self.norm = None
        self.rank = self.rank_pad = 0

    def tensors(self) -> Dict[str, TensorDecl]:
        n, R = self.names, self.rank_hint
        return {n["q"]: TensorDecl((self.Nk, self.E)), n["k"]: TensorDecl((self.Nk, self.E)), n["v"]: TensorDecl((self.Nv, self.E)),
                n["gate"]: TensorDecl((self.Nv, self.E)), n["out"]: TensorDecl((self.E, self.Nv)),
                n["norm"]: TensorDecl((self.dv,), kind="vector", init="norm"),
                n["a1"]: TensorDecl((-1, self.E), random_shape=(R, self.E)),
                n["a2"]: TensorDecl((self.Nk, -1), random_shape=(self.Nk, R), std=0.5),
                n["a2_bias"]: TensorDecl((self.Nk,), kind="vector", std=1.0)}

    def load(self, src) -> None:
        f, n = src.fetch, self.names
        a1, a2 = f(n["a1"]), f(n["a2"])
        if a1.shape[0] != a2.shape[1]:
            raise ValueError(f"{n['a1']} has {a1.shape[0]} rows, {n['a2']} {a2.shape[1]} columns")
        self.rank = a1.shape[0]
        # the low-rank part sits first in the packed projection, padded with zero rows (and zero columns of the second
        # matrix) to a multiple of 32, the inner size that the product for a few tokens takes; the packed rows end in zero rows
        # up to a multiple of 16
        self.rank_pad = self.rank + (-self.rank % 32)
        if self.rank_pad != self.rank:
            a1 = torch.cat((a1, a1.new_zeros((self.rank_pad - self.rank, a1.shape[1]))), dim=0)
            a2 = torch.cat((a2, a2.new_zeros((a2.shape[0], self.rank_pad - self.rank))), dim=1)
        w_in = torch.cat((a1, f(n["q"]), f(n["k"]), f(n["v"]), f(n["gate"])), dim=0)
        pad = -w_in.shape[0] % 16
        if pad:
            w_in = torch.cat((w_in, w_in.new_zeros((pad, w_in.shape[1]))), dim=0)
        self.w_in, self.w_a2 = w_in.contiguous(), a2.contiguous()
        self.a2_bias = f(n["a2_bias"]).float().contiguous()
        self.w_out = f(n["out"]).contiguous()
        self.norm = f(n["norm"]).float().contiguous()

    def cache_need(self):
        return StateNeed((self.heads, self.dk, self.dv), "float32")

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        Nk, Nv = self.Nk, self.Nv
        proj = ops.linear(x, self.w_in)
        R = self.rank_pad
        z = ops.linear(proj[:, :R], self.w_a2, out_dtype=torch.float32)
        o = ops.gated_decay_attention(proj[:, R:R + Nk], proj[:, R + Nk:R + 2 * Nk], proj[:, R + 2 * Nk:R + 2 * Nk + Nv], z,
                                      self.a2_bias, heads=self.heads, tau=self.tau, q_scale=self.dk ** -0.5, state=cache.state,
                                      q_start=ctx.q_start, slots=ctx.slots,
                                      q_lens=None if ctx.uniform_decode else ctx.host_q_lens, workspace=ctx.workspace)
        act = torch.empty((x.shape[0], Nv), dtype=x.dtype, device=x.device)
        ops.group_rms_gate(o, self.heads, self.norm, self.eps, proj[:, R + 2 * Nk + Nv:R + 2 * Nk + 2 * Nv], act, ops.ACT_SILU)
        return ops.linear(act, self.w_out)
