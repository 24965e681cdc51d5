from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..cache.manager import StateNeed
from ..weights.loader import TensorDecl
from .base import Mixer, Projected, register_mixer


@register_mixer("decay_linear_attention")
class DecayLinearAttention(Mixer, Projected):
    """Linear attention with one fixed decay per head.

    q = silu(Wq x), k = silu(Wk x) [heads, key_dim], v = silu(Wv x) [heads, value_dim]; per head and request a state
    S [key_dim, value_dim] in float32 that starts at zero: S <- decay_h S + k v^T, o = S^T q, token by token; the heads side
    by side get one RMS norm (plain weight), times sigmoid(Wg x), then the output projection.

    params: hidden_size, num_heads, key_dim, value_dim, decay (one number per head), norm_eps, names.
    """

    graph_safe = True

    def __init__(self, spec, prefix, env, position=None):
        super().__init__(spec, prefix, env)
        s = spec
        self.E, self.heads, self.dk, self.dv = int(s["hidden_size"]), int(s["num_heads"]), int(s["key_dim"]), int(s["value_dim"])
        self.decay_values = [float(a) for a in s["decay"]]
        if len(self.decay_values) != self.heads:
            raise ValueError("one decay per head wanted")
        if self.dk > ops.DECAY_ATTENTION_MAX_KEY_DIM:
            raise ValueError(f"key size {self.dk}: the kernel takes key sizes up to {ops.DECAY_ATTENTION_MAX_KEY_DIM}")
        self.eps = float(s["norm_eps"])
        names = {"q": "q", "k": "k", "v": "v", "gate": "gate", "out": "out", "norm": "norm"}
        names.update(s.get("names") or {})
        self.names = {k: self.name(v) for k, v in names.items()}
        self.Nk, self.Nv = self.heads * self.dk, self.heads * self.dv
        self.w_in = self.w_out = self.norm = self.decay = None

    def tensors(self) -> Dict[str, TensorDecl]:
        n = self.names
        return {n["q"]: TensorDecl((self.Nk, self.E)), n["k"]: TensorDecl((self.Nk, self.E)), n["v"]: TensorDecl((self.Nv, self.E)),
                n["gate"]: TensorDecl((self.Nv, self.E)), n["out"]: TensorDecl((self.E, self.Nv)),
                n["norm"]: TensorDecl((self.Nv,), kind="vector", init="norm")}

    def load(self, src) -> None:
        f, n = src.fetch, self.names
        self.w_in = torch.cat((f(n["q"]), f(n["k"]), f(n["v"]), f(n["gate"])), dim=0).contiguous()
        self.w_out = f(n["out"]).contiguous()
        self.norm = f(n["norm"]).float().contiguous()
        self.decay = torch.tensor(self.decay_values, dtype=torch.float32, device=self.w_in.device)

    def in_weight(self):
        return self.w_in

    def out_weight(self):
        return self.w_out

    def cache_need(self):
        return StateNeed((self.heads, self.dk, self.dv), "float32")

    def middle(self, proj, act, ctx, cache=None, writes_cache=True, out_scale=1.0):
        Nk, Nv = self.Nk, self.Nv
        o = ops.decay_attention(proj[:, :Nk], proj[:, Nk:2 * Nk], proj[:, 2 * Nk:2 * Nk + Nv], heads=self.heads, decay=self.decay,
                                state=cache.state, q_start=ctx.q_start, slots=ctx.slots,
                                q_lens=None if ctx.uniform_decode else ctx.host_q_lens, workspace=ctx.workspace)
        ops.rms_gate(o, self.norm, self.eps, proj[:, 2 * Nk + Nv:2 * Nk + 2 * Nv], act, out_scale)

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        return self.forward_projected(x, ctx, cache, writes_cache)
