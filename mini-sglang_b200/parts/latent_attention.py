from __future__ import annotations

from typing import Dict

import torch

from .. import ops
from ..cache.manager import PagedKVNeed
from ..weights.loader import TensorDecl
from .attention import paged_attend
from .base import Mixer, register_mixer
from .context import KVCacheView


@register_mixer("latent_attention")
class LatentAttention(Mixer):
    """Softmax attention whose keys and values are made from one low-rank latent per token; only the latent (and one
    rotated key part shared by all heads) is cached.

    q = Wq x, or through a latent of its own: q = Wuq rmsnorm(Wdq x) (`q_rank`); per head [key_dim | rot_dim].
    Wdkv x has kv_rank + rot_dim rows: the first kv_rank, RMS-normed, are the latent c; the last rot_dim are the rotated key
    part.  Per head k = Wuk_h c, v = Wuv_h c; score = (q_plain . k + q_rot . k_rot) * scale; causal, optionally only the last
    `window` keys; softmax; optionally the heads side by side times sigmoid(Wg x); output projection.

    Computed with the up-projections folded into the query and the output: score = (Wuk_h^T q_plain | q_rot) . (c | k_rot), so a
    token's cache row [c | k_rot] is key and value at once for all heads (one kv head of size kv_rank + rot_dim, its values the
    row itself: `PagedKVNeed.shared_kv`), and head h's output is Wuv_h applied to the first kv_rank elements of what the
    attention kernels return.  The attention launches are the paged ones every other softmax mixer of the engine uses.

    params: hidden_size, num_heads, key_dim, rot_dim (0: no rotated part), value_dim, kv_rank, q_rank (None: no query latent),
            scale, window (None: all keys), gate (None | "sigmoid"), norm_eps, names.  The position encoding (a part with
            `inv_freq`, `magnitude`, `rotary_dim`) comes from the layer.
    """

    graph_safe = True

    def __init__(self, spec, prefix, env, position=None):
        super().__init__(spec, prefix, env)
        s = spec
        self.E, self.H = int(s["hidden_size"]), int(s["num_heads"])
        self.dk, self.rd, self.dv = int(s["key_dim"]), int(s.get("rot_dim") or 0), int(s["value_dim"])
        self.r, self.rq = int(s["kv_rank"]), int(s.get("q_rank") or 0)
        self.scale = float(s["scale"])
        self.window = int(s["window"]) if s.get("window") else None
        self.gate = s.get("gate")
        if self.gate not in (None, "sigmoid"):
            raise ValueError(f"unknown output gate {self.gate!r}; known: sigmoid")
        self.eps = float(s["norm_eps"])
        self.position = position if self.rd else None
        if self.rd and (position is None or not hasattr(position, "inv_freq")):
            raise ValueError("a latent attention with a rotated part needs a position encoding that gives its frequencies")
        self.rot_dims = int(self.position.rotary_dim) if self.rd else 0
        if self.rot_dims > self.rd:
            raise ValueError(f"{self.rot_dims} rotated dimensions, the rotated part has {self.rd}")
        self.D = self.r + self.rd                     # a cache row
        if self.D > 512:
            raise ValueError(f"latent size {self.r} + rotated part {self.rd}: the attention kernels take rows up to 512")
        names = {"q": "q", "dq": "dq", "dq_norm": "dq.norm", "uq": "uq", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk",
                 "uv": "uv", "gate": "g", "out": "o"}
        names.update(s.get("names") or {})
        self.names = {k: self.name(v) for k, v in names.items()}
        self.use_mma = ops.mma_supported(self.D, env.dtype)
        self.w_in = self.w_uq = self.w_ukT = self.w_uvT = self.w_o = self.dq_norm = self.dkv_norm = None

    # -- weights -----------------------------------------------------------------------
    def tensors(self) -> Dict[str, TensorDecl]:
        n, qd = self.names, self.H * (self.dk + self.rd)
        t = {n["dkv"]: TensorDecl((self.r + self.rd, self.E)), n["dkv_norm"]: TensorDecl((self.r,), kind="vector", init="norm"),
             n["uk"]: TensorDecl((self.H * self.dk, self.r)), n["uv"]: TensorDecl((self.H * self.dv, self.r)),
             n["out"]: TensorDecl((self.E, self.H * self.dv))}
        if self.rq:
            t[n["dq"]] = TensorDecl((self.rq, self.E))
            t[n["dq_norm"]] = TensorDecl((self.rq,), kind="vector", init="norm")
            t[n["uq"]] = TensorDecl((qd, self.rq))
        else:
            t[n["q"]] = TensorDecl((qd, self.E))
        if self.gate:
            t[n["gate"]] = TensorDecl((self.H * self.dv, self.E))
        return t

    def load(self, src) -> None:
        f, n = src.fetch, self.names
        first = f(n["dq"]) if self.rq else f(n["q"])
        rows = [first, f(n["dkv"])] + ([f(n["gate"])] if self.gate else [])
        self.q_w = first.shape[0]                      # columns of the packed projection: [q or its latent | dkv | gate]
        w_in = torch.cat(rows, dim=0)
        pad = -w_in.shape[0] % 16                      # the weight-streaming product for a few tokens takes rows in sixteens
        if pad:
            w_in = torch.cat((w_in, w_in.new_zeros((pad, w_in.shape[1]))), dim=0)
        self.w_in = w_in.contiguous()
        if self.rq:
            self.w_uq = f(n["uq"]).contiguous()
            self.dq_norm = f(n["dq_norm"]).float().contiguous()
        self.dkv_norm = f(n["dkv_norm"]).float().contiguous()
        self.w_ukT = f(n["uk"]).view(self.H, self.dk, self.r).contiguous()                    # q_plain [H, T, dk] @ -> [H, T, r]
        self.w_uvT = f(n["uv"]).view(self.H, self.dv, self.r).transpose(1, 2).contiguous()    # o_lat [H, T, r] @ -> [H, T, dv]
        self.w_o = f(n["out"]).contiguous()

    def cache_need(self):
        # every request's keys are cut by themselves: with one kv head for all query heads the decode launch reads a
        # thirteenth of a grouped-query cache, and dealing the keys out evenly over the blocks has nothing to even out
        return PagedKVNeed(1, self.D, self.window, q_heads=self.H, shared_kv=True, even_cut=False)

    # -- compute -----------------------------------------------------------------------
    def forward(self, x: torch.Tensor, ctx, cache: KVCacheView, writes_cache: bool = True) -> torch.Tensor:
        T, H, dk, rd, r, D = ctx.T, self.H, self.dk, self.rd, self.r, self.D
        proj = ops.linear(x, self.w_in)
        freq = self.position.inv_freq if rd else None
        mag = float(self.position.magnitude) if rd else 1.0
        cq = ops.latent_prep(proj, dq_off=0, q_rank=self.rq, dkv_off=self.q_w, kv_rank=r, rot_dim=rd, rot_dims=self.rot_dims,
                             dq_norm=self.dq_norm, dkv_norm=self.dkv_norm, eps=self.eps, freq=freq, mag=mag,
                             positions=ctx.positions, out_loc=cache.group.out_loc if writes_cache else None,
                             cache=cache.k if writes_cache else None, page_size=cache.page_size)
        q = ops.linear(cq, self.w_uq) if self.rq else proj[:, :self.q_w]
        q3 = q.view(T, H, dk + rd) if q.is_contiguous() else q.unflatten(1, (H, dk + rd))
        # the key up-projection folded into the query: per head [T, dk] x [dk, r], written in place into the query rows
        qf = torch.empty((T, H, D), dtype=x.dtype, device=x.device)
        torch.bmm(q3[:, :, :dk].transpose(0, 1), self.w_ukT, out=qf[:, :, :r].transpose(0, 1))
        if rd:
            ops.rope_heads(q3, dk, qf, r, rot_dim=rd, rot_dims=self.rot_dims, freq=freq, mag=mag, positions=ctx.positions)
        of = torch.empty_like(qf)
        view = KVCacheView(cache.k, cache.k, cache.group, cache.page_size)
        paged_attend(qf, of, ctx, view, n_q=H, n_kv=1, d=D, window=int(self.window or 0), scale=self.scale, use_mma=self.use_mma)
        # the value up-projection on what the heads gathered of the latent
        heads = torch.empty((T, H * self.dv), dtype=x.dtype, device=x.device)
        torch.bmm(of[:, :, :r].transpose(0, 1), self.w_uvT, out=heads.view(T, H, self.dv).transpose(0, 1))
        if self.gate:
            g0 = self.q_w + r + rd
            ops.gate_mul(proj[:, g0:g0 + H * self.dv], heads, heads, ops.ACT_SIGMOID)
        return ops.linear(heads, self.w_o)
