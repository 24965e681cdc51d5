from __future__ import annotations

import math
from typing import Dict

import torch

from .. import ops
from ..cache.manager import PagedKVNeed, StateNeed
from ..weights.loader import TensorDecl
from .attention import paged_attend
from .base import Mixer, Projected, register_mixer


def distance_buckets(rows: int, far: float, n: int) -> torch.Tensor:
    """Row of a distance-bias table for every distance 0 .. n-1: the first rows // 2 distances have a row each, the
    larger ones share rows whose width grows logarithmically so that distance `far` reaches the last row."""
    half = rows // 2
    out = []
    for dist in range(n):
        if dist < half or half == 0:
            out.append(min(dist, rows - 1))
        else:
            out.append(min(rows - 1, half + int(math.floor(math.log(dist / half) / math.log(far / half) * (rows - half)))))
    return torch.tensor(out, dtype=torch.long)


@register_mixer("conv_window_attention")
class ConvWindowAttention(Mixer, Projected):
    """Grouped-query softmax attention over a sliding window and the first tokens of the sequence, whose values are its keys.

    q = Wq x, k = Wk x; a short causal convolution over time on every channel of q and of k (taps per channel, no bias; the
    last taps - 1 inputs of a request are its state); v = k as it leaves the convolution; RMS norm over the whole of q and
    over the whole of k (one weight per channel, all heads at once); no rotation.  The query at position i sees key j <= i if
    i - j < window or j < keep_first.  score = q . k * scale + bias[bucket(i - j), head] with a learned table of `rows`
    buckets (`distance_buckets`); softmax; the head's output times sigmoid(Wg x)[head]; output projection.

    params: hidden_size, num_heads, num_kv_heads, head_dim, scale, conv_taps, norm_eps, window, keep_first, bias_far,
            bias_rows (for random weights only: the checkpoint's table gives the number of rows), names.
    """

    graph_safe = True

    def __init__(self, spec, prefix, env, position=None):
        super().__init__(spec, prefix, env)
        s = spec
        self.E, self.n_q, self.n_kv, self.d = int(s["hidden_size"]), int(s["num_heads"]), int(s["num_kv_heads"]), int(s["head_dim"])
        if self.n_q % self.n_kv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.d > ops.WINDOW_ATTENTION_MAX_HEAD_DIM:
            raise ValueError(f"head size {self.d}: the windowed attention kernel takes head sizes up to {ops.WINDOW_ATTENTION_MAX_HEAD_DIM}")
        self.scale = float(s["scale"])
        self.taps = int(s.get("conv_taps", 1))
        if not 1 <= self.taps <= ops.CONV_MAX_TAPS:
            raise ValueError(f"{self.taps} taps: the convolution kernel takes 1 to {ops.CONV_MAX_TAPS}")
        self.eps = float(s["norm_eps"])
        self.window = int(s["window"]) if s.get("window") else None
        self.keep_first = int(s.get("keep_first", 0)) if self.window else 0
        self.bias_far = float(s["bias_far"])
        self.bias_rows = int(s.get("bias_rows", 48))
        self.Cq, self.Ck = self.n_q * self.d, self.n_kv * self.d
        names = {"q": "q", "k": "k", "q_norm": "q_norm", "k_norm": "k_norm", "q_conv": "q_conv", "k_conv": "k_conv",
                 "bias": "distance_bias", "gate": "gate", "out": "out"}
        names.update(s.get("names") or {})
        self.names = {k: self.name(v) for k, v in names.items()}
        # bfloat16 at head sizes the mma kernels of csrc/attention.cu take: those, with the step's kv splits; otherwise (true
        # float32, other head sizes) the float32-arithmetic kernel of csrc/mixers.cu, which takes every request whole
        self.use_mma = ops.window_bias_supported(self.d, env.dtype, self.n_q // self.n_kv)
        self.w_in = self.w_out = self.q_taps = self.k_taps = self.q_norm = self.k_norm = self.bias = self.bias_log2 = None

    # -- weights -----------------------------------------------------------------------
    def tensors(self) -> Dict[str, TensorDecl]:
        n = self.names
        return {n["q"]: TensorDecl((self.Cq, self.E)), n["k"]: TensorDecl((self.Ck, self.E)),
                n["q_norm"]: TensorDecl((self.Cq,), kind="vector", init="norm"),
                n["k_norm"]: TensorDecl((self.Ck,), kind="vector", init="norm"),
                n["q_conv"]: TensorDecl((self.Cq, self.taps), kind="vector", std=0.5),
                n["k_conv"]: TensorDecl((self.Ck, self.taps), kind="vector", std=0.5),
                n["bias"]: TensorDecl((-1, self.n_q), kind="vector", std=0.5, random_shape=(self.bias_rows, self.n_q)),
                n["gate"]: TensorDecl((self.n_q, self.E)), n["out"]: TensorDecl((self.E, self.Cq))}

    def load(self, src) -> None:
        f, n = src.fetch, self.names
        self.w_in = torch.cat((f(n["q"]), f(n["k"]), f(n["gate"])), dim=0).contiguous()
        self.w_out = f(n["out"]).contiguous()
        # [taps, channels]: the kernel reads a tap's weights of neighbouring channels with one access
        self.q_taps, self.k_taps = f(n["q_conv"]).float().t().contiguous(), f(n["k_conv"]).float().t().contiguous()
        self.q_norm, self.k_norm = f(n["q_norm"]).float().contiguous(), f(n["k_norm"]).float().contiguous()
        table = f(n["bias"]).float()                                   # [rows, heads]
        rows = table.shape[0]
        if rows > 1 and self.bias_far <= rows // 2:
            raise ValueError(f"{n['bias']}: {rows} rows need a far distance beyond {rows // 2}, not {self.bias_far}")
        # by distance, ready to be looked up: every distance from `far` on falls into the last row
        n_dist = int(math.ceil(self.bias_far)) + 1 if rows > 1 else 1
        idx = distance_buckets(rows, self.bias_far, n_dist).to(table.device)
        self.bias = table[idx].t().contiguous()                         # [heads, distances]
        self.bias_log2 = (self.bias * math.log2(math.e)).contiguous() if self.use_mma else None

    def in_weight(self):
        return self.w_in

    def out_weight(self):
        return self.w_out

    def cache_need(self):
        return (PagedKVNeed(self.n_kv, self.d, self.window, q_heads=self.n_q, keep_first=self.keep_first,
                            library="attention" if self.use_mma else "mixers", even_cut=False),
                StateNeed((self.taps - 1, self.Cq + self.Ck), "compute"))

    # -- compute -----------------------------------------------------------------------
    def middle(self, proj, act, ctx, cache=None, writes_cache=True, out_scale=1.0):
        kv, conv = cache
        Cq, Ck = self.Cq, self.Ck
        q = ops.conv_norm_kvwrite(proj[:, :Cq], proj[:, Cq:Cq + Ck], n_kv=self.n_kv, head_dim=self.d, q_taps=self.q_taps,
                                  k_taps=self.k_taps, q_norm=self.q_norm, k_norm=self.k_norm, eps=self.eps, state=conv.state,
                                  token_req=ctx.token_req, q_start=ctx.q_start, slots=ctx.slots,
                                  out_loc=kv.group.out_loc if writes_cache else None, k_cache=kv.k if writes_cache else None,
                                  v_cache=kv.v if writes_cache else None, page_size=kv.page_size, one_token=ctx.uniform_decode)
        gate = proj[:, Cq + Ck:Cq + Ck + self.n_q]
        if self.use_mma:
            q3 = q.view(ctx.T, self.n_q, self.d)
            o = torch.empty_like(q3)
            paged_attend(q3, o, ctx, kv, n_q=self.n_q, n_kv=self.n_kv, d=self.d, window=int(self.window or 0), scale=self.scale,
                         use_mma=True, keep_first=self.keep_first, bias_log2=self.bias_log2)
            ops.head_gate(o, gate, act, out_scale)
            return
        ops.window_attention(q.view(ctx.T, self.n_q, self.d), act, kv.k, kv.v, q_start=ctx.q_start, kv_len=ctx.kv_len,
                             block_table=kv.group.block_table, n_kv=self.n_kv, page_size=kv.page_size,
                             window=int(self.window or 0), keep_first=self.keep_first, scale=self.scale,
                             q_lens=None if ctx.uniform_decode else ctx.host_q_lens, bias=self.bias, gate=gate,
                             out_scale=out_scale)

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        return self.forward_projected(x, ctx, cache, writes_cache)
