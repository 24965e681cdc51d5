"""Nametar, plain and slow: one function per mechanism, written from the design's equations in float64 on the CPU.

Shares no code with the engine package.  Notation: x [T, E] the stream, h the normed input of a sublayer, W stored
[out, in] and applied as h @ W.T.  Everything is computed per sequence, every position from all earlier ones (no cache,
no state carried between calls except where a function says so).
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch

F64 = torch.float64


def rms_scale(x: torch.Tensor, w: Optional[torch.Tensor], eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) (* w) over the last dimension."""
    y = x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)
    return y if w is None else y * w


def silu(z: torch.Tensor) -> torch.Tensor:
    return z * torch.sigmoid(z)


def rotary_frequencies(dims: int, base: float, scaling: Optional[dict]):
    """-> (frequencies [dims / 2], factor on cos and sin).  With scaling = {factor, original, fast, slow} the frequencies
    whose wavelength is long against `original` are divided by `factor`, with a linear ramp between the two bounds."""
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(dims // 2)], dtype=F64)
    if not scaling:
        return f, 1.0
    def dim_of(turns):
        return dims * math.log(scaling["original"] / (2 * math.pi * turns)) / (2 * math.log(base))
    lo = max(math.floor(dim_of(scaling["fast"])), 0)
    hi = min(math.ceil(dim_of(scaling["slow"])), dims - 1)
    out = []
    for i in range(dims // 2):
        ramp = min(max((i - lo) / max(hi - lo, 0.001), 0.0), 1.0)
        out.append(float(f[i]) / scaling["factor"] * ramp + float(f[i]) * (1 - ramp))
    return torch.tensor(out, dtype=F64), 0.1 * math.log(scaling["factor"]) + 1.0


def rotate(vec: torch.Tensor, pos: int, freq: torch.Tensor, mag: float, dims: int) -> torch.Tensor:
    """One vector at one position: element i of the first `dims` pairs with element i + dims / 2; the rest pass."""
    out = vec.clone()
    for i in range(dims // 2):
        a = float(torch.tensor(pos * float(freq[i].to(torch.float32)), dtype=torch.float32))      # the angle is a float32 product
        c, s = math.cos(a) * mag, math.sin(a) * mag
        u, v = vec[i], vec[i + dims // 2]
        out[i] = u * c - v * s
        out[i + dims // 2] = v * c + u * s
    return out


def visible(i: int, j: int, window: Optional[int]) -> bool:
    return j <= i and (window is None or i - j < window)


def latent_attention(W: Dict[str, torch.Tensor], pre: str, m: dict, h: torch.Tensor, eps: float, gated: bool) -> torch.Tensor:
    """Keys and values of every head from one latent per token; an optional rotated part of the query heads against one
    rotated key part shared by all heads; optional window; optional sigmoid gate on the heads side by side."""
    T = h.shape[0]
    H, dim, vdim, r = m["heads"], m["dim"], m["vdim"], m["kv_rank"]
    rd = m.get("rot_dim", 0) or 0
    if m.get("q_rank"):
        q = rms_scale(h @ W[pre + "dq"].T, W[pre + "dq.norm"], eps) @ W[pre + "uq"].T
    else:
        q = h @ W[pre + "q"].T
    q = q.view(T, H, dim + rd)
    down = h @ W[pre + "dkv"].T
    c = rms_scale(down[:, :r], W[pre + "dkv.norm"], eps)
    k = (c @ W[pre + "uk"].T).view(T, H, dim)
    v = (c @ W[pre + "uv"].T).view(T, H, vdim)
    window = (m.get("mask") or {}).get("size")
    if rd:
        rot = m["rot"]
        freq, mag = rotary_frequencies(rot["dims"], rot["base"], rot.get("scaling"))
        kr = torch.stack([rotate(down[t, r:], t, freq, mag, rot["dims"]) for t in range(T)])
        qr = torch.stack([torch.stack([rotate(q[t, hh, dim:], t, freq, mag, rot["dims"]) for hh in range(H)]) for t in range(T)])
    out = torch.zeros(T, H, vdim, dtype=F64)
    for i in range(T):
        js = [j for j in range(T) if visible(i, j, window)]
        for hh in range(H):
            s = k[js, hh] @ q[i, hh, :dim]
            if rd:
                s = s + kr[js] @ qr[i, hh]
            p = torch.softmax(s * m["scale"], 0)
            out[i, hh] = p @ v[js, hh]
    o = out.reshape(T, H * vdim)
    if gated:
        o = o * torch.sigmoid(h @ W[pre + "g"].T)
    return o @ W[pre + "o"].T


def gated_linear_attention(W: Dict[str, torch.Tensor], pre: str, m: dict, h: torch.Tensor, eps: float) -> torch.Tensor:
    """S_t = diag(alpha_t) S_(t-1) + k_t v_t^T, o_t = S_t^T q_t with alpha = sigmoid(z)^(1/tau) per key channel."""
    T = h.shape[0]
    H, dim, vdim, tau = m["heads"], m["dim"], m["vdim"], m["tau"]
    q = (h @ W[pre + "q"].T).view(T, H, dim) * dim ** -0.5
    k = (h @ W[pre + "k"].T).view(T, H, dim)
    v = (h @ W[pre + "v"].T).view(T, H, vdim)
    z = ((h @ W[pre + "a1"].T) @ W[pre + "a2"].T + W[pre + "a2.b"]).view(T, H, dim)
    alpha = torch.sigmoid(z) ** (1.0 / tau)
    o = torch.zeros(T, H, vdim, dtype=F64)
    for hh in range(H):
        S = torch.zeros(dim, vdim, dtype=F64)
        for t in range(T):
            S = alpha[t, hh][:, None] * S + k[t, hh][:, None] * v[t, hh][None, :]
            o[t, hh] = S.T @ q[t, hh]
    o = rms_scale(o, W[pre + "norm"], eps).reshape(T, H * vdim)
    return (o * silu(h @ W[pre + "g"].T)) @ W[pre + "o"].T


def feed_forward(W, pre: str, h: torch.Tensor) -> torch.Tensor:
    return (silu(h @ W[pre + "gate"].T) * (h @ W[pre + "up"].T)) @ W[pre + "down"].T


def layer(cfg: dict, W, i: int, x: torch.Tensor) -> torch.Tensor:
    """x <- x + m norm1b(mixer(norm1 x)); x <- x + m norm2b(ff(norm2 x))."""
    L, p, eps, mult = cfg["layers"][i], f"l{i}.", cfg["norm"]["eps"], cfg.get("residual_mult", 1.0)
    h = rms_scale(x, W[p + "norm1"], eps)
    if L["type"] == "gla":
        a = gated_linear_attention(W, p + "mix.", L["mixer"], h, eps)
    else:
        a = latent_attention(W, p + "mix.", L["mixer"], h, eps, gated=L["type"] == "latent_attention")
    x = x + mult * rms_scale(a, W[p + "norm1b"], eps)
    if L.get("mlp") is not None:
        f = feed_forward(W, p + "mlp.", rms_scale(x, W[p + "norm2"], eps))
        x = x + mult * rms_scale(f, W[p + "norm2b"], eps)
    return x


def forward_sequence(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], mutate=None) -> torch.Tensor:
    """Logits [T, vocab] of every position of one sequence.  `mutate(cfg)` may return a changed copy of the configuration
    (a window one token wider, say) to show what a test's bound tells apart."""
    if mutate is not None:
        cfg = mutate(cfg)
    W = {k: v.to(F64) for k, v in weights.items()}
    x = W["embed"][torch.tensor(tokens)] * (cfg.get("embedding") or {}).get("scale", 1.0)
    for i in range(len(cfg["layers"])):
        x = layer(cfg, W, i, x)
    return rms_scale(x, W["final.norm"], cfg["norm"]["eps"]) @ W["head"].T


def greedy_generate(cfg: dict, weights, prompt: List[int], n: int) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(n):
        t = int(forward_sequence(cfg, weights, toks)[-1].argmax())
        out.append(t)
        toks.append(t)
    return out
