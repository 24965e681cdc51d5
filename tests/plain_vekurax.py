"""A plain, slow implementation of the Vekurax decoder, one function per mechanism, written from the
architecture's equations and sharing no code with the engine.  It takes the content of a config.json and a
dict of tensors by checkpoint name and runs one whole sequence at a time on the CPU; there is no cache: every
function sees all tokens of the sequence.

Notation: T tokens, width E, x the residual stream [T, E], u the normed input of a layer's sublayers.
"""

from __future__ import annotations

import math
from typing import Dict, List, Optional

import torch


def gelu_tanh(z: torch.Tensor) -> torch.Tensor:
    return 0.5 * z * (1.0 + torch.tanh(math.sqrt(2.0 / math.pi) * (z + 0.044715 * z ** 3)))


def dynamic_tanh(x: torch.Tensor, alpha: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor) -> torch.Tensor:
    """tanh(alpha x) * weight + bias, element by element; no statistics of the row."""
    return torch.tanh(alpha * x) * weight + bias


def rms_scale(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """x / sqrt(mean(x^2) + eps) * weight over the last dimension."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * weight


def short_causal_conv(u: torch.Tensor, taps: torch.Tensor) -> torch.Tensor:
    """u [T, C], taps [C, K]: y[t, c] = sum_j taps[c, j] * u[t - K + 1 + j, c], zeros before the sequence."""
    T, C = u.shape
    K = taps.shape[1]
    padded = torch.cat((torch.zeros(K - 1, C, dtype=u.dtype), u), dim=0)
    y = torch.zeros_like(u)
    for j in range(K):
        y = y + taps[:, j] * padded[j:j + T]
    return y


def distance_bucket(n: int, rows: int, far: int) -> int:
    """Row of the distance-bias table for a distance n >= 0: one row per distance below rows/2, then
    logarithmically wider buckets that reach the last row at distance `far`."""
    half = rows // 2
    if n < half:
        return n
    return min(rows - 1, half + int(math.floor(math.log(n / half) / math.log(far / half) * (rows - half))))


def visible(i: int, j: int, window: int, keep_first: int) -> bool:
    return j <= i and (i - j < window or j < keep_first)


def left_attention(u: torch.Tensor, w: Dict[str, torch.Tensor], p: str, c: dict, eps: float) -> torch.Tensor:
    """Windowed softmax attention whose values are its keys (before the key norm), with a short convolution and a
    whole-projection RMS norm on q and k, a learned bias by bucketed distance and one output gate per head."""
    T = u.shape[0]
    H, G, d = c["heads"], c["kv_heads"], c["dim"]
    q = short_causal_conv(u @ w[p + ".q"].T, w[p + ".q.conv"])
    k = short_causal_conv(u @ w[p + ".k"].T, w[p + ".k.conv"])
    v = k.view(T, G, d)
    q = rms_scale(q, w[p + ".q.norm"], eps).view(T, H, d)
    k = rms_scale(k, w[p + ".k.norm"], eps).view(T, G, d)
    rel = w[p + ".rel"]
    rows = rel.shape[0]
    gate = torch.sigmoid(u @ w[p + ".g"].T)                       # [T, H]
    out = torch.zeros(T, H, d, dtype=u.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            js = [j for j in range(i + 1) if visible(i, j, c["mask"]["size"], c["mask"]["keep_first"])]
            s = torch.stack([(q[i, h] * k[j, g]).sum() * c["scale"] + rel[distance_bucket(i - j, rows, c["bias_max"]), h]
                             for j in js])
            a = torch.softmax(s, dim=0)
            out[i, h] = (a[:, None] * v[js, g]).sum(dim=0) * gate[i, h]
    return out.reshape(T, H * d) @ w[p + ".o"].T


def right_attention(u: torch.Tensor, w: Dict[str, torch.Tensor], p: str, c: dict, eps: float) -> torch.Tensor:
    """Linear attention with a fixed decay per head: S <- decay * S + k v^T, o = S^T q, token by token."""
    T = u.shape[0]
    H, dk, dv = c["heads"], c["dim"], c["vdim"]
    silu = torch.nn.functional.silu
    q = silu(u @ w[p + ".q"].T).view(T, H, dk)
    k = silu(u @ w[p + ".k"].T).view(T, H, dk)
    v = silu(u @ w[p + ".v"].T).view(T, H, dv)
    o = torch.zeros(T, H, dv, dtype=u.dtype)
    for h in range(H):
        S = torch.zeros(dk, dv, dtype=u.dtype)
        for t in range(T):
            S = c["decay"][h] * S + k[t, h][:, None] * v[t, h][None, :]
            o[t, h] = S.T @ q[t, h]
    y = rms_scale(o.reshape(T, H * dv), w[p + ".norm"], eps) * torch.sigmoid(u @ w[p + ".g"].T)
    return y @ w[p + ".o"].T


def pair_mixer(u, w, p, c, eps):
    return c["left_scale"] * left_attention(u, w, p + ".left", c["left"], eps) + \
        c["right_scale"] * right_attention(u, w, p + ".right", c["right"], eps)


def feed_forward(u, w, p, c):
    if c["kind"] != "dense":
        raise ValueError(c["kind"])
    return (gelu_tanh(u @ w[p + ".gate"].T) * (u @ w[p + ".up"].T)) @ w[p + ".down"].T


def forward_sequence(cfg: dict, weights: Dict[str, torch.Tensor], tokens: List[int], dtype=torch.float64,
                     streams: Optional[list] = None) -> torch.Tensor:
    """-> logits [T, vocab]; `streams`, if given, receives the residual stream after every layer."""
    w = {k: (v.to(dtype) if v.is_floating_point() else v) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        src = layer.get("weights_of", i)
        p = f"l{src}"
        if layer["type"] != "parallel":
            raise ValueError(layer["type"])
        u = dynamic_tanh(x, w[p + ".norm1.alpha"], w[p + ".norm1"], w[p + ".norm1.b"])
        y = pair_mixer(u, w, p + ".mix", layer["mixer"], eps)
        if layer.get("mlp") is not None:
            y = y + feed_forward(u, w, p + ".mlp", layer["mlp"])
        x = x + y
        if streams is not None:
            streams.append(x.clone())
    x = dynamic_tanh(x, w["final.norm.alpha"], w["final.norm"], w["final.norm.b"])
    return x @ w["embed"].T


def greedy_generate(cfg, weights, prompt: List[int], n_new: int, dtype=torch.float64) -> List[int]:
    toks, out = list(prompt), []
    for _ in range(n_new):
        t = int(forward_sequence(cfg, weights, toks, dtype)[-1].argmax())
        out.append(t)
        toks.append(t)
    return out
