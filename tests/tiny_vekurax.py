"""Small Vekurax configurations with seeded random weights for the tests.

Sizes differ from configuration to configuration in everything the design lets differ: width, vocabulary, heads and
groups, head sizes that are no multiple of 32 or of 8, taps (also 1: no convolution state), windows (also 1, and wider
than any test sequence), kept first tokens (also 0), rows of the distance table, decays, scales (also 1), layers without
a feed-forward, and layers that run another layer's weights.  Weights are drawn in float32 from a generator seeded by
(seed, tensor name), sized so that every sublayer moves the stream visibly, and rounded to bfloat16 so that both engines
and the plain implementation hold the same numbers.  This file shares nothing with the engine package.
"""

from __future__ import annotations

import copy
import hashlib
import math
from typing import Dict

import torch


def _layer(width, *, heads, kv_heads, dim, window, keep_first, taps, far, scale=None, r_heads, r_dim, r_vdim, decay, ff,
           left_scale=0.9, right_scale=0.6, weights_of=None):
    entry = {"type": "parallel",
             "mixer": {"left": {"heads": heads, "kv_heads": kv_heads, "dim": dim, "vdim": dim, "conv": taps, "bias_max": far,
                                "scale": scale if scale is not None else dim ** -0.5,
                                "mask": {"size": window, "keep_first": keep_first}},
                       "right": {"heads": r_heads, "dim": r_dim, "vdim": r_vdim, "decay": list(decay)},
                       "left_scale": left_scale, "right_scale": right_scale},
             "mlp": {"kind": "dense", "ff": ff} if ff else None}
    if weights_of is not None:
        entry["weights_of"] = weights_of
    return entry


def _model(width, vocab, eps, layers, rows):
    return {"architecture": "Vekurax", "width": width, "vocab": vocab, "norm": {"eps": eps}, "layers": layers,
            "_rows": rows}          # "_rows": rows of every layer's distance table (a tensor's shape, not a config key)


def _again(layer, of):
    out = copy.deepcopy(layer)
    out["weights_of"] = of
    return out


_A0 = _layer(64, heads=6, kv_heads=3, dim=24, window=9, keep_first=3, taps=3, far=37, r_heads=3, r_dim=12, r_vdim=20,
             decay=(0.5, 0.9, 0.99), ff=48, left_scale=1.3, right_scale=0.7)
_A1 = _layer(64, heads=2, kv_heads=1, dim=40, window=5, keep_first=0, taps=2, far=64, scale=0.21, r_heads=2, r_dim=8, r_vdim=33,
             decay=(0.8, 0.999), ff=None)
# A: two layers with tensors, each run twice in an order of their own; one has no feed-forward and keeps no first tokens
TINY_VA = _model(64, 97, 1e-5, [_A0, _A1, _again(_A1, 1), _again(_A0, 0)], rows=10)

# B: one head per kv head, one tap (no convolution state), a window of one token beside four kept ones, unit scales,
#    a distance table of two rows, one head in the linear attention, key size above 32
TINY_VB = _model(48, 61, 1e-6, [
    _layer(48, heads=3, kv_heads=3, dim=16, window=1, keep_first=4, taps=1, far=5, r_heads=1, r_dim=36, r_vdim=8, decay=(0.95,),
           ff=80, left_scale=1.0, right_scale=1.0),
    _layer(48, heads=3, kv_heads=3, dim=16, window=1, keep_first=4, taps=1, far=5, r_heads=1, r_dim=36, r_vdim=8, decay=(0.95,),
           ff=80, left_scale=1.0, right_scale=1.0)], rows=2)

# C: sixteen heads on one kv head (two blocks of heads in the attention kernel), a window wider than the test sequences
#    with kept tokens inside it, five taps, head size 64, an odd number of table rows
TINY_VC = _model(96, 131, 1e-5, [
    _layer(96, heads=16, kv_heads=1, dim=64, window=300, keep_first=7, taps=5, far=200, r_heads=2, r_dim=32, r_vdim=64,
           decay=(0.9, 0.97), ff=64),
    _layer(96, heads=4, kv_heads=2, dim=32, window=33, keep_first=17, taps=4, far=100, r_heads=4, r_dim=16, r_vdim=16,
           decay=(0.3, 0.6, 0.9, 1.0), ff=32, left_scale=0.5, right_scale=2.0)], rows=15)

CONFIGS_V = {"VA": TINY_VA, "VB": TINY_VB, "VC": TINY_VC}


def config_json(cfg: dict) -> dict:
    return {k: v for k, v in cfg.items() if not k.startswith("_")}


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    E, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, E), "final.norm": (E,), "final.norm.b": (E,), "final.norm.alpha": ()}
    for i, layer in enumerate(cfg["layers"]):
        if "weights_of" in layer:
            continue
        p = f"l{i}."
        lf, rt = layer["mixer"]["left"], layer["mixer"]["right"]
        Cq, Ck = lf["heads"] * lf["dim"], lf["kv_heads"] * lf["dim"]
        Nk, Nv = rt["heads"] * rt["dim"], rt["heads"] * rt["vdim"]
        out.update({p + "norm1": (E,), p + "norm1.b": (E,), p + "norm1.alpha": (),
                    p + "mix.left.q": (Cq, E), p + "mix.left.k": (Ck, E), p + "mix.left.q.norm": (Cq,), p + "mix.left.k.norm": (Ck,),
                    p + "mix.left.q.conv": (Cq, lf["conv"]), p + "mix.left.k.conv": (Ck, lf["conv"]),
                    p + "mix.left.rel": (cfg["_rows"], lf["heads"]), p + "mix.left.g": (lf["heads"], E), p + "mix.left.o": (E, Cq),
                    p + "mix.right.q": (Nk, E), p + "mix.right.k": (Nk, E), p + "mix.right.v": (Nv, E), p + "mix.right.g": (Nv, E),
                    p + "mix.right.o": (E, Nv), p + "mix.right.norm": (Nv,)})
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            out.update({p + "mlp.gate": (ff, E), p + "mlp.up": (ff, E), p + "mlp.down": (E, ff)})
    return out


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors by checkpoint name."""
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
        g = torch.Generator(device="cpu").manual_seed(int.from_bytes(h[:7], "little"))
        r = torch.randn(shape, generator=g, dtype=torch.float32)
        if name.endswith(".alpha"):
            t = 0.7 + 0.2 * r
        elif name.endswith(".b"):
            t = 0.1 * r
        elif name.endswith("norm1") or name.endswith(".norm"):
            t = 1.0 + 0.1 * r
        elif name.endswith(".conv"):
            t = 0.6 * r
        elif name.endswith(".rel"):
            t = 1.0 * r
        elif name == "embed":
            t = 0.7 * r
        else:
            t = r / math.sqrt(shape[1])           # a projection: outputs about as large as its inputs
        out[name] = t.to(torch.bfloat16)
    return out
