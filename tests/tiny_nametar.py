"""Small Nametar configurations with seeded random weights for the tests.

The configurations differ in everything the design lets differ: width, vocabulary, order and number of layers, heads,
key / value / latent sizes (cache rows of 32, 48, 64 and 128 elements, and 28, which no tensor-core kernel takes), a query
latent or none, a rotated part with fewer rotated dimensions than it has elements, frequency scaling or none, windows (1, 9,
wider than any test sequence), layers without a feed-forward, unit factors (residual factor and embedding scale 1, tau 1),
ranks of the decay's projection that are no multiple of anything.  Weights are drawn in float32 from a generator seeded by
(seed, tensor name) and rounded to bfloat16, so that the engine in both precisions and the plain implementation hold the
same numbers.  This file shares nothing with the engine package.
"""

from __future__ import annotations

import hashlib
import math
from typing import Dict

import torch


def _la(heads, dim, vdim, kv_rank, scale=None):
    return {"type": "latent_attention", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "kv_rank": kv_rank,
                                                  "scale": scale if scale is not None else dim ** -0.5}}


def _la2(heads, dim, rot_dim, vdim, kv_rank, window, q_rank=None, dims=None, base=10000.0, scaling=None, scale=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": kv_rank,
         "scale": scale if scale is not None else (dim + rot_dim) ** -0.5,
         "rot": {"base": base, "dims": dims if dims is not None else rot_dim}}
    if window:
        m["mask"] = {"size": window}
    if q_rank:
        m["q_rank"] = q_rank
    if scaling:
        m["rot"]["scaling"] = scaling
    return {"type": "latent_attention_2", "mixer": m}


def _gla(heads, dim, vdim, tau, rank):
    return {"type": "gla", "mixer": {"heads": heads, "dim": dim, "vdim": vdim, "tau": tau}, "_rank": rank}


def _with(layer, ff):
    out = dict(layer)
    out["mlp"] = {"kind": "dense", "ff": ff} if ff else None
    return out


def _model(width, vocab, eps, mult, emb_scale, layers):
    return {"architecture": "Nametar", "width": width, "vocab": vocab, "norm": {"eps": eps}, "residual_mult": mult,
            "embedding": {"scale": emb_scale}, "layers": layers}


YARN = {"factor": 4.0, "original": 32, "fast": 8.0, "slow": 1.0}
# A: window of 9 with a query latent and scaled frequencies (cache row 24 + 8 = 32), a linear attention without
#    feed-forward, a gated latent attention (row 48), a second linear attention
TINY_NA = _model(64, 97, 1e-5, 0.7, 3.0, [
    _with(_la2(3, 8, 8, 12, 24, window=9, q_rank=20, scaling=YARN), 48),
    _with(_gla(2, 12, 20, 4.0, rank=6), None),
    _with(_la(4, 16, 8, 48), 40),
    _with(_gla(3, 8, 8, 16.0, rank=3), 32)])
# B: unit factors, one head, a window of one token, no query latent, no frequency scaling, 4 of the 8 elements of the rotated
#    part rotated, a cache row of 28 elements, key size above 32 and tau 1 in the linear attention
TINY_NB = _model(48, 61, 1e-6, 1.0, 1.0, [
    _with(_gla(1, 36, 8, 1.0, rank=5), 80),
    _with(_la2(1, 20, 8, 16, 20, window=1, dims=4, base=100.0), 24),
    _with(_la2(2, 12, 8, 10, 20, window=4, dims=8, base=50.0, scale=0.4), None),
    _with(_la(2, 10, 14, 28, scale=0.3), 24)])
# C: sixteen heads on a cache row of 112 + 16 = 128 elements with a window wider than the test sequences (the tcgen05 prefill
#    kernel in bfloat16), no window at all on the next, a gated latent attention with a row of 64
TINY_NC = _model(96, 131, 1e-5, 0.5, 9.0, [
    _with(_la2(16, 16, 16, 24, 112, window=300, q_rank=40, scaling={"factor": 2.0, "original": 64, "fast": 16.0, "slow": 2.0}), 64),
    _with(_la2(4, 24, 8, 16, 56, window=None, q_rank=None, scaling=YARN), None),
    _with(_gla(2, 32, 64, 8.0, rank=32), 32),
    _with(_la(2, 32, 40, 64), 64),
    _with(_la2(5, 8, 16, 8, 32, window=33, q_rank=12), 32)])

CONFIGS_N = {"NA": TINY_NA, "NB": TINY_NB, "NC": TINY_NC}


def config_json(cfg: dict) -> dict:
    out = dict(cfg)
    out["layers"] = [{k: v for k, v in l.items() if not k.startswith("_")} for l in cfg["layers"]]
    return out


def tensor_shapes(cfg: dict) -> Dict[str, tuple]:
    E, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, E), "final.norm": (E,), "head": (V, E)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        out.update({p + "norm1": (E,), p + "norm1b": (E,)})
        if layer["type"] == "gla":
            Nk, Nv, R = m["heads"] * m["dim"], m["heads"] * m["vdim"], layer["_rank"]
            out.update({p + "mix.q": (Nk, E), p + "mix.k": (Nk, E), p + "mix.v": (Nv, E), p + "mix.g": (Nv, E), p + "mix.o": (E, Nv),
                        p + "mix.norm": (m["vdim"],), p + "mix.a1": (R, E), p + "mix.a2": (Nk, R), p + "mix.a2.b": (Nk,)})
        else:
            H, rd, r = m["heads"], m.get("rot_dim", 0), m["kv_rank"]
            qd = H * (m["dim"] + rd)
            if m.get("q_rank"):
                out.update({p + "mix.dq": (m["q_rank"], E), p + "mix.dq.norm": (m["q_rank"],), p + "mix.uq": (qd, m["q_rank"])})
            else:
                out[p + "mix.q"] = (qd, E)
            out.update({p + "mix.dkv": (r + rd, E), p + "mix.dkv.norm": (r,), p + "mix.uk": (H * m["dim"], r),
                        p + "mix.uv": (H * m["vdim"], r), p + "mix.o": (E, H * m["vdim"])})
            if layer["type"] == "latent_attention":
                out[p + "mix.g"] = (H * m["vdim"], E)
        if layer["mlp"] is not None:
            ff = layer["mlp"]["ff"]
            out.update({p + "mlp.gate": (ff, E), p + "mlp.up": (ff, E), p + "mlp.down": (E, ff)})
            out.update({p + "norm2": (E,), p + "norm2b": (E,)})
    return out


def make_weights(cfg: dict, seed: int) -> Dict[str, torch.Tensor]:
    """bfloat16 tensors by checkpoint name."""
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
        g = torch.Generator(device="cpu").manual_seed(int.from_bytes(h[:7], "little"))
        r = torch.randn(shape, generator=g, dtype=torch.float32)
        if name.endswith(".a2.b"):
            t = 1.0 + 2.0 * r                     # decays from nearly none to strong
        elif len(shape) == 1:
            t = 1.0 + 0.1 * r                     # norm weights
        elif name == "embed":
            t = 0.5 * r
        elif name.endswith(".uq") or name.endswith(".uk"):
            t = 2.0 * r / math.sqrt(shape[1])     # scores spread enough for the softmax to prefer some keys
        else:
            t = r / math.sqrt(shape[1])           # a projection: outputs about as large as its inputs
        out[name] = t.to(torch.bfloat16)
    return out
