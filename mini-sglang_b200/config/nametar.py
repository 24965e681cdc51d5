"""Nametar: typed configuration and model description.

A decoder whose layers are listed one by one in config.json (`layers`): every entry names the kind of its mixer (`type`),
the mixer's sizes and constants (`mixer`) and its feed-forward (`mlp`, or null for none).  The embedding is scaled by a
constant; every sublayer has an RMS norm before and after it, and what it adds to the float32 stream is multiplied by one
constant of the model (`residual_mult`).  Mixers:

  latent_attention     softmax attention from one low-rank key/value latent per token, no positions, all earlier keys, the
                       heads' outputs times a sigmoid gate
  latent_attention_2   the same kind with a query latent, a rotated key part shared by all heads (rotary encoding in halves
                       with YaRN's frequency scaling) and a sliding window
  gla                  linear attention with a decay per token and key channel made from the input

The feed-forward is down(silu(gate x) * up x).  The head is a matrix of its own.  Everything that differs between models of
the design is read here; nothing else in the engine knows the design's name.
"""

from __future__ import annotations

import dataclasses
from typing import Any, Dict, List, Optional

from .registry import ConfigError, register_architecture
from .spec import LayerSpec, ModelSpec, PartSpec, Run

DEFAULT_MAX_CONTEXT = 1 << 20       # the design has no position table: the engine's own limit bounds a request


def _need(d: Dict[str, Any], key: str, where: str):
    if not isinstance(d, dict) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} has no {key!r}")
    return d[key]


@dataclasses.dataclass
class NametarLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]


@dataclasses.dataclass
class NametarConfig:
    width: int
    vocab: int
    norm_eps: float
    residual_mult: float
    embedding_scale: float
    layers: List[NametarLayer]
    max_context_len: int = DEFAULT_MAX_CONTEXT
    eos_token_ids: List[int] = dataclasses.field(default_factory=list)
    raw: Dict[str, Any] = dataclasses.field(default_factory=dict, repr=False)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "NametarConfig":
        layers = []
        for i, entry in enumerate(_need(raw, "layers", "the model")):
            where = f"layer {i}"
            layers.append(NametarLayer(type=str(_need(entry, "type", where)), mixer=dict(_need(entry, "mixer", where)),
                                       mlp=dict(entry["mlp"]) if entry.get("mlp") is not None else None))
        eos = raw.get("eos_token_id", [])
        eos = [] if eos is None else ([int(e) for e in eos] if isinstance(eos, (list, tuple)) else [int(eos)])
        emb = raw.get("embedding") or {}
        cfg = cls(width=int(_need(raw, "width", "the model")), vocab=int(_need(raw, "vocab", "the model")),
                  norm_eps=float(_need(_need(raw, "norm", "the model"), "eps", "norm")),
                  residual_mult=float(raw.get("residual_mult", 1.0)), embedding_scale=float(emb.get("scale", 1.0)),
                  layers=layers, max_context_len=int(raw.get("max_context_len", DEFAULT_MAX_CONTEXT)), eos_token_ids=eos,
                  raw=dict(raw))
        cfg.check()
        return cfg

    def check(self) -> None:
        if self.width <= 0 or self.vocab <= 0 or not self.layers:
            raise ConfigError("width, vocab and the number of layers must be positive")
        for i, l in enumerate(self.layers):
            if l.type not in _MIXERS:
                raise ConfigError(f"config.json: layer {i} has type {l.type!r}; known: " + ", ".join(sorted(_MIXERS)))
            if l.mlp is not None and l.mlp.get("kind") != "dense":
                raise ConfigError(f"config.json: layer {i} has a feed-forward of kind {l.mlp.get('kind')!r}; known: dense")

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)


def _latent(cfg: NametarConfig, m: Dict[str, Any], where: str, gate: Optional[str]):
    """-> (mixer, position encoding or None) of a latent attention.  A query latent, a rotated part and a window are there
    when the entry gives their sizes (`q_rank`, `rot_dim` with `rot`, `mask.size`)."""
    rot_dim = int(m.get("rot_dim") or 0)
    position = None
    if rot_dim:
        rot = _need(m, "rot", where)
        dims = int(rot.get("dims", rot_dim))
        if dims > rot_dim or dims % 2:
            raise ConfigError(f"config.json: {where}.rot: {dims} rotated dimensions must be even and at most rot_dim = {rot_dim}")
        sc = rot.get("scaling")
        scaling = None
        if sc:
            scaling = {k: float(_need(sc, k, where + ".rot.scaling")) for k in ("factor", "original", "fast", "slow")}
        position = PartSpec("rope_yarn", {"rotary_dim": dims, "theta": float(_need(rot, "base", where + ".rot")), "scaling": scaling})
    mask = m.get("mask") or {}
    mixer = PartSpec("latent_attention", {
        "hidden_size": cfg.width, "num_heads": int(_need(m, "heads", where)), "key_dim": int(_need(m, "dim", where)),
        "rot_dim": rot_dim, "value_dim": int(_need(m, "vdim", where)), "kv_rank": int(_need(m, "kv_rank", where)),
        "q_rank": int(m["q_rank"]) if m.get("q_rank") else None, "scale": float(_need(m, "scale", where)),
        "window": int(mask["size"]) if mask.get("size") else None, "gate": gate, "norm_eps": cfg.norm_eps})
    return mixer, position


def _latent_gated(cfg, m, where):
    return _latent(cfg, m, where, "sigmoid")


def _latent_plain(cfg, m, where):
    return _latent(cfg, m, where, None)


def _gla(cfg: NametarConfig, m: Dict[str, Any], where: str):
    return PartSpec("gated_linear_attention", {
        "hidden_size": cfg.width, "num_heads": int(_need(m, "heads", where)), "key_dim": int(_need(m, "dim", where)),
        "value_dim": int(_need(m, "vdim", where)), "tau": float(_need(m, "tau", where)), "norm_eps": cfg.norm_eps,
        "decay_rank": int(m.get("decay_rank", 16))}), None


_MIXERS = {"latent_attention": _latent_gated, "latent_attention_2": _latent_plain, "gla": _gla}
NAMETAR_LAYER_NAMES = {"mixer": "mix", "feed_forward": "mlp"}


def build_nametar_spec(cfg: NametarConfig) -> ModelSpec:
    """scaled embedding -> layers of (norm, mixer, norm, scaled sum; norm, feed-forward, norm, scaled sum) -> norm -> head;
    every entry of config.json's list is one layer with tensors `l<i>.*` and one run with a cache of its own."""
    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", {"size": cfg.width, "eps": cfg.norm_eps, "name": name})

    layers = []
    for i, l in enumerate(cfg.layers):
        mixer, position = _MIXERS[l.type](cfg, l.mixer, f"layer {i}.mixer")
        norms = {"input": norm(f"l{i}.norm1"), "mixer_out": norm(f"l{i}.norm1b")}
        ffn = None
        if l.mlp is not None:
            ffn = PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": int(_need(l.mlp, "ff", f"layer {i}.mlp")),
                                         "activation": "silu", "names": {"gate": "gate", "up": "up", "down": "down"}})
            norms.update({"ffn_in": norm(f"l{i}.norm2"), "ffn_out": norm(f"l{i}.norm2b")})
        layers.append(LayerSpec(prefix=f"l{i}", mixer=mixer, feed_forward=ffn, norms=norms, position=position,
                                block="sandwich_residual", names=NAMETAR_LAYER_NAMES,
                                block_params={"residual_scale": cfg.residual_mult}))
    return ModelSpec(
        architecture="Nametar", hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "embed",
                                               "scale": cfg.embedding_scale}),
        final_norm=norm("final.norm"),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied": False, "name": "head"}),
        layers=layers, schedule=[Run(layer=i, cache=i) for i in range(len(cfg.layers))],
        max_context_len=cfg.max_context_len, eos_token_ids=list(cfg.eos_token_ids), checkpoint_dtype="bfloat16")


register_architecture("Nametar", NametarConfig, build_nametar_spec)
