"""Vekurax: typed configuration and model description.

A decoder whose layers are listed one by one in config.json (`layers`): every entry names the kind of its
mixer (`type`), the mixer's sizes and constants (`mixer`) and its feed-forward (`mlp`, or null for none).  An
entry with `weights_of: j` is another run of layer j's weights with a cache and state of its own.  The one
kind of layer so far, "parallel", norms the stream once with a Dynamic-Tanh norm and lets a mixer and a gated
feed-forward read that output side by side; its mixer is a weighted pair of a windowed softmax attention
(short convolution on q and k, whole-projection RMS norm, values = keys, distance bias, kept first tokens,
one output gate per head) and a linear attention with a fixed decay per head.  The output head is the
embedding table.  Everything that differs between models of the design is read here; nothing else in the
engine knows the design's name.
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
class VekuraxLayer:
    type: str
    mixer: Dict[str, Any]
    mlp: Optional[Dict[str, Any]]
    weights_of: Optional[int]


@dataclasses.dataclass
class VekuraxConfig:
    width: int
    vocab: int
    norm_eps: float
    layers: List[VekuraxLayer]
    max_context_len: int = DEFAULT_MAX_CONTEXT
    eos_token_ids: List[int] = dataclasses.field(default_factory=list)
    raw: Dict[str, Any] = dataclasses.field(default_factory=dict, repr=False)

    @classmethod
    def from_dict(cls, raw: Dict[str, Any]) -> "VekuraxConfig":
        layers = []
        for i, entry in enumerate(_need(raw, "layers", "the model")):
            where = f"layer {i}"
            wo = entry.get("weights_of")
            layers.append(VekuraxLayer(type=str(_need(entry, "type", where)), mixer=dict(_need(entry, "mixer", where)),
                                       mlp=dict(entry["mlp"]) if entry.get("mlp") is not None else None,
                                       weights_of=int(wo) if wo is not None else None))
        eos = raw.get("eos_token_id", [])
        eos = [] if eos is None else ([int(e) for e in eos] if isinstance(eos, (list, tuple)) else [int(eos)])
        cfg = cls(width=int(_need(raw, "width", "the model")), vocab=int(_need(raw, "vocab", "the model")),
                  norm_eps=float(_need(_need(raw, "norm", "the model"), "eps", "norm")), layers=layers,
                  max_context_len=int(raw.get("max_context_len", DEFAULT_MAX_CONTEXT)), eos_token_ids=eos, raw=dict(raw))
        cfg.check()
        return cfg

    def owner(self, i: int) -> int:
        """The layer whose tensors layer i uses (itself, unless it is another run of an earlier layer's weights)."""
        seen = set()
        while self.layers[i].weights_of is not None:
            if i in seen:
                raise ConfigError(f"config.json: the weights_of entries from layer {i} on form a circle")
            seen.add(i)
            i = self.layers[i].weights_of
        return i

    def check(self) -> None:
        if self.width <= 0 or self.vocab <= 0 or not self.layers:
            raise ConfigError("width, vocab and the number of layers must be positive")
        for i, l in enumerate(self.layers):
            if l.weights_of is not None and not 0 <= l.weights_of < len(self.layers):
                raise ConfigError(f"config.json: layer {i} names weights_of {l.weights_of}, the model has {len(self.layers)} layers")
            self.owner(i)
            if l.type not in _MIXERS:
                raise ConfigError(f"config.json: layer {i} has type {l.type!r}; known: " + ", ".join(sorted(_MIXERS)))
            if l.mlp is not None and l.mlp.get("kind") != "dense":
                raise ConfigError(f"config.json: layer {i} has a feed-forward of kind {l.mlp.get('kind')!r}; known: dense")

    def to_dict(self) -> Dict[str, Any]:
        return dict(self.raw)


def _pair_mixer(cfg: VekuraxConfig, m: Dict[str, Any], where: str) -> PartSpec:
    """The "parallel" mixer: left_scale * windowed attention + right_scale * decaying linear attention."""
    lf, rt = _need(m, "left", where), _need(m, "right", where)
    mask = _need(lf, "mask", where + ".left")
    dim = int(_need(lf, "dim", where + ".left"))
    if int(lf.get("vdim", dim)) != dim:
        raise ConfigError(f"config.json: {where}.left: the values are the keys, so vdim must equal dim")
    heads = int(_need(lf, "heads", where + ".left"))
    left = PartSpec("conv_window_attention", {
        "hidden_size": cfg.width, "num_heads": heads, "num_kv_heads": int(lf.get("kv_heads") or heads), "head_dim": dim,
        "scale": float(_need(lf, "scale", where + ".left")), "conv_taps": int(_need(lf, "conv", where + ".left")),
        "norm_eps": cfg.norm_eps, "window": int(_need(mask, "size", where + ".left.mask")),
        "keep_first": int(mask.get("keep_first", 0)), "bias_far": float(_need(lf, "bias_max", where + ".left")),
        "max_positions": cfg.max_context_len,
        "names": {"q": "q", "k": "k", "q_norm": "q.norm", "k_norm": "k.norm", "q_conv": "q.conv", "k_conv": "k.conv",
                  "bias": "rel", "gate": "g", "out": "o"}})
    decay = [float(x) for x in _need(rt, "decay", where + ".right")]
    r_heads = int(_need(rt, "heads", where + ".right"))
    if len(decay) != r_heads:
        raise ConfigError(f"config.json: {where}.right: {len(decay)} decays for {r_heads} heads")
    right = PartSpec("decay_linear_attention", {
        "hidden_size": cfg.width, "num_heads": r_heads, "key_dim": int(_need(rt, "dim", where + ".right")),
        "value_dim": int(_need(rt, "vdim", where + ".right")), "decay": decay, "norm_eps": cfg.norm_eps,
        "names": {"q": "q", "k": "k", "v": "v", "gate": "g", "out": "o", "norm": "norm"}})
    return PartSpec("weighted_pair", {"hidden_size": cfg.width, "first": left, "second": right,
                                      "first_scale": float(_need(m, "left_scale", where)),
                                      "second_scale": float(_need(m, "right_scale", where)),
                                      "first_name": "left", "second_name": "right"})


_MIXERS = {"parallel": _pair_mixer}
VEKURAX_LAYER_NAMES = {"input": "norm1", "mixer": "mix", "feed_forward": "mlp"}


def build_vekurax_spec(cfg: VekuraxConfig) -> ModelSpec:
    """embed -> runs of (one norm; mixer and feed-forward side by side; sum) -> norm -> the embedding as head.
    Layers that own tensors become the model's layers; every entry of config.json's list is one run, in order, with
    a cache id of its own."""
    owners = sorted({cfg.owner(i) for i in range(len(cfg.layers))})
    index = {o: k for k, o in enumerate(owners)}
    layers = []
    for o in owners:
        l = cfg.layers[o]
        norm = PartSpec("dynamic_tanh", {"size": cfg.width, "name": f"l{o}.norm1"})
        ffn = None
        if l.mlp is not None:
            ffn = PartSpec("gated_mlp", {"hidden_size": cfg.width, "intermediate_size": int(_need(l.mlp, "ff", f"layer {o}.mlp")),
                                         "activation": "gelu_tanh", "names": {"gate": "gate", "up": "up", "down": "down"}})
        layers.append(LayerSpec(prefix=f"l{o}", mixer=_MIXERS[l.type](cfg, l.mixer, f"layer {o}.mixer"), feed_forward=ffn,
                                norms={"input": norm}, position=None, block="parallel_shared_norm",
                                names=VEKURAX_LAYER_NAMES))
    return ModelSpec(
        architecture="Vekurax", hidden_size=cfg.width, vocab_size=cfg.vocab,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "name": "embed"}),
        final_norm=PartSpec("dynamic_tanh", {"size": cfg.width, "name": "final.norm"}),
        head=PartSpec("lm_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.width, "tied": True, "name": "head",
                                  "tied_to": "embed"}),
        layers=layers,
        schedule=[Run(layer=index[cfg.owner(i)], cache=i) for i in range(len(cfg.layers))],
        max_context_len=cfg.max_context_len, eos_token_ids=list(cfg.eos_token_ids), checkpoint_dtype="bfloat16")


register_architecture("Vekurax", VekuraxConfig, build_vekurax_spec)
