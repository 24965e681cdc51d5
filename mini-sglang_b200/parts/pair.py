from __future__ import annotations

from typing import Dict

import torch

from ..weights.loader import TensorDecl
from .base import MIXERS, Mixer, Projected, build_part, register_mixer


@register_mixer("weighted_pair")
class WeightedPair(Mixer, Projected):
    """Two mixers side by side on the same input: first_scale * first(x) + second_scale * second(x).

    Both are `Projected` parts, so their input projections are one product and their output projections another: the
    scales go onto what enters the output product.  What each keeps between steps is kept side by side too: the pair
    declares the needs of the first followed by those of the second.

    params: hidden_size, first, second (PartSpecs of registered mixers), first_scale, second_scale, first_name, second_name
            (what the checkpoint calls them below the pair's prefix).
    """

    def __init__(self, spec, prefix, env, position=None):
        super().__init__(spec, prefix, env)
        self.subs = []
        for which in ("first", "second"):
            part = build_part(MIXERS, "mixer", spec[which], self.name(spec.get(which + "_name", which)), env, position=position)
            if not isinstance(part, Projected):
                raise ValueError(f"a weighted pair takes mixers that are given by their projections; {spec[which].kind!r} is not")
            self.subs.append(part)
        self.scales = [float(spec.get("first_scale", 1.0)), float(spec.get("second_scale", 1.0))]
        self.graph_safe = all(p.graph_safe for p in self.subs)
        self.w_in = self.w_out = None
        self._needs = []
        for p in self.subs:
            need = p.cache_need()
            self._needs.append(() if need is None else (need if isinstance(need, tuple) else (need,)))

    def tensors(self) -> Dict[str, TensorDecl]:
        out: Dict[str, TensorDecl] = {}
        for p in self.subs:
            out.update(p.tensors())
        return out

    def load(self, src) -> None:
        for p in self.subs:
            p.load(src)
        self.w_in = torch.cat([p.in_weight() for p in self.subs], dim=0).contiguous()
        self.w_out = torch.cat([p.out_weight() for p in self.subs], dim=1).contiguous()
        self.in_widths = [p.in_weight().shape[0] for p in self.subs]
        self.mid_widths = [p.out_weight().shape[1] for p in self.subs]

    def in_weight(self):
        return self.w_in

    def out_weight(self):
        return self.w_out

    def cache_need(self):
        needs = tuple(n for ns in self._needs for n in ns)
        return needs if needs else None

    def middle(self, proj, act, ctx, cache=None, writes_cache=True, out_scale=1.0):
        caches = tuple(cache) if isinstance(cache, tuple) else ((cache,) if cache is not None else ())
        a = m = c = 0
        for p, scale, ns, wi, wm in zip(self.subs, self.scales, self._needs, self.in_widths, self.mid_widths):
            mine = caches[c:c + len(ns)]
            sub_cache = None if not ns else (mine if isinstance(p.cache_need(), tuple) else mine[0])
            p.middle(proj[:, a:a + wi], act[:, m:m + wm], ctx, sub_cache, writes_cache, out_scale * scale)
            a, m, c = a + wi, m + wm, c + len(ns)

    def forward(self, x, ctx, cache, writes_cache: bool = True):
        return self.forward_projected(x, ctx, cache, writes_cache)
