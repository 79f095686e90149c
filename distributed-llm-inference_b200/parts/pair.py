"""Two mixers side by side on the same input."""

from __future__ import annotations

import dataclasses

from ..cache.needs import needs_of, state_needs_of
from .base import Part, WeightedPair, build_part, register_part


@register_part("mixer", "weighted_pair")
class WeightedPairMixer(Part):
    """first_scale * first(x) + second_scale * second(x): two mixers read the same input; each keeps a cache or state of its
    own kind in the same run step (at most one of them pages).  The sum is left to whoever adds the result to the stream
    (``WeightedPair``), where it is formed in float32.
    params: first, second (PartSpecs of mixers), first_scale, second_scale."""

    graph_capturable = True

    def __init__(self, spec, env) -> None:
        super().__init__(spec, env)
        p = spec.params
        self.first = build_part("mixer", p["first"], env)
        self.second = build_part("mixer", p["second"], env)
        self.fa, self.fb = float(p["first_scale"]), float(p["second_scale"])
        if not (self.first.graph_capturable and self.second.graph_capturable):
            self.graph_capturable = False
        self._first_states = len(state_needs_of(self.first.cache_need()))

    def children(self):
        return [self.first, self.second]

    def cache_need(self):
        return needs_of(self.first.cache_need()) + needs_of(self.second.cache_need())

    def forward(self, x, batch, cache):
        n = self._first_states
        a = self.first.forward(x, batch, dataclasses.replace(cache, states=cache.states[:n]))
        b = self.second.forward(x, batch, dataclasses.replace(cache, states=cache.states[n:]))
        return WeightedPair(a, self.fa, b, self.fb)
