"""Several mixers on the same input, their results summed with fixed factors."""
from __future__ import annotations

from .base import Mixer
from .registry import lookup, register
from .spec import PartSpec


@register("mixer", "parallel_mixers")
class ParallelMixers(Mixer):
    """residual += sum_m scale_m * mixer_m(x).  `members` lists (PartSpec, scale) pairs; a member's
    tensors sit below its spec's prefix, its factor is handed to it as `out_scale` (members apply it to
    their result in float32, before their output projection), and its cache is the member of the same
    place in the layer's composite cache request: an attention member keeps keys and values, a
    recurrent one a state, both in one cache layer."""

    def __init__(self, *, members, hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        self.members = []
        for spec, scale in members:
            if not isinstance(spec, PartSpec):
                raise TypeError("parallel_mixers: a member is a (PartSpec, scale) pair")
            part = lookup("mixer", spec.kind)(hidden_size=hidden_size, dtype=dtype, device=device,
                                              **dict(spec.params, out_scale=float(scale)))
            self.members.append((spec.prefix, part))
        if not self.members:
            raise ValueError("parallel_mixers: no members")
        self.graph_safe = all(getattr(p, "graph_safe", True) for _, p in self.members)

    def tensor_specs(self):
        out = {}
        for prefix, part in self.members:
            for local, ts in part.tensor_specs().items():
                if prefix + local in out:
                    raise ValueError(f"parallel_mixers: two members declare {prefix + local!r}")
                out[prefix + local] = ts
        return out

    def set_tensors(self, tensors):
        for prefix, part in self.members:
            part.set_tensors({local: tensors[prefix + local] for local in part.tensor_specs()})

    def get_tensors(self):
        return {prefix + local: t for prefix, part in self.members for local, t in part.get_tensors().items()}

    def prepare(self, max_positions):
        for _, part in self.members:
            part.prepare(max_positions)

    def cache_request(self):
        return tuple(part.cache_request() for _, part in self.members)

    def forward(self, x, residual, ctx, cache_layer, writes_cache):
        for (_, part), sub in zip(self.members, cache_layer.parts):
            part.forward(x, residual, ctx, sub, writes_cache)
