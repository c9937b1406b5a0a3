"""Typed configuration of the Lulisun decoder, read from config.json.

config.json gives every size and every constant that can differ between models of the design:

    {"architecture": "Lulisun", "vocab": V, "width": D, "norm": {"eps": e},
     "layers": [{"type": "parallel",
                 "mixer": {"left":  {"heads", "kv_heads", "dim", "vdim", "scale",
                                     "mask": {"size"}, "rot": {"base", "dims"}},
                           "right": {"heads", "dim", "vdim"},
                           "left_scale", "right_scale"},
                 "mlp": null | {"kind": "moe", "expert": {"ff"},
                                "router": {"experts", "top", "groups": {"count", "keep"}},
                                "shared": {"ff"}},
                 "weights_of": j (optional: the layer runs layer j's tensors with a cache of its own)},
                ...]}

Nothing has a default: a missing key is an error that names it.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .model_config import ConfigError

ARCHITECTURE = "Lulisun"


def _get(d: Mapping, key: str, where: str):
    if not isinstance(d, Mapping) or key not in d or d[key] is None:
        raise ConfigError(f"config.json: {where} lacks '{key}'")
    return d[key]


def _int(d: Mapping, key: str, where: str, minimum: int = 1) -> int:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, int) or v < minimum:
        raise ConfigError(f"config.json: {where}.{key} must be an integer >= {minimum}, found {v!r}")
    return v


def _float(d: Mapping, key: str, where: str) -> float:
    v = _get(d, key, where)
    if isinstance(v, bool) or not isinstance(v, (int, float)):
        raise ConfigError(f"config.json: {where}.{key} must be a number, found {v!r}")
    return float(v)


@dataclass(frozen=True)
class ChunkedAttentionConfig:
    heads: int
    kv_heads: int
    dim: int                 # size of a query / key head
    vdim: int                # size of a value head
    scale: float             # on the scores
    chunk: int               # positions per block of mutually visible tokens
    rot_base: float
    rot_dims: int            # rotated channels of a head (the first ones)


@dataclass(frozen=True)
class RecurrenceConfig:
    heads: int
    dim: int
    vdim: int


@dataclass(frozen=True)
class RoutedExpertsConfig:
    experts: int
    top: int
    expert_ff: int
    groups: int
    keep: int
    shared_ff: int | None


@dataclass(frozen=True)
class LulisunLayerConfig:
    left: ChunkedAttentionConfig
    right: RecurrenceConfig
    left_scale: float
    right_scale: float
    mlp: RoutedExpertsConfig | None
    weights_of: int | None
    raw: Any = None          # the entry as config.json gives it


@dataclass(frozen=True)
class LulisunConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    layers: tuple
    raw: Any = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "LulisunConfig":
        entries = _get(d, "layers", "the model")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            kind = _get(entry, "type", where)
            if kind != "parallel":
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design (have: 'parallel')")
            mixer = _get(entry, "mixer", where)
            left, right = _get(mixer, "left", where + ".mixer"), _get(mixer, "right", where + ".mixer")
            lw, rw = where + ".mixer.left", where + ".mixer.right"
            a = ChunkedAttentionConfig(
                heads=_int(left, "heads", lw), kv_heads=_int(left, "kv_heads", lw), dim=_int(left, "dim", lw),
                vdim=_int(left, "vdim", lw), scale=_float(left, "scale", lw),
                chunk=_int(_get(left, "mask", lw), "size", lw + ".mask"),
                rot_base=_float(_get(left, "rot", lw), "base", lw + ".rot"),
                rot_dims=_int(_get(left, "rot", lw), "dims", lw + ".rot", minimum=2))
            if a.heads % a.kv_heads:
                raise ConfigError(f"config.json: {lw}: {a.heads} heads are not a multiple of {a.kv_heads} kv heads")
            if a.rot_dims % 2 or a.rot_dims > a.dim:
                raise ConfigError(f"config.json: {lw}.rot.dims {a.rot_dims} must be even and at most dim {a.dim}")
            r = RecurrenceConfig(heads=_int(right, "heads", rw), dim=_int(right, "dim", rw), vdim=_int(right, "vdim", rw))
            mlp = entry.get("mlp")
            m = None
            if mlp is not None:
                mw = where + ".mlp"
                if _get(mlp, "kind", mw) != "moe":
                    raise ConfigError(f"config.json: {mw}.kind {mlp['kind']!r} is not a feed-forward of this design (have: 'moe')")
                router = _get(mlp, "router", mw)
                groups = router.get("groups")
                shared = mlp.get("shared")
                m = RoutedExpertsConfig(
                    experts=_int(router, "experts", mw + ".router"), top=_int(router, "top", mw + ".router"),
                    expert_ff=_int(_get(mlp, "expert", mw), "ff", mw + ".expert"),
                    groups=1 if groups is None else _int(groups, "count", mw + ".router.groups"),
                    keep=1 if groups is None else _int(groups, "keep", mw + ".router.groups"),
                    shared_ff=None if shared is None else _int(shared, "ff", mw + ".shared"))
                if m.experts % m.groups or m.keep > m.groups or m.keep * (m.experts // m.groups) < m.top or m.top > m.experts:
                    raise ConfigError(f"config.json: {mw}.router: {m.experts} experts in {m.groups} groups, {m.keep} kept, "
                                      f"cannot give {m.top} choices")
            of = entry.get("weights_of")
            seen = {i}
            while of is not None:                 # a layer may name one that itself runs another's tensors: follow to the owner
                if isinstance(of, bool) or not isinstance(of, int) or not 0 <= of < len(entries) or of in seen:
                    raise ConfigError(f"config.json: {where}.weights_of {entry.get('weights_of')!r} names no other layer "
                                      "with tensors of its own")
                if entries[of].get("weights_of") is None:
                    break
                seen.add(of)
                of = entries[of].get("weights_of")
            layers.append(LulisunLayerConfig(a, r, _float(mixer, "left_scale", where + ".mixer"),
                                             _float(mixer, "right_scale", where + ".mixer"), m, of, raw=entry))
        eps = _float(_get(d, "norm", "the model"), "eps", "norm")
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        return cls(architecture=ARCHITECTURE, vocab_size=_int(d, "vocab", "the model"),
                   hidden_size=_int(d, "width", "the model"), norm_eps=eps, layers=tuple(layers), raw=dict(d))

    def to_dict(self) -> dict:
        """The config.json form."""
        layers = []
        for L in self.layers:
            a, r, m = L.left, L.right, L.mlp
            entry = {"type": "parallel", "mixer": {
                "left": {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale,
                         "mask": {"size": a.chunk}, "rot": {"base": a.rot_base, "dims": a.rot_dims}},
                "right": {"heads": r.heads, "dim": r.dim, "vdim": r.vdim},
                "left_scale": L.left_scale, "right_scale": L.right_scale}}
            entry["mlp"] = None if m is None else {
                "kind": "moe", "expert": {"ff": m.expert_ff},
                "router": {"experts": m.experts, "top": m.top, "groups": {"count": m.groups, "keep": m.keep}},
                "shared": None if m.shared_ff is None else {"ff": m.shared_ff}}
            if L.weights_of is not None:
                entry["weights_of"] = L.weights_of
            layers.append(entry)
        return {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                "norm": {"eps": self.norm_eps}, "layers": layers}
