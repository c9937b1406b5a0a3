"""Typed configuration of the Vadodra decoder, read from config.json.

config.json gives every size and every constant that can differ between models of the design:

    {"architecture": "Vadodra", "vocab": V, "width": D, "norm": {"eps": e}, "embedding": {"scale": s},
     "layers": [{"type": "attention",
                 "mixer": {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size"},
                           "rot": {"base", "dims", "scaling": {"factor"}}},
                 "mlp": null | {"kind": "dense", "ff", "limit"}},
                {"type": "latent_attention",
                 "mixer": {"heads", "dim", "rot_dim", "vdim", "kv_rank", "scale", "rot": {"base", "dims"},
                           "kv_from": j (optional: the layer reads layer j's cached latent)},
                 "mlp": ...},
                ...]}

Sizes and constants have no defaults: a missing key is an error that names it.  Optional are only the
things a layer may lack: `mask` (no window: every earlier position is visible), `rot.scaling`, `kv_from`, `mlp`.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Mapping

from .lulisun_config import _float, _get, _int
from .model_config import ConfigError

ARCHITECTURE = "Vadodra"


@dataclass(frozen=True)
class RotaryConfig:
    base: float
    dims: int                # rotated channels (the first ones of the rotated vector)
    factor: float            # every frequency is divided by it (1: no scaling)


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int                 # size of a query / key head; the values are the unrotated keys, so also theirs
    vdim: int
    scale: float
    window: int | None       # a query sees itself and the window - 1 positions before it (None: all)
    rot: RotaryConfig


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int                 # unrotated query / key channels of a head
    rot_dim: int             # rotated ones (the key's are shared by the heads)
    vdim: int
    kv_rank: int
    scale: float
    rot: RotaryConfig
    kv_from: int | None      # the layer whose cached latent this one reads (None: its own)


@dataclass(frozen=True)
class DenseMlpConfig:
    ff: int
    limit: float


@dataclass(frozen=True)
class VadodraLayerConfig:
    kind: str                # "attention" | "latent_attention"
    mixer: Any
    mlp: DenseMlpConfig | None
    raw: Any = None


def _rot(d: Mapping, where: str) -> RotaryConfig:
    r = _get(d, "rot", where)
    w = where + ".rot"
    dims = _int(r, "dims", w, minimum=2)
    if dims % 2:
        raise ConfigError(f"config.json: {w}.dims {dims} must be even")
    factor = 1.0
    if r.get("scaling") is not None:
        factor = _float(r["scaling"], "factor", w + ".scaling")
        if not factor > 0:
            raise ConfigError(f"config.json: {w}.scaling.factor must be positive, found {factor}")
    base = _float(r, "base", w)
    if not base > 0:
        raise ConfigError(f"config.json: {w}.base must be positive, found {base}")
    return RotaryConfig(base=base, dims=dims, factor=factor)


@dataclass(frozen=True)
class VadodraConfig:
    architecture: str
    vocab_size: int
    hidden_size: int
    norm_eps: float
    embedding_scale: float
    layers: tuple
    raw: Any = None

    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "VadodraConfig":
        entries = _get(d, "layers", "the model")
        if not isinstance(entries, (list, tuple)) or not entries:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, entry in enumerate(entries):
            where = f"layers[{i}]"
            kind = _get(entry, "type", where)
            m = _get(entry, "mixer", where)
            mw = where + ".mixer"
            if kind == "attention":
                mask = m.get("mask")
                a = WindowAttentionConfig(
                    heads=_int(m, "heads", mw), kv_heads=_int(m, "kv_heads", mw), dim=_int(m, "dim", mw),
                    vdim=_int(m, "vdim", mw), scale=_float(m, "scale", mw),
                    window=None if mask is None else _int(mask, "size", mw + ".mask"), rot=_rot(m, mw))
                if a.heads % a.kv_heads:
                    raise ConfigError(f"config.json: {mw}: {a.heads} heads are not a multiple of {a.kv_heads} kv heads")
                if a.vdim != a.dim:
                    raise ConfigError(f"config.json: {mw}: the values are the keys, so vdim {a.vdim} must equal dim {a.dim}")
                if a.rot.dims > a.dim:
                    raise ConfigError(f"config.json: {mw}.rot.dims {a.rot.dims} exceeds dim {a.dim}")
                mixer = a
            elif kind == "latent_attention":
                src = m.get("kv_from")
                a = LatentAttentionConfig(
                    heads=_int(m, "heads", mw), dim=_int(m, "dim", mw), rot_dim=_int(m, "rot_dim", mw, minimum=2),
                    vdim=_int(m, "vdim", mw), kv_rank=_int(m, "kv_rank", mw), scale=_float(m, "scale", mw),
                    rot=_rot(m, mw), kv_from=src)
                if a.rot.dims > a.rot_dim:
                    raise ConfigError(f"config.json: {mw}.rot.dims {a.rot.dims} exceeds rot_dim {a.rot_dim}")
                if src is not None:
                    if isinstance(src, bool) or not isinstance(src, int) or not 0 <= src < i:
                        raise ConfigError(f"config.json: {mw}.kv_from {src!r} must name an earlier layer")
                    owner = layers[src]
                    o = owner.mixer
                    if owner.kind != "latent_attention" or o.kv_from is not None:
                        raise ConfigError(f"config.json: {mw}.kv_from {src}: that layer keeps no latent of its own")
                    if (o.kv_rank, o.rot_dim, o.rot) != (a.kv_rank, a.rot_dim, a.rot):
                        raise ConfigError(f"config.json: {mw}.kv_from {src}: kv_rank, rot_dim and rot must equal that layer's")
                mixer = a
            else:
                raise ConfigError(f"config.json: {where}.type {kind!r} is not a mixer of this design "
                                  "(have: 'attention', 'latent_attention')")
            mlp = entry.get("mlp")
            ff = None
            if mlp is not None:
                fw = where + ".mlp"
                if _get(mlp, "kind", fw) != "dense":
                    raise ConfigError(f"config.json: {fw}.kind {mlp['kind']!r} is not a feed-forward of this design (have: 'dense')")
                ff = DenseMlpConfig(ff=_int(mlp, "ff", fw), limit=_float(mlp, "limit", fw))
                if not ff.limit > 0:
                    raise ConfigError(f"config.json: {fw}.limit must be positive, found {ff.limit}")
            layers.append(VadodraLayerConfig(kind, mixer, ff, raw=entry))
        eps = _float(_get(d, "norm", "the model"), "eps", "norm")
        if eps <= 0:
            raise ConfigError("config.json: norm.eps must be positive")
        return cls(architecture=ARCHITECTURE, vocab_size=_int(d, "vocab", "the model"),
                   hidden_size=_int(d, "width", "the model"), norm_eps=eps,
                   embedding_scale=_float(_get(d, "embedding", "the model"), "scale", "embedding"),
                   layers=tuple(layers), raw=dict(d))

    def to_dict(self) -> dict:
        """The config.json form."""
        def rot(r: RotaryConfig) -> dict:
            out = {"base": r.base, "dims": r.dims}
            if r.factor != 1.0:
                out["scaling"] = {"factor": r.factor}
            return out

        layers = []
        for L in self.layers:
            a = L.mixer
            if L.kind == "attention":
                mixer = {"heads": a.heads, "kv_heads": a.kv_heads, "dim": a.dim, "vdim": a.vdim, "scale": a.scale,
                         "rot": rot(a.rot)}
                if a.window is not None:
                    mixer["mask"] = {"size": a.window}
            else:
                mixer = {"heads": a.heads, "dim": a.dim, "rot_dim": a.rot_dim, "vdim": a.vdim, "kv_rank": a.kv_rank,
                         "scale": a.scale, "rot": rot(a.rot)}
                if a.kv_from is not None:
                    mixer["kv_from"] = a.kv_from
            layers.append({"type": L.kind, "mixer": mixer,
                           "mlp": None if L.mlp is None else {"kind": "dense", "ff": L.mlp.ff, "limit": L.mlp.limit}})
        return {"architecture": self.architecture, "vocab": self.vocab_size, "width": self.hidden_size,
                "norm": {"eps": self.norm_eps}, "embedding": {"scale": self.embedding_scale}, "layers": layers}
