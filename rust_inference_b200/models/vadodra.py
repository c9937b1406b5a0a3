"""The Vadodra decoder as a `ModelSpec`.

Every layer is x <- x + (mixer(h) + ff(h)) with h = norm(x) (`parallel_shared_norm`): one layer norm with a
weight and no bias, whose output both branches read.  The mixer is either grouped-query softmax attention
over a sliding window whose values are the keys as projected (no value projection), with an RMS norm of
every query and key head before the rotation, interleaved rotary pairs on the first channels of a head and
linearly scaled positions (`gqa_attention` with `values_from_keys`, `qk_norm_eps`, `window`); or causal
attention over a low-rank latent shared by the heads, with an output gate per head (`latent_attention`),
which may read the latent another layer cached: that is the schedule.  The feed-forward is the bounded
gated form (`bounded_glu`) or absent.  The embedding's rows are scaled as they enter the stream; the head is
the embedding table itself, unscaled, after the model's norm.

Tensor names: `embed`, `l<i>.norm1`, `l<i>.mix.{q,k,q.norm,k.norm,o}` or
`l<i>.mix.{q,dkv,dkv.norm,uk,uv,g,o}`, `l<i>.mlp.{gate,up,down}`, `final.norm`.
"""
from __future__ import annotations

from ..config.vadodra_config import ARCHITECTURE, VadodraConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# the configuration gives no context length: positions are bounded by the cache a run is given
MAX_POSITIONS = 1 << 17

GATE_ALPHA, UP_SHIFT = 1.702, 1.0          # the design's constants of the gated feed-forward

_ATTENTION_NAMES = {"q": "q", "k": "k", "o": "o", "q_norm": "q.norm", "k_norm": "k.norm"}
_LATENT_NAMES = {"q": "q", "dkv": "dkv", "dkv_norm": "dkv.norm", "uk": "uk", "uv": "uv", "gate": "g", "o": "o"}
_MLP_NAMES = {"gate": "gate", "up": "up", "down": "down"}


def _norm(cfg: VadodraConfig, prefix: str) -> PartSpec:
    return PartSpec("layernorm", {"eps": cfg.norm_eps, "weight_name": ""}, prefix=prefix)


def build_spec(cfg: VadodraConfig) -> ModelSpec:
    layers, schedule = [], []
    for i, L in enumerate(cfg.layers):
        a = L.mixer
        if L.kind == "attention":
            rope = PartSpec("rope", {"head_dim": a.dim, "base": a.rot.base, "style": "interleaved", "rot_dims": a.rot.dims,
                                     "exact_angles": True, "scaling_factor": a.rot.factor})
            mixer = PartSpec("gqa_attention", {
                "n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim, "qkv_bias": False, "position": rope,
                "scale": a.scale, "window": a.window, "qk_norm_eps": cfg.norm_eps, "values_from_keys": True,
                "names": _ATTENTION_NAMES}, prefix="mix.")
            cache = i
        else:
            rope = PartSpec("rope", {"head_dim": a.rot_dim, "base": a.rot.base, "style": "half", "rot_dims": a.rot.dims,
                                     "exact_angles": True, "scaling_factor": a.rot.factor})
            mixer = PartSpec("latent_attention", {
                "n_heads": a.heads, "head_dim": a.dim, "rot_dim": a.rot_dim, "v_head_dim": a.vdim, "kv_rank": a.kv_rank,
                "eps": cfg.norm_eps, "position": rope, "scale": a.scale, "own_latent": a.kv_from is None,
                "gated": True, "names": _LATENT_NAMES}, prefix="mix.")
            cache = i if a.kv_from is None else a.kv_from
        parts = {"mixer": mixer, "norm": _norm(cfg, "norm1")}
        if L.mlp is not None:
            parts["feed_forward"] = PartSpec("bounded_glu", {
                "intermediate_size": L.mlp.ff, "limit": L.mlp.limit, "alpha": GATE_ALPHA, "shift": UP_SHIFT,
                "names": _MLP_NAMES}, prefix="mlp.")
        layers.append(LayerSpec(prefix=f"l{i}.", arrangement="parallel_shared_norm", parts=parts))
        schedule.append(ScheduleEntry(layer=i, cache=cache))
    head = PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "norm": _norm(cfg, "final.norm"), "tied": True,
                                    "weight_prefix": None})
    embedding = PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "weight_name": "",
                                             "scale": cfg.embedding_scale}, prefix="embed")
    return ModelSpec(hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, max_positions=MAX_POSITIONS,
                     layers=tuple(layers), schedule=tuple(schedule), embedding=embedding, head=head)


register_architecture(ARCHITECTURE, VadodraConfig.from_dict, build_spec, replace=True)
