"""The Lulisun decoder as a `ModelSpec`.

Every layer is x <- x + mixer(norm1(x)) + ff(norm2(x)) (`parallel_two_norms`), the norms RMS norms whose
stored weight is an offset from one.  The mixer is two mixers on the same input (`parallel_mixers`): grouped-query
softmax attention whose keys are limited to the query's own chunk of positions, with rotary positions
on the first channels of every head, a value head size of its own and a score scale from the
configuration; and a gated linear recurrence with a matrix state per head.  The feed-forward is a
routed mixture of gated experts with grouped choice and a gated shared expert (`routed_experts`), or
absent.  A layer may run another layer's tensors with a cache of its own: that is the schedule.

Tensor names: `embed`, `l<i>.norm1`, `l<i>.norm2`, `l<i>.mix.left.{q,k,v,o}`,
`l<i>.mix.right.{q,f,f.b,lower,v,norm,o}`, `l<i>.mlp.e<k>.{gate,up,down}`, `l<i>.mlp.router`,
`l<i>.mlp.correction`, `l<i>.mlp.shared.{gate,up,down,sg}`, `final.norm`, `head`.
"""
from __future__ import annotations

from ..config.lulisun_config import ARCHITECTURE, LulisunConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, ScheduleEntry

# the configuration gives no context length: positions are bounded by the cache a run is given
MAX_POSITIONS = 1 << 17

_ATTENTION_NAMES = {"q": "q", "k": "k", "v": "v", "o": "o"}
_RECURRENCE_NAMES = {"q": "q", "f": "f", "f_bias": "f.b", "lower": "lower", "v": "v", "norm": "norm", "o": "o"}
_EXPERT_NAMES = {"router": "router", "correction": "correction", "gate": "e{e}.gate", "up": "e{e}.up",
                 "down": "e{e}.down", "shared_gate": "shared.gate", "shared_up": "shared.up",
                 "shared_down": "shared.down", "shared_mix": "shared.sg"}


def _norm(cfg: LulisunConfig, prefix: str) -> PartSpec:
    return PartSpec("rmsnorm", {"eps": cfg.norm_eps, "unit_offset": True, "weight_name": ""}, prefix=prefix)


def build_spec(cfg: LulisunConfig) -> ModelSpec:
    layers, index_of, schedule = [], {}, []
    for i, L in enumerate(cfg.layers):
        if L.weights_of is not None:
            continue
        a, r, m = L.left, L.right, L.mlp
        rope = PartSpec("rope", {"head_dim": a.dim, "base": a.rot_base, "style": "half", "rot_dims": a.rot_dims,
                                 "exact_angles": True})
        left = PartSpec("gqa_attention", {
            "n_heads": a.heads, "n_kv_heads": a.kv_heads, "head_dim": a.dim, "v_head_dim": a.vdim, "qkv_bias": False,
            "position": rope, "scale": a.scale, "chunk": a.chunk, "names": _ATTENTION_NAMES}, prefix="left.")
        right = PartSpec("gated_linear_recurrence", {
            "n_heads": r.heads, "head_dim": r.dim, "v_head_dim": r.vdim, "eps": cfg.norm_eps,
            "names": _RECURRENCE_NAMES}, prefix="right.")
        parts = {
            "mixer": PartSpec("parallel_mixers", {"members": ((left, L.left_scale), (right, L.right_scale))}, prefix="mix."),
            "mixer_norm": _norm(cfg, "norm1"),
        }
        if m is not None:
            parts["feed_forward"] = PartSpec("routed_experts", {
                "n_experts": m.experts, "top": m.top, "expert_size": m.expert_ff, "n_groups": m.groups,
                "group_keep": m.keep, "shared_size": m.shared_ff, "names": _EXPERT_NAMES}, prefix="mlp.")
            parts["feed_forward_norm"] = _norm(cfg, "norm2")
        index_of[i] = len(layers)
        layers.append(LayerSpec(prefix=f"l{i}.", arrangement="parallel_two_norms", parts=parts))
    for i, L in enumerate(cfg.layers):
        schedule.append(ScheduleEntry(layer=index_of[i if L.weights_of is None else L.weights_of], cache=i))
    head = PartSpec("linear_head", {"vocab_size": cfg.vocab_size, "norm": _norm(cfg, "final.norm"), "tied": False,
                                    "weight_prefix": "head", "weight_name": ""})
    embedding = PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "weight_name": ""}, prefix="embed")
    return ModelSpec(hidden_size=cfg.hidden_size, vocab_size=cfg.vocab_size, max_positions=MAX_POSITIONS,
                     layers=tuple(layers), schedule=tuple(schedule), embedding=embedding, head=head)


register_architecture(ARCHITECTURE, LulisunConfig.from_dict, build_spec, replace=True)
