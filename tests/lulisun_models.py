"""Small Lulisun configurations for the tests, and model folders made from them.

The configurations differ from one another in every size and constant; they include values that
make two sizes equal or 1 (one kv head per head, one recurrent head, one expert chosen, groups of
one expert, no groups, no shared expert, a layer without feed-forward, a chunk shorter than a page
and one longer, rotary positions on a part of a head and on all of it, odd value head sizes)."""
import json
import os

import torch

import plain_lulisun


def _layer(*, heads, kv, dim, vdim, scale, chunk, base, rot, rh, rdim, rvdim, ls, rs, mlp, of=None):
    entry = {"type": "parallel", "mixer": {
        "left": {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": vdim, "scale": scale, "mask": {"size": chunk},
                 "rot": {"base": base, "dims": rot}},
        "right": {"heads": rh, "dim": rdim, "vdim": rvdim}, "left_scale": ls, "right_scale": rs}, "mlp": mlp}
    if of is not None:
        entry["weights_of"] = of
    return entry


def _moe(experts, top, ff, groups=None, shared=None):
    router = {"experts": experts, "top": top}
    if groups is not None:
        router["groups"] = {"count": groups[0], "keep": groups[1]}
    out = {"kind": "moe", "expert": {"ff": ff}, "router": router}
    if shared is not None:
        out["shared"] = {"ff": shared}
    return out


_A0 = dict(heads=4, kv=2, dim=32, vdim=16, scale=0.21, chunk=24, base=10000.0, rot=16, rh=3, rdim=24, rvdim=40,
           ls=0.7, rs=1.3)
_B0 = dict(heads=6, kv=3, dim=16, vdim=24, scale=0.3, chunk=100, base=777.0, rot=8, rh=2, rdim=8, rvdim=16, ls=1.1, rs=0.6)

CONFIGS = {
    # four layer runs: own weights; no feed-forward, other head shapes, no GQA, one recurrent head of an odd
    # width; layer 0 once more; one expert chosen of five without groups or shared expert
    "A": {"architecture": "Lulisun", "vocab": 300, "width": 128, "norm": {"eps": 1e-5}, "layers": [
        _layer(**_A0, mlp=_moe(12, 3, 48, groups=(3, 2), shared=80)),
        _layer(heads=2, kv=2, dim=64, vdim=64, scale=0.125, chunk=7, base=50000.0, rot=64, rh=1, rdim=72, rvdim=33,
               ls=1.0, rs=0.4, mlp=None),
        _layer(**_A0, mlp=_moe(12, 3, 48, groups=(3, 2), shared=80), of=0),
        _layer(heads=1, kv=1, dim=8, vdim=8, scale=0.5, chunk=65, base=100.0, rot=2, rh=2, rdim=16, rvdim=8,
               ls=0.9, rs=0.9, mlp=_moe(5, 1, 24)),
    ]},
    # a looped model: one set of weights run three times; groups of one expert; width not a multiple of 32
    "B": {"architecture": "Lulisun", "vocab": 157, "width": 72, "norm": {"eps": 1e-6}, "layers": [
        _layer(**_B0, mlp=_moe(6, 2, 20, groups=(6, 3), shared=12), of=1),
        _layer(**_B0, mlp=_moe(6, 2, 20, groups=(6, 3), shared=12)),
        _layer(**_B0, mlp=_moe(6, 2, 20, groups=(6, 3), shared=12), of=1),
    ]},
}


def pin_routing(cfg, weights):
    """Corrections that decide the choice by themselves: 1.5 apart within a group of experts and 20 apart
    from group to group, so neither the order of the groups' top-2 sums nor the order of the experts hangs
    on the router's sigmoid (which lies in (0, 1)), and a bfloat16 run and the plain one choose the same
    experts at every token (the weights of the chosen still come from the router)."""
    out = dict(weights)
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is None and layer.get("mlp") is not None:
            router = layer["mlp"]["router"]
            n = router["experts"]
            groups = (router.get("groups") or {"count": 1})["count"]
            size = n // groups
            g = torch.Generator().manual_seed(i)
            group_rank = torch.randperm(groups, generator=g).float()
            c = torch.cat([20.0 * group_rank[k] + 1.5 * torch.randperm(size, generator=g).float() for k in range(groups)])
            out[f"l{i}.mlp.correction"] = (c - 8.0).to(torch.bfloat16)
    return out


class LulisunModel:
    def __init__(self, folder, cfg, weights):
        self.folder, self.cfg = folder, cfg
        self.weights = {k: v.float() for k, v in weights.items()}       # the stored bfloat16 values, widened

    def plain_logits(self, tokens, **kw):
        return plain_lulisun.forward(self.cfg, self.weights, tokens, **kw)


def make(tmp_path, name, seed=0, pinned=False, cfg=None, edit=None):
    from rust_inference_b200.weights.safetensors_io import write_safetensors
    cfg = cfg or CONFIGS[name]
    weights = plain_lulisun.random_weights(cfg, seed)
    if pinned:
        weights = pin_routing(cfg, weights)
    if edit is not None:
        edit(weights)
    folder = str(tmp_path / f"lulisun_{name}_{seed}_{int(pinned)}")
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights)
    return LulisunModel(folder, cfg, weights)
