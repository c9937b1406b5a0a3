"""Lulisun configurations drawn at random (seeded): every size and constant varies, including the ones the
fixed test models happen to make equal, and head sizes of 64 and 128 that send bfloat16 runs to the
tensor-core attention kernels.  Each model runs a prompt whole, its tail token by token, and a batch of
two unequal requests, in float32 (free routing) and bfloat16 (pinned routing), against the plain model."""
import random

import pytest
import torch

import lulisun_models
from conftest import random_tokens, rel_err

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-4, "bfloat16": 8e-2}


def draw_config(seed: int) -> dict:
    rng = random.Random(seed)
    width = rng.choice([40, 64, 72, 96, 100, 128, 136])
    n_kinds = rng.choice([1, 2, 2])

    def kind():
        kv = rng.choice([1, 2, 3])
        dim = rng.choice([8, 16, 24, 40, 64, 64, 128])
        same = dim in (64, 128) and rng.random() < 0.7
        vdim = dim if same else rng.choice([8, 12, 20, 32, 48])
        rot = rng.choice([d for d in (2, 4, 8, 16, 32, 64, 128) if d <= dim] + [dim])
        rdim, rvdim = rng.choice([4, 8, 20, 36, 64]), rng.choice([4, 9, 16, 40])
        experts = rng.choice([2, 4, 6, 8, 12])
        groups = rng.choice([g for g in (1, 2, 3, 4, 6) if experts % g == 0])
        keep = rng.randint(1, groups)
        top = rng.randint(1, min(3, keep * (experts // groups)))
        mlp = None
        if rng.random() < 0.85:
            mlp = lulisun_models._moe(experts, top, rng.choice([8, 20, 24, 40]),
                                      groups=None if (groups == 1 and rng.random() < 0.5) else (groups, keep),
                                      shared=rng.choice([None, 16, 28]))
        return dict(heads=kv * rng.choice([1, 2, 4]), kv=kv, dim=dim, vdim=vdim, scale=rng.uniform(0.05, 0.4),
                    chunk=rng.choice([1, 5, 33, 64, 90, 128, 1000]), base=rng.choice([100.0, 1e4, 5e5]), rot=rot,
                    rh=rng.choice([1, 2, 3]), rdim=rdim, rvdim=rvdim, ls=rng.uniform(0.3, 1.5), rs=rng.uniform(0.3, 1.5), mlp=mlp)

    kinds = [kind() for _ in range(n_kinds)]
    layers, owner = [], {}
    for i in range(rng.choice([2, 3, 4])):
        k = rng.randrange(n_kinds)
        if k in owner and rng.random() < 0.6:
            layers.append(lulisun_models._layer(**kinds[k], of=owner[k]))
        else:
            layers.append(lulisun_models._layer(**kinds[k]))
            owner.setdefault(k, i)
    # a sharer may come before its owner in the file
    if rng.random() < 0.3 and len(layers) > 1 and "weights_of" not in layers[0] and "weights_of" not in layers[-1] \
            and layers[0]["mixer"] == layers[-1]["mixer"] and layers[0]["mlp"] == layers[-1]["mlp"]:
        layers[0]["weights_of"] = len(layers) - 1
        for L in layers[1:-1]:
            if L.get("weights_of") == 0:
                L["weights_of"] = len(layers) - 1
    return {"architecture": "Lulisun", "vocab": rng.choice([97, 160, 301]), "width": width,
            "norm": {"eps": rng.choice([1e-5, 1e-6])}, "layers": layers}


@pytest.mark.parametrize("seed", list(range(14)))
def test_random_configuration(seed, tmp_path):
    from rust_inference_b200.engine.engine import Engine
    cfg = draw_config(seed)
    vocab = cfg["vocab"]
    a, b = random_tokens(150, vocab, seed), random_tokens(37, vocab, seed + 100)
    for dtype in ("float32", "bfloat16"):
        model = lulisun_models.make(tmp_path, f"r{seed}", seed=seed, pinned=dtype == "bfloat16", cfg=cfg)
        want_a, want_b = model.plain_logits(a), model.plain_logits(b)
        eng = Engine.from_pretrained(model.folder, dtype=dtype, max_tokens=1024, n_slots=4)
        s = eng.alloc_slot()
        assert rel_err(eng.step([s], [a], "all"), want_a) < TOL[dtype], (seed, dtype, "whole", cfg)
        eng.free_slot(s)
        sa, sb = eng.alloc_slot(), eng.alloc_slot()
        out = eng.step([sa, sb], [a[:131], b[:30]], "all").cpu()
        rows_a, rows_b = [out[:131]], [out[131:]]
        for p in range(7):
            out = eng.step([sa, sb], [[a[131 + p]], [b[30 + p]]], "last").cpu()
            rows_a.append(out[0:1])
            rows_b.append(out[1:2])
        eng.free_slot(sb)
        for p in range(138, 150):
            rows_a.append(eng.step([sa], [[a[p]]], "last").cpu())
        assert rel_err(torch.cat(rows_a), want_a) < TOL[dtype], (seed, dtype, "batch a", cfg)
        assert rel_err(torch.cat(rows_b), want_b) < TOL[dtype], (seed, dtype, "batch b", cfg)
        eng.check_device_status()
