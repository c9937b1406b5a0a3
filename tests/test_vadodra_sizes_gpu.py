"""Vadodra configurations drawn at random (seeded): every size and constant varies, including the ones the fixed
test models happen to make equal, head sizes of 64 and 128 that send bfloat16 runs to the tensor-core attention
kernels, latents whose sizes are no multiple of 8 (the per-head products then run on the FFMA pipe), windows from
one position to more than the prompt, any order of layers.  Each model runs a prompt whole, its tail token by token,
and a batch of two unequal requests, in float32 and bfloat16, against the plain model."""
import random

import pytest
import torch

import vadodra_models as vm
from conftest import random_tokens, rel_err

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-4, "bfloat16": 6e-2}


def draw_config(seed: int) -> dict:
    rng = random.Random(1000 + seed)
    width = rng.choice([40, 64, 72, 96, 100, 128, 136])

    def ff():
        return (None, None) if rng.random() < 0.15 else (rng.choice([8, 20, 24, 40, 72]), rng.choice([0.5, 1.0, 2.5, 7.0]))

    def window_layer():
        kv = rng.choice([1, 2, 3])
        dim = rng.choice([8, 16, 24, 40, 64, 64, 128])
        rot = rng.choice([r for r in (2, 4, 8, 16, 32, 64, 128) if r <= dim] + [dim])
        return vm.layer("attention", vm.attn(
            heads=kv * rng.choice([1, 2, 4]), kv=kv, dim=dim, scale=rng.uniform(0.05, 0.4),
            window=rng.choice([1, 5, 33, 64, 65, 90, 128, 1000, None]), base=rng.choice([100.0, 1e4, 5e5]), rot=rot,
            factor=rng.choice([None, 2.0, 4.0, 0.5])), *ff())

    owners = {}

    def latent_layer(i):
        if owners and rng.random() < 0.5:
            src = rng.choice(list(owners))
            rank, rd, base = owners[src]
        else:
            src, rank, rd, base = None, rng.choice([8, 12, 20, 40, 64, 100]), rng.choice([2, 4, 8, 16, 32]), rng.choice([100.0, 1e4])
            owners[i] = (rank, rd, base)
        return vm.layer("latent_attention", vm.latent(
            heads=rng.choice([1, 2, 3, 5, 8]), dim=rng.choice([4, 8, 12, 24, 64]), rot_dim=rd, vdim=rng.choice([4, 8, 20, 32, 72]),
            rank=rank, scale=rng.uniform(0.05, 0.3), base=base, kv_from=src), *ff())

    layers = []
    for i in range(rng.choice([2, 3, 4, 5])):
        layers.append(latent_layer(i) if rng.random() < 0.5 else window_layer())
    return {"architecture": "Vadodra", "vocab": rng.choice([97, 160, 301]), "width": width,
            "norm": {"eps": rng.choice([1e-5, 1e-6])}, "embedding": {"scale": rng.choice([1.0, 6.5, 12.0])}, "layers": layers}


@pytest.mark.parametrize("seed", list(range(14)))
def test_random_configuration(seed, tmp_path):
    from rust_inference_b200.engine.engine import Engine
    cfg = draw_config(seed)
    vocab = cfg["vocab"]
    a, b = random_tokens(150, vocab, seed), random_tokens(37, vocab, seed + 100)
    model = vm.make(tmp_path, f"r{seed}", seed=seed, cfg=cfg)
    want_a, want_b = model.plain_logits(a), model.plain_logits(b)
    for dtype in ("float32", "bfloat16"):
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
