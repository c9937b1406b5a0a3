"""Small Vadodra configurations for the tests, and model folders made from them.

They differ from one another in every size and constant and include values that make two sizes equal or 1: one
kv head per query head and one kv head for all, a single head, a window of one position, of less than a page and
of more than two pages, no window, rotation of a whole head and of two channels, scaled and unscaled positions,
a latent narrower and wider than the heads it feeds, layers that read an earlier layer's latent (also two of
them, also as the last layer), layers without feed-forward, widths that are no multiple of 32."""
import json
import os

import plain_vadodra


def attn(*, heads, kv, dim, scale, window, base, rot, factor=None):
    r = {"base": base, "dims": rot}
    if factor is not None:
        r["scaling"] = {"factor": factor}
    m = {"heads": heads, "kv_heads": kv, "dim": dim, "vdim": dim, "scale": scale, "rot": r}
    if window is not None:
        m["mask"] = {"size": window}
    return m


def latent(*, heads, dim, rot_dim, vdim, rank, scale, base, kv_from=None):
    m = {"heads": heads, "dim": dim, "rot_dim": rot_dim, "vdim": vdim, "kv_rank": rank, "scale": scale,
         "rot": {"base": base, "dims": rot_dim}}
    if kv_from is not None:
        m["kv_from"] = kv_from
    return m


def layer(kind, mixer, ff=None, limit=None):
    return {"type": kind, "mixer": mixer, "mlp": None if ff is None else {"kind": "dense", "ff": ff, "limit": limit}}


CONFIGS = {
    # windows of 20 (inside a page) and 150 (more than two pages); a latent layer read by two later ones, the last
    # of them without feed-forward
    "A": {"architecture": "Vadodra", "vocab": 310, "width": 128, "norm": {"eps": 1e-5}, "embedding": {"scale": 9.5}, "layers": [
        layer("latent_attention", latent(heads=4, dim=16, rot_dim=8, vdim=24, rank=40, scale=0.2, base=10000.0), 96, 1.5),
        layer("attention", attn(heads=4, kv=2, dim=32, scale=0.18, window=20, base=50000.0, rot=8, factor=2.0), 72, 3.0),
        layer("latent_attention", latent(heads=2, dim=24, rot_dim=8, vdim=16, rank=40, scale=0.15, base=10000.0, kv_from=0), 96, 1.5),
        layer("attention", attn(heads=6, kv=1, dim=16, scale=0.25, window=150, base=300.0, rot=16), None),
        layer("latent_attention", latent(heads=5, dim=8, rot_dim=8, vdim=8, rank=40, scale=0.3, base=10000.0, kv_from=0), None),
    ]},
    # width 72; a single query head; a window of one position; no window at all; a latent wider than the width
    "B": {"architecture": "Vadodra", "vocab": 157, "width": 72, "norm": {"eps": 1e-6}, "embedding": {"scale": 1.0}, "layers": [
        layer("attention", attn(heads=1, kv=1, dim=24, scale=0.2, window=1, base=777.0, rot=2, factor=8.0), 40, 0.75),
        layer("latent_attention", latent(heads=1, dim=40, rot_dim=2, vdim=72, rank=96, scale=0.11, base=500.0), 40, 7.0),
        layer("attention", attn(heads=3, kv=3, dim=8, scale=0.35, window=None, base=1e6, rot=8), 56, 2.0),
        layer("latent_attention", latent(heads=3, dim=8, rot_dim=16, vdim=8, rank=16, scale=0.2, base=80.0), 24, 1.0),
    ]},
    # sizes the tensor-core kernels take: heads of 64 and 128, windows across pages, a latent of 64 + 32
    "C": {"architecture": "Vadodra", "vocab": 264, "width": 256, "norm": {"eps": 1e-6}, "embedding": {"scale": 16.0}, "layers": [
        layer("attention", attn(heads=4, kv=2, dim=64, scale=0.125, window=70, base=500000.0, rot=32, factor=4.0), 384, 2.0),
        layer("latent_attention", latent(heads=4, dim=64, rot_dim=32, vdim=64, rank=64, scale=0.1, base=10000.0), 384, 2.0),
        layer("attention", attn(heads=2, kv=1, dim=128, scale=0.09, window=129, base=10000.0, rot=128), 256, 4.0),
        layer("latent_attention", latent(heads=8, dim=32, rot_dim=32, vdim=32, rank=64, scale=0.12, base=10000.0, kv_from=1), 128, 2.0),
    ]},
}


class VadodraModel:
    def __init__(self, folder, cfg, weights):
        self.folder, self.cfg = folder, cfg
        self.weights = {k: v.float() for k, v in weights.items()}       # the stored bfloat16 values, widened

    def plain_logits(self, tokens, **kw):
        return plain_vadodra.forward(self.cfg, self.weights, tokens, **kw)


def make(tmp_path, name, seed=0, cfg=None, edit=None, hot=1.0):
    from rust_inference_b200.weights.safetensors_io import write_safetensors
    cfg = cfg or CONFIGS[name]
    weights = plain_vadodra.random_weights(cfg, seed, hot=hot)
    if edit is not None:
        edit(weights)
    folder = str(tmp_path / f"vadodra_{name}_{seed}")
    os.makedirs(folder, exist_ok=True)
    with open(os.path.join(folder, "config.json"), "w") as f:
        json.dump(cfg, f)
    write_safetensors(os.path.join(folder, "model.safetensors"), weights)
    return VadodraModel(folder, cfg, weights)
