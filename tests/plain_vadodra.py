"""The Vadodra decoder restated plainly: float64 torch on the CPU, whole sequences at once, one function per
mechanism, no cache, no batching, no code shared with the library.  The tests compare the engine with this.

Notation: T tokens, D the stream's width; W["name"] the tensors under the names of the weight file
(matrices [out, in]); positions count from 0.
"""
import math

import torch


# ---- small pieces ---------------------------------------------------------------------------------------
def centred_norm(x, w, eps):
    """(x - mean) / sqrt(mean of squared deviations + eps) * w over the last axis."""
    mu = x.mean(-1, keepdim=True)
    dev = x - mu
    return dev / torch.sqrt((dev * dev).mean(-1, keepdim=True) + eps) * w


def rms_norm(x, w, eps):
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps) * w


def angles(positions, base, dims, factor):
    """[T, dims / 2]: position * base^(-2 i / dims) / factor."""
    i = torch.arange(dims // 2, dtype=torch.float64)
    freq = torch.pow(torch.tensor(float(base), dtype=torch.float64), -2.0 * i / dims) / factor
    return positions.double()[:, None] * freq[None, :]


def rotate_adjacent(x, positions, base, dims, factor=1.0):
    """x [T, heads, d]: channels (2i, 2i + 1) of the first `dims` turn by the i-th angle; the rest pass."""
    a = angles(positions, base, dims, factor)
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    out = x.clone()
    u, v = x[..., 0:dims:2], x[..., 1:dims:2]
    out[..., 0:dims:2] = u * c - v * s
    out[..., 1:dims:2] = v * c + u * s
    return out


def rotate_halves(x, positions, base, dims, factor=1.0):
    """x [T, heads, d]: channels (i, i + dims / 2) of the first `dims` turn by the i-th angle; the rest pass."""
    a = angles(positions, base, dims, factor)
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    h = dims // 2
    out = x.clone()
    u, v = x[..., :h], x[..., h:dims]
    out[..., :h] = u * c - v * s
    out[..., h:dims] = v * c + u * s
    return out


def softmax_attention(scores, values, visible):
    """scores [heads, T, T], values [T, heads, dv], visible bool [T, T] -> [T, heads, dv]."""
    scores = scores.masked_fill(~visible[None], float("-inf"))
    return torch.einsum("hij,jhd->ihd", torch.softmax(scores, dim=-1), values)


def _factor(rot):
    return float((rot.get("scaling") or {}).get("factor", 1.0))


# ---- mixers -----------------------------------------------------------------------------------------------
def window_attention(h, W, p, m, eps):
    """Grouped-query attention whose values are the keys as projected; per-head RMS norm of q and k, adjacent-pair
    rotation of their first channels; a query sees itself and the mask.size - 1 positions before it."""
    T = h.shape[0]
    H, G, d = m["heads"], m["kv_heads"], m["dim"]
    pos = torch.arange(T)
    q = (h @ W[p + "q"].T).view(T, H, d)
    k = (h @ W[p + "k"].T).view(T, G, d)
    v = k
    rot = m["rot"]
    q = rotate_adjacent(rms_norm(q, W[p + "q.norm"], eps), pos, rot["base"], rot["dims"], _factor(rot))
    k = rotate_adjacent(rms_norm(k, W[p + "k.norm"], eps), pos, rot["base"], rot["dims"], _factor(rot))
    k, v = k.repeat_interleave(H // G, dim=1), v.repeat_interleave(H // G, dim=1)
    gap = pos[:, None] - pos[None, :]
    visible = gap >= 0
    if m.get("mask") is not None:
        visible = visible & (gap < m["mask"]["size"])
    o = softmax_attention(torch.einsum("ihd,jhd->hij", q, k) * m["scale"], v, visible)
    return o.reshape(T, -1) @ W[p + "o"].T


def latent_rows(h, W, p, m, eps):
    """What a layer with a down-projection keeps per position: the normalised latent [T, rank] and the rotated
    key part [T, rot_dim]."""
    T = h.shape[0]
    rank, rot = m["kv_rank"], m["rot"]
    down = h @ W[p + "dkv"].T
    c = rms_norm(down[:, :rank], W[p + "dkv.norm"], eps)
    k_rot = rotate_halves(down[:, None, rank:], torch.arange(T), rot["base"], rot["dims"], _factor(rot))[:, 0]
    return c, k_rot


def latent_attention(h, W, p, m, eps, rows):
    """Causal attention whose keys and values are per-head maps of the shared latent (`rows` = latent_rows of this
    layer or of the one it reads), with an output gate per head."""
    T = h.shape[0]
    H, d, rd, vd = m["heads"], m["dim"], m["rot_dim"], m["vdim"]
    c, k_rot = rows
    pos = torch.arange(T)
    q = (h @ W[p + "q"].T).view(T, H, d + rd)
    q_plain = q[..., :d]
    q_rot = rotate_halves(q[..., d:], pos, m["rot"]["base"], m["rot"]["dims"], _factor(m["rot"]))
    k_plain = (c @ W[p + "uk"].T).view(T, H, d)
    v = (c @ W[p + "uv"].T).view(T, H, vd)
    scores = (torch.einsum("ihd,jhd->hij", q_plain, k_plain) + torch.einsum("ihd,jd->hij", q_rot, k_rot)) * m["scale"]
    o = softmax_attention(scores, v, (pos[:, None] - pos[None, :]) >= 0)
    gate = torch.sigmoid(h @ W[p + "g"].T)
    return (o * gate[:, :, None]).reshape(T, -1) @ W[p + "o"].T


def bounded_glu(h, W, p, mlp):
    lim = mlp["limit"]
    g = torch.clamp(h @ W[p + "gate"].T, max=lim)
    u = torch.clamp(h @ W[p + "up"].T, min=-lim, max=lim)
    return (g * torch.sigmoid(1.702 * g) * (u + 1.0)) @ W[p + "down"].T


# ---- the model ----------------------------------------------------------------------------------------------
def forward(cfg, weights, tokens, streams=None):
    """float64 logits [T, vocab] of a whole sequence; `streams` (a list) receives the stream after every layer."""
    W = {k: v.double() for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens, dtype=torch.long)] * cfg["embedding"]["scale"]
    kept = {}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        h = centred_norm(x, W[p + "norm1"], eps)
        if layer["type"] == "attention":
            mixed = window_attention(h, W, p + "mix.", m, eps)
        else:
            if m.get("kv_from") is None:
                kept[i] = latent_rows(h, W, p + "mix.", m, eps)
            mixed = latent_attention(h, W, p + "mix.", m, eps, kept[i if m.get("kv_from") is None else m["kv_from"]])
        ff = bounded_glu(h, W, p + "mlp.", layer["mlp"]) if layer.get("mlp") is not None else 0.0
        x = x + (mixed + ff)
        if streams is not None:
            streams.append(x.clone())
    return centred_norm(x, W["final.norm"], eps) @ W["embed"].T


def greedy(cfg, weights, prompt, n_new):
    tokens = list(prompt)
    for _ in range(n_new):
        tokens.append(int(forward(cfg, weights, tokens)[-1].argmax()))
    return tokens[len(prompt):]


# ---- tensors ------------------------------------------------------------------------------------------------
def tensor_shapes(cfg):
    D = cfg["width"]
    shapes = {"embed": (cfg["vocab"], D), "final.norm": (D,)}
    for i, layer in enumerate(cfg["layers"]):
        p, m = f"l{i}.", layer["mixer"]
        shapes[p + "norm1"] = (D,)
        if layer["type"] == "attention":
            H, G, d = m["heads"], m["kv_heads"], m["dim"]
            shapes.update({p + "mix.q": (H * d, D), p + "mix.k": (G * d, D), p + "mix.q.norm": (d,), p + "mix.k.norm": (d,),
                           p + "mix.o": (D, H * d)})
        else:
            H, d, rd, vd, r = m["heads"], m["dim"], m["rot_dim"], m["vdim"], m["kv_rank"]
            shapes[p + "mix.q"] = (H * (d + rd), D)
            if m.get("kv_from") is None:
                shapes[p + "mix.dkv"] = (r + rd, D)
                shapes[p + "mix.dkv.norm"] = (r,)
            shapes.update({p + "mix.uk": (H * d, r), p + "mix.uv": (H * vd, r), p + "mix.g": (H, D), p + "mix.o": (D, H * vd)})
        if layer.get("mlp") is not None:
            F = layer["mlp"]["ff"]
            shapes.update({p + "mlp.gate": (F, D), p + "mlp.up": (F, D), p + "mlp.down": (D, F)})
    return shapes


def random_weights(cfg, seed, hot=1.0):
    """bfloat16 tensors: matrices N(0, hot^2 / in) (the latent's up-maps a little larger, so that the heads' keys
    differ), norm weights 1 + N(0, 0.2), the embedding N(0, 1) / its scale (a stream of unit size)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith("norm") or name.endswith("norm1"):
            t = 1.0 + 0.2 * torch.randn(shape, generator=g)
        elif name == "embed":
            t = torch.randn(shape, generator=g) / cfg["embedding"]["scale"]
        else:
            t = torch.randn(shape, generator=g) * (hot / math.sqrt(shape[1]))
        out[name] = t.to(torch.bfloat16)
    return out
