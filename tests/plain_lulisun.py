"""A plain, slow restatement of the Lulisun decoder, one function per mechanism, written from its
equations and sharing nothing with the library: whole sequences at once, no cache, no
batching, float64 unless told otherwise.  Tests compare the engine with it.

Notation: x_t is the stream at token t (width D), h the normalised input of a block.  A layer is
    x <- x + mixer(n1(x)) + ff(n2(x))          n(x) = x / sqrt(mean(x^2) + eps) * (1 + w)
The mixer is a * A(h) + b * R(h) with A a chunk-local softmax attention and R a gated linear
recurrence; the feed-forward is a routed mixture of gated experts plus an always-on shared expert.
"""
from __future__ import annotations

import math

import torch


def unit_offset_rmsnorm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * (1 + w): the file holds the factor minus one."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * (1.0 + w)


def plain_rmsnorm(x, w, eps):
    """x / sqrt(mean(x^2) + eps) * w."""
    return x / torch.sqrt((x * x).mean(dim=-1, keepdim=True) + eps) * w


def rotate_partial(x, positions, base, rot_dims):
    """x [T, heads, dim]: the first rot_dims channels of every head are rotated, channel i with
    channel i + rot_dims/2 by the angle p * base^(-2i/rot_dims); the rest pass."""
    half = rot_dims // 2
    i = torch.arange(half, dtype=x.dtype)
    freq = torch.pow(torch.tensor(float(base), dtype=x.dtype), -2.0 * i / rot_dims)
    ang = positions.to(x.dtype)[:, None] * freq[None, :]              # [T, half]
    c, s = torch.cos(ang)[:, None, :], torch.sin(ang)[:, None, :]
    u, v = x[..., :half], x[..., half:rot_dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., rot_dims:]], dim=-1)


def chunk_visible(n, chunk):
    """vis[i, j]: j <= i and both lie in the same block of `chunk` positions counted from 0."""
    i = torch.arange(n)[:, None]
    j = torch.arange(n)[None, :]
    return (j <= i) & ((i // chunk) == (j // chunk))


def chunked_attention(h, w, pre, *, heads, kv_heads, dim, vdim, scale, chunk, rot_base, rot_dims):
    """Grouped-query softmax attention whose keys are limited to the query's own chunk."""
    n = h.shape[0]
    q = (h @ w[pre + "q"].T).view(n, heads, dim)
    k = (h @ w[pre + "k"].T).view(n, kv_heads, dim)
    v = (h @ w[pre + "v"].T).view(n, kv_heads, vdim)
    pos = torch.arange(n)
    q = rotate_partial(q, pos, rot_base, rot_dims)
    k = rotate_partial(k, pos, rot_base, rot_dims)
    vis = chunk_visible(n, chunk)
    rep = heads // kv_heads
    out = torch.zeros(n, heads, vdim, dtype=h.dtype)
    for head in range(heads):
        g = head // rep
        s = (q[:, head] @ k[:, g].T) * scale
        s = s.masked_fill(~vis, float("-inf"))
        out[:, head] = torch.softmax(s, dim=-1) @ v[:, g]
    return out.reshape(n, heads * vdim) @ w[pre + "o"].T


def gated_recurrence(h, w, pre, *, heads, dim, vdim, eps, state=None):
    """Per head a matrix state S [dim, vdim]:  S <- diag(f) S + (1 - f) v^T,  o = S^T q, with
    q = silu(Wq h), f = l + (1 - l) sigmoid(Wf h + b); o is RMS-normed per head with one weight."""
    n = h.shape[0]
    q = torch.nn.functional.silu(h @ w[pre + "q"].T).view(n, heads, dim)
    f = torch.sigmoid(h @ w[pre + "f"].T + w[pre + "f.b"])
    low = w[pre + "lower"]
    f = (low + (1.0 - low) * f).view(n, heads, dim)
    v = (h @ w[pre + "v"].T).view(n, heads, vdim)
    S = torch.zeros(heads, dim, vdim, dtype=h.dtype) if state is None else state.clone()
    o = torch.zeros(n, heads, vdim, dtype=h.dtype)
    for t in range(n):
        S = f[t][:, :, None] * S + (1.0 - f[t])[:, :, None] * v[t][:, None, :]
        o[t] = torch.einsum("hkv,hk->hv", S, q[t])
    o = plain_rmsnorm(o, w[pre + "norm"], eps)
    return o.reshape(n, heads * vdim) @ w[pre + "o"].T, S


def gated_expert(h, w, pre):
    """down( silu(gate h) * (up h) )."""
    return (torch.nn.functional.silu(h @ w[pre + "gate"].T) * (h @ w[pre + "up"].T)) @ w[pre + "down"].T


def route(h, w, pre, *, experts, top, groups, keep):
    """ids [T, top] and weights [T, top]: s = sigmoid(router h); c = s + correction ranks; groups of
    experts / groups consecutive experts rank by their top-2 sum of c and only the `keep` highest stay in
    the ranking; the `top` highest c are taken with weights s / sum(s of the taken)."""
    s = torch.sigmoid(h @ w[pre + "router"].T)                          # [T, E]
    choice = s + w[pre + "correction"]
    n = h.shape[0]
    size = experts // groups
    grouped = choice.view(n, groups, size)
    gscore = grouped.topk(min(2, size), dim=-1).values.sum(dim=-1)      # [T, groups]
    kept = gscore.topk(keep, dim=-1).indices
    allowed = torch.zeros(n, groups, dtype=torch.bool)
    allowed.scatter_(1, kept, True)
    masked = grouped.masked_fill(~allowed[:, :, None], float("-inf")).view(n, experts)
    ids = masked.topk(top, dim=-1).indices                              # [T, top]
    picked = s.gather(1, ids)
    return ids, picked / (picked.sum(dim=-1, keepdim=True) + 1e-20), s


def routed_feed_forward(h, w, pre, mlp):
    r = mlp["router"]
    g = r.get("groups") or {"count": 1, "keep": 1}
    ids, weights, _ = route(h, w, pre, experts=r["experts"], top=r["top"], groups=g["count"], keep=g["keep"])
    out = torch.zeros(h.shape[0], w[pre + "e0.down"].shape[0], dtype=h.dtype)
    for t in range(h.shape[0]):
        for c in range(ids.shape[1]):
            e = int(ids[t, c])
            out[t] += weights[t, c] * gated_expert(h[t:t + 1], w, pre + f"e{e}.")[0]
    if mlp.get("shared"):
        gate = torch.sigmoid(h @ w[pre + "shared.sg"].T)               # [T, 1]
        out = out + gate * gated_expert(h, w, pre + "shared.")
    return out


def layer_weights_index(cfg, i):
    j = cfg["layers"][i].get("weights_of")
    return i if j is None else j


def forward(cfg, weights, tokens, dtype=torch.float64, streams=None):
    """Logits [T, vocab] of one whole sequence.  `streams`, a list, receives the stream after every layer."""
    w = {k: v.to(dtype) for k, v in weights.items()}
    eps = cfg["norm"]["eps"]
    x = w["embed"][torch.tensor(tokens, dtype=torch.long)]
    for i, layer in enumerate(cfg["layers"]):
        pre = f"l{layer_weights_index(cfg, i)}."
        m = layer["mixer"]
        h1 = unit_offset_rmsnorm(x, w[pre + "norm1"], eps)
        L, R = m["left"], m["right"]
        a = chunked_attention(h1, w, pre + "mix.left.", heads=L["heads"], kv_heads=L["kv_heads"], dim=L["dim"],
                              vdim=L["vdim"], scale=L["scale"], chunk=L["mask"]["size"], rot_base=L["rot"]["base"],
                              rot_dims=L["rot"]["dims"])
        r, _ = gated_recurrence(h1, w, pre + "mix.right.", heads=R["heads"], dim=R["dim"], vdim=R["vdim"], eps=eps)
        y = m["left_scale"] * a + m["right_scale"] * r
        if layer.get("mlp") is not None:
            h2 = unit_offset_rmsnorm(x, w[pre + "norm2"], eps)
            y = y + routed_feed_forward(h2, w, pre + "mlp.", layer["mlp"])
        x = x + y
        if streams is not None:
            streams.append(x.clone())
    x = unit_offset_rmsnorm(x, w["final.norm"], eps)
    return x @ w["head"].T


def greedy(cfg, weights, prompt, n_new):
    """Greedy continuation by re-running the whole sequence for every new token."""
    toks = list(prompt)
    for _ in range(n_new):
        toks.append(int(forward(cfg, weights, toks)[-1].argmax()))
    return toks[len(prompt):]


def tensor_shapes(cfg):
    """Name -> shape of every tensor a model of this configuration stores."""
    D, V = cfg["width"], cfg["vocab"]
    out = {"embed": (V, D), "final.norm": (D,), "head": (V, D)}
    for i, layer in enumerate(cfg["layers"]):
        if layer.get("weights_of") is not None:
            continue
        p = f"l{i}."
        L, R = layer["mixer"]["left"], layer["mixer"]["right"]
        out[p + "norm1"] = (D,)
        out[p + "mix.left.q"] = (L["heads"] * L["dim"], D)
        out[p + "mix.left.k"] = (L["kv_heads"] * L["dim"], D)
        out[p + "mix.left.v"] = (L["kv_heads"] * L["vdim"], D)
        out[p + "mix.left.o"] = (D, L["heads"] * L["vdim"])
        out[p + "mix.right.q"] = (R["heads"] * R["dim"], D)
        out[p + "mix.right.f"] = (R["heads"] * R["dim"], D)
        out[p + "mix.right.f.b"] = (R["heads"] * R["dim"],)
        out[p + "mix.right.lower"] = (R["heads"] * R["dim"],)
        out[p + "mix.right.v"] = (R["heads"] * R["vdim"], D)
        out[p + "mix.right.norm"] = (R["vdim"],)
        out[p + "mix.right.o"] = (D, R["heads"] * R["vdim"])
        mlp = layer.get("mlp")
        if mlp is not None:
            out[p + "norm2"] = (D,)
            ff = mlp["expert"]["ff"]
            for e in range(mlp["router"]["experts"]):
                out[p + f"mlp.e{e}.gate"] = (ff, D)
                out[p + f"mlp.e{e}.up"] = (ff, D)
                out[p + f"mlp.e{e}.down"] = (D, ff)
            out[p + "mlp.router"] = (mlp["router"]["experts"], D)
            out[p + "mlp.correction"] = (mlp["router"]["experts"],)
            if mlp.get("shared"):
                sf = mlp["shared"]["ff"]
                out[p + "mlp.shared.gate"] = (sf, D)
                out[p + "mlp.shared.up"] = (sf, D)
                out[p + "mlp.shared.down"] = (D, sf)
                out[p + "mlp.shared.sg"] = (1, D)
    return out


def random_weights(cfg, seed, std=None):
    """Random weights in the stored precision (bfloat16 values held as float32 is the caller's
    business): matrices N(0, 1/sqrt(in)), norm weights and biases small, lower bounds in (0, 1)."""
    g = torch.Generator().manual_seed(seed)
    out = {}
    for name, shape in tensor_shapes(cfg).items():
        if name.endswith(".lower"):
            t = torch.rand(shape, generator=g) * 0.9
        elif name.endswith(("norm1", "norm2", "final.norm")):
            t = torch.randn(shape, generator=g) * 0.2
        elif name.endswith(".norm"):
            t = 1.0 + torch.randn(shape, generator=g) * 0.2
        elif name.endswith(("f.b", "correction")):
            t = torch.randn(shape, generator=g) * 0.5
        elif name == "embed":
            t = torch.randn(shape, generator=g)
        else:
            s = std if std is not None else 1.0 / math.sqrt(shape[-1])
            t = torch.randn(shape, generator=g) * s
        out[name] = t.to(torch.bfloat16)
    return out
