"""Causal attention over a low-rank latent that all heads share.

Every position keeps ONE row for all heads: the latent c (kv_rank values, RMS-normalised) and one
rotated key part (rot_dim values).  Head h's keys and values are linear maps of the latent,
k_h = [Uk_h c, k_rot] and v_h = Uv_h c, and its queries are q_h = [q_nope_h, q_rot_h]; the score of a
query against a cached position is (q_nope_h . Uk_h c + q_rot_h . k_rot) * scale.

The per-head keys and values are never formed.  The query is carried into the latent space instead,
q_lat_h = Uk_h^T q_nope_h, so that the score is [q_lat_h, q_rot_h] . [c, k_rot]: attention of `heads` query
heads over ONE kv head whose key is the cached row and whose value is the row's first kv_rank channels.
A head's output is then Uv_h applied to its weighted sum of latents, times its output gate
sigmoid(W_g x)_h, and the output projection adds the heads onto the stream.  The two per-head maps are
grouped contractions (a head is a group of rows), the ones routed experts use.

A layer may read another layer's cached rows (the schedule gives it that layer's cache and
`writes_cache` false): it then has no down-projection of its own, only its own queries, Uk, Uv, gate
and output projection.
"""
from __future__ import annotations

import math

import torch

from ..cache.sequence_cache import KVRequest
from ..kernels import linear, ops, attention as attn_kernels
from .base import Mixer
from .registry import register, lookup
from .spec import TensorSpec, PartSpec


@register("mixer", "latent_attention")
class LatentAttention(Mixer):
    """n_heads heads of head_dim unrotated and rot_dim rotated query / key channels and v_head_dim value
    channels over a latent of kv_rank channels.  `position`: the rotary encoding of the rot_dim part (its
    tables, pairing and rotated channels).  `own_latent` false: the layer has no down-projection and reads
    the cache of the layer the schedule names.  `gated`: an output gate per head.  `scale`: on the scores
    (default 1 / sqrt(head_dim + rot_dim)).  `names`: q, dkv, dkv_norm, uk, uv, gate, o below the prefix."""

    _NAMES = {"q": "q_proj.weight", "dkv": "kv_a_proj.weight", "dkv_norm": "kv_a_norm.weight",
              "uk": "k_b_proj.weight", "uv": "v_b_proj.weight", "gate": "g_proj.weight", "o": "o_proj.weight"}

    def __init__(self, *, n_heads: int, head_dim: int, rot_dim: int, v_head_dim: int, kv_rank: int, eps: float,
                 position: PartSpec, scale: float | None = None, own_latent: bool = True, gated: bool = True,
                 names: dict | None = None, hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        self.n_heads, self.head_dim, self.rot_dim = int(n_heads), int(head_dim), int(rot_dim)
        self.v_head_dim, self.kv_rank = int(v_head_dim), int(kv_rank)
        if min(self.n_heads, self.head_dim, self.v_head_dim, self.kv_rank) <= 0 or self.rot_dim < 2 or self.rot_dim % 2:
            raise ValueError("latent attention: sizes must be positive and the rotated part even")
        self.eps = float(eps)
        self.scale = 1.0 / math.sqrt(float(head_dim + rot_dim)) if scale is None else float(scale)
        self.own_latent, self.gated = bool(own_latent), bool(gated)
        self.names = dict(self._NAMES, **(names or {}))
        self.position = lookup("position", position.kind)(hidden_size=hidden_size, dtype=dtype, device=device,
                                                          **position.params)
        if getattr(self.position, "head_dim", self.rot_dim) != self.rot_dim:
            raise ValueError("latent attention: the position encoding must be built for the rotated part's size")
        self.q_dim = self.n_heads * (self.head_dim + self.rot_dim)
        self.wide = self.kv_rank + self.rot_dim
        self.w_in = self.w_o = self.w_uk_t = self.w_uv = self.latent_norm = None

    # ---- tensors -----------------------------------------------------------------------------------------
    def tensor_specs(self):
        h, nm, H = self.hidden_size, self.names, self.n_heads
        specs = {nm["q"]: TensorSpec((self.q_dim, h))}
        if self.own_latent:
            specs[nm["dkv"]] = TensorSpec((self.wide, h))
            specs[nm["dkv_norm"]] = TensorSpec((self.kv_rank,), role="vector", init="ones")
        specs[nm["uk"]] = TensorSpec((H * self.head_dim, self.kv_rank))
        specs[nm["uv"]] = TensorSpec((H * self.v_head_dim, self.kv_rank))
        if self.gated:
            specs[nm["gate"]] = TensorSpec((H, h))
        specs[nm["o"]] = TensorSpec((h, H * self.v_head_dim))
        return specs

    def set_tensors(self, tensors):
        nm, H = self.names, self.n_heads
        # one matrix for everything that reads x: queries, then the latent with its key part, then the gates
        mats = [tensors[nm["q"]]]
        if self.own_latent:
            mats.append(tensors[nm["dkv"]])
            self.latent_norm = tensors[nm["dkv_norm"]].contiguous()
        if self.gated:
            mats.append(tensors[nm["gate"]])
        self.w_in = linear.Weight(torch.cat(mats, dim=0))
        # Uk per head, transposed: q_lat_h = Uk_h^T q_nope_h is x W^T with W = Uk_h^T [kv_rank, head_dim]
        self.w_uk_t = tensors[nm["uk"]].view(H, self.head_dim, self.kv_rank).transpose(1, 2).contiguous()
        self.w_uv = tensors[nm["uv"]].view(H, self.v_head_dim, self.kv_rank).contiguous()
        self.w_o = linear.Weight(tensors[nm["o"]])

    def get_tensors(self):
        nm, H = self.names, self.n_heads
        w = self.w_in.t
        out = {nm["q"]: w[:self.q_dim]}
        at = self.q_dim
        if self.own_latent:
            out[nm["dkv"]] = w[at:at + self.wide]
            out[nm["dkv_norm"]] = self.latent_norm
            at += self.wide
        if self.gated:
            out[nm["gate"]] = w[at:at + H]
        out[nm["uk"]] = self.w_uk_t.transpose(1, 2).reshape(H * self.head_dim, self.kv_rank)
        out[nm["uv"]] = self.w_uv.view(H * self.v_head_dim, self.kv_rank)
        out[nm["o"]] = self.w_o.t
        return out

    def prepare(self, max_positions):
        self.position.prepare(max_positions)

    def cache_request(self):
        return KVRequest(1, self.wide, None, self.kv_rank, True)

    # ---- the step ------------------------------------------------------------------------------------------
    def _grouped(self, x, w, out, lists, n_rows):
        """out<float32>[rows of head h] = x[rows of head h] w[h]^T for every head: on the tensor cores when the
        sizes allow (bfloat16, K a multiple of 8), else on the FFMA pipe."""
        offsets, order, tiles, n_tiles, fast = lists
        if fast:
            from ..kernels import tcgen05
            return tcgen05.grouped_gemm(x, w, None, out, offsets, tiles, n_tiles, n_pairs=n_rows)
        return ops.moe_grouped_simt(x, w, None, out, offsets, order, tiles, n_tiles, n_pairs=n_rows, top=1)

    def forward(self, x, residual, ctx, cache_layer, writes_cache):
        if writes_cache != self.own_latent:
            raise RuntimeError("latent attention: a layer with a down-projection writes its cache, one without reads another's")
        n, H, d, rd, kr, vd = x.shape[0], self.n_heads, self.head_dim, self.rot_dim, self.kv_rank, self.v_head_dim
        rows = n * H
        pos = self.position
        if pos.cos is None or pos.cos.shape[0] < ctx.max_len:
            raise RuntimeError("rope tables do not cover the step's positions; call prepare() first")
        proj = ctx.buffer("latent_proj", (n, self.w_in.n), self.dtype)
        linear.project(x, self.w_in, proj, ctx)

        fast = False
        if self.dtype == torch.bfloat16:
            from ..kernels import tcgen05
            fast = tcgen05.grouped_supports(self.dtype, self.w_uk_t) and tcgen05.grouped_supports(self.dtype, self.w_uv)
        if fast:
            tile_rows = tcgen05.GROUPED_TILE_ROWS
        else:
            tile_rows = ops.moe_tile_rows()
        per_head = -(-n // tile_rows)
        offsets = ctx.buffer("latent_offsets", (H + 1,), torch.int32)
        order = ctx.buffer("latent_order", (rows,), torch.int32)
        tiles = ctx.buffer("latent_tiles", (2 * H * per_head,), torch.int32)
        n_tiles = ctx.buffer("latent_n_tiles", (1,), torch.int32)
        lists = (offsets, order, tiles, n_tiles, fast)
        q_nope = ctx.buffer("latent_q_nope", (rows, d), self.dtype)              # [heads, T, head_dim]
        q_wide = ctx.buffer("latent_q_wide", (n, H * self.wide), self.dtype)     # [T, heads, kv_rank + rot_dim]
        ops.latent_prepare(proj, pos.cos, pos.sin, self.latent_norm, self.eps, ctx.token_pos, ctx.token_seq,
                           ctx.seq_slot, ctx.page_table, cache_layer.k, q_nope, q_wide, offsets, order, tiles, n_tiles,
                           n_heads=H, head_dim=d, rot_dim=rd, rank=kr, rot_dims=pos.rot_dims, style=pos.style,
                           page_size=ctx.page_size, write_kv=writes_cache, tile_rows=tile_rows)
        # the queries into the latent space, head by head
        if fast:
            # on the tensor cores the product's epilogue rounds and writes the wide rows itself
            tcgen05.grouped_gemm_spread(q_nope, self.w_uk_t, q_wide, self.wide, offsets, tiles, n_tiles, n_pairs=rows)
        else:
            q_lat = ctx.buffer("latent_q_lat", (rows, kr), torch.float32)
            self._grouped(q_nope, self.w_uk_t, q_lat, lists, rows)
            ops.latent_widen(q_lat, q_wide, n_tokens=n, n_heads=H, rank=kr, rot_dim=rd)
        # attention of all heads over the one cached row per position; the weighted latents head by head
        o_lat = ctx.buffer("latent_o_lat", (rows, kr), self.dtype)              # [heads, T, kv_rank]
        attn_kernels.latent_attention(q_wide, cache_layer, o_lat, ctx, n_heads=H, key_dim=self.wide, rank=kr,
                                      scale=self.scale)
        v = ctx.buffer("latent_v", (rows, vd), torch.float32)                    # [heads, T, v_head_dim]
        self._grouped(o_lat, self.w_uv, v, lists, rows)
        gated = ctx.buffer("attn_out", (n, H * vd), self.dtype)
        gates = proj[:, self.w_in.n - H:] if self.gated else None
        ops.latent_gate(v, gates, gated, n_tokens=n, n_heads=H, v_head_dim=vd)
        linear.into_residual(gated, self.w_o, residual, ctx)
