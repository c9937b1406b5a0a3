"""A gated linear recurrence with a matrix state per head (the HGRN2 form of linear attention)."""
from __future__ import annotations

import torch

from ..cache.sequence_cache import StateRequest
from ..kernels import linear, ops
from .base import Mixer
from .registry import register
from .spec import TensorSpec


@register("mixer", "gated_linear_recurrence")
class GatedLinearRecurrence(Mixer):
    """Per head a state S [dim, vdim] in float32, zero at the start of a sequence and carried from
    token to token in the slot's state area:

        q = silu(Wq x)            f = low + (1 - low) * sigmoid(Wf x + b)        v = Wv x
        S <- diag(f) S + (1 - f) v^T          o = S^T q

    The forget gate f lies in [low, 1) per head and channel, and the write is tied to it (weight 1 - f),
    which takes the place of a key.  Every head's o is RMS-normed over vdim with one weight shared by the heads,
    the heads are concatenated and projected by Wo onto the residual stream.  The three projections
    run as one product with float32 results; gates, state and norm are float32 in both precisions.
    `out_scale` multiplies the mixer's result (applied to the normed o, in float32).  `names` gives
    the tensors' names below the part's prefix."""

    _NAMES = {"q": "q_proj.weight", "f": "f_proj.weight", "f_bias": "f_proj.bias", "lower": "lower_bound",
              "v": "v_proj.weight", "norm": "o_norm.weight", "o": "o_proj.weight"}

    def __init__(self, *, n_heads: int, head_dim: int, v_head_dim: int, eps: float, out_scale: float = 1.0,
                 names: dict | None = None, hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        self.n_heads, self.head_dim, self.v_head_dim = n_heads, head_dim, v_head_dim
        self.q_dim, self.v_dim = n_heads * head_dim, n_heads * v_head_dim
        self.eps = float(eps)
        self.out_scale = float(out_scale)
        self.names = dict(self._NAMES, **(names or {}))
        self.w_qfv = self.w_o = self.f_bias = self.lower = self.norm = None

    def tensor_specs(self):
        h, nm = self.hidden_size, self.names
        return {
            nm["q"]: TensorSpec((self.q_dim, h)),
            nm["f"]: TensorSpec((self.q_dim, h)),
            nm["f_bias"]: TensorSpec((self.q_dim,), role="vector"),
            nm["lower"]: TensorSpec((self.q_dim,), role="vector", init="zeros"),
            nm["v"]: TensorSpec((self.v_dim, h)),
            nm["norm"]: TensorSpec((self.v_head_dim,), role="vector", init="ones"),
            nm["o"]: TensorSpec((h, self.v_dim)),
        }

    def set_tensors(self, tensors):
        nm = self.names
        self.w_qfv = linear.Weight(torch.cat([tensors[nm["q"]], tensors[nm["f"]], tensors[nm["v"]]], dim=0))
        self.w_o = linear.Weight(tensors[nm["o"]])
        self.f_bias, self.lower, self.norm = tensors[nm["f_bias"]], tensors[nm["lower"]], tensors[nm["norm"]]

    def get_tensors(self):
        nm, q = self.names, self.q_dim
        w = self.w_qfv.t
        return {nm["q"]: w[:q], nm["f"]: w[q:2 * q], nm["f_bias"]: self.f_bias, nm["lower"]: self.lower,
                nm["v"]: w[2 * q:], nm["norm"]: self.norm, nm["o"]: self.w_o.t}

    def cache_request(self):
        return StateRequest((self.n_heads, self.head_dim, self.v_head_dim), torch.float32)

    def forward(self, x, residual, ctx, cache_layer, writes_cache):
        if not writes_cache:
            raise ValueError("a recurrent state has one writer: a layer cannot read another layer's state")
        n = x.shape[0]
        z = ctx.buffer("recurrence_z", (n, 2 * self.q_dim + self.v_dim), torch.float32)
        linear.logits(x, self.w_qfv, z, ctx)                       # float32 results in both precisions
        o = ctx.buffer("recurrence_o", (n, self.v_dim), self.dtype)
        o_raw = ctx.buffer("recurrence_o_raw", (n, self.v_dim), torch.float32)
        # long runs of new tokens are cut into pieces that are scanned side by side
        piece, most = ops.recurrence_pieces(ctx.max_new, ctx.n_seqs, self.n_heads, self.head_dim, self.v_head_dim)
        scratch = None
        if piece:
            scratch = ctx.buffer("recurrence_pieces", (ctx.n_seqs * most * self.n_heads * self.head_dim
                                                       * (self.v_head_dim + 1),), torch.float32)
        ops.gated_recurrence(z, self.f_bias, self.lower, self.norm, cache_layer.state, ctx.cu_seqlens, ctx.seq_slot, o,
                             n_seqs=ctx.n_seqs, heads=self.n_heads, dim=self.head_dim, vdim=self.v_head_dim,
                             eps=self.eps, out_scale=self.out_scale, o_raw=o_raw, piece=piece, max_pieces=most,
                             scratch=scratch, longest_run=ctx.max_new)
        linear.into_residual(o, self.w_o, residual, ctx)
