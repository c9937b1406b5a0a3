"""The token embedding: a row of the table per token, widened to float32 (transformer.rs:74-75), times a
factor when the model has one (the table itself stays unscaled: a tied head reads it as it is)."""
from __future__ import annotations

from ..kernels import ops
from .base import Embedding
from .registry import register
from .spec import TensorSpec


@register("embedding", "token_embedding")
class TokenEmbedding(Embedding):
    def __init__(self, *, vocab_size: int, weight_name: str = "weight", scale: float = 1.0, hidden_size: int, dtype, device):
        super().__init__(hidden_size=hidden_size, dtype=dtype, device=device)
        self.vocab_size = vocab_size
        self.scale = float(scale)           # on the rows as they enter the float32 stream
        self.weight_name = weight_name      # the table's name below the part's prefix
        self.weight = None

    def tensor_specs(self):
        return {self.weight_name: TensorSpec((self.vocab_size, self.hidden_size))}

    def set_tensors(self, tensors):
        self.weight = tensors[self.weight_name]

    def get_tensors(self):
        return {self.weight_name: self.weight}

    def table(self):
        return self.weight

    def forward(self, ctx, residual):
        ops.embed_gather(self.weight, ctx.token_ids, residual, self.scale)
