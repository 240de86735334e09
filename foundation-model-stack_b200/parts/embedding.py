"""Embeddings: how a step's token ids become the first rows of the float32 residual stream.

Interface of an embedding (what the decoder calls):

    cache_request() -> StateRequest | None       what it keeps per sequence between steps
    forward(batch, state_view, scale) -> [tokens, dim] float32

``TableEmbedding`` ("table"): the token's row of the table (fms/models/llama.py:332).

``PairHashEmbedding`` ("pair_hash"): the token's row plus a row of a second, hashed table of token pairs,
e(t) = table[token_t] + pairs[(token_(t-1) * mul_prev + token_t * mul_cur) mod buckets], and pairs[buckets] (the
last row) for the first token of a sequence.  The token before a step's first row is the sequence's own state: one
int32 per slot that the kernel reads and then sets to the step's last token.
"""
from __future__ import annotations

import torch

from ..cache.requests import StateRequest
from ..config.specs import EmbeddingSpec
from ..kernels import ops
from .base import Part
from .registry import register_embedding


class TableEmbedding(Part):
    def __init__(self, spec: EmbeddingSpec, vocab_size: int, dim: int) -> None:
        super().__init__()
        self.vocab_size, self.dim = vocab_size, dim
        self.declare("weight", (vocab_size, dim), role="matrix")

    def cache_request(self):
        return None

    def forward(self, batch, state_view, scale: float = 1.0):
        return ops.embed(self.tensor("weight"), batch.tokens, scale)

    def kernel_libraries(self, dtype):
        return ["elementwise"]


class PairHashEmbedding(TableEmbedding):
    def __init__(self, spec: EmbeddingSpec, vocab_size: int, dim: int) -> None:
        super().__init__(spec, vocab_size, dim)
        options = dict(spec.options)
        self.buckets = int(options["buckets"])
        self.mul_prev, self.mul_cur = int(options["mul_prev"]), int(options["mul_cur"])
        if self.buckets <= 0:
            raise ValueError(f"pair_hash embedding: {self.buckets} buckets")
        self.pairs_name = options.get("name", "pairs")
        self.declare(self.pairs_name, (self.buckets + 1, dim), role="matrix")

    def cache_request(self):
        return StateRequest((1,), torch.int32, "previous_token")

    def forward(self, batch, state_view, scale: float = 1.0):
        return ops.embed_pair_hash(self.tensor("weight"), self.tensor(self.pairs_name), batch, state_view.state,
                                   self.buckets, self.mul_prev, self.mul_cur, scale)


register_embedding("table", TableEmbedding)
register_embedding("pair_hash", PairHashEmbedding)
