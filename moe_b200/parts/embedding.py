"""Token embedding and the output projection.

x_i = embed[token_i] (src/model.rs:662-665; an id outside the vocabulary is an
error here, the reference wraps it).  logits = W_lm norm(x) on the requested
rows only; W_lm is the embedding when the model ties them (src/model.rs:350).
"""
from __future__ import annotations

import torch

from ..ops import core
from ..ops.linear import linear
from .base import Part, TensorSpec, register_part


class TokenEmbedding(Part):
    category, kind = "embedding", "token_embedding"
    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(self.params["vocab_size"])
        self.hidden = int(self.params["hidden_size"])

    def tensors(self):
        return {"weight": TensorSpec((self.vocab, self.hidden))}

    def step_elements(self, num_tokens):
        return float(num_tokens * self.hidden)            # one row a token

    def bind(self, tensors, rt):
        super().bind(tensors, rt)
        self.weight = tensors["weight"].contiguous()

    def forward(self, rt, token_ids, num_tokens, batch=None):
        """With a batch that carries ``last_token`` (the per-slot table of the tokens sampled last),
        a token id of -1 is read from there."""
        x = rt.empty((num_tokens, self.hidden), torch.float32)
        last = getattr(batch, "last_token", None)
        if last is not None:
            core.embed(self.weight, token_ids, x, rt.status, last, batch.seq_of_token, batch.slots)
        else:
            core.embed(self.weight, token_ids, x, rt.status)
        return x


class LMHead(Part):
    category, kind = "head", "lm_head"
    graph_safe = True

    def __init__(self, spec):
        super().__init__(spec)
        self.vocab = int(self.params["vocab_size"])
        self.hidden = int(self.params["hidden_size"])
        self.tied = bool(self.params.get("tied", False))

    def tensors(self):
        return {} if self.tied else {"weight": TensorSpec((self.vocab, self.hidden))}

    def describe(self):
        return "output projection" + (" (the embedding)" if self.tied else "")

    def step_elements(self, num_tokens):
        return float(self.vocab * self.hidden)            # the whole matrix, tied or not

    def bind(self, tensors, rt, embedding: TokenEmbedding = None):
        super().bind(tensors, rt)
        self.weight = embedding.weight if self.tied else tensors["weight"].contiguous()

    def forward(self, rt, h):
        """h: Activations of the wanted rows -> logits [rows, vocab] float32."""
        return linear(rt, h.act, self.weight)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "lm_head", LMHead)
