"""Token embedding and the output head.

x0[r] = table[ids[r]] (engine/model.py:291,315 of willzeng274/kernel-rush-kawk);
logits = h W^T at the wanted rows only, with W the embedding table when the
head is tied (engine/model.py:103-107,303). Logits leave in 32-bit.
"""

from __future__ import annotations

from .base import Embedding, Head, StateNeed, TensorSpec, register_embedding, register_head


class TokenEmbedding(Embedding):
    """params: vocab, hidden."""

    def __init__(self, params):
        super().__init__(params)
        self.vocab = int(params["vocab"])
        self.hidden = int(params["hidden"])
        self.table = None

    def tensor_specs(self):
        return {"table": TensorSpec((self.vocab, self.hidden), "table")}

    def bind(self, tensors, runtime):
        self.table = tensors["table"]

    def forward(self, ctx):
        return ctx.ops.embed(self.table, ctx.batch.tokens, ctx.batch.n_rows)


class BigramEmbedding(Embedding):
    """x[r] = table[id_r] + pairs[(id_prev * mul_prev + id_r * mul_cur) mod buckets], with the pair table's last row
    (number ``buckets``) for a sequence's first token; the sum and the rows are 32-bit. The sequence's last token id
    is kept as fixed-size state, so that a step may start anywhere. params: vocab, hidden, buckets, mul_prev, mul_cur."""

    def __init__(self, params):
        super().__init__(params)
        self.vocab = int(params["vocab"])
        self.hidden = int(params["hidden"])
        self.buckets = int(params["buckets"])
        self.mul_prev = int(params["mul_prev"])
        self.mul_cur = int(params["mul_cur"])
        self.table = self.pairs = None

    def tensor_specs(self):
        return {"table": TensorSpec((self.vocab, self.hidden), "table"),
                "pairs": TensorSpec((self.buckets + 1, self.hidden), "table")}

    def cache_need(self):
        return StateNeed((1,), "int32")

    def bind(self, tensors, runtime):
        self.table, self.pairs = tensors["table"], tensors["pairs"]

    def forward(self, ctx, cache):
        return ctx.ops.embed_bigram(self.table, self.pairs, cache.state, self.buckets, self.mul_prev, self.mul_cur, ctx.batch)


class OutputHead(Head):
    """params: vocab, hidden, scale (default 1: the logits are multiplied by it). The plan points
    "weight" at the embedding table's checkpoint name when the head is tied."""

    def __init__(self, params):
        super().__init__(params)
        self.vocab = int(params["vocab"])
        self.hidden = int(params["hidden"])
        self.scale = float(params.get("scale", 1.0))
        self.weight = None

    def tensor_specs(self):
        return {"weight": TensorSpec((self.vocab, self.hidden), "table")}

    def bind(self, tensors, runtime):
        self.weight = tensors["weight"]

    def forward(self, ctx, h):
        """h: normalised rows (a Normed or a tensor) of the wanted positions."""
        logits = ctx.ops.linear(h, self.weight, out_float32=True)
        return logits if self.scale == 1.0 else logits.mul_(self.scale)


register_embedding("token_embedding", TokenEmbedding)
register_embedding("bigram_embedding", BigramEmbedding)
register_head("output_head", OutputHead)
