"""Token embedding and output head.

embedding: residual[t,:] = E[id_t,:] * scale (fp32 residual stream; scale 1 unless the design gives one).  lm_head: logits = x . W^T in fp32, with
W = E when the embeddings are tied and the file has no head of its own
(reference: src/inference/engines/transformer_engine.cpp:495-522, src/model/model_weights.cpp:28-33).
"""
from .. import kernels
from ..weights.loader import TensorSpec
from .base import Part, register_part
from .linear import Linear


class TokenEmbedding(Part):
    graph_safe = True
    def __init__(self, rt, vocab_size, hidden_size, names=None, scale=1.0):
        self.rt, self.vocab_size, self.hidden_size, self.scale = rt, vocab_size, hidden_size, float(scale)
        self.names = {"weight": "weight", **(names or {})}
        self.table = None

    def tensor_specs(self):
        return {self.names["weight"]: TensorSpec((self.vocab_size, self.hidden_size), role="embedding")}

    def bind(self, tensors):
        self.table = self._matrix(tensors[self.names["weight"]])

    def output_table(self):
        """The table as an output head reads it when the two are tied: [vocab, hidden] in the compute dtype."""
        return self.table

    def forward(self, token_ids, status=None, add_into=None):
        """The tokens' rows as a new fp32 stream, or (``add_into``) added to an existing one."""
        return kernels.embedding(token_ids, self.table, out=add_into, status=status, scale=self.scale, add=add_into is not None)


class PairEmbedding(TokenEmbedding):
    """The token's row plus a row of a second table that the token and the one before it choose together:
    row (previous * mul_prev + token * mul_cur) mod buckets, or the row after the hashed ones for a sequence's first token.
    The last token of a request's portion is state: one int32 per request slot (``cache_spec``), so that the next portion,
    or the next single token, finds its predecessor whatever the cut.  ``forward_step`` takes the step's batch."""
    needs_batch = True

    def __init__(self, rt, vocab_size, hidden_size, buckets, mul_prev, mul_cur, names=None):
        super().__init__(rt, vocab_size, hidden_size, names={"weight": "embed", "pair": "bigram", **(names or {})})
        if buckets <= 0:
            from ..config.base import ConfigError
            raise ConfigError(f"the second embedding table needs a positive number of hashed rows, not {buckets}")
        self.buckets, self.mul_prev, self.mul_cur = int(buckets), int(mul_prev), int(mul_cur)
        self.pair_table = None

    def tensor_specs(self):
        specs = super().tensor_specs()
        specs[self.names["pair"]] = TensorSpec((self.buckets + 1, self.hidden_size), role="embedding")
        return specs

    def bind(self, tensors):
        super().bind(tensors)
        self.pair_table = self._matrix(tensors[self.names["pair"]])

    def cache_spec(self):
        import torch
        from .base import StateSpec
        return StateSpec((1,), torch.int32)

    def forward(self, token_ids, status=None, add_into=None):
        raise RuntimeError("this embedding looks at the token before: it runs on a step's batch (forward_step)")

    def forward_step(self, batch, cache):
        return kernels.embedding_pair(batch, self.table, self.pair_table, cache.state, self.buckets, self.mul_prev, self.mul_cur,
                                      status=batch.status)


class LMHead(Part):
    graph_safe = True
    def __init__(self, rt, vocab_size, hidden_size, tied=False, names=None):
        self.rt, self.vocab_size, self.hidden_size, self.tied = rt, vocab_size, hidden_size, bool(tied)
        self.names = {"weight": "weight", **(names or {})}
        self.linear = None

    def tensor_specs(self):
        return {self.names["weight"]: TensorSpec((self.vocab_size, self.hidden_size), required=not self.tied)}

    def bind(self, tensors, shared_table=None):
        w = tensors.get(self.names["weight"])
        if w is None:
            if not self.tied or shared_table is None:
                raise ValueError("lm_head: no weight and nothing to tie to")
            self.linear = Linear(shared_table, None, self.rt)
        else:
            self.linear = Linear(self._matrix(w), None, self.rt)

    def forward(self, x):
        return self.linear.forward(x)


register_part("embedding", "embedding", TokenEmbedding, replace=True)
register_part("embedding", "pair_embedding", PairEmbedding, replace=True)
register_part("lm_head", "lm_head", LMHead, replace=True)
