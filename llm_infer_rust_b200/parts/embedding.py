"""Token embedding and output head."""
from __future__ import annotations

import torch

from ..kernels import ops
from .base import ParamDecl, Part
from .registry import register_part


class TokenEmbedding(Part):
    """h[t] = table[ids[t]], unscaled (reference: src/layers/linear.rs:9-11)."""
    category = "embedding"

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])

    def param_decls(self):
        return {"weight": ParamDecl((self.vocab, self.hidden))}

    def forward(self, token_ids):
        return ops.embedding(token_ids, self.params["weight"], self.env.dtype)


class LinearHead(Part):
    """logits = x W^T in float32, no scale and no soft-cap (reference: src/layers/linear.rs:15-20).

    With ``tied`` and no stored head the weight is the embedding table itself.
    """
    category = "head"
    chainable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.vocab = int(spec["vocab_size"])
        self.hidden = int(spec["hidden_size"])
        self.tied = bool(spec.get("tied", False))

    def param_decls(self):
        return {"weight": ParamDecl((self.vocab, self.hidden))}

    def takes_pending(self, rows: int) -> bool:
        return ops.few_row_takes(rows, self.params["weight"], self.env.dtype, ops.EPI_PLAIN_F32)

    def forward(self, x):
        if isinstance(x, ops.PendingNorm):
            if self.takes_pending(x.shape[0]):
                return ops.few_row_linear(x, self.params["weight"], ops.EPI_PLAIN_F32, lazy=True)
            x = x.materialize()
        return ops.linear(x, self.params["weight"], out_dtype=torch.float32)


register_part("embedding", "token_embedding", TokenEmbedding)
register_part("head", "linear_head", LinearHead)
