"""Arrangements of a layer's parts."""
from __future__ import annotations

from ..kernels import ops
from .registry import build_part, register_part


class PreNormDeferredAdd:
    """Pre-norm residual block whose adds are folded into the following norm.

    x = norm_in(h + residual); a = mixer(x); x = norm_post(a + residual);
    h = feed_forward(x).  The feed-forward's output is NOT added here: the next
    block's input norm (or the model's final norm) adds it.  The first block gets
    ``residual is None``: then residual = h and x = norm_in(h).
    Reference: src/models/qwen3/model.rs:424-460, :516-534 and :181-208.
    """
    category = "block"

    def __init__(self, layer_spec, env):
        self.spec = layer_spec
        self.input_norm = build_part("norm", layer_spec["input_norm"], env)
        self.post_mixer_norm = build_part("norm", layer_spec["post_mixer_norm"], env)
        self.mixer = build_part("mixer", layer_spec["mixer"], env)
        self.feed_forward = build_part("feed_forward", layer_spec["feed_forward"], env)

    def children(self):
        return {"input_norm": self.input_norm, "mixer": self.mixer,
                "post_mixer_norm": self.post_mixer_norm, "feed_forward": self.feed_forward}

    @staticmethod
    def _fuses(norm, consumer, tokens):
        """A norm is handed on unrun when it can be (``pending_add``) and its consumer ``takes_pending``."""
        takes = getattr(consumer, "takes_pending", None)
        return hasattr(norm, "pending_add") and takes is not None and takes(tokens)

    @staticmethod
    def _settle(part):
        """Products of few rows may wait to be launched together (``ops.few_row_linear``).  A part that says
        ``chainable = True`` touches activations through ``ops`` alone and may be handed such tensors; before any
        other part runs, everything that waits is launched."""
        if not getattr(part, "chainable", False):
            ops.flush_chain()

    def forward(self, h, residual, ctx, cache):
        tokens = h.shape[0]
        self._settle(self.input_norm)
        self._settle(self.mixer)
        if residual is None:
            residual = h
            if hasattr(self.input_norm, "pending") and self._fuses(self.input_norm, self.mixer, tokens):
                x = self.input_norm.pending(h)
            else:
                x = self.input_norm.forward(h)
        elif self._fuses(self.input_norm, self.mixer, tokens):
            x = self.input_norm.pending_add(h, residual)
            residual = x.residual_out
        else:
            x = self.input_norm.forward_add(h, residual, out=h)
        a = self.mixer.forward(x, ctx, cache)
        self._settle(self.post_mixer_norm)
        self._settle(self.feed_forward)
        if self._fuses(self.post_mixer_norm, self.feed_forward, tokens):
            x = self.post_mixer_norm.pending_add(a, residual)
            residual = x.residual_out
        else:
            x = self.post_mixer_norm.forward_add(a, residual, out=a)
        return self.feed_forward.forward(x), residual


register_part("block", "pre_norm_deferred_add", PreNormDeferredAdd)
