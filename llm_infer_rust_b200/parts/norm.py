"""RMSNorm with an optional fused residual add."""
from __future__ import annotations

from ..kernels import ops
from .base import ParamDecl, Part
from .registry import register_part


class RMSNorm(Part):
    """y = x * rsqrt(mean(x^2) + eps) * weight, in float, rounded once.

    ``forward_add`` adds a residual first: the float sum is normalised unrounded
    and stored rounded as the new residual (reference: src/layers/ops.rs:8-35,
    src/layers/fused_ops.cu:49-106).
    """
    category = "norm"
    chainable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.width = int(spec["width"])
        self.eps = float(spec["eps"])

    def param_decls(self):
        return {"weight": ParamDecl((self.width,), "vector")}

    def forward(self, x, out=None, rows=None):
        return ops.rms_norm(x, self.params["weight"], self.eps, out=out, rows=rows)

    def forward_add(self, x, residual, out=None, rows=None, write_residual=True):
        return ops.add_rms_norm(x, residual, self.params["weight"], self.eps, out=out, rows=rows,
                                write_residual=write_residual)

    def pending_add(self, x, residual, rows=None, write_residual=True):
        """The same add + norm, not run yet: a consumer that ``takes_pending`` fuses it into its product.
        The new residual will be in ``.residual_out`` of the result (``residual`` itself is left alone)."""
        return ops.PendingNorm(x, residual, self.params["weight"], self.eps, rows=rows,
                               write_residual=write_residual)


    def pending(self, x, rows=None):
        """The plain norm of ``x``, not run yet (for a consumer that ``takes_pending``)."""
        return ops.PendingNorm(x, None, self.params["weight"], self.eps, rows=rows, write_residual=False)


register_part("norm", "rms_norm", RMSNorm)
