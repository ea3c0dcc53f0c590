"""Feed-forward parts."""
from __future__ import annotations

from ..kernels import ops
from .base import ParamDecl, Part
from .registry import register_part


class SwiGLU(Part):
    """down(silu(gate(x)) * up(x)) with gate and up packed into one matrix, no bias.

    ``gate_up_proj`` is [2 I, H] with the gate rows first (reference:
    src/layers/mlp.rs:7-25, packing src/models/qwen3/model.rs:577-586).
    """
    category = "feed_forward"
    chainable = True

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])

    def param_decls(self):
        return {"gate_up_proj": ParamDecl((2 * self.inter, self.hidden)),
                "down_proj": ParamDecl((self.hidden, self.inter))}

    def takes_pending(self, tokens: int) -> bool:
        """Whether a step of ``tokens`` tokens runs the norm before it as the prologue of the gate/up product."""
        return ops.few_row_takes(tokens, self.params["gate_up_proj"], self.env.dtype, ops.EPI_SWIGLU)

    def forward(self, x):
        if ops.few_row_takes(x.shape[0], self.params["gate_up_proj"], self.env.dtype, ops.EPI_SWIGLU):
            # few tokens: norm (if pending), gate and up projections and silu(gate) * up in one kernel
            return ops.linear(ops.few_row_linear(x, self.params["gate_up_proj"], ops.EPI_SWIGLU, lazy=True),
                              self.params["down_proj"], lazy=True)
        if isinstance(x, ops.PendingNorm):
            x = x.materialize()
        if ops.gemm_tc_pays(x, self.params["gate_up_proj"], ops.GEMM_SWIGLU):
            # many tokens, large matrices: gate and up projections with silu(gate) * up as the epilogue, on tcgen05
            return ops.linear(ops.gemm_tc(x, self.params["gate_up_proj"], ops.GEMM_SWIGLU), self.params["down_proj"])
        gate_up = ops.linear(x, self.params["gate_up_proj"])
        return ops.linear(ops.silu_mul(gate_up), self.params["down_proj"])


register_part("feed_forward", "swiglu", SwiGLU)
