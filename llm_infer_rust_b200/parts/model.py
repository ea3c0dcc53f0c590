"""The generic decoder: embedding, the run list of blocks, final norm, head."""
from __future__ import annotations

from typing import Dict, List

import torch

from ..config.spec import ModelSpec
from ..kernels import ops
from .base import BuildEnv, Part
from .registry import build_part


class DecoderModel:
    """Built from a ``ModelSpec`` alone; knows no architecture.

    Parameter paths: ``embedding.weight``, ``layers.<i>.<child>.<name>`` (children as
    the block names them), ``final_norm.weight``, ``lm_head.weight``.
    """

    def __init__(self, spec: ModelSpec, dtype: torch.dtype, device: torch.device):
        spec.validate()
        self.spec = spec
        self.dtype = dtype
        self.device = torch.device(device)
        env = BuildEnv(dtype, self.device, {})
        for name, pe in spec.position_encodings.items():
            env.position_encodings[name] = build_part("position_encoding", pe, env)
        self.position_encodings = env.position_encodings
        self.embedding = build_part("embedding", spec.embedding, env)
        self.blocks = [build_part("block", layer, env) for layer in spec.layers]
        self.final_norm = build_part("norm", spec.final_norm, env)
        self.lm_head = build_part("head", spec.lm_head, env)
        self.run_list = list(spec.run_list)
        for e, entry in enumerate(self.run_list):
            if entry.reads is not None:
                mine = self.blocks[entry.layer].mixer.cache_spec()
                theirs = self.blocks[self.run_list[entry.reads].layer].mixer.cache_spec()
                if mine != theirs:
                    raise ValueError(f"run list entry {e} reads the cache of entry {entry.reads}, "
                                     f"whose keys and values have another shape or window")

    # ------------------------------------------------------------------ parameters
    def _owners(self) -> Dict[str, Part]:
        owners = {"embedding": self.embedding, "final_norm": self.final_norm, "lm_head": self.lm_head}
        for i, block in enumerate(self.blocks):
            for child, part in block.children().items():
                owners[f"layers.{i}.{child}"] = part
        return owners

    def parameter_shapes(self) -> Dict[str, tuple]:
        return {f"{prefix}.{name}": decl.shape
                for prefix, part in self._owners().items() for name, decl in part.param_decls().items()}

    def bind_parameter(self, path: str, tensor: torch.Tensor) -> None:
        prefix, _, name = path.rpartition(".")
        owner = self._owners().get(prefix)
        if owner is None:
            raise KeyError(f"the model has no part {prefix!r} (parameter {path!r})")
        owner.bind(name, tensor)

    def parameter(self, path: str) -> torch.Tensor:
        prefix, _, name = path.rpartition(".")
        return self._owners()[prefix].params[name]

    def unbound_parameters(self) -> List[str]:
        return [f"{prefix}.{name}" for prefix, part in self._owners().items()
                for name in part.missing_params()]

    def parameter_bytes(self) -> int:
        seen, total = set(), 0
        for part in self._owners().values():
            for t in part.params.values():
                if t.data_ptr() not in seen:
                    seen.add(t.data_ptr())
                    total += t.numel() * t.element_size()
        return total

    # ------------------------------------------------------------------ one step
    def forward(self, ctx, caches) -> torch.Tensor:
        """Run the step's tokens; float32 logits [ctx.num_logits, vocab] at ``ctx.logit_rows``."""
        h = self.embedding.forward(ctx.token_ids)
        residual = None
        for e, entry in enumerate(self.run_list):
            h, residual = self.blocks[entry.layer].forward(h, residual, ctx, caches[e])
        takes = getattr(self.lm_head, "takes_pending", None)
        if not (getattr(self.final_norm, "chainable", False) and getattr(self.lm_head, "chainable", False)):
            ops.flush_chain()
        if residual is None:
            x = self.final_norm.forward(h, rows=ctx.logit_rows)
        elif hasattr(self.final_norm, "pending_add") and takes is not None and takes(ctx.num_logits):
            x = self.final_norm.pending_add(h, residual, rows=ctx.logit_rows, write_residual=False)
        else:
            x = self.final_norm.forward_add(h, residual, rows=ctx.logit_rows, write_residual=False)
        logits = self.lm_head.forward(x)
        ops.flush_chain()                 # nothing waits when the step's logits are handed out
        return logits
