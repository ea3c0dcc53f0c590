"""Grouped-query attention over the paged cache."""
from __future__ import annotations

import math

import torch

from ..kernels import ops
from .base import PagedKVSpec, ParamDecl, Part
from .registry import register_part

_KEYS_PER_CTA_AT_LEAST = 512      # fewer keys per CTA leave its warps' copy pipelines half empty


def decode_splits(ctas_per_split: int, kv_len_bound: int, sm_count: int) -> int:
    """How many CTAs share one row's keys.

    With ``ctas_per_split`` CTAs for each split, the number of splits is chosen so that the
    grid fills whole waves of SMs as well as it can while every CTA keeps at least 512 keys.
    """
    ctas_per_split = max(1, ctas_per_split)
    if 8 * ctas_per_split >= 7 * sm_count:
        # A grid that fills the SMs without splits stays whole: with several waves the splits are combined by a kernel
        # of its own, which costs more than the last wave's idle SMs (measured at 4,096 keys a row: 32 rows x 8 KV
        # heads 90.8 us whole against 103.8 us in the four splits that fill the waves best, 64 rows 177.5 against
        # 182.3 us in two).
        return 1
    most = max(1, min(64, kv_len_bound // _KEYS_PER_CTA_AT_LEAST))
    best, best_fill = 1, 0.0
    for splits in range(1, most + 1):
        if splits == 8 and 2 * ctas_per_split * splits > sm_count:
            # Eight splits of a grid that fits one wave are the CTAs of one cluster, and more than a handful of clusters
            # of eight do not find room side by side: measured at 2 rows x 8 KV heads, 18.1 us against 12.4 us with six
            # splits (one row: 8 clusters of eight, 9.6 us, the best there).
            continue
        ctas = ctas_per_split * splits
        fill = ctas / (sm_count * -(-ctas // sm_count))
        if fill > best_fill * 1.05:
            best, best_fill = splits, fill
    return best


class GQAttention(Part):
    """q, k, v = x W_qkv^T; per-head RMSNorm of q and k; rotary encoding; keys and
    values go to the cache; causal (optionally windowed) attention over the cache;
    output projection.  No bias.

    Order and formulas: src/models/qwen3/model.rs:462-534 of the reference; one
    packed QKV matrix with q rows, then k rows, then v rows (src/layers/linear.rs:25-78).
    Parameters of the part: head counts, head size, the norm's eps (None: no QK
    norm), the window (None: all keys), the softmax scale and the name of the
    model's position encoding.
    """
    category = "mixer"
    chainable = True          # reads its input through ops.* only, and may return a product that still waits (ops.few_row_linear)

    def __init__(self, spec, env):
        super().__init__(spec, env)
        self.hidden = int(spec["hidden_size"])
        self.nh = int(spec["num_heads"])
        self.nkv = int(spec["num_kv_heads"])
        self.d = int(spec["head_dim"])
        self.qk_eps = spec.get("qk_norm_eps")
        self.window = spec.get("window")
        self.scale = float(spec.get("softmax_scale", 1.0 / math.sqrt(self.d)))
        if self.nh % self.nkv:
            raise ValueError("num_heads must be a multiple of num_kv_heads")
        if self.d % 2 or not 2 <= self.d <= 512:
            raise ValueError(f"head_dim {self.d} is refused: the attention kernels take even head sizes up to 512")
        name = spec.get("position_encoding")
        self.rope = env.position_encodings[name] if name else None

    def param_decls(self):
        decls = {"qkv_proj": ParamDecl(((self.nh + 2 * self.nkv) * self.d, self.hidden)),
                 "o_proj": ParamDecl((self.hidden, self.nh * self.d))}
        if self.qk_eps is not None:
            decls["q_norm"] = ParamDecl((self.d,), "vector")
            decls["k_norm"] = ParamDecl((self.d,), "vector")
        return decls

    def cache_spec(self):
        return PagedKVSpec(self.nkv, self.d, self.window)

    def state_spec(self):
        return None

    def takes_pending(self, tokens: int) -> bool:
        """Whether a step of ``tokens`` tokens runs the input norm as the prologue of the QKV product."""
        return ops.few_row_takes(tokens, self.params["qkv_proj"], self.env.dtype, ops.EPI_QKV, self.d)

    def forward(self, x, ctx, cache):
        p = self.params
        tokens = x.shape[0]
        rope = self.rope
        q = torch.empty((tokens, self.nh * self.d), dtype=x.dtype, device=x.device)
        slots = ctx.slots[cache.group] if cache.writes else None
        if ops.few_row_takes(tokens, p["qkv_proj"], self.env.dtype, ops.EPI_QKV, self.d):
            # few tokens: norm (if pending), projection, per-head norm, rotation and cache store in one kernel
            ops.few_row_linear(x, p["qkv_proj"], ops.EPI_QKV, qkv=dict(
                head_dim=self.d, num_heads=self.nh, num_kv_heads=self.nkv, q_out=q, k_cache=cache.k, v_cache=cache.v,
                q_weight=p.get("q_norm"), k_weight=p.get("k_norm"), eps=float(self.qk_eps or 0.0),
                cos=rope.cos if rope else None, sin=rope.sin if rope else None,
                rot_dim=rope.rot_dim if rope else 0, positions=ctx.positions, slots=slots), lazy=True)
        else:
            if isinstance(x, ops.PendingNorm):
                x = x.materialize()
            qkv = ops.linear(x, p["qkv_proj"])
            ops.qkv_post(qkv, q, cache.k, cache.v, p.get("q_norm"), p.get("k_norm"),
                         float(self.qk_eps or 0.0), rope.cos if rope else None, rope.sin if rope else None,
                         rope.rot_dim if rope else 0, ctx.positions, slots, self.nh, self.nkv, self.d)
        out = torch.empty_like(q)
        g = cache.group
        page = ctx.page_sizes[g]
        if ctx.num_prefill:
            ops.prefill_attention(q, cache.k, cache.v, out, ctx.block_tables[g], ctx.cu_q, ctx.kv_len,
                                  ctx.prefix_len, ctx.prefill_rows, ctx.num_prefill, ctx.max_q_len,
                                  self.nh, self.nkv, self.d, page, self.window, self.scale)
        if ctx.num_decode:
            bound = min(ctx.kv_len_bound, self.window) if self.window else ctx.kv_len_bound
            per_split = ops.decode_ctas_per_split(q.dtype, ctx.num_decode, self.nh, self.nkv, self.d, page)
            splits = decode_splits(per_split, bound, ctx.sm_count)
            need = ops.decode_scratch_floats(ctx.num_decode, self.nh, self.d, splits)
            scratch = ctx.scratch(need) if need else None
            ops.decode_attention(q, cache.k, cache.v, out, scratch, ctx.block_tables[g], ctx.cu_q,
                                 ctx.kv_len, ctx.decode_rows, ctx.num_decode, self.nh, self.nkv, self.d,
                                 page, self.window, self.scale, splits)
        return ops.linear(out, p["o_proj"], lazy=True)


register_part("mixer", "gqa_attention", GQAttention)
