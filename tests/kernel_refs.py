"""Plain PyTorch float32 references of the engine's kernels, one function per op.

Each mirrors the semantics of one kernel of ``llm_infer_rust_b200/csrc`` (and,
through it, of the reference's kernels: src/layers/fused_ops.cu,
src/models/attention/kv_store.cu, src/models/attention/backend.rs:1455-1498) with
straightforward tensor code, on whatever device the inputs live.  They share no
code with the package.
"""
from __future__ import annotations

from typing import Optional

import torch


def ref_embedding(ids, table, out_dtype):
    return table.float()[ids.long()].to(out_dtype)


def ref_rms_norm(x, w, eps):
    xf = x.float()
    y = xf * torch.rsqrt((xf * xf).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype)


def ref_add_rms_norm(x, residual, w, eps):
    """Returns (normed, new residual): the float sum is normalised unrounded, stored rounded."""
    s = x.float() + residual.float()
    y = s * torch.rsqrt((s * s).mean(-1, keepdim=True) + eps) * w.float()
    return y.to(x.dtype), s.to(x.dtype)


def ref_silu_mul(gate_up):
    width = gate_up.shape[-1] // 2
    g, u = gate_up[..., :width].float(), gate_up[..., width:].float()
    return (g / (1.0 + torch.exp(-g)) * u).to(gate_up.dtype)


def ref_qkv_post(qkv, q_w, k_w, eps, cos, sin, rot_dim, positions, nh, nkv, d):
    """(q, k, v) as [T, heads, d] in qkv's dtype: per-head norm and rotation in float, one rounding."""
    t = qkv.shape[0]
    x = qkv.float().view(t, nh + 2 * nkv, d)
    q, k, v = x[:, :nh], x[:, nh:nh + nkv], x[:, nh + nkv:]

    def norm(a, w):
        if w is None:
            return a
        return a * torch.rsqrt((a * a).mean(-1, keepdim=True) + eps) * w.float()

    def rope(a):
        if cos is None or rot_dim == 0:
            return a
        half = rot_dim // 2
        c = cos[positions.long()][:, None, :]
        s = sin[positions.long()][:, None, :]
        a1, a2, rest = a[..., :half], a[..., half:rot_dim], a[..., rot_dim:]
        return torch.cat([a1 * c - a2 * s, a2 * c + a1 * s, rest], dim=-1)

    q = rope(norm(q, q_w)).to(qkv.dtype)
    k = rope(norm(k, k_w)).to(qkv.dtype)
    return q, k, v.to(qkv.dtype)


def ref_store_kv(k_cache, v_cache, k, v, slots):
    """cache[page, :, offset] = row for every token (slot = page * page_size + offset); slot 0 (the
    sink) is skipped.  Caches are [pages + 1, kv_heads, page_size, head_dim]."""
    page_size = k_cache.shape[2]
    keep = slots != 0
    page, off = (slots[keep] // page_size).long(), (slots[keep] % page_size).long()
    k_cache[page, :, off] = k[keep]
    v_cache[page, :, off] = v[keep]


def ref_paged_attention(q, k_cache, v_cache, block_table, cu_q, kv_len, prefix_len, nh, nkv, d,
                        page_size, window: Optional[int], scale, rows=None):
    """Causal attention of every listed row over the paged cache; out like q ([T, nh * d]).

    Query i of a row sits at position prefix + i and sees keys j <= that position
    (and > position - window)."""
    out = torch.zeros_like(q)
    qv = q.float().view(-1, nh, d)
    ov = out.view(-1, nh, d)
    # [pages + 1, kv_heads, page_size, d] -> one row of all KV heads per slot
    flat_k = k_cache.float().permute(0, 2, 1, 3).reshape(-1, nkv, d)
    flat_v = v_cache.float().permute(0, 2, 1, 3).reshape(-1, nkv, d)
    g = nh // nkv
    n_rows = cu_q.numel() - 1
    for r in (range(n_rows) if rows is None else [int(x) for x in rows]):
        b, e = int(cu_q[r]), int(cu_q[r + 1])
        total, prefix = int(kv_len[r]), int(prefix_len[r])
        pos = torch.arange(total, device=q.device)
        slot = block_table[r][(pos // page_size).long()].long() * page_size + pos % page_size
        k = flat_k[slot].repeat_interleave(g, dim=1)           # [total, nh, d]
        v = flat_v[slot].repeat_interleave(g, dim=1)
        s = torch.einsum("qhd,khd->hqk", qv[b:e], k) * scale
        p = (prefix + torch.arange(e - b, device=q.device))[:, None]
        blocked = pos[None, :] > p
        if window:
            blocked = blocked | (pos[None, :] <= p - window)
        s = s.masked_fill(blocked[None], float("-inf"))
        ov[b:e] = torch.einsum("hqk,khd->qhd", torch.softmax(s, -1), v).to(q.dtype)
    return out


def ref_linear(x, w, out_dtype=None):
    return (x.float() @ w.float().t()).to(out_dtype or x.dtype)


def ref_filtered_probs(logits, temperature, top_k, top_p):
    """The distribution that joint top-k / top-p sampling draws from (ties at a cut-off kept)."""
    probs = torch.softmax(logits.double() / temperature, -1)
    vocab = logits.shape[-1]
    keep = torch.ones_like(probs, dtype=torch.bool)
    if 0 < top_k < vocab:
        keep &= probs >= torch.topk(probs, top_k, -1).values[..., -1:]
    if top_p < 1.0:
        srt = torch.sort(probs, -1, descending=True).values
        crossing = (srt.cumsum(-1) < top_p).sum(-1, keepdim=True).clamp_max(vocab - 1)
        keep &= probs >= srt.gather(-1, crossing)
    kept = torch.where(keep, probs, torch.zeros_like(probs))
    return kept / kept.sum(-1, keepdim=True)
