"""Plain, slow, whole-sequence implementation of the dense Qwen3 decoder.

This file is the oracle of the test-suite.  It shares no code with the product
package: it reads ``config.json`` keys and checkpoint tensor names by itself,
keeps no cache, runs one sequence at a time and has one function per part.

It rests on the formulas of the reference project (MabinogiX/llm_infer_rust),
not on running it: the reference is Rust over libtorch and neither ``cargo``
nor ``rustc`` exists where these tests are written, so its model code can be
neither imported nor compiled here.  Every function cites the lines of the
reference that give the formula (paths are relative to the reference's root).

All arithmetic runs in ``dtype`` (float64 by default: the ground truth that the
float32 engine is compared with).  ``round_to`` optionally rounds the values at
the places where an engine with 16-bit activations stores a tensor, so that a
bfloat16 engine can be compared with a model of its own rounding.

Two options go beyond what the reference accepts, because the engine's parts
take them as parameters: a sliding window on chosen layers (the reference
rejects ``use_sliding_window``, src/models/qwen3/config.rs:105-126; the mask used
here is ``p - W < j <= p``), and a run list that may name a layer twice or let a
layer read the keys and values that an earlier entry of the list wrote.
"""
from __future__ import annotations

import math
from typing import Dict, List, Optional, Sequence

import torch


def _round(x: torch.Tensor, round_to: Optional[torch.dtype]) -> torch.Tensor:
    if round_to is None:
        return x
    return x.to(round_to).to(x.dtype)


# --------------------------------------------------------------------------- config
def plain_config(raw: dict) -> dict:
    """Sizes and constants from config.json keys with the reference's defaults.

    src/models/qwen3/config.rs:30-41 (defaults: max_position_embeddings 8192,
    rope_theta 10000, rms_norm_eps 1e-6, tie_word_embeddings false),
    :70-94 (num_key_value_heads defaults to the head count, head_dim to
    hidden_size / heads).
    """
    heads = int(raw["num_attention_heads"])
    hidden = int(raw["hidden_size"])
    cfg = {
        "hidden": hidden,
        "layers": int(raw["num_hidden_layers"]),
        "heads": heads,
        "kv_heads": int(raw.get("num_key_value_heads", heads)),
        "head_dim": int(raw.get("head_dim", hidden // heads)),
        "inter": int(raw["intermediate_size"]),
        "vocab": int(raw["vocab_size"]),
        "theta": float(raw.get("rope_theta", 10000.0)),
        "eps": float(raw.get("rms_norm_eps", 1e-6)),
        "tie": bool(raw.get("tie_word_embeddings", False)),
        "max_pos": int(raw.get("max_position_embeddings", 8192)),
    }
    windows: List[Optional[int]] = [None] * cfg["layers"]
    if raw.get("use_sliding_window", False):
        w = int(raw["sliding_window"])
        types = raw.get("layer_types")
        if types is not None:
            windows = [w if t == "sliding_attention" else None for t in types]
        else:
            first = int(raw.get("max_window_layers", 0))
            windows = [w if i >= first else None for i in range(cfg["layers"])]
    cfg["windows"] = windows
    return cfg


# --------------------------------------------------------------------------- parts
def plain_embedding(ids: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """h[t] = E[ids[t]], no scaling.  src/layers/linear.rs:9-11, src/models/qwen3/model.rs:176."""
    return table[ids.long()]


def plain_rms_norm(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * w; the weight multiplies directly.

    src/layers/ops.rs:13-17 (eager), src/layers/fused_ops.cu:49-56 (CUDA).
    """
    var = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(var + eps) * w


def plain_add_rms_norm(x, residual, w, eps, round_to=None):
    """s = x + r; r' = round(s); y = rms_norm(s) on the UNROUNDED sum.

    src/layers/ops.rs:32-34, src/layers/fused_ops.cu:95-105; the fixture that
    tells the two roundings apart is src/layers/ops.rs:455-479.
    """
    s = x + residual
    return _round(plain_rms_norm(s, w, eps), round_to), _round(s, round_to)


def plain_rope_angles(positions: torch.Tensor, rot_dim: int, theta: float, dtype) -> torch.Tensor:
    """phi[p, i] = p * exp(-ln(theta) * 2i / d), i in [0, d/2).  src/layers/ops.rs:84-88."""
    i = torch.arange(0, rot_dim, 2, dtype=dtype)
    inv_freq = torch.exp(i * (-(math.log(theta) / rot_dim)))
    return positions.to(dtype)[:, None] * inv_freq[None, :]


def plain_rope(x: torch.Tensor, positions: torch.Tensor, theta: float) -> torch.Tensor:
    """Half-split rotation of [T, heads, d] over the full head size.

    out[:d/2] = x[:d/2] cos - x[d/2:] sin; out[d/2:] = x[d/2:] cos + x[:d/2] sin.
    src/layers/ops.rs:120-127, src/layers/fused_ops.cu:125-132.
    """
    d = x.shape[-1]
    phi = plain_rope_angles(positions, d, theta, x.dtype)
    cos, sin = torch.cos(phi)[:, None, :], torch.sin(phi)[:, None, :]
    a, b = x[..., : d // 2], x[..., d // 2:]
    return torch.cat([a * cos - b * sin, b * cos + a * sin], dim=-1)


def plain_qkv(x, wq, wk, wv, heads, kv_heads, head_dim):
    """q, k, v = x Wq^T, x Wk^T, x Wv^T without bias, viewed [T, heads, d].

    src/layers/linear.rs:61-77 (one packed weight, three views),
    src/models/qwen3/model.rs:563-576 (row order q, k, v).
    """
    t = x.shape[0]
    q = (x @ wq.T).view(t, heads, head_dim)
    k = (x @ wk.T).view(t, kv_heads, head_dim)
    v = (x @ wv.T).view(t, kv_heads, head_dim)
    return q, k, v


def plain_qk_norm(q, k, wq_norm, wk_norm, eps):
    """RMSNorm over head_dim of every q and k head, before RoPE; v untouched.

    src/models/qwen3/model.rs:474-480, src/layers/ops.rs:39-51.
    """
    return plain_rms_norm(q, wq_norm, eps), plain_rms_norm(k, wk_norm, eps)


def plain_attention(q, k, v, window: Optional[int] = None, round_to=None) -> torch.Tensor:
    """Causal grouped-query attention of one whole sequence.

    Query head h reads KV head h // (heads / kv_heads); S = q k^T / sqrt(d);
    key j is visible to the query at position p iff j <= p (and p - W < j with
    a window); softmax over keys; o = P v.
    src/models/attention/backend.rs:1463-1498 (scale, repeat_interleave, -inf
    mask, softmax, P v), :1455-1461 (mask j > prefix + i).
    """
    t, heads, d = q.shape
    g = heads // k.shape[1]
    kk = k.repeat_interleave(g, dim=1).transpose(0, 1)      # [heads, T, d]
    vv = v.repeat_interleave(g, dim=1).transpose(0, 1)
    qq = q.transpose(0, 1)
    s = (qq @ kk.transpose(1, 2)) * (1.0 / math.sqrt(d))
    p = torch.arange(t)[:, None]
    j = torch.arange(t)[None, :]
    blocked = j > p
    if window is not None:
        blocked = blocked | (j <= p - window)
    s = s.masked_fill(blocked[None], float("-inf"))
    prob = torch.softmax(s, dim=-1)
    o = prob @ vv
    return _round(o.transpose(0, 1).reshape(t, heads * d), round_to)


def plain_swiglu(x, w_gate, w_up, w_down, round_to=None):
    """down(silu(x Wg^T) * (x Wu^T)), silu(z) = z / (1 + exp(-z)), no bias.

    src/layers/mlp.rs:21-24, src/layers/ops.rs:54-61, src/layers/fused_ops.cu:142-144.
    """
    g = _round(x @ w_gate.T, round_to)
    u = _round(x @ w_up.T, round_to)
    m = _round(g / (1.0 + torch.exp(-g)) * u, round_to)
    return _round(m @ w_down.T, round_to)


def plain_lm_head(x, w_lm):
    """logits = x W_lm^T, no scale and no soft-cap.  src/layers/linear.rs:15-20."""
    return x @ w_lm.T


# --------------------------------------------------------------------------- model
def plain_forward(weights: Dict[str, torch.Tensor], raw_config: dict, ids: Sequence[int],
                  dtype=torch.float64, round_to: Optional[torch.dtype] = None,
                  run_list: Optional[Sequence[dict]] = None) -> torch.Tensor:
    """Logits [T, vocab] of one whole sequence.

    Order of operations: src/models/qwen3/model.rs:155-221 (embedding, layers,
    final norm, head) and :424-534 (one layer: input norm, QKV, QK norm, RoPE,
    attention, o_proj, post-attention add-norm, SwiGLU).  The output of the
    feed-forward is not added inside the layer: the add is folded into the next
    layer's input norm and the last one into the final norm (:181-208).

    ``run_list``: entries ``{"layer": i, "reads": e}``; ``layer`` is the index
    of the weights to run, ``reads`` (optional) the index of an earlier ENTRY
    whose keys and values this entry attends to instead of its own.
    """
    cfg = plain_config(raw_config)
    w = {n: t.to(dtype) for n, t in weights.items()}
    ids_t = torch.as_tensor(list(ids), dtype=torch.long)
    pos = torch.arange(len(ids_t))
    if run_list is None:
        run_list = [{"layer": i} for i in range(cfg["layers"])]

    h = plain_embedding(ids_t, w["model.embed_tokens.weight"])
    residual = None
    kv_of_entry = []
    for entry in run_list:
        li = entry["layer"]
        pre = f"model.layers.{li}."
        if residual is None:
            residual = h
            x = _round(plain_rms_norm(h, w[pre + "input_layernorm.weight"], cfg["eps"]), round_to)
        else:
            x, residual = plain_add_rms_norm(h, residual, w[pre + "input_layernorm.weight"],
                                             cfg["eps"], round_to)
        q, k, v = plain_qkv(x, w[pre + "self_attn.q_proj.weight"], w[pre + "self_attn.k_proj.weight"],
                            w[pre + "self_attn.v_proj.weight"], cfg["heads"], cfg["kv_heads"],
                            cfg["head_dim"])
        q, k, v = _round(q, round_to), _round(k, round_to), _round(v, round_to)
        q, k = plain_qk_norm(q, k, w[pre + "self_attn.q_norm.weight"],
                             w[pre + "self_attn.k_norm.weight"], cfg["eps"])
        q = _round(plain_rope(q, pos, cfg["theta"]), round_to)
        k = _round(plain_rope(k, pos, cfg["theta"]), round_to)
        kv_of_entry.append((k, v))
        if entry.get("reads") is not None:
            k, v = kv_of_entry[entry["reads"]]
        a = plain_attention(q, k, v, cfg["windows"][li], round_to)
        o = _round(a @ w[pre + "self_attn.o_proj.weight"].T, round_to)
        x, residual = plain_add_rms_norm(o, residual, w[pre + "post_attention_layernorm.weight"],
                                         cfg["eps"], round_to)
        h = plain_swiglu(x, w[pre + "mlp.gate_proj.weight"], w[pre + "mlp.up_proj.weight"],
                         w[pre + "mlp.down_proj.weight"], round_to)
    if residual is None:
        x = _round(plain_rms_norm(h, w["model.norm.weight"], cfg["eps"]), round_to)
    else:
        x, _ = plain_add_rms_norm(h, residual, w["model.norm.weight"], cfg["eps"], round_to)
    w_lm = w.get("lm_head.weight")
    if w_lm is None:
        # src/models/qwen3/model.rs:250-263: a stored lm_head wins; else tied; else an error.
        if not cfg["tie"]:
            raise KeyError("lm_head.weight is missing and tie_word_embeddings is false")
        w_lm = w["model.embed_tokens.weight"]
    return plain_lm_head(x, w_lm)


# --------------------------------------------------------------------------- sampling
def plain_greedy(logits: torch.Tensor) -> torch.Tensor:
    """argmax over the vocabulary.  src/engine/sampling.rs:244-246."""
    return logits.argmax(dim=-1)


def plain_filtered_probs(logits: torch.Tensor, temperature: float, top_k: int, top_p: float) -> torch.Tensor:
    """Distribution that temperature sampling with joint top-k / top-p draws from.

    probs = softmax(logits / T); both cut-offs are found on that one
    distribution and ties at a cut-off are kept: the k-th largest value, and
    the value at which the descending cumulative sum first reaches top_p;
    what is below either is removed and the rest renormalised.
    src/engine/sampling.rs:251-268 and :409-428.
    """
    scaled = logits.double() / temperature
    probs = torch.softmax(scaled, dim=-1)
    vocab = logits.shape[-1]
    keep = torch.ones_like(probs, dtype=torch.bool)
    if 0 < top_k < vocab:
        kth = torch.topk(probs, top_k, dim=-1).values[..., -1:]
        keep &= probs >= kth
    if top_p < 1.0:
        srt = torch.sort(probs, dim=-1, descending=True).values
        crossing = (srt.cumsum(-1) < top_p).sum(-1, keepdim=True).clamp_max(vocab - 1)
        keep &= probs >= srt.gather(-1, crossing)
    kept = torch.where(keep, probs, torch.zeros_like(probs))
    return kept / kept.sum(-1, keepdim=True)


def plain_generate_greedy(weights, raw_config, prompt: Sequence[int], new_tokens: int,
                          dtype=torch.float64) -> List[int]:
    """Greedy continuation by re-running the whole sequence for every token."""
    seq = list(prompt)
    out = []
    for _ in range(new_tokens):
        nxt = int(plain_greedy(plain_forward(weights, raw_config, seq, dtype)[-1]))
        out.append(nxt)
        seq.append(nxt)
    return out
