"""Dense Qwen3 as a registry entry: configuration, parts and checkpoint names.

Checkpoint names and packing follow the reference
(src/models/qwen3/model.rs:229-263, :543-586): per layer ``input_layernorm``,
``self_attn.{q,k,v,o}_proj``, ``self_attn.{q,k}_norm``,
``post_attention_layernorm``, ``mlp.{gate,up,down}_proj``; q, k, v rows are
packed in that order into one matrix, gate rows before up rows.  A stored
``lm_head.weight`` is loaded even when the embeddings are tied; without one a
tied model shares the embedding table and an untied one is in error.
"""
from __future__ import annotations

from typing import List

from ..config.qwen3 import Qwen3Config
from ..config.registry import Architecture, register_architecture
from ..weights.plan import SourceTensor, WeightBinding


def qwen3_weight_plan(c: Qwen3Config) -> List[WeightBinding]:
    h, d = c.hidden_size, c.head_dim
    q_rows, kv_rows = c.num_attention_heads * d, c.num_key_value_heads * d
    plan = [WeightBinding("embedding.weight",
                          (SourceTensor("model.embed_tokens.weight", (c.vocab_size, h)),))]
    for i in range(c.num_hidden_layers):
        src, dst = f"model.layers.{i}.", f"layers.{i}."
        plan += [
            WeightBinding(dst + "input_norm.weight",
                          (SourceTensor(src + "input_layernorm.weight", (h,), "norm"),)),
            WeightBinding(dst + "mixer.qkv_proj", (
                SourceTensor(src + "self_attn.q_proj.weight", (q_rows, h)),
                SourceTensor(src + "self_attn.k_proj.weight", (kv_rows, h)),
                SourceTensor(src + "self_attn.v_proj.weight", (kv_rows, h)))),
            WeightBinding(dst + "mixer.q_norm",
                          (SourceTensor(src + "self_attn.q_norm.weight", (d,), "norm"),)),
            WeightBinding(dst + "mixer.k_norm",
                          (SourceTensor(src + "self_attn.k_norm.weight", (d,), "norm"),)),
            WeightBinding(dst + "mixer.o_proj",
                          (SourceTensor(src + "self_attn.o_proj.weight", (h, q_rows)),)),
            WeightBinding(dst + "post_mixer_norm.weight",
                          (SourceTensor(src + "post_attention_layernorm.weight", (h,), "norm"),)),
            WeightBinding(dst + "feed_forward.gate_up_proj", (
                SourceTensor(src + "mlp.gate_proj.weight", (c.intermediate_size, h)),
                SourceTensor(src + "mlp.up_proj.weight", (c.intermediate_size, h)))),
            WeightBinding(dst + "feed_forward.down_proj",
                          (SourceTensor(src + "mlp.down_proj.weight", (h, c.intermediate_size)),)),
        ]
    plan.append(WeightBinding("final_norm.weight", (SourceTensor("model.norm.weight", (h,), "norm"),)))
    plan.append(WeightBinding("lm_head.weight", (SourceTensor("lm_head.weight", (c.vocab_size, h)),),
                              optional=c.tie_word_embeddings,
                              alias_of="embedding.weight" if c.tie_word_embeddings else None))
    return plan


QWEN3 = Architecture(name=Qwen3Config.architecture, model_type=Qwen3Config.model_type,
                     parse_config=Qwen3Config.parse, model_spec=Qwen3Config.model_spec,
                     weight_plan=qwen3_weight_plan, checkpoint_dtype=lambda c: c.checkpoint_dtype,
                     stop_ids=lambda c: c.eos_token_ids)

register_architecture(QWEN3, replace=True)
