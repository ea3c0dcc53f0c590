"""Shared fixtures: the tiny configurations, their random weights and model folders.

Tests marked ``gpu`` need a CUDA device; everything else runs on the CPU.
Model folders are written into temporary folders and never kept.
"""
from __future__ import annotations

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        have_gpu = torch.cuda.is_available()
    except Exception:
        have_gpu = False
    if have_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device is visible")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def _base(**kw):
    raw = {"model_type": "qwen3", "architectures": ["Qwen3ForCausalLM"], "eos_token_id": None,
           "hidden_act": "silu", "attention_bias": False}
    raw.update(kw)
    return raw


# Three tiny configurations that differ in every size and option.  A and B are the two
# that the benchmark description names; C adds what the parts take beyond them: a window on
# some layers, one query head per KV head and a head size that is no power of two.
TINY = {
    "A": dict(raw=_base(num_hidden_layers=2, hidden_size=64, num_attention_heads=4, num_key_value_heads=2,
                        head_dim=16, intermediate_size=128, vocab_size=256, rope_theta=10000.0,
                        rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=128),
              seed=0, norm_std=0.0, page_size=4),
    "B": dict(raw=_base(num_hidden_layers=3, hidden_size=96, num_attention_heads=6, num_key_value_heads=2,
                        head_dim=32, intermediate_size=224, vocab_size=509, rope_theta=1e6,
                        rms_norm_eps=1e-5, tie_word_embeddings=False, max_position_embeddings=256),
              seed=1, norm_std=0.1, page_size=16),
    "C": dict(raw=_base(num_hidden_layers=4, hidden_size=80, num_attention_heads=5, num_key_value_heads=5,
                        head_dim=48, intermediate_size=176, vocab_size=301, rope_theta=50000.0,
                        rms_norm_eps=3e-6, tie_word_embeddings=False, max_position_embeddings=320,
                        use_sliding_window=True, sliding_window=40,
                        layer_types=["sliding_attention", "full_attention", "sliding_attention",
                                     "full_attention"]),
              seed=2, norm_std=0.05, page_size=8),
    # D has a head size (64) for which the bfloat16 engine fuses norm, QKV product, per-head norm, rotation
    # and cache store into one kernel when a step brings few tokens.
    "D": dict(raw=_base(num_hidden_layers=2, hidden_size=136, num_attention_heads=4, num_key_value_heads=2,
                        head_dim=64, intermediate_size=200, vocab_size=333, rope_theta=1e5,
                        rms_norm_eps=2e-6, tie_word_embeddings=False, max_position_embeddings=256),
              seed=3, norm_std=0.1, page_size=16),
    # E has the head size (128) of the tcgen05 attention kernels: portions of 64 tokens or more go through them,
    # shorter ones and decoded tokens through the mma.sync kernels and the fused QKV product.
    "E": dict(raw=_base(num_hidden_layers=2, hidden_size=192, num_attention_heads=4, num_key_value_heads=2,
                        head_dim=128, intermediate_size=328, vocab_size=307, rope_theta=1e6,
                        rms_norm_eps=1e-6, tie_word_embeddings=True, max_position_embeddings=512),
              seed=4, norm_std=0.1, page_size=16),
}


@pytest.fixture(scope="session")
def tiny():
    return TINY


@pytest.fixture(scope="session")
def tiny_weights():
    """name -> checkpoint tensors (float32, on the CPU) of each tiny configuration."""
    from llm_infer_rust_b200 import random_tensors
    return {k: random_tensors(v["raw"], v["seed"], norm_std=v["norm_std"]) for k, v in TINY.items()}


@pytest.fixture(scope="session")
def tiny_dirs(tmp_path_factory):
    """name -> a model folder (config.json, model.safetensors) of each tiny configuration."""
    from llm_infer_rust_b200 import write_random_model
    out = {}
    for k, v in TINY.items():
        d = tmp_path_factory.mktemp(f"tiny_{k}")
        write_random_model(str(d), v["raw"], v["seed"], norm_std=v["norm_std"])
        out[k] = str(d)
    return out
