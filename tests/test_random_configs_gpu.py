"""Configurations drawn at random: the engine against the plain implementation, in 32-bit and in bfloat16.

The tiny configurations of conftest.py are chosen by hand; these are not.  Widths, feed-forward sizes and
vocabularies are any number (odd ones too: no vector load may assume a multiple of 8), head counts and groups
are free, pages hold 1 to 64 tokens, some layers have a window.  Head sizes are mostly those that other tests compile
anyway; two are even numbers that are no multiple of 16 (40 and 72: the all-sizes kernels pad them).  Each sequence is run whole, with its last 24 tokens decoded one by
one, and in portions; tolerances as in the replay tests.
"""
import random

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu

HEAD_SIZES = [16, 32, 48, 64, 128, 40, 72]
TOL = {"float32": 1e-5, "bfloat16": 2.0 ** -5}
T = 200
PLANS = {"whole": [T], "last 24 decoded": [T - 24] + [1] * 24, "portions": [2, 17, 3, 64, 2, 9, 31, 5, 67]}


def drawn(index):
    rng = random.Random(1000 + index)
    layers = rng.choice([1, 2, 3])
    nkv, group = rng.choice([1, 2, 3, 4]), rng.choice([1, 2, 3, 4, 5, 7, 8])
    raw = {"model_type": "qwen3", "architectures": ["Qwen3ForCausalLM"], "eos_token_id": None, "hidden_act": "silu",
           "attention_bias": False, "num_hidden_layers": layers,
           "hidden_size": rng.choice([rng.randrange(32, 320, 2), rng.randrange(32, 320, 8), rng.randrange(33, 321, 2)]),
           "num_attention_heads": nkv * group, "num_key_value_heads": nkv, "head_dim": HEAD_SIZES[index % len(HEAD_SIZES)],
           "intermediate_size": rng.choice([rng.randrange(48, 400, 2), rng.randrange(48, 400, 8), rng.randrange(49, 401, 2)]),
           "vocab_size": rng.randrange(97, 1200), "rope_theta": rng.choice([1e4, 5e4, 1e6]),
           "rms_norm_eps": rng.choice([1e-6, 1e-5, 3e-6]), "tie_word_embeddings": rng.random() < 0.5,
           "max_position_embeddings": 512}
    if rng.random() < 0.4:
        raw.update(use_sliding_window=True, sliding_window=rng.randrange(5, 90),
                   layer_types=[rng.choice(["sliding_attention", "full_attention"]) for _ in range(layers)])
    return raw, rng.choice([1, 2, 4, 8, 16, 16, 32, 64])


def run_plan(engine, ids, sizes):
    from llm_infer_rust_b200.engine import StepEntry
    engine.open_request(1)
    got, at = [], 0
    for n in sizes:
        got.append(engine.step([StepEntry(1, ids[at: at + n], list(range(n)))]).float().cpu().numpy())
        at += n
    engine.check_kernel_errors()
    engine.close_request(1)
    return np.concatenate(got)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("index", range(14))
def test_a_configuration_drawn_at_random(index, dtype, tmp_path):
    from llm_infer_rust_b200 import random_tensors, write_random_model
    from llm_infer_rust_b200.engine import Engine
    raw, page = drawn(index)
    what = {k: raw[k] for k in ("head_dim", "num_attention_heads", "num_key_value_heads", "hidden_size",
                                "intermediate_size", "vocab_size", "num_hidden_layers")}
    what.update(page=page, window=raw.get("sliding_window"))
    g = torch.Generator().manual_seed(index)
    ids = torch.randint(0, raw["vocab_size"], (T,), generator=g).tolist()
    weights = random_tensors(raw, index, norm_std=0.1)
    if dtype == "bfloat16":
        weights = {k: t.to(torch.bfloat16) for k, t in weights.items()}
    want = P.plain_forward(weights, raw, ids).numpy()
    folder = write_random_model(str(tmp_path / "model"), raw, index, norm_std=0.1, dtype=dtype)
    engine = Engine(folder, dtype=dtype, max_running_req=2, page_size=page, max_total_tokens=512, max_seq_len=256,
                    cuda_graph_bs=2 if dtype == "bfloat16" else 0)
    scale = max(1.0, float(np.abs(want).max()))
    for name, sizes in PLANS.items():
        assert sum(sizes) == T
        err = np.abs(run_plan(engine, ids, sizes).astype(np.float64) - want).max(axis=1)
        worst = int(err.argmax())
        assert err[worst] <= TOL[dtype] * scale, \
            f"{what}, {name}: position {worst} is off by {err[worst]:.3e} (allowed {TOL[dtype] * scale:.3e}); " \
            f"first position beyond the bound: {int(np.argmax(err > TOL[dtype] * scale))}"
