"""Layers of real size: the bfloat16 engine against the plain implementation and against the float32 engine.

The tiny configurations do not reach what only real sizes switch on: the tcgen05 attention kernels with a grid
larger than the machine (two query tiles per CTA), cluster split-K in the few-row product, the tcgen05 product with
the SwiGLU epilogue, the decode kernel with several splits, CUDA graphs over real layer sizes.  Here models with
the layer sizes of Qwen3-0.6B and Qwen3-8B (fewer layers, a smaller vocabulary) run the same token sequences through
the float32 engine (true 32-bit kernels) and through the bfloat16 engine; both read the same bfloat16-rounded weights,
and both are compared with the plain implementation on those weights (in float32 on the CPU: a fault that the two
engines share, in the batch arrays, in block tables beyond 2,048 tokens or in page arithmetic at width 4,096, would
pass a comparison of one engine with the other).

Tolerances as in the replay tests: 2^-5 of the logits' scale for the bfloat16 engine; 1e-4 for the float32 engine
against the float32 plain implementation (two float32 computations of sums of up to 12,288 terms in different orders).
"""
import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu

BASE = {"model_type": "qwen3", "architectures": ["Qwen3ForCausalLM"], "eos_token_id": None, "hidden_act": "silu",
        "attention_bias": False, "head_dim": 128, "vocab_size": 4099, "rope_theta": 1e6, "rms_norm_eps": 1e-6,
        "max_position_embeddings": 4096}
SHAPES = {
    # the layer sizes of Qwen3-0.6B and of Qwen3-8B (where the tcgen05 product with the SwiGLU epilogue pays)
    "0.6b": dict(BASE, num_hidden_layers=3, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8,
                 intermediate_size=3072, tie_word_embeddings=True),
    "8b": dict(BASE, num_hidden_layers=1, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
               intermediate_size=12288, tie_word_embeddings=False),
}


def tokens(n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, BASE["vocab_size"], (n,), generator=g).tolist()


def run(engine, plan, seqs):
    """plan: steps of (request, count); every fed position's logits come back, per request in order."""
    from llm_infer_rust_b200.engine import StepEntry
    fed = {r: 0 for r in seqs}
    got = {r: [] for r in seqs}
    places = {r: [] for r in seqs}
    for step in plan:
        entries = []
        for r, n in step:
            if fed[r] == 0:
                engine.open_request(r)
            # all positions of short portions, the last position of long ones (a logits row is 16 KB)
            want = list(range(n)) if n <= 64 else [n - 1]
            entries.append((r, n, want, StepEntry(r, seqs[r][fed[r]: fed[r] + n], want)))
            places[r] += [fed[r] + i for i in want]
            fed[r] += n
        logits = engine.step([e[3] for e in entries]).float().cpu().numpy()
        at = 0
        for r, n, want, _ in entries:
            got[r].append(logits[at: at + len(want)])
            at += len(want)
    engine.check_kernel_errors()
    for r in seqs:
        engine.close_request(r)
    run.places = places                                       # positions of the rows that came back, per request
    return {r: np.concatenate(v) for r, v in got.items()}


@pytest.mark.parametrize("shape", sorted(SHAPES))
def test_bfloat16_engine_agrees_with_the_float32_engine_at_real_layer_sizes(shape, tmp_path):
    import json
    from llm_infer_rust_b200 import random_tensors
    from llm_infer_rust_b200.engine import Engine
    from llm_infer_rust_b200.weights import write_safetensors
    # stored in bfloat16: the float32 engine widens the same values (drawn once, written as a model folder by hand)
    stored = random_tensors(SHAPES[shape], 11, std=0.03 if shape == "0.6b" else 0.015, norm_std=0.1, dtype="bfloat16")
    folder = str(tmp_path)
    with open(tmp_path / "config.json", "w") as fh:
        json.dump(dict(SHAPES[shape], torch_dtype="bfloat16"), fh)
    write_safetensors(str(tmp_path / "model.safetensors"), stored.items())
    weights = {n: t.float() for n, t in stored.items()}
    seqs = {1: tokens(2700, 1), 2: tokens(333, 2), 3: tokens(40, 3)}
    # request 1: 2,560 tokens at once (160 pairs of tiles for 8 KV heads: the two-tile attention kernel), then a
    # portion of 100 over that prefix, then single tokens; request 2: whole (one tile per CTA), request 3 beside
    # decoded tokens of the others, in steps of at most 16 tokens (the few-row product, the decode kernel in splits)
    plan = [[(1, 2560)], [(1, 100), (2, 333)], [(1, 1), (3, 14)], [(1, 1), (3, 1)]] + [[(1, 1), (3, 1)]] * 6 + \
           [[(1, 1)]] * 8 + [[(3, 8)]]
    common = dict(max_running_req=4, page_size=16, max_total_tokens=4096, max_seq_len=2800)
    ref = run(Engine(folder, dtype="float32", cuda_graph_bs=0, **common), plan, seqs)
    eng = Engine(folder, dtype="bfloat16", cuda_graph_bs=4, **common)
    from llm_infer_rust_b200.kernels import ops
    one_before, two_before = ops.tcgen05_attention_launches()
    got = run(eng, plan, seqs)
    one_after, two_after = ops.tcgen05_attention_launches()
    assert two_after > two_before and one_after > one_before, "both tcgen05 attention kernels must have run"
    again = run(eng, plan, seqs)                       # (graphs replay in both runs: they exist since the engine was built)
    for r in seqs:
        plain = P.plain_forward(weights, SHAPES[shape], seqs[r], dtype=torch.float32).numpy()[run.places[r]]
        bound = max(1.0, float(np.abs(plain).max()))
        for name, g, tol in (("float32 engine", ref[r], 1e-4), ("bfloat16 engine", got[r], 2.0 ** -5)):
            err = np.abs(g - plain).max(axis=1)
            worst = int(err.argmax())
            assert err[worst] <= tol * bound, \
                f"request {r}, {name} against the plain implementation: row {worst} (position {run.places[r][worst]}) " \
                f"is off by {err[worst]:.3e} (allowed {tol * bound:.3e})"
        scale = max(1.0, float(np.abs(ref[r]).max()))
        for name, g in (("first run", got[r]), ("with graphs replayed", again[r])):
            assert g.shape == ref[r].shape
            err = np.abs(g - ref[r]).max(axis=1)
            worst = int(err.argmax())
            assert err[worst] <= 2.0 ** -5 * scale, \
                f"request {r}, {name}: row {worst} is off by {err[worst]:.3e} (allowed {2.0 ** -5 * scale:.3e})"
        # the same kernels ran both times
        assert np.abs(got[r] - again[r]).max() <= 2.0 ** -7 * scale
