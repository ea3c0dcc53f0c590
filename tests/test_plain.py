"""Self-checks of the plain implementation and fixed vectors from the reference's tests.

The plain implementation is the oracle of every other test, so it is checked
against properties that follow from the formulas alone (causality, the GQA head
mapping, the relative-position property of the rotation, tied and untied heads)
and against the fixtures that the reference's own unit tests spell out
(src/layers/ops.rs:455-523, src/engine/sampling.rs:455-548, :736-757).
"""
import math

import pytest
import torch

import plain_qwen3 as P


def test_causality(tiny, tiny_weights):
    for name in ("A", "B", "C", "D", "E"):
        raw, w = tiny[name]["raw"], tiny_weights[name]
        g = torch.Generator().manual_seed(3)
        ids = torch.randint(0, raw["vocab_size"], (50,), generator=g).tolist()
        base = P.plain_forward(w, raw, ids)
        changed = list(ids)
        changed[30] = (changed[30] + 1) % raw["vocab_size"]
        other = P.plain_forward(w, raw, changed)
        assert torch.equal(base[:30], other[:30])
        assert not torch.allclose(base[30:], other[30:])
        assert torch.allclose(P.plain_forward(w, raw, ids[:20]), base[:20], atol=1e-12)


def test_gqa_head_mapping_and_scale():
    t, heads, kv, d = 5, 6, 2, 8
    g = torch.Generator().manual_seed(0)
    q = torch.randn(t, heads, d, generator=g, dtype=torch.float64)
    k = torch.randn(t, kv, d, generator=g, dtype=torch.float64)
    v = torch.randn(t, kv, d, generator=g, dtype=torch.float64)
    out = P.plain_attention(q, k, v).view(t, heads, d)
    for h in range(heads):
        kh = h // (heads // kv)
        for p in range(t):
            s = (k[: p + 1, kh] @ q[p, h]) / math.sqrt(d)
            want = torch.softmax(s, 0) @ v[: p + 1, kh]
            assert torch.allclose(out[p, h], want, atol=1e-12)


def test_window_mask():
    t, d, W = 12, 4, 3
    g = torch.Generator().manual_seed(1)
    q, k, v = (torch.randn(t, 1, d, generator=g, dtype=torch.float64) for _ in range(3))
    out = P.plain_attention(q, k, v, window=W).view(t, d)
    for p in range(t):
        lo = max(0, p - W + 1)
        s = (k[lo: p + 1, 0] @ q[p, 0]) / math.sqrt(d)
        assert torch.allclose(out[p], torch.softmax(s, 0) @ v[lo: p + 1, 0], atol=1e-12)


def test_rope_formula_and_relative_positions():
    # src/layers/ops.rs:497-523: inv_freq = exp(arange(0, d, 2) * (-ln(theta) / d)), positions [0, 15, 3, 15]
    d, theta = 4, 10000.0
    pos = torch.tensor([0, 15, 3, 15])
    phi = P.plain_rope_angles(pos, d, theta, torch.float64)
    want = pos.double()[:, None] * torch.tensor([1.0, theta ** (-0.5)], dtype=torch.float64)[None]
    assert torch.allclose(phi, want, atol=1e-12)
    x = torch.arange(16, dtype=torch.float64).view(4, 1, 4) + 1
    y = P.plain_rope(x, pos, theta)
    assert torch.equal(y[0], x[0])                                  # position 0: no rotation
    c, s = math.cos(15.0), math.sin(15.0)
    assert abs(y[1, 0, 0] - (x[1, 0, 0] * c - x[1, 0, 2] * s)) < 1e-12   # pairs (i, i + d/2)
    assert abs(y[1, 0, 2] - (x[1, 0, 2] * c + x[1, 0, 0] * s)) < 1e-12
    # q.k after rotation depends on the distance only
    g = torch.Generator().manual_seed(2)
    q = torch.randn(1, 1, 16, generator=g, dtype=torch.float64)
    k = torch.randn(1, 1, 16, generator=g, dtype=torch.float64)
    dots = []
    for a, b in ((3, 1), (10, 8), (57, 55)):
        qa = P.plain_rope(q, torch.tensor([a]), 1e6)
        kb = P.plain_rope(k, torch.tensor([b]), 1e6)
        dots.append((qa * kb).sum().item())
    assert max(dots) - min(dots) < 1e-10


def test_residual_add_norm_uses_the_unrounded_sum():
    # src/layers/ops.rs:455-479
    x = torch.ones(1, 1024, dtype=torch.float64)
    r = torch.tensor([0.00390625, 0.0078125], dtype=torch.float64).repeat(512)[None]
    w = torch.ones(1024, dtype=torch.float64)
    y, new_r = P.plain_add_rms_norm(x, r, w, 1e-6, round_to=torch.bfloat16)
    assert torch.equal(y, torch.ones_like(y))
    assert new_r[0, :2].tolist() == [1.0, 1.0078125]
    rounded_first = P._round(P.plain_rms_norm(new_r, w, 1e-6), torch.bfloat16)
    assert not torch.equal(rounded_first, torch.ones_like(y))


def test_rms_norm_weight_multiplies_directly():
    x = torch.tensor([[3.0, 4.0]], dtype=torch.float64)
    y = P.plain_rms_norm(x, torch.tensor([2.0, 0.0], dtype=torch.float64), 0.0)
    assert torch.allclose(y, torch.tensor([[2 * 3 / math.sqrt(12.5), 0.0]], dtype=torch.float64))


def test_tied_and_untied_heads(tiny, tiny_weights):
    raw, w = tiny["A"]["raw"], tiny_weights["A"]
    ids = [1, 2, 3, 4]
    tied = P.plain_forward(w, raw, ids)
    w2 = dict(w)
    w2["lm_head.weight"] = w["model.embed_tokens.weight"] * 2.0
    assert torch.allclose(P.plain_forward(w2, raw, ids), 2.0 * tied)     # a stored head wins
    untied = dict(raw, tie_word_embeddings=False)
    with pytest.raises(KeyError):
        P.plain_forward(w, untied, ids)


def test_run_list_twice_and_shared_cache(tiny, tiny_weights):
    raw, w = tiny["B"]["raw"], tiny_weights["B"]
    ids = list(range(20))
    base = P.plain_forward(w, raw, ids)
    same = P.plain_forward(w, raw, ids, run_list=[{"layer": 0}, {"layer": 1}, {"layer": 2}])
    assert torch.equal(base, same)
    twice = P.plain_forward(w, raw, ids, run_list=[{"layer": 0}, {"layer": 1}, {"layer": 1}, {"layer": 2}])
    shared = P.plain_forward(w, raw, ids, run_list=[{"layer": 0}, {"layer": 1}, {"layer": 2, "reads": 0}])
    assert not torch.allclose(base, twice) and not torch.allclose(base, shared)


def test_greedy_and_filtered_probabilities():
    logits = torch.tensor([[0.1, 2.0, 0.2], [3.0, 1.0, 0.5]])
    assert P.plain_greedy(logits).tolist() == [1, 0]
    probs = torch.tensor([[0.4, 0.3, 0.2, 0.1]])
    f = P.plain_filtered_probs(probs.log(), 1.0, 2, 0.5)
    assert torch.allclose(f, torch.tensor([[4 / 7, 3 / 7, 0, 0]], dtype=torch.float64), atol=1e-9)
    f = P.plain_filtered_probs(probs.log(), 1.0, -1, 1.0)
    assert torch.allclose(f, probs.double(), atol=1e-7)
    # ties at a cut-off are kept
    f = P.plain_filtered_probs(torch.tensor([[0.3, 0.3, 0.3, 0.1]]).log(), 1.0, 1, 1.0)
    assert torch.allclose(f, torch.tensor([[1 / 3, 1 / 3, 1 / 3, 0]], dtype=torch.float64), atol=1e-7)
    # a lower temperature sharpens
    f = P.plain_filtered_probs(probs.log(), 0.5, -1, 1.0)
    assert torch.allclose(f, (probs ** 2 / (probs ** 2).sum()).double(), atol=1e-7)


def test_plain_generation_is_self_consistent(tiny, tiny_weights):
    raw, w = tiny["A"]["raw"], tiny_weights["A"]
    out = P.plain_generate_greedy(w, raw, [5, 9, 17], 4)
    seq = [5, 9, 17] + out
    logits = P.plain_forward(w, raw, seq[:-1])
    assert logits[2:].argmax(-1).tolist() == out


@pytest.mark.parametrize("name", ["A", "B"])
def test_the_plain_implementation_has_not_drifted(name):
    """Against the logits that tests/golden/make_golden.py recorded from this same implementation (see its header for
    what that does and does not prove): same weights, same ids, same logits to float32 rounding."""
    import os
    import sys
    import numpy as np
    here = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
    sys.path.insert(0, here)
    import make_golden
    stored = np.load(os.path.join(here, f"tiny_{name}.npz"))
    ids, logits = make_golden.golden_case(name)
    assert np.array_equal(ids, stored["ids"])
    assert np.abs(logits - stored["logits"]).max() <= 1e-6 * max(1.0, float(np.abs(logits).max()))
