"""Trace replay against the plain implementation, in 32-bit and in bfloat16.

The same requests are replayed whole; with the last 32 tokens decoded one by one;
in portions of changing size, down to two tokens; and mixed, up to four live
requests with portions of some beside decoded tokens of others, in a pool so
small that pages are used again.  Every position's logits are compared with the
plain implementation's whole-sequence logits.

Tolerances.  float32 engine against the float64 plain implementation: 1e-5 of
the logits' scale (the reference's own bound for its float path,
src/models/qwen3/model.rs:796).  bfloat16 engine: the plain implementation runs
on the same bfloat16-rounded weights in float64; activations are rounded to
bfloat16 (2^-9 relative) after every operation of 2 to 4 layers, which stays
within 2^-5 of the logits' scale (the reference tests its 16-bit kernels with
0.03125 = 2^-5 absolute, src/layers/ops.rs:280).
"""
import numpy as np
import pytest
import torch

import plain_qwen3 as P
from replay_driver import Replay, mixed_schedule, run_alone

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-5, "bfloat16": 2.0 ** -5}
LENGTHS = {"A": 120, "B": 250, "C": 300, "D": 250, "E": 380}


def tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def oracle(weights, raw, ids, dtype):
    if dtype == "bfloat16":
        weights = {n: t.to(torch.bfloat16) for n, t in weights.items()}
    return P.plain_forward(weights, raw, ids).numpy()


def check(got, want, dtype, what):
    scale = max(1.0, float(np.abs(want).max()))
    err = np.abs(got.astype(np.float64) - want).max(axis=1)
    worst = int(err.argmax())
    assert err[worst] <= TOL[dtype] * scale, \
        f"{what}: position {worst} is off by {err[worst]:.3e} (allowed {TOL[dtype] * scale:.3e}); " \
        f"first position beyond the bound: {int(np.argmax(err > TOL[dtype] * scale))}"


def model_dir(tiny_dirs, tiny, tiny_weights, name, dtype, tmp_path):
    """float32 engine: the float32 folder.  bfloat16 engine: a folder stored in bfloat16."""
    if dtype == "float32":
        return tiny_dirs[name]
    from llm_infer_rust_b200 import write_random_model
    v = tiny[name]
    return write_random_model(str(tmp_path / "bf16_model"), v["raw"], v["seed"], norm_std=v["norm_std"],
                              dtype="bfloat16")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_alone_whole_decoded_and_in_portions(name, dtype, tiny, tiny_weights, tiny_dirs, tmp_path):
    raw, page = tiny[name]["raw"], tiny[name]["page_size"]
    vocab, T = raw["vocab_size"], LENGTHS[name]
    ids = tokens(vocab, T, 10)
    want = oracle(tiny_weights[name], raw, ids, dtype)
    rp = Replay(model_dir(tiny_dirs, tiny, tiny_weights, name, dtype, tmp_path), dtype, 2 * T, str(tmp_path / "out"),
                vocab, ["--page-size", str(page)])
    try:
        whole = run_alone(rp, "whole", ids, [T])
        check(whole, want, dtype, "whole")
        decoded = run_alone(rp, "decoded", ids, [T - 32] + [1] * 32)
        check(decoded, want, dtype, "last 32 decoded")
        sizes, left, k = [], T, 0
        pattern = [2, 17, 3, 2, page, page + 1, 31, 2, 5, 64, 2, 9]
        while left:
            n = min(pattern[k % len(pattern)], left)
            if left - n == 1:
                n += 1
            sizes.append(n)
            left -= n
            k += 1
        portions = run_alone(rp, "portions", ids, sizes)
        check(portions, want, dtype, f"portions {sizes}")
        one_by_one = run_alone(rp, "first", ids[:40], [1] * 40)        # the first tokens of a sequence
        check(one_by_one, want[:40], dtype, "the first 40 tokens one by one")
        if dtype == "float32":
            # the same arithmetic runs however the tokens are cut: far below the bound
            for other, what in ((decoded, "decoded"), (portions, "portions")):
                assert np.abs(other - whole).max() <= 2e-6 * max(1.0, np.abs(want).max()), what
    finally:
        assert rp.close() == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D", "E"])
def test_mixed_with_pages_used_again(name, dtype, tiny, tiny_weights, tiny_dirs, tmp_path):
    raw, page = tiny[name]["raw"], tiny[name]["page_size"]
    vocab, longest = raw["vocab_size"], LENGTHS[name]
    lengths = [longest, 33, longest - 37, 64, 70, 2, longest // 2, 45, 65, longest - 1]
    requests = {}
    for k, n in enumerate(lengths):
        ids = tokens(vocab, n, 100 + k)
        requests[f"r{k}"] = (ids, max(1, n - 32 if k % 2 == 0 else n // 2))
    pool = 2 * (-(-longest // 64) * 64) + 128                 # far less than all requests together
    assert sum(-(-n // 64) * 64 for n in lengths) > 2 * pool
    want = {r: oracle(tiny_weights[name], raw, ids, dtype) for r, (ids, _) in requests.items()}
    got = {r: [] for r in requests}
    rp = Replay(model_dir(tiny_dirs, tiny, tiny_weights, name, dtype, tmp_path), dtype, pool, str(tmp_path / "out"),
                vocab, ["--page-size", str(page)])
    try:
        steps = mixed = 0
        for entries, end in mixed_schedule(requests, pool, seed=5):
            logits = rp.step(entries, end)
            at = 0
            for r, toks, _ in entries:
                got[r].append(logits[at:at + len(toks)])
                at += len(toks)
            steps += 1
            kinds = {len(t) == 1 for _, t, _ in entries}
            mixed += kinds == {True, False}
        assert mixed >= 10, "the schedule must hold steps with portions beside decoded tokens"
    finally:
        assert rp.close() == 0
    for r in requests:
        check(np.concatenate(got[r]), want[r], dtype, f"request {r} of the mixed run")


@pytest.mark.parametrize("name", ["B", "E"])
def test_a_checkpoint_stored_in_32_bit_under_the_bfloat16_engine(name, tiny, tiny_weights, tiny_dirs, tmp_path):
    """A checkpoint that is 32-bit as a whole is converted to the engine's dtype when it is bound (the reference:
    src/models/qwen3/model.rs:616): the logits are those of the weights rounded to bfloat16, and the bfloat16
    products (few-row kernels, tensor-core attention) run, not the 32-bit ones."""
    raw, page = tiny[name]["raw"], tiny[name]["page_size"]
    vocab, T = raw["vocab_size"], LENGTHS[name]
    ids = tokens(vocab, T, 12)
    want = oracle(tiny_weights[name], raw, ids, "bfloat16")
    rp = Replay(tiny_dirs[name], "bfloat16", 2 * T, str(tmp_path / "out"), vocab, ["--page-size", str(page)])
    try:
        check(run_alone(rp, "whole", ids, [T]), want, "bfloat16", "whole")
        check(run_alone(rp, "decoded", ids, [T - 32] + [1] * 32), want, "bfloat16", "last 32 decoded")
        check(run_alone(rp, "portions", ids, [2, 17, 3, 64, T - 86]), want, "bfloat16", "portions")
    finally:
        assert rp.close() == 0


def test_replay_refuses_what_it_cannot_hold(tiny, tiny_dirs, tmp_path):
    raw = tiny["A"]["raw"]
    rp = Replay(tiny_dirs["A"], "float32", 64, str(tmp_path / "out"), raw["vocab_size"], ["--page-size", "4"])
    rp.step([("a", tokens(256, 60, 1), [59])])
    with pytest.raises(RuntimeError, match="ended early"):
        rp.step([("b", tokens(256, 60, 2), [59])])            # the pool holds 64 tokens
    assert rp.proc.wait() != 0
