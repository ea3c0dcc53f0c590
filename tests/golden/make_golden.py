#!/usr/bin/env python3
"""Writes the golden logits of the plain implementation for the two tiny configurations.

What these files are, and what they are not.  The reference project (MabinogiX/llm_infer_rust) is a Rust binary over
libtorch; neither cargo nor rustc exists where these tests are written, so its model code can be neither compiled nor
imported and no output of it can be recorded.  The plain implementation (tests/plain_qwen3.py) therefore rests on the
reference's formulas and on the fixed vectors of its own tests.  The files written here come from the plain
implementation ITSELF (float64, rounded to float32): they pin it against drift (an edit that changes a formula, a
default or an order of operations shows up as a changed logit), they do not anchor it to anyone else's code.

    python tests/golden/make_golden.py          # rewrites tests/golden/tiny_A.npz and tiny_B.npz

Weights: llm_infer_rust_b200.random_tensors of the tiny configurations of tests/conftest.py (a counter-based
generator: the same bits everywhere); token ids: torch.randint with the seeds below.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

CASES = {"A": (17, 7), "B": (70, 8)}         # tiny configuration -> (sequence length, seed of the token ids)


def golden_case(name):
    import plain_qwen3 as P
    from conftest import TINY
    from llm_infer_rust_b200 import random_tensors
    v = TINY[name]
    length, seed = CASES[name]
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, v["raw"]["vocab_size"], (length,), generator=g).tolist()
    weights = random_tensors(v["raw"], v["seed"], norm_std=v["norm_std"])
    logits = P.plain_forward(weights, v["raw"], ids).numpy()
    return np.asarray(ids, dtype=np.int32), logits


if __name__ == "__main__":
    for name in CASES:
        ids, logits = golden_case(name)
        np.savez_compressed(os.path.join(HERE, f"tiny_{name}.npz"), ids=ids, logits=logits.astype(np.float32))
        print(f"tiny_{name}.npz: {logits.shape}")
