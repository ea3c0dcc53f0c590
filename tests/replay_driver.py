"""Drives ``bin/trace_run`` as a user does: a child process, steps on its standard
input, ``done <step>`` lines back, logits read from the files it writes."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from typing import Dict, List, Sequence, Tuple

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TRACE_RUN = os.path.join(ROOT, "bin", "trace_run")


class Replay:
    def __init__(self, model_dir: str, dtype: str, max_tokens: int, out_dir: str, vocab: int,
                 extra: Sequence[str] = ()):
        self.out_dir, self.vocab, self.next_step = out_dir, vocab, 0
        cmd = [sys.executable, TRACE_RUN, "--model", model_dir, "--dtype", dtype, "--out", out_dir,
               "--max-tokens", str(max_tokens), *extra]
        self.proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, bufsize=1)

    def step(self, entries: Sequence[Tuple[str, Sequence[int], Sequence[int]]], end: Sequence[str] = ()):
        """entries: (id, tokens, want).  Returns float32 logits [wanted, vocab] (or None)."""
        n = self.next_step
        self.next_step += 1
        rec = {"step": n, "entries": [{"id": i, "tokens": list(t), "want": list(w)} for i, t, w in entries],
               "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        while True:
            line = self.proc.stdout.readline()
            if not line:
                raise RuntimeError(f"trace_run ended early with code {self.proc.wait()}")
            if line.strip() == f"done {n}":
                break
        wanted = sum(len(w) for _, _, w in entries)
        path = os.path.join(self.out_dir, f"{n}.f32")
        if wanted == 0:
            assert not os.path.exists(path)
            return None
        data = np.fromfile(path, dtype="<f4")
        assert data.size == wanted * self.vocab, (data.size, wanted, self.vocab)
        return data.reshape(wanted, self.vocab)

    def close(self) -> int:
        self.proc.stdin.close()
        code = self.proc.wait(timeout=120)
        self.proc.stdout.close()
        return code


def run_alone(rp: Replay, rid: str, ids: Sequence[int], portions: Sequence[int]) -> np.ndarray:
    """Feed one request in the given portions (all positions wanted), end it; logits [T, vocab]."""
    assert sum(portions) == len(ids)
    out, at = [], 0
    for k, n in enumerate(portions):
        last = k == len(portions) - 1
        out.append(rp.step([(rid, ids[at:at + n], range(n))], end=[rid] if last else []))
        at += n
    return np.concatenate(out)


def mixed_schedule(requests: Dict[str, Tuple[Sequence[int], int]], pool_tokens: int, seed: int,
                   max_live: int = 4):
    """A deterministic schedule of mixed steps.

    requests: id -> (token ids, prompt length): the prompt goes in portions of 2 to 24
    tokens, the rest one token a step.  Up to ``max_live`` requests are live, as long as
    their lengths, each rounded up to 64, fit ``pool_tokens``; now and then a live request
    sits a step out.  Yields (entries, end) with every position wanted.
    """
    rng = np.random.default_rng(seed)
    waiting = list(requests)
    live: List[str] = []
    fed = {r: 0 for r in requests}

    def rounded(r):
        return -(-len(requests[r][0]) // 64) * 64

    while waiting or live:
        while waiting and len(live) < max_live and sum(map(rounded, live)) + rounded(waiting[0]) <= pool_tokens:
            live.append(waiting.pop(0))
        entries, end = [], []
        for r in list(live):
            ids, prompt = requests[r]
            if len(live) > 1 and rng.random() < 0.15:
                continue                                      # left out of this step
            at = fed[r]
            if at < prompt:
                n = int(min(prompt - at, rng.integers(2, 25)))
                if prompt - at - n == 1:                      # never leave a prompt portion of one token
                    n += 1
            else:
                n = 1
            entries.append((r, ids[at:at + n], range(n)))
            fed[r] = at + n
            if fed[r] == len(ids):
                end.append(r)
                live.remove(r)
        if entries:
            yield entries, end
