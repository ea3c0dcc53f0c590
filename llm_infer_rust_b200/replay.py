"""Trace replay: feed given token ids through the engine step by step and write logits.

It samples nothing and owns no forward pass, cache or loader: it drives
``Engine.step``, the step function that generation uses.

Input, one JSON object a line:
    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}
For a step in which something is wanted, ``<out>/<step>.f32`` receives the logits
at the wanted places, little-endian float32 [wanted, vocab], in the order of the
entries and of ``want``.  After every step a line ``done <step>`` is printed.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Dict, Optional, List


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


def main(argv: Optional[List[str]] = None) -> int:
    ap = argparse.ArgumentParser(prog="trace_run")
    ap.add_argument("--model", required=True)
    ap.add_argument("--dtype", required=True, choices=["bfloat16", "float32"])
    ap.add_argument("--out", required=True)
    ap.add_argument("--max-tokens", type=int, required=True)
    ap.add_argument("--page-size", type=int, default=16)
    args = ap.parse_args(argv)
    os.makedirs(args.out, exist_ok=True)

    from .engine import Engine, StepEntry
    page = args.page_size
    # Each live request's count is rounded up to a multiple of 64 (or of the page, if larger).
    unit = _round_up(64, page)
    pool_tokens = _round_up(max(args.max_tokens, unit), unit)
    engine = Engine(args.model, dtype=args.dtype, max_running_req=8, page_size=page,
                    max_total_tokens=pool_tokens, max_seq_len=None, cuda_graph_bs=0,
                    max_prefill_tokens_per_batch=0, chunked_prefill_size=0)
    ids: Dict[str, int] = {}
    next_id = 1
    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        entries = []
        for e in rec.get("entries", []):
            key = str(e["id"])
            if key not in ids:
                ids[key] = next_id
                engine.open_request(next_id)
                next_id += 1
            entries.append(StepEntry(ids[key], [int(t) for t in e["tokens"]],
                                     [int(i) for i in e.get("want", [])]))
        if entries:
            logits = engine.step(entries)
            if logits.shape[0] > 0:
                data = logits.detach().to("cpu").contiguous().numpy().astype("<f4", copy=False)
                path = os.path.join(args.out, f"{rec['step']}.f32")
                with open(path + ".tmp", "wb") as fh:
                    fh.write(data.tobytes())
                os.replace(path + ".tmp", path)
            engine.check_kernel_errors()
        for key in rec.get("end", []):
            key = str(key)
            if key in ids:
                engine.close_request(ids.pop(key))
        print(f"done {rec['step']}", flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
