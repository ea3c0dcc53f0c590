#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200, with its share of the roofline.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--shape 0.6b|8b|32b] [--layers L]
                    [--batch B] [--context C] [--point-shapes 8b,32b] [--no-points] [--impl ours|reference]

A step is one decode step of a batch of B requests whose context ends at C tokens: the
requests are prefilled with random token ids up to C - W - K tokens, W + K tokens are
decoded greedily, and the last K steps are timed.  One JSON line is printed:

* ``value``: decoded tokens a second, timed on the device (CUDA events around K steps that are
  queued back to back: each step's sampled tokens go to the next step on the device);
* ``e2e``: the same through ``Engine.add_request`` / ``Engine.schedule_step``: prompts go in as
  host token ids, every step's index arrays are copied from pinned host memory, its sampled ids
  are read back to the host and returned to the caller step by step (the scheduler loop launches
  the next decode step before it has read the running one's ids, so a decoded token reaches the
  next step on the device as well as the host);
* ``prefill``: one step of 2,048 prompt tokens; ``frac`` = its FLOPs / time / the bfloat16 peak;
* ``roofline``: bytes that a decode step must read (every weight once and the cache of the live
  requests) / its time, against the measured copy bandwidth;
* ``points``: decoded tokens a second at batch 1 and 64 at the same context and at the headline batch at half the
  context, each with ``_frac``, its share of the roofline (bytes as above / time / measured copy bandwidth); then the
  same figures (``<shape>_decode_b1`` ... ``<shape>_prefill_frac``) for the other shapes of ``--point-shapes``, by
  default the Qwen3-8B and Qwen3-32B layer sizes with all their layers (each engine is built, measured with a quarter
  of the steps and released before the next);
* ``routing``: which products of a decode step ran on this package's few-row kernels and which on the library (a
  rule of sizes, not a measurement: the same line again on the same machine takes the same kernels).

Peaks come from MEASURED_PEAKS.json beside this file when it is there.  Weights are random
(drawn on the device), token ids are synthetic.  One GPU only.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

SHAPES = {
    "0.6b": dict(num_hidden_layers=28, hidden_size=1024, num_attention_heads=16, num_key_value_heads=8,
                 head_dim=128, intermediate_size=3072, vocab_size=151936, tie_word_embeddings=True,
                 max_position_embeddings=40960),
    "8b": dict(num_hidden_layers=36, hidden_size=4096, num_attention_heads=32, num_key_value_heads=8,
               head_dim=128, intermediate_size=12288, vocab_size=151936, tie_word_embeddings=False,
               max_position_embeddings=40960),
    "32b": dict(num_hidden_layers=64, hidden_size=5120, num_attention_heads=64, num_key_value_heads=8,
                head_dim=128, intermediate_size=25600, vocab_size=151936, tie_word_embeddings=False,
                max_position_embeddings=40960),
}
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
REFERENCE_UNAVAILABLE = ("the reference is a Rust binary over libtorch: pip install --no-deps of it succeeds but installs "
                         "metadata only (no module, no binary); building it needs cargo/rustc and torch==2.13.0, "
                         "neither of which this image has")


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.isfile(path):
        with open(path) as fh:
            p = json.load(fh)
        return {k: float(p.get(k, FALLBACK_PEAKS[k])) for k in FALLBACK_PEAKS}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""
    QUERY = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    NAMES = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")

    def __init__(self):
        self.samples, self.proc, self.thread = [], None, None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}",
                                          "--format=csv,noheader,nounits", "-lms", "100"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [x.strip() for x in line.split(",")]
            if len(parts) == 6 and parts[0].isdigit():
                self.samples.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.proc.wait()
        self.thread.join(timeout=2)
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no sample"]}
        reasons = [n for i, n in enumerate(self.NAMES) if any(s[2 + i] == "Active" for s in self.samples)]
        return {"sm_mhz": statistics.median(int(s[0]) for s in self.samples),
                "sm_max_mhz": int(self.samples[0][1]), "reasons": reasons, "samples": len(self.samples)}


def model_numbers(raw):
    """Parameter counts and per-token cache bytes of a dense Qwen3 shape (bfloat16)."""
    L, H, nh, nkv, d = (raw["num_hidden_layers"], raw["hidden_size"], raw["num_attention_heads"],
                        raw["num_key_value_heads"], raw["head_dim"])
    I, V = raw["intermediate_size"], raw["vocab_size"]
    layer_matrix = (nh + 2 * nkv) * d * H + H * nh * d + 3 * I * H
    layer_params = layer_matrix + 2 * H + 2 * d
    head = V * H
    embed = 0 if raw["tie_word_embeddings"] else V * H
    return dict(layer_matrix=layer_matrix, params=L * layer_params + head + embed + H,
                decode_weight_bytes=2 * (L * layer_params + head + H), kv_bytes_per_token=L * 2 * nkv * d * 2)


def prefill_flops(raw, T):
    n = model_numbers(raw)
    L, nh, d = raw["num_hidden_layers"], raw["num_attention_heads"], raw["head_dim"]
    return 2.0 * T * n["layer_matrix"] * L + L * nh * 4.0 * d * T * (T + 1) / 2 + 2.0 * raw["vocab_size"] * raw["hidden_size"]


def random_prompt(vocab, n, seed):
    import torch
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def fill_requests(engine, ids, prompt_len, vocab, chunk=4096):
    """Open the requests and run their prompts through the step function, in portions."""
    from llm_infer_rust_b200.engine import StepEntry
    for r in ids:
        engine.open_request(r)
        prompt = random_prompt(vocab, prompt_len, 1000 + r)
        for at in range(0, prompt_len, chunk):
            engine.step([StepEntry(r, prompt[at:at + chunk], [])])


def decode_device_timed(engine, batch, context, steps, warmup, vocab):
    """Tokens a second of `steps` decode steps that end at `context` tokens, timed on the device."""
    import torch
    from llm_infer_rust_b200 import SamplingParams
    from llm_infer_rust_b200.engine import StepEntry
    from llm_infer_rust_b200.kernels import ops
    ids = list(range(1, batch + 1))
    fill_requests(engine, ids, context - steps - warmup, vocab)
    rows = [(SamplingParams(), 0, 0)] * batch
    entries = [StepEntry(r, [0], [0]) for r in ids]
    tokens = torch.zeros(batch, dtype=torch.int32, device=engine.device)
    for _ in range(warmup):
        tokens = engine.sampler.sample_device(engine.step(entries, device_tokens=tokens), rows)
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = ops.launch_count()
    start.record()
    for _ in range(steps):
        tokens = engine.sampler.sample_device(engine.step(entries, device_tokens=tokens), rows)
    end.record()
    torch.cuda.synchronize()
    launches = ops.launch_count() - launches
    ms = start.elapsed_time(end) / steps
    engine.check_kernel_errors()
    mean_context = context - (steps + 1) / 2.0
    for r in ids:
        engine.close_request(r)
    return dict(tokens_per_s=batch * 1000.0 / ms, ms_per_step=ms, launches=launches, mean_context=mean_context)


def decode_end_to_end(engine, batch, context, steps, warmup, vocab):
    """The same through the public scheduler loop: host token ids in, host token ids out, every step."""
    import torch
    from llm_infer_rust_b200 import SamplingParams
    # prompts enter one a step, so the first request decodes up to `batch` tokens before the last is in
    prompt_len = context - steps - warmup - batch
    sp = SamplingParams(max_tokens=steps + warmup + 2 * batch + 8, ignore_eos=True)
    for r in range(batch):
        engine.add_request(random_prompt(vocab, prompt_len, 2000 + r), sp)
    while engine.scheduler.num_pending() or any(
            engine.scheduler.status_of(u) != engine._rt.Status.Decoding for u in list(engine._params)):
        engine.schedule_step()                               # prompts, in portions
    for _ in range(warmup - 1):
        engine.schedule_step()
    h2d = engine.last_upload_bytes
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    produced = 0
    for _ in range(steps):
        produced += len(engine.schedule_step())
    torch.cuda.synchronize()
    elapsed = time.perf_counter() - t0
    for u in list(engine._params):
        engine.abort_request(u)
    while not engine.is_idle():
        engine.schedule_step()
    assert produced == batch * steps, (produced, batch, steps)
    return dict(tokens_per_s=produced / elapsed, h2d=h2d, d2h=4 * batch)


def prefill_timed(engine, T, vocab, repeats=3):
    import torch
    from llm_infer_rust_b200.engine import StepEntry
    best = None
    for k in range(repeats + 1):
        prompt = random_prompt(vocab, T, 3000 + k)
        engine.open_request(9000 + k)
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        engine.step([StepEntry(9000 + k, prompt, [T - 1])])
        end.record()
        torch.cuda.synchronize()
        engine.close_request(9000 + k)
        if k > 0:                                             # the first run warms up
            ms = start.elapsed_time(end)
            best = ms if best is None else min(best, ms)
    return best


def step_bytes(numbers, batch, mean_context):
    """Bytes that a decode step has to read: every weight once and the cache of the live requests."""
    return numbers["decode_weight_bytes"] + batch * mean_context * numbers["kv_bytes_per_token"]


def routing_of(engine, rows):
    """Which way the products of a step of `rows` tokens go: this package's few-row kernels (the ring kernel, or the
    streaming kernel for the largest weights) or the library."""
    from llm_infer_rust_b200.kernels import ops
    block = engine.model.blocks[0]
    mixer, ff = block.mixer, block.feed_forward
    products = {"qkv": (mixer.params["qkv_proj"], ops.EPI_QKV, mixer.d), "o": (mixer.params["o_proj"], ops.EPI_PLAIN_BF16, 0),
                "gate_up": (ff.params["gate_up_proj"], ops.EPI_SWIGLU, 0), "down": (ff.params["down_proj"], ops.EPI_PLAIN_BF16, 0),
                "head": (engine.model.lm_head.params["weight"], ops.EPI_PLAIN_F32, 0)}
    library = [name for name, (w, mode, d) in products.items() if not ops.few_row_takes(rows, w, engine.dtype, mode, d)]
    streamed = [name for name, (w, mode, d) in products.items()
                if name not in library and mode != ops.EPI_QKV and ops.stream_takes(rows, w, engine.dtype, mode)]
    return (f"{ops.few_row_route} kernel" + (f", streaming kernel for {'+'.join(streamed)}" if streamed else "")
            + (f", library for {'+'.join(library)}" if library else ""))


def build_engine(shape_name, layers, biggest, context):
    from llm_infer_rust_b200.engine import Engine
    shape = dict(SHAPES[shape_name])
    full_layers = shape["num_hidden_layers"]
    if layers:
        shape["num_hidden_layers"] = min(layers, full_layers)
    raw = dict(model_type="qwen3", architectures=["Qwen3ForCausalLM"], rope_theta=1e6, rms_norm_eps=1e-6,
               torch_dtype="bfloat16", eos_token_id=None, **shape)
    pool_tokens = biggest * (context + 128) + 4096
    engine = Engine(None, random_weights_config=raw, random_weights_seed=0, dtype="bfloat16",
                    max_running_req=biggest, max_seq_len=context + 64, page_size=16,
                    max_total_tokens=pool_tokens, cuda_graph_bs=biggest, chunked_prefill_size=4096,
                    prefill_cuda_graph_max_tokens=2048, log_level="warn")
    return engine, raw, full_layers


def release():
    """Give the memory of an engine that the caller has just dropped back to the device (the next engine sizes its
    cache pool from what is free)."""
    import gc
    import torch
    gc.collect()
    torch.cuda.synchronize()
    torch.cuda.empty_cache()


def measure_point_shape(shape_name, context, steps, warmup, peak):
    """Decode at batch 1 / 8 / 64 and a prefill of 2,048 tokens at another shape, each with its share of the roofline."""
    engine, raw, _ = build_engine(shape_name, None, 64, context)
    numbers, vocab = model_numbers(raw), raw["vocab_size"]
    out = {}
    prefill_ms = prefill_timed(engine, 2048, vocab)
    tag = shape_name.replace(".", "")
    out[f"{tag}_prefill_tok_s"] = round(2048 * 1000.0 / prefill_ms, 1)
    out[f"{tag}_prefill_frac"] = round(prefill_flops(raw, 2048) / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)
    for b in (1, 8, 64):
        run = decode_device_timed(engine, b, context, steps, warmup, vocab)
        out[f"{tag}_decode_b{b}"] = round(run["tokens_per_s"], 1)
        out[f"{tag}_decode_b{b}_frac"] = round(step_bytes(numbers, b, run["mean_context"]) / (run["ms_per_step"] * 1e-3) / 1e9
                                               / peak["hbm_gbs"], 4)
    routing = f"{shape_name}: {routing_of(engine, 8)}"
    del engine
    release()
    return out, routing


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--shape", default="0.6b", choices=sorted(SHAPES))
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the shape has")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--context", type=int, default=4096)
    ap.add_argument("--no-points", action="store_true", help="only the headline shape at the headline batch")
    ap.add_argument("--point-shapes", default="8b,32b",
                    help="other shapes measured into `points` (decode at batch 1 / 8 / 64, prefill), comma separated")
    ap.add_argument("--only", choices=["decode", "prefill"], default=None,
                    help="run one phase alone and print a short line (for profiling)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps({"impl": "reference", "unavailable": REFERENCE_UNAVAILABLE}))
        return 0
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)

    biggest = args.batch if (args.no_points or args.only) else max(64, args.batch)
    engine, raw, full_layers = build_engine(args.shape, args.layers, biggest, args.context)
    vocab = raw["vocab_size"]
    numbers = model_numbers(raw)
    peak, peak_source = peaks()

    if args.only == "decode":
        run = decode_device_timed(engine, args.batch, args.context, args.steps, args.warmup, vocab)
        print(json.dumps({"only": "decode", "batch": args.batch, **{k: round(v, 4) for k, v in run.items()}}))
        return 0
    if args.only == "prefill":
        ms = prefill_timed(engine, 2048, vocab, repeats=max(1, args.steps))
        print(json.dumps({"only": "prefill", "tokens": 2048, "ms": round(ms, 3)}))
        return 0
    prefill_ms = prefill_timed(engine, 2048, vocab)
    flops = prefill_flops(raw, 2048)
    points = {}

    def fraction(batch, run):
        return round(step_bytes(numbers, batch, run["mean_context"]) / (run["ms_per_step"] * 1e-3) / 1e9 / peak["hbm_gbs"], 4)

    if not args.no_points:
        for b in (1, 64):
            run = decode_device_timed(engine, b, args.context, args.steps, args.warmup, vocab)
            points[f"decode_b{b}"] = round(run["tokens_per_s"], 1)
            points[f"decode_b{b}_frac"] = fraction(b, run)
        # the same batch at half the context (the decode of a 2,048-token prompt starts there and ends at the headline's)
        half = decode_device_timed(engine, args.batch, args.context // 2, args.steps, args.warmup, vocab)
        points[f"decode_b{args.batch}_c{args.context // 2}"] = round(half["tokens_per_s"], 1)
        points[f"decode_b{args.batch}_c{args.context // 2}_frac"] = fraction(args.batch, half)
    e2e = decode_end_to_end(engine, args.batch, args.context, args.steps, args.warmup, vocab)
    clocks = ClockSampler()
    clocks.start()
    main_run = decode_device_timed(engine, args.batch, args.context, args.steps, args.warmup, vocab)
    clock_record = clocks.stop()
    routing = [f"{args.shape}: {routing_of(engine, args.batch)}"]
    del engine
    release()
    if not args.no_points:
        for name in [n for n in args.point_shapes.split(",") if n and n != args.shape]:
            more, way = measure_point_shape(name, args.context, max(8, args.steps // 4), args.warmup, peak)
            points.update(more)
            routing.append(way)

    achieved = step_bytes(numbers, args.batch, main_run["mean_context"]) / (main_run["ms_per_step"] * 1e-3) / 1e9
    line = {
        "metric": "decode tokens/s", "value": round(main_run["tokens_per_s"], 1), "unit": "tokens/s", "n_gpus": 1,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(main_run["ms_per_step"], 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic token ids, random weights", "impl": "ours",
        "config": {"model": f"Qwen3-{args.shape.upper()} shape", "layers": raw["num_hidden_layers"],
                   "layers_of_shape": full_layers, "hidden": raw["hidden_size"], "heads": raw["num_attention_heads"],
                   "kv_heads": raw["num_key_value_heads"], "head_dim": raw["head_dim"],
                   "intermediate": raw["intermediate_size"], "vocab": vocab, "tied": raw["tie_word_embeddings"],
                   "global_batch": args.batch, "seq_len": args.context,
                   "prompt_len": args.context - args.steps - args.warmup, "page_size": 16,
                   "parallelism": "single GPU", "decode_graphs": True, "prefill_graph": True,
                   "l2": "inputs exceed L2: every step reads all weights and the live cache",
                   "peaks": peak_source},
        "clocks": clock_record,
        "e2e": {"value": round(e2e["tokens_per_s"], 1), "unit": "tokens/s", "h2d_bytes_per_step": e2e["h2d"],
                "d2h_bytes_per_step": e2e["d2h"]},
        "gpu_launches": main_run["launches"],
        "prefill": {"value": round(2048 * 1000.0 / prefill_ms, 1), "tokens": 2048, "ms": round(prefill_ms, 3),
                    "frac": round(flops / (prefill_ms * 1e-3) / (peak["bf16_tflops"] * 1e12), 4)},
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": peak["hbm_gbs"], "unit": "GB/s",
                     "frac": round(achieved / peak["hbm_gbs"], 4)},
        "points": points,
        "routing": "; ".join(routing),
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
