"""Command line of the engine.

Option names and meanings are the reference's where it has them
(src/server/cli.rs:13-36, defaults src/engine/engine.rs:64-86).  The reference
serves HTTP; this engine has no server and no tokenizer, so prompts come as
token ids (``--prompt-ids`` or one JSON list per line on standard input) and
results leave as one JSON object per prompt on standard output.
"""
from __future__ import annotations

import argparse
import json
import sys
from typing import List, Optional

USAGE = """Usage: python -m llm_infer_rust_b200 --model-path PATH [options]
Engine options (names and defaults follow the reference's command line):
  --model-path PATH         folder that holds config.json and model.safetensors
  --memory-ratio R          share of the GPU's memory that weights and cache together may take (0.9)
  --max-total-tokens N      upper limit of the cache pool in tokens; whole pages only (none)
  --max-running-req N       how many requests may be live at once (256)
  --max-prefill-tokens-per-batch N  prompt tokens that one step may bring, 0 for no limit (8192)
  --chunked-prefill-size N  prompts longer than this are cut into portions; -1 or 0 never cuts; left out,
                            it is chosen from the GPU's memory
  --cuda-graph-bs N         largest decode batch that replays a CUDA graph, 0 for none (max-running-req)
  --prefill-cuda-graph-max-tokens N  steps with prompt tokens up to this size are captured as a graph when their
                            shape comes again, 0 for none (2048)
  --disable-cpu-gpu-overlap wait for every step's tokens before the next step goes to the GPU (by default a
                            step of decoded tokens is launched while the one before still reports)
  --max-seq-len N           longest sequence of a request, prompt and outputs; no more than the model's
                            max_position_embeddings (8192)
  --page-size N             tokens per cache page (16)
  --dtype NAME              auto (the checkpoint's), bfloat16 or float32
  --device NAME             auto or cuda; there is no CPU path (auto)
  --log-level LEVEL         error, warn, info, debug or trace (info)
  --tp-size N               must be 1: the engine runs on one GPU
Read for the sake of launch scripts written for the reference, and without effect (no HTTP server, one attention
backend, one way of uploading a step's index arrays):
  --host IP  --port PORT  --log-dir PATH  --trust-remote-code  --attention-backend fa|pt|flashinfer
  --enable-consecutive-prefill-overlap  --disable-async-metadata
Prompts and sampling (token ids in, token ids out):
  --prompt-ids IDS          comma-separated token ids; may be given several times (else JSON lists on stdin)
  --temperature T  --top-k K  --top-p P  --max-tokens N  --ignore-eos  --seed S
Random-weights mode (writes the model folder, then serves it if prompts are given):
  --random-weights          write config.json and model.safetensors into --model-path
  --config PATH             config.json to build the random model from
  --seed S                  seed of the random weights (and of sampling)
  --init-std X  --norm-std X   N(0, X) matrices (default 0.02); norm weights 1 + N(0, X) (default 0)
  -h, --help                this text"""


# Options of the reference's server (src/server/cli.rs:13-36) that a launch script may carry over: they are read
# and have no effect.
WITHOUT_EFFECT_VALUED = {"--host": None, "--port": None, "--log-dir": None,
                         "--attention-backend": ["fa", "pt", "flashinfer"]}
WITHOUT_EFFECT_SWITCHES = ("--trust-remote-code", "--enable-consecutive-prefill-overlap", "--disable-async-metadata")


def given_without_effect(args: argparse.Namespace) -> List[str]:
    """The options of the reference's server that were given and do nothing here."""
    def dest(flag):
        return flag.lstrip("-").replace("-", "_")
    return [f for f in WITHOUT_EFFECT_VALUED if getattr(args, dest(f)) is not None] + \
           [f for f in WITHOUT_EFFECT_SWITCHES if getattr(args, dest(f))]


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(prog="llm_infer_rust_b200", usage=USAGE, add_help=False)
    p.add_argument("-h", "--help", action="store_true")
    p.add_argument("--model-path")
    p.add_argument("--memory-ratio", type=float, default=0.9)
    p.add_argument("--max-total-tokens", type=int, default=None)
    p.add_argument("--max-running-req", type=int, default=256)
    p.add_argument("--max-prefill-tokens-per-batch", type=int, default=8192)
    p.add_argument("--chunked-prefill-size", type=int, default=None)
    p.add_argument("--cuda-graph-bs", type=int, default=None)
    p.add_argument("--prefill-cuda-graph-max-tokens", type=int, default=2048)
    p.add_argument("--disable-cpu-gpu-overlap", action="store_true")
    p.add_argument("--max-seq-len", type=int, default=None)
    p.add_argument("--page-size", type=int, default=16)
    p.add_argument("--dtype", default="auto", choices=["auto", "bfloat16", "float32"])
    p.add_argument("--device", default="auto", choices=["auto", "cuda"])
    p.add_argument("--log-level", default="info", type=lambda v: "warn" if v.lower() == "warning" else v.lower(),
                   choices=["trace", "debug", "info", "warn", "error"])
    p.add_argument("--tp-size", type=int, default=1)
    for flag in WITHOUT_EFFECT_VALUED:
        p.add_argument(flag, default=None, choices=WITHOUT_EFFECT_VALUED[flag])
    for flag in WITHOUT_EFFECT_SWITCHES:
        p.add_argument(flag, action="store_true")
    p.add_argument("--prompt-ids", action="append", default=[])
    p.add_argument("--temperature", type=float, default=0.0)
    p.add_argument("--top-k", type=int, default=-1)
    p.add_argument("--top-p", type=float, default=1.0)
    p.add_argument("--max-tokens", type=int, default=1024)
    p.add_argument("--ignore-eos", action="store_true")
    p.add_argument("--seed", type=int, default=0)
    p.add_argument("--random-weights", action="store_true")
    p.add_argument("--config")
    p.add_argument("--init-std", type=float, default=0.02)
    p.add_argument("--norm-std", type=float, default=0.0)
    return p


def parse_args(argv: Optional[List[str]] = None) -> argparse.Namespace:
    return build_parser().parse_args(argv)


def read_prompts(args: argparse.Namespace) -> List[List[int]]:
    prompts = [[int(t) for t in text.split(",") if t.strip()] for text in args.prompt_ids]
    if not prompts and not sys.stdin.isatty():
        for line in sys.stdin:
            line = line.strip()
            if line:
                prompts.append([int(t) for t in json.loads(line)])
    return prompts


def main(argv: Optional[List[str]] = None) -> int:
    args = parse_args(argv)
    if args.help:
        print(USAGE)
        return 0
    if not args.model_path:
        print("--model-path is required\n" + USAGE, file=sys.stderr)
        return 2
    if args.tp_size != 1:
        print("--tp-size: only 1 is supported (this engine runs on one GPU)", file=sys.stderr)
        return 2
    ignored = given_without_effect(args)
    if ignored and args.log_level in ("trace", "debug", "info"):
        print("note: " + ", ".join(ignored) + " accepted, without effect here", file=sys.stderr)
    if args.random_weights:
        if not args.config:
            print("--random-weights needs --config PATH", file=sys.stderr)
            return 2
        from .weights.random_init import write_random_model
        with open(args.config) as fh:
            raw = json.load(fh)
        write_random_model(args.model_path, raw, args.seed, std=args.init_std, norm_std=args.norm_std)
        print(f"wrote {args.model_path}/config.json and model.safetensors", file=sys.stderr)
    prompts = read_prompts(args)
    if not prompts:
        return 0
    from .engine import Engine
    from .sampling import SamplingParams
    engine = Engine(args.model_path, dtype=args.dtype, device=args.device,
                    max_running_req=args.max_running_req, max_seq_len=args.max_seq_len,
                    page_size=args.page_size, memory_ratio=args.memory_ratio,
                    max_total_tokens=args.max_total_tokens,
                    max_prefill_tokens_per_batch=args.max_prefill_tokens_per_batch,
                    chunked_prefill_size=args.chunked_prefill_size, cuda_graph_bs=args.cuda_graph_bs,
                    prefill_cuda_graph_max_tokens=args.prefill_cuda_graph_max_tokens,
                    cpu_gpu_overlap=not args.disable_cpu_gpu_overlap, seed=args.seed, log_level=args.log_level)
    params = SamplingParams(args.temperature, args.top_k, args.top_p, args.ignore_eos, args.max_tokens,
                            args.seed if args.seed else None)
    for prompt, result in zip(prompts, engine.generate(prompts, params)):
        print(json.dumps({"prompt_ids": prompt, "output_ids": result.tokens,
                          "finish_reason": result.finish_reason}), flush=True)
    return 0
