"""What the entry points decide on the host: option names and defaults of the command line, the sizes that
follow from them, and the refusals that need no GPU.

Option names, meanings and defaults are the reference's (src/server/cli.rs:13-36, src/engine/engine.rs:64-86);
the graph buckets follow src/engine/graph.rs:93-97 and the automatic portion size src/engine/engine.rs:600-610.
"""
import json
import subprocess
import sys

import pytest
import torch

import plain_qwen3 as P
from llm_infer_rust_b200 import cli
from llm_infer_rust_b200.engine.engine import Engine, auto_chunked_prefill_size, graph_batch_sizes
from llm_infer_rust_b200.sampling import SamplingParams


def test_option_names_and_defaults_are_the_references():
    a = cli.parse_args(["--model-path", "m"])
    assert (a.model_path, a.max_running_req, a.page_size, a.memory_ratio) == ("m", 256, 16, 0.9)
    assert (a.max_seq_len, a.max_total_tokens, a.chunked_prefill_size, a.cuda_graph_bs) == (None, None, None, None)
    assert (a.max_prefill_tokens_per_batch, a.prefill_cuda_graph_max_tokens) == (8192, 2048)
    assert (a.dtype, a.device, a.log_level, a.disable_cpu_gpu_overlap) == ("auto", "auto", "info", False)
    assert (a.temperature, a.top_k, a.top_p, a.max_tokens, a.ignore_eos) == (0.0, -1, 1.0, 1024, False)
    a = cli.parse_args(["--model-path", "m", "--max-running-req", "4", "--max-seq-len", "99", "--page-size", "8",
                        "--dtype", "float32", "--memory-ratio", "0.5", "--max-total-tokens", "640",
                        "--max-prefill-tokens-per-batch", "0", "--chunked-prefill-size", "-1", "--cuda-graph-bs", "0",
                        "--prefill-cuda-graph-max-tokens", "0", "--disable-cpu-gpu-overlap", "--device", "cuda",
                        "--prompt-ids", "1,2,3", "--prompt-ids", "4", "--temperature", "0.8", "--top-k", "5",
                        "--top-p", "0.9", "--max-tokens", "7", "--ignore-eos", "--seed", "3"])
    assert (a.max_running_req, a.max_seq_len, a.page_size, a.dtype, a.memory_ratio) == (4, 99, 8, "float32", 0.5)
    assert (a.max_total_tokens, a.max_prefill_tokens_per_batch, a.chunked_prefill_size, a.cuda_graph_bs) == (640, 0, -1, 0)
    assert a.disable_cpu_gpu_overlap and a.ignore_eos and a.seed == 3
    assert cli.read_prompts(a) == [[1, 2, 3], [4]]
    # the reference's server options that a launch script may carry over are read and do nothing
    a = cli.parse_args(["--model-path", "m", "--host", "0.0.0.0", "--port", "9001", "--tp-size", "1", "--log-dir", "l",
                        "--attention-backend", "flashinfer", "--trust-remote-code", "--disable-async-metadata",
                        "--enable-consecutive-prefill-overlap", "--log-level", "WARNING"])
    assert a.log_level == "warn" and a.tp_size == 1
    assert cli.given_without_effect(a) == ["--host", "--port", "--log-dir", "--attention-backend", "--trust-remote-code",
                                           "--enable-consecutive-prefill-overlap", "--disable-async-metadata"]
    assert cli.given_without_effect(cli.parse_args(["--model-path", "m"])) == []
    for refused in (["--dtype", "float16"], ["--device", "cpu"], ["--log-level", "loud"], ["--attention-backend", "x"]):
        with pytest.raises(SystemExit):
            cli.parse_args(["--model-path", "m"] + refused)


def test_the_command_line_without_a_model_or_prompts(tmp_path, capsys):
    assert cli.main(["--help"]) == 0 and "--max-running-req" in capsys.readouterr().out
    assert cli.main([]) == 2 and "--model-path is required" in capsys.readouterr().err
    assert cli.main(["--model-path", str(tmp_path), "--random-weights"]) == 2
    assert cli.main(["--model-path", str(tmp_path), "--tp-size", "2"]) == 2 and "only 1" in capsys.readouterr().err
    # random-weights mode writes a model folder and, with no prompts, stops there (no GPU is asked for)
    raw = {"model_type": "qwen3", "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 1, "hidden_size": 32,
           "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 16, "intermediate_size": 48,
           "vocab_size": 61, "tie_word_embeddings": False}
    (tmp_path / "c.json").write_text(json.dumps(raw))
    out = subprocess.run([sys.executable, "-m", "llm_infer_rust_b200", "--model-path", str(tmp_path / "model"),
                          "--random-weights", "--config", str(tmp_path / "c.json"), "--seed", "5"],
                         stdin=subprocess.DEVNULL, capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    assert json.loads((tmp_path / "model" / "config.json").read_text())["vocab_size"] == 61
    assert (tmp_path / "model" / "model.safetensors").stat().st_size > 61 * 32 * 2 * 2


def test_graph_buckets_and_the_automatic_portion_size():
    assert graph_batch_sizes(256) == [1, 2, 4, 8, 16, 32, 64, 128, 256]
    assert graph_batch_sizes(5) == [1, 2, 4, 5] and graph_batch_sizes(1) == [1] and graph_batch_sizes(0) == []
    assert graph_batch_sizes(300) == [1, 2, 4, 8, 16, 32, 64, 128, 256, 300]
    gib = 1024
    assert [auto_chunked_prefill_size(m) for m in (16 * gib, 20 * gib, 59 * gib, 60 * gib, 159 * gib, 183359)] == \
        [2048, 4096, 4096, 8192, 8192, 16384]


def test_sampling_params_of_the_python_entry_point():
    p = SamplingParams()
    assert (p.temperature, p.top_k, p.top_p, p.ignore_eos, p.max_tokens) == (0.0, -1, 1.0, False, 1024)
    n = SamplingParams(0.7, 5, 7.5, False, 0).normalized()
    assert n.top_p == 1.0 and n.max_tokens == 1 and n.top_k == 5


@pytest.mark.skipif(torch.cuda.is_available(), reason="needs a machine without a GPU")
def test_without_a_gpu_the_engine_refuses_loudly(tmp_path):
    raw = {"model_type": "qwen3", "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 1, "hidden_size": 32,
           "num_attention_heads": 2, "intermediate_size": 48, "vocab_size": 61}
    with pytest.raises(RuntimeError, match="no CPU path"):
        Engine(None, random_weights_config=raw)
    out = subprocess.run([sys.executable, "bin/trace_run", "--model", str(tmp_path), "--dtype", "float32",
                          "--out", str(tmp_path / "o"), "--max-tokens", "64"], stdin=subprocess.DEVNULL,
                         capture_output=True, text=True, timeout=120, cwd=str(P.__file__).rsplit("/tests/", 1)[0])
    assert out.returncode != 0 and "config.json" in out.stderr


def test_the_references_all_ones_fixture_on_the_plain_implementation():
    """src/server/components/builder.rs:281-341: a tiny model whose weights are all ones gives equal logits, so greedy
    decoding returns token 0 twice for the prompt [1]."""
    raw = {"model_type": "qwen3", "architectures": ["Qwen3ForCausalLM"], "num_hidden_layers": 1, "hidden_size": 8,
           "num_attention_heads": 2, "num_key_value_heads": 1, "head_dim": 4, "intermediate_size": 16,
           "vocab_size": 11, "tie_word_embeddings": True, "max_position_embeddings": 16}
    from llm_infer_rust_b200 import random_tensors
    weights = {name: torch.ones_like(t) for name, t in random_tensors(raw, 0).items()}
    assert P.plain_generate_greedy(weights, raw, [1], 2) == [0, 0]
    logits = P.plain_forward(weights, raw, [1, 0])
    assert torch.allclose(logits, logits[:, :1].expand_as(logits))
