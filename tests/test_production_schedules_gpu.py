"""Steps as serving produces them, each against the plain implementation.

The replay tests cut prompts into portions of 2 to 24 tokens; a server's portions are hundreds or thousands of tokens
long and stand beside the decoded tokens of other requests, decode steps replay graphs, and equal portions of a long
prompt replay a graph of their shape.  At head size 128 those steps take other kernels (tcgen05 attention from one
full tile of 128 query vectors on) than anything the small portions reach.  Here:

* portions of 64 to 200 tokens beside one to three decoded tokens and a second, shorter portion, with so few pages
  that they are used again, and a check that the tcgen05 attention kernel ran in steps that also held decoded tokens;
* equal portions replayed as a graph over a growing prefix (``prefill_cuda_graph_max_tokens``);
* decode graphs of 1, 2 and 4 rows and a batch of 3 padded to 4;
* an engine whose weights were drawn on the device (``random_weights_config``), read back and given to the plain
  implementation, and compared with the folder that the same configuration and seed write.

Tolerances as in the replay tests: 1e-5 of the logits' scale in float32, 2^-5 in bfloat16.
"""
import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-5, "bfloat16": 2.0 ** -5}


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


def folder_for(tiny, name, dtype, tmp_path):
    from llm_infer_rust_b200 import write_random_model
    v = tiny[name]
    return write_random_model(str(tmp_path / f"{name}_{dtype}"), v["raw"], v["seed"], norm_std=v["norm_std"], dtype=dtype)


def large_portion_schedule(requests, pool_tokens, seed, max_live=4):
    """Like the replay tests' mixed schedule, with a server's portions: the request that entered last is fed 64 to 200
    prompt tokens a step, one other may get a shorter portion (2 to 40), the rest decode."""
    rng = np.random.default_rng(seed)
    waiting, live, fed = list(requests), [], {r: 0 for r in requests}

    def rounded(r):
        return -(-len(requests[r][0]) // 64) * 64

    while waiting or live:
        while waiting and len(live) < max_live and sum(map(rounded, live)) + rounded(waiting[0]) <= pool_tokens:
            live.append(waiting.pop(0))
        entries, end, short_given = [], [], False
        for r in list(live):
            ids, prompt = requests[r]
            at = fed[r]
            if at < prompt:
                if r == live[-1] or rng.random() < 0.3:
                    n = int(min(prompt - at, rng.integers(64, 201)))
                elif not short_given:
                    n, short_given = int(min(prompt - at, rng.integers(2, 41))), True
                else:
                    continue                                  # waits for a later step
                if prompt - at - n == 1:
                    n += 1
            else:
                n = 1
            entries.append((r, ids[at:at + n]))
            fed[r] = at + n
            if fed[r] == len(ids):
                end.append(r)
                live.remove(r)
        if entries:
            yield entries, end


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_large_portions_beside_decoded_tokens_with_pages_used_again(dtype, tiny, tiny_weights, tmp_path):
    from llm_infer_rust_b200.engine import Engine, StepEntry
    from llm_infer_rust_b200.kernels import ops
    raw, page = tiny["E"]["raw"], tiny["E"]["page_size"]
    vocab = raw["vocab_size"]
    lengths = [420, 130, 500, 96, 333, 260, 70, 480]
    requests = {}
    for k, n in enumerate(lengths):
        ids = tokens(vocab, n, 300 + k)
        requests[k + 1] = (ids, n - (24 if k % 2 == 0 else 9))        # the prompt; the rest is decoded
    pool = 2 * 512 + 128                                               # far less than all requests together
    assert sum(-(-n // 64) * 64 for n in lengths) > 2 * pool
    want = {r: oracle(tiny_weights["E"], raw, ids, dtype) for r, (ids, _) in requests.items()}
    engine = Engine(folder_for(tiny, "E", dtype, tmp_path), dtype=dtype, max_running_req=4, page_size=page,
                    max_total_tokens=pool, cuda_graph_bs=0, max_prefill_tokens_per_batch=0, chunked_prefill_size=0)
    got = {r: [] for r in requests}
    opened = set()
    tcgen05_beside_decoded = with_two_portions = 0
    for entries, end in large_portion_schedule(requests, pool, seed=9):
        for r, _ in entries:
            if r not in opened:
                engine.open_request(r)
                opened.add(r)
        before = sum(ops.tcgen05_attention_launches())
        logits = engine.step([StepEntry(r, toks, list(range(len(toks)))) for r, toks in entries]).float().cpu().numpy()
        ran = sum(ops.tcgen05_attention_launches()) - before
        sizes = [len(t) for _, t in entries]
        if ran and 1 in sizes:
            tcgen05_beside_decoded += 1
        if sum(1 for n in sizes if n > 1) >= 2 and 1 in sizes:
            with_two_portions += 1
        at = 0
        for r, toks in entries:
            got[r].append(logits[at:at + len(toks)])
            at += len(toks)
        for r in end:
            engine.close_request(r)
    engine.check_kernel_errors()
    assert engine.cache.manager.live_requests() == 0 and engine.cache.manager.check() == ""
    assert with_two_portions >= 3, "the schedule must hold steps with two portions beside decoded tokens"
    if dtype == "bfloat16":
        assert tcgen05_beside_decoded >= 5, "the tcgen05 attention kernel must run in steps that also decode"
    for r in requests:
        check(np.concatenate(got[r]), want[r], dtype, f"request {r}")


def test_equal_portions_replay_a_graph_over_a_growing_prefix(tiny, tiny_weights, tmp_path):
    """Head size 128, portions of 128 tokens: from the second portion on the step is captured and replayed (its
    arrays say how long the prefix is); the logits are those of the plain implementation and of the eager engine."""
    from llm_infer_rust_b200.engine import Engine, StepEntry
    raw, page = tiny["E"]["raw"], tiny["E"]["page_size"]
    ids = tokens(raw["vocab_size"], 3 * 128 + 2, 77)          # (the model has 512 positions)
    want = oracle(tiny_weights["E"], raw, ids, "bfloat16")
    folder = folder_for(tiny, "E", "bfloat16", tmp_path)
    common = dict(dtype="bfloat16", max_running_req=2, page_size=page, max_total_tokens=2048, cuda_graph_bs=0,
                  max_prefill_tokens_per_batch=0, chunked_prefill_size=0)
    rows = {}
    for name, graph_tokens in (("eager", 0), ("graphs", 256)):
        engine = Engine(folder, prefill_cuda_graph_max_tokens=graph_tokens, **common)
        engine.open_request(1)
        out = []
        for at in range(0, 3 * 128, 128):
            out.append(engine.step([StepEntry(1, ids[at:at + 128], list(range(128)))]).float().cpu().numpy())
        out.append(engine.step([StepEntry(1, ids[384:386], [0, 1])]).float().cpu().numpy())
        engine.check_kernel_errors()
        rows[name] = np.concatenate(out)
        replayed = [g for g in engine._shape_graphs.values() if g.graph is not None]
        assert len(replayed) == (1 if graph_tokens else 0)
        engine.close_request(1)
    check(rows["graphs"], want, "bfloat16", "portions replayed as a graph")
    check(rows["eager"], want, "bfloat16", "eager portions")
    assert np.abs(rows["graphs"] - rows["eager"]).max() <= 2.0 ** -7 * max(1.0, float(np.abs(want).max()))


@pytest.mark.parametrize("name", ["B", "E"])
def test_decode_graphs_of_every_bucket_against_the_plain_implementation(name, tiny, tiny_weights, tmp_path):
    """Buckets 1, 2 and 4, and three rows padded to four (the padding row points at the sink page): each request's
    logits are the plain implementation's, whatever else sat in the batch."""
    from llm_infer_rust_b200.engine import Engine, StepEntry
    raw, page = tiny[name]["raw"], tiny[name]["page_size"]
    vocab = raw["vocab_size"]
    engine = Engine(folder_for(tiny, name, "bfloat16", tmp_path), dtype="bfloat16", max_running_req=4, page_size=page,
                    max_total_tokens=1024, cuda_graph_bs=4, max_prefill_tokens_per_batch=0, chunked_prefill_size=0)
    assert sorted(engine._graphs) == [1, 2, 4]
    uid = 0
    for rows in (1, 2, 3, 4, 3, 1):
        seqs = {}
        for _ in range(rows):
            uid += 1
            seqs[uid] = tokens(vocab, 37 + 9 * (uid % 5), 500 + uid)
        decoded = 12
        got = {r: [] for r in seqs}
        for r, ids in seqs.items():
            engine.open_request(r)
            n = len(ids) - decoded
            got[r].append(engine.step([StepEntry(r, ids[:n], list(range(n)))]).float().cpu().numpy())
        for k in range(decoded):
            logits = engine.step([StepEntry(r, [ids[len(ids) - decoded + k]], [0]) for r, ids in seqs.items()])
            logits = logits.float().cpu().numpy()
            for i, r in enumerate(seqs):
                got[r].append(logits[i:i + 1])
        engine.check_kernel_errors()
        bucket = next(b for b in sorted(engine._graphs) if b >= rows)
        assert engine._graphs[bucket].graph is not None, f"the graph of {bucket} rows was not captured"
        for r, ids in seqs.items():
            check(np.concatenate(got[r]), oracle(tiny_weights[name], raw, ids, "bfloat16"), "bfloat16",
                  f"{rows} rows in the graph of {bucket}, request {r}")
            engine.close_request(r)
    assert engine.cache.manager.check() == ""


@pytest.mark.parametrize("name", ["A", "B", "E"])
def test_the_streaming_kernel_in_every_place_it_fits(name, tiny, tiny_weights, tmp_path, monkeypatch):
    """The rule of sizes sends only the largest weights to the streaming kernel (csrc/stream_linear.cu), which no tiny
    model has.  With the rule's size set to nothing, every few-row product that fits goes there (output projection,
    gate/up, down projection, head; behind a norm, handing the next norm to the ring kernel's QKV, with 9 to 16 rows
    and rows of x fetched beside the weights): decoded tokens in batches of 1 to 12 rows, eager and as graphs, against
    the plain implementation."""
    from llm_infer_rust_b200.engine import Engine, StepEntry
    from llm_infer_rust_b200.kernels import ops
    monkeypatch.setattr(ops, "stream_min_bytes", 0)
    streamed, real = [0], ops.stream_linear

    def counting(*args, **kwargs):
        streamed[0] += 1
        return real(*args, **kwargs)
    monkeypatch.setattr(ops, "stream_linear", counting)
    raw, page = tiny[name]["raw"], tiny[name]["page_size"]
    vocab = raw["vocab_size"]
    for graphs in (0, 4):
        engine = Engine(folder_for(tiny, name, "bfloat16", tmp_path), dtype="bfloat16", max_running_req=12, page_size=page,
                        max_total_tokens=2048, cuda_graph_bs=graphs, max_prefill_tokens_per_batch=0, chunked_prefill_size=0)
        before = ops.launch_count()
        uid = 0
        for rows in (1, 3, 12):
            seqs = {}
            for _ in range(rows):
                uid += 1
                seqs[uid] = tokens(vocab, 21 + 5 * (uid % 4), 900 + uid)
            decoded = 6
            got = {r: [] for r in seqs}
            for r, ids in seqs.items():
                engine.open_request(r)
                n = len(ids) - decoded
                got[r].append(engine.step([StepEntry(r, ids[:n], list(range(n)))]).float().cpu().numpy())
            for k in range(decoded):
                logits = engine.step([StepEntry(r, [ids[len(ids) - decoded + k]], [0]) for r, ids in seqs.items()])
                logits = logits.float().cpu().numpy()
                for i, r in enumerate(seqs):
                    got[r].append(logits[i:i + 1])
            engine.check_kernel_errors()
            for r, ids in seqs.items():
                check(np.concatenate(got[r]), oracle(tiny_weights[name], raw, ids, "bfloat16"), "bfloat16",
                      f"{rows} rows, graphs {graphs}, request {r}")
                engine.close_request(r)
        assert ops.launch_count() > before and engine.cache.manager.check() == ""
        del engine
    assert streamed[0] > 0                                     # (the rule did route there)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_weights_drawn_on_the_device_are_the_folder_s_weights(dtype, tiny, tmp_path):
    """``Engine(None, random_weights_config=...)`` (the constructor of the benchmark) draws on the device what
    ``write_random_model`` writes for the same configuration and seed; a step on those weights is the plain
    implementation's."""
    from llm_infer_rust_b200 import random_tensors
    from llm_infer_rust_b200.engine import Engine, StepEntry
    v = tiny["D"]
    raw = dict(v["raw"], torch_dtype=dtype)
    engine = Engine(None, random_weights_config=raw, random_weights_seed=v["seed"], dtype=dtype, max_running_req=2,
                    page_size=v["page_size"], max_total_tokens=512, cuda_graph_bs=0)
    written = random_tensors(raw, v["seed"])                   # norm_std 0, as the device draw's default
    plan = engine.arch.weight_plan(engine.config)
    for binding in plan:
        if binding.optional and binding.alias_of is not None:
            continue
        want = torch.cat([written[s.name] for s in binding.sources]).to(engine.dtype)
        assert torch.equal(engine.model.parameter(binding.param).cpu(), want), binding.param
    ids = tokens(raw["vocab_size"], 90, 5)
    engine.open_request(1)
    got = np.concatenate([engine.step([StepEntry(1, ids[:70], list(range(70)))]).float().cpu().numpy()] +
                         [engine.step([StepEntry(1, [t], [0])]).float().cpu().numpy() for t in ids[70:]])
    engine.check_kernel_errors()
    check(got, P.plain_forward({n: t.to(engine.dtype) for n, t in written.items()}, raw, ids).numpy(), dtype,
          "a step on weights drawn on the device")
