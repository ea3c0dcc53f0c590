"""The engine through its entry points: ``generate``, the scheduler loop, the command line,
decode graphs, long decoding, and what happens when pages run out."""
import json
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def tokens(vocab, n, seed):
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def engine(folder, **kw):
    from llm_infer_rust_b200.engine import Engine
    kw.setdefault("cuda_graph_bs", 0)
    kw.setdefault("max_running_req", 4)
    return Engine(folder, **kw)


def confident_greedy(weights, raw, prompt, n):
    """Greedy continuation by the plain implementation, and the margin between its two best logits."""
    seq, out, margin = list(prompt), [], float("inf")
    for _ in range(n):
        last = P.plain_forward(weights, raw, seq)[-1]
        top = torch.topk(last, 2).values
        margin = min(margin, float(top[0] - top[1]))
        out.append(int(last.argmax()))
        seq.append(out[-1])
    return out, margin


def test_greedy_generation_matches_the_plain_implementation(tiny, tiny_weights, tiny_dirs):
    from llm_infer_rust_b200 import SamplingParams
    raw = tiny["A"]["raw"]
    prompts = [tokens(256, n, 20 + n) for n in (5, 9, 17)]
    eng = engine(tiny_dirs["A"], dtype="float32", page_size=4, max_total_tokens=256)
    got = eng.generate(prompts, SamplingParams(max_tokens=8, ignore_eos=True))
    for prompt, res in zip(prompts, got):
        want, margin = confident_greedy(tiny_weights["A"], raw, prompt, 8)
        assert margin > 1e-4, "the test's own prompt leaves a near tie; choose another seed"
        assert res.tokens == want and res.finish_reason == "length"
    assert eng.cache.manager.live_requests() == 0 and eng.cache.manager.check() == ""
    # a stop id ends a request with the id emitted
    stop = got[0].tokens[3]
    eng2 = engine(tiny_dirs["A"], dtype="float32", page_size=4, max_total_tokens=256, eos_token_ids=[stop])
    res = eng2.generate([prompts[0]], SamplingParams(max_tokens=8))[0]
    first = got[0].tokens.index(stop)
    assert res.tokens == got[0].tokens[: first + 1] and res.finish_reason == "stop"
    res = eng2.generate([prompts[0]], SamplingParams(max_tokens=8, ignore_eos=True))[0]
    assert res.tokens == got[0].tokens


# ----------------------------------------------------------------------------- temperature sampling
def philox_uniform(seed, counter):
    """Philox4x32-10 with counter (counter, 0, 0x1234567, 0) and key (seed lo, seed hi): the first word / 2^24."""
    M0, M1, W0, W1, mask = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85, 0xFFFFFFFF
    c = [counter & mask, 0, 0x1234567, 0]
    k0, k1 = seed & mask, (seed >> 32) & mask
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [(p1 >> 32) ^ c[1] ^ k0, p1 & mask, (p0 >> 32) ^ c[3] ^ k1, p0 & mask]
        k0, k1 = (k0 + W0) & mask, (k1 + W1) & mask
    return (c[0] >> 8) / 16777216.0


def test_temperature_sampling_is_the_inverse_cdf_of_a_keyed_uniform(tiny, tiny_weights, tiny_dirs):
    """Tiny B: prompts 1/7/33/70, portions of 16, mixed batches, temperature 0.8, a fixed seed, 12 tokens.
    Every sampled token is where the plain distribution's cumulative sum passes the uniform number
    that (seed, output index) give; so it cannot depend on the batch."""
    from llm_infer_rust_b200 import SamplingParams
    raw, w = tiny["B"]["raw"], tiny_weights["B"]
    prompts = [tokens(509, n, 40 + n) for n in (1, 7, 33, 70)]
    sp = [SamplingParams(temperature=0.8, max_tokens=12, ignore_eos=True, seed=1000 + i) for i in range(4)]
    eng = engine(tiny_dirs["B"], dtype="float32", page_size=16, max_total_tokens=512, chunked_prefill_size=16)
    together = eng.generate(prompts, sp)
    alone = [eng.generate([p], [s])[0] for p, s in zip(prompts, sp)]
    assert [r.tokens for r in together] == [r.tokens for r in alone]
    other_seed = eng.generate([prompts[3]], [SamplingParams(temperature=0.8, max_tokens=12, ignore_eos=True, seed=7)])[0]
    assert other_seed.tokens != together[3].tokens
    checked = 0
    for i, (prompt, res) in enumerate(zip(prompts, together)):
        assert len(res.tokens) == 12
        logits = P.plain_forward(w, raw, prompt + res.tokens[:-1])[len(prompt) - 1:]
        cdf = torch.softmax(logits / 0.8, -1).cumsum(-1)
        for k, tok in enumerate(res.tokens):
            u = philox_uniform(1000 + i, k) * float(cdf[k, -1])
            want = int((cdf[k] <= u).sum())
            gap = float((cdf[k] - u).abs().min())
            if gap > 1e-5:                                    # away from a boundary the draw is unambiguous
                assert tok == want, (i, k, tok, want, gap)
                checked += 1
    assert checked >= 40


def test_when_pages_run_out_requests_wait_and_results_do_not_change(tiny, tiny_dirs):
    from llm_infer_rust_b200 import SamplingParams
    prompts = [tokens(301, n, 60 + n) for n in (50, 20, 64, 9, 33, 41, 70, 5)]
    sp = SamplingParams(max_tokens=20, ignore_eos=True)
    roomy = engine(tiny_dirs["C"], dtype="float32", page_size=8, max_total_tokens=2048, max_running_req=8,
                   chunked_prefill_size=32)
    want = [r.tokens for r in roomy.generate(prompts, sp)]
    # 24 pages of 8 = 192 tokens: two or three requests fit at a time, the rest wait at the head of the queue
    tight = engine(tiny_dirs["C"], dtype="float32", page_size=8, max_total_tokens=192, max_running_req=8,
                   chunked_prefill_size=32)
    uids = [tight.add_request(p, sp) for p in prompts]
    out = {u: [] for u in uids}
    most_running, steps = 0, 0
    while not tight.is_idle():
        for o in tight.schedule_step():
            out[o.uid].append(o.token)
        most_running = max(most_running, tight.scheduler.num_running())
        assert tight.cache.manager.check() == ""
        steps += 1
        assert steps < 2000
    assert [out[u] for u in uids] == want
    assert most_running < 8 and tight.cache.manager.free_pages(0) == 24
    # a request that can never fit is aborted, the others are served
    res = tight.generate([tokens(301, 150, 1), prompts[3]], SamplingParams(max_tokens=100, ignore_eos=True))
    assert res[0].finish_reason == "abort" and res[0].tokens == [] and len(res[1].tokens) == 100


def test_long_decoding_stays_on_the_plain_logits(tiny, tiny_weights, tiny_dirs, tmp_path):
    """Three hundred tokens decoded one by one (windows slide, pages are given back on the way)."""
    from llm_infer_rust_b200.engine import StepEntry
    raw, w = tiny["C"]["raw"], tiny_weights["C"]
    ids = tokens(301, 318, 77)
    want = P.plain_forward(w, raw, ids).numpy()
    for dtype, tol in (("float32", 1e-5), ("bfloat16", 2.0 ** -5)):
        ww = w if dtype == "float32" else {n: t.to(torch.bfloat16) for n, t in w.items()}
        ref = want if dtype == "float32" else P.plain_forward(ww, raw, ids).numpy()
        folder = tiny_dirs["C"]
        if dtype == "bfloat16":                               # a checkpoint stored in bfloat16
            from llm_infer_rust_b200 import write_random_model
            v = tiny["C"]
            folder = write_random_model(str(tmp_path / "bf16"), v["raw"], v["seed"], norm_std=v["norm_std"],
                                        dtype="bfloat16")
        eng = engine(folder, dtype=dtype, page_size=8, max_total_tokens=512)
        eng.open_request(1)
        rows = [eng.step([StepEntry(1, ids[:18], list(range(18)))]).cpu().numpy()]
        for t in range(18, 318):
            rows.append(eng.step([StepEntry(1, [ids[t]], [0])]).cpu().numpy())
        eng.check_kernel_errors()
        got = np.concatenate(rows)
        held = eng.cache.manager.pages_held(1, [g.window for g in eng.cache_plan.groups].index(40))
        assert held <= 40 // 8 + 2                            # the windowed group kept only its window
        err = np.abs(got - ref).max(axis=1)
        assert err.max() <= tol * max(1.0, np.abs(ref).max()), (dtype, int(err.argmax()), err.max())


def test_decode_graphs_give_the_eager_logits(tiny, tiny_dirs, tmp_path):
    from llm_infer_rust_b200 import SamplingParams, write_random_model
    from llm_infer_rust_b200.engine import StepEntry
    v = tiny["B"]
    folder = write_random_model(str(tmp_path / "m"), v["raw"], v["seed"], norm_std=v["norm_std"], dtype="bfloat16")
    prompts = [tokens(509, n, 80 + n) for n in (3, 40, 17)]
    eager = engine(folder, dtype="bfloat16", max_total_tokens=512)
    graph = engine(folder, dtype="bfloat16", max_total_tokens=512, cuda_graph_bs=4)
    assert sorted(graph._graphs) == [1, 2, 4]
    for eng in (eager, graph):
        for r, p in enumerate(prompts):
            eng.open_request(r + 1)
            eng.step([StepEntry(r + 1, p, [])])
    nxt = [5, 6, 7]
    for step in range(20):
        live = [r for r in range(3) if not (r == 1 and step >= 10)]        # the batch shrinks: another bucket, padded rows
        entries = [StepEntry(r + 1, [nxt[r]], [0]) for r in live]
        a = eager.step(entries).clone()
        b = graph.step(entries).clone()
        # the padded batch may take another library matrix kernel: equal up to bfloat16 rounding
        assert (a - b).abs().max() <= 2.0 ** -6 * max(1.0, float(a.abs().max())), step
        nxt = [int(x) % 509 for x in (a.argmax(-1).tolist() + [0, 0, 0])[:3]]
    assert graph._graphs[4].graph is not None and graph._graphs[2].graph is not None
    graph.check_kernel_errors()
    sp = SamplingParams(max_tokens=16, ignore_eos=True)
    for eng in (eager, graph):
        for r in range(3):
            eng.close_request(r + 1)
    res = graph.generate(prompts, sp)
    assert [len(r.tokens) for r in res] == [16, 16, 16] and graph.cache.manager.live_requests() == 0


def test_graphs_of_repeated_prompt_portions_give_the_eager_logits(tiny, tmp_path):
    from llm_infer_rust_b200 import write_random_model
    from llm_infer_rust_b200.engine import StepEntry
    v = tiny["C"]
    folder = write_random_model(str(tmp_path / "m"), v["raw"], v["seed"], norm_std=v["norm_std"], dtype="bfloat16")
    eager = engine(folder, dtype="bfloat16", page_size=8, max_total_tokens=1024)
    graph = engine(folder, dtype="bfloat16", page_size=8, max_total_tokens=1024, prefill_cuda_graph_max_tokens=64)
    prompts = {1: tokens(301, 96, 1), 2: tokens(301, 112, 2)}
    for eng in (eager, graph):
        eng.open_request(1)
        eng.open_request(2)
    # portions of 16 alone, then 16 beside a decoded token of the other request, then an odd tail
    plan = [[(1, 16)]] * 4 + [[(2, 16)]] * 3 + [[(1, 16), (2, 1)]] * 2 + [[(2, 31)], [(2, 31)]]
    fed = {1: 0, 2: 0}
    for step, rows in enumerate(plan):
        entries = [StepEntry(r, prompts[r][fed[r]: fed[r] + n], [n - 1, 0]) for r, n in rows]
        for r, n in rows:
            fed[r] += n
        a = eager.step(entries).clone()
        b = graph.step(entries).clone()
        assert (a - b).abs().max() <= 2.0 ** -6 * max(1.0, float(a.abs().max())), step
    assert len(graph._shape_graphs) == 3 and all(g.graph is not None for g in graph._shape_graphs.values())
    graph.check_kernel_errors()


def test_command_line(tiny, tiny_dirs, tmp_path):
    from llm_infer_rust_b200 import SamplingParams
    want = engine(tiny_dirs["A"], dtype="float32", page_size=4, max_total_tokens=256).generate(
        [[1, 2, 3], [9, 8, 7, 6]], SamplingParams(max_tokens=5, ignore_eos=True))
    cmd = [sys.executable, "-m", "llm_infer_rust_b200", "--model-path", tiny_dirs["A"], "--dtype", "float32",
           "--page-size", "4", "--max-total-tokens", "256", "--max-running-req", "4", "--max-seq-len", "64",
           "--cuda-graph-bs", "0", "--prompt-ids", "1,2,3", "--prompt-ids", "9,8,7,6", "--max-tokens", "5", "--ignore-eos"]
    done = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr
    lines = [json.loads(x) for x in done.stdout.strip().splitlines()]
    assert [x["output_ids"] for x in lines] == [r.tokens for r in want]
    assert lines[0]["prompt_ids"] == [1, 2, 3] and lines[0]["finish_reason"] == "length"
    # random-weights mode writes the folder and serves it
    cfg = tmp_path / "cfg.json"
    cfg.write_text(json.dumps(tiny["A"]["raw"]))
    out_dir = tmp_path / "made"
    cmd = [sys.executable, "-m", "llm_infer_rust_b200", "--model-path", str(out_dir), "--random-weights", "--config",
           str(cfg), "--seed", "0", "--dtype", "float32", "--page-size", "4", "--max-total-tokens", "256",
           "--max-running-req", "4", "--cuda-graph-bs", "0", "--prompt-ids", "1,2,3", "--max-tokens", "5", "--ignore-eos"]
    done = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert done.returncode == 0, done.stderr
    assert sorted(os.listdir(out_dir)) == ["config.json", "model.safetensors"]
    assert json.loads(done.stdout.strip())["output_ids"] == want[0].tokens      # seed 0 is the fixture's seed
    bad = subprocess.run([sys.executable, "-m", "llm_infer_rust_b200", "--model-path", tiny_dirs["A"],
                          "--max-seq-len", "4096", "--prompt-ids", "1"], cwd=ROOT, capture_output=True, text=True)
    assert bad.returncode != 0 and "max_position_embeddings" in bad.stderr


def test_refusals_at_start_up_and_in_a_step(tiny, tiny_dirs, tmp_path):
    from llm_infer_rust_b200 import ConfigError
    from llm_infer_rust_b200.engine import Engine, StepEntry
    with pytest.raises(ConfigError, match="max_position_embeddings"):
        Engine(tiny_dirs["A"], max_seq_len=129)
    with pytest.raises(ConfigError, match="CUDA only"):
        Engine(tiny_dirs["A"], device="cpu")
    unsupported = tmp_path / "moe"
    unsupported.mkdir()
    (unsupported / "config.json").write_text(json.dumps(dict(tiny["A"]["raw"], model_type="qwen3_moe",
                                                             architectures=["Qwen3MoeForCausalLM"])))
    with pytest.raises(ConfigError, match="unsupported model"):       # before any weight is looked for
        Engine(str(unsupported))
    eng = engine(tiny_dirs["A"], dtype="float32", page_size=4, max_total_tokens=32)
    eng.open_request(1)
    with pytest.raises(MemoryError, match="no pages left"):
        eng.step([StepEntry(1, list(range(40)), [])])
    with pytest.raises(ValueError, match="at least one token"):
        eng.step([StepEntry(1, [], [])])
    eng.step([StepEntry(1, [1, 2, 300], [])])                          # 300 is outside the vocabulary of 256
    with pytest.raises(Exception, match="token id"):
        eng.check_kernel_errors()


@pytest.mark.parametrize("dtype,graphs", [("float32", 0), ("bfloat16", 4)])
def test_steps_launched_ahead_give_the_same_tokens(dtype, graphs, tiny, tiny_dirs, tmp_path):
    """With the next step put on the GPU before this step's tokens are read, every request gets the tokens it
    gets with one step at a time: requests of different lengths, stop ids that end some of them while their
    next step already runs, sampled and greedy rows, requests that arrive and are aborted in between."""
    from llm_infer_rust_b200 import SamplingParams, write_random_model
    v = tiny["B"]
    folder = tiny_dirs["B"] if dtype == "float32" else \
        write_random_model(str(tmp_path / "m"), v["raw"], v["seed"], norm_std=v["norm_std"], dtype="bfloat16")
    prompts = [tokens(509, n, 70 + n) for n in (3, 11, 40, 7, 25, 2)]
    params = [SamplingParams(max_tokens=m, temperature=t, seed=5 + i, ignore_eos=ig)
              for i, (m, t, ig) in enumerate([(30, 0.0, False), (12, 0.9, False), (9, 0.0, True), (1, 0.0, False),
                                              (40, 1.1, False), (17, 0.0, False)])]

    def run(overlap, stops):
        eng = engine(folder, dtype=dtype, page_size=v["page_size"], max_total_tokens=1024, max_running_req=4,
                     cuda_graph_bs=graphs, eos_token_ids=stops, cpu_gpu_overlap=overlap)
        got = eng.generate(prompts, params)
        assert eng.cache.manager.live_requests() == 0 and eng.cache.manager.check() == ""
        # requests that come and go while steps are in flight
        uids = [eng.add_request(p, sp) for p, sp in zip(prompts[:3], params[:3])]
        seen = {u: [] for u in uids}
        steps = 0
        while not eng.is_idle():
            for o in eng.schedule_step():
                if o.token >= 0:
                    seen[o.uid].append(o.token)
            steps += 1
            if steps == 4:
                assert eng.abort_request(uids[0])
                uids.append(eng.add_request(prompts[4], params[4]))
                seen[uids[-1]] = []
        assert eng.cache.manager.live_requests() == 0 and eng.cache.manager.check() == ""
        return [(r.tokens, r.finish_reason) for r in got], [seen[u] for u in uids]

    serial, serial_loop = run(False, [])
    # stop ids taken from what the requests really produce, so that some of them end early
    stops = sorted({serial[0][0][5], serial[4][0][9], serial[5][0][3]})
    for stop_ids in ([], stops):
        a, a_loop = run(False, stop_ids)
        b, b_loop = run(True, stop_ids)
        assert a == b
        assert a_loop[1:] == b_loop[1:]                       # (the aborted request may have got one token more or less)
        assert b_loop[0] == a_loop[0][:len(b_loop[0])] or a_loop[0] == b_loop[0][:len(a_loop[0])]
    assert any(reason == "stop" for _, reason in b) and any(reason == "length" for _, reason in b)


def test_many_requests_arriving_and_ending_at_random_with_and_without_steps_ahead(tiny, tiny_dirs):
    """Sixty requests of random lengths arrive between steps, some are aborted, stop ids end others: with steps
    launched ahead every request that was not aborted gets the tokens it gets one step at a time, and the cache
    ends empty both ways."""
    import random
    from llm_infer_rust_b200 import SamplingParams
    v = tiny["A"]
    vocab = v["raw"]["vocab_size"]

    def run(overlap):
        rnd = random.Random(7)
        eng = engine(tiny_dirs["A"], dtype="float32", page_size=v["page_size"], max_total_tokens=640,
                     max_running_req=6, max_seq_len=100, eos_token_ids=[3, 17, 101, 200], cpu_gpu_overlap=overlap)
        todo = [(tokens(vocab, rnd.randint(1, 40), 300 + i),
                 SamplingParams(max_tokens=rnd.randint(1, 30), temperature=rnd.choice([0.0, 0.0, 0.8]), seed=i,
                                ignore_eos=rnd.random() < 0.3)) for i in range(60)]
        abort_at = {i: rnd.randint(1, 12) for i in rnd.sample(range(60), 8)}    # request -> steps after its arrival
        results, uid_of, age, aborted = {}, {}, {}, set()
        step = 0
        while todo or not eng.is_idle():
            for _ in range(rnd.randint(0, 2)):
                if todo:
                    i = 60 - len(todo)
                    prompt, sp = todo.pop(0)
                    uid_of[i] = eng.add_request(prompt, sp)
                    results[uid_of[i]] = ([], None)
                    age[i] = 0
            for o in eng.schedule_step():
                toks, _ = results[o.uid]
                if o.token >= 0:
                    toks.append(o.token)
                if o.finished:
                    results[o.uid] = (toks, o.reason.name)
            for i in list(age):
                age[i] += 1
                if abort_at.get(i) == age[i] and results[uid_of[i]][1] is None:
                    eng.abort_request(uid_of[i])
                    aborted.add(i)
            step += 1
            assert step < 5000
        assert eng.cache.manager.live_requests() == 0 and eng.cache.manager.check() == ""
        return {i: results[u] for i, u in uid_of.items()}, aborted

    serial, aborted_a = run(False)
    ahead, aborted_b = run(True)
    assert len(serial) == len(ahead) == 60
    reasons = set()
    for i in range(60):
        if i in aborted_a or i in aborted_b:
            continue                                          # an aborted request may be a token further one way
        assert serial[i] == ahead[i], i
        reasons.add(serial[i][1])
    assert {"Stop", "Length"} <= reasons


def test_a_dropped_engine_in_a_dead_cycle_does_not_break_the_next_capture(tiny, tmp_path):
    """An engine that was dropped while a reference cycle still held it is freed by Python's cycle collector, at
    whatever allocation starts a collection.  Inside a graph capture that would destroy CUDA graphs and return
    their memory, which a capturing stream does not permit: the capture collects first and holds the collector
    off.  Here the collector is off until the second engine's capture, where the model's forward pass (wrapped)
    asks for a collection in the middle of it."""
    import gc
    from llm_infer_rust_b200 import SamplingParams, write_random_model
    v = tiny["B"]
    folder = write_random_model(str(tmp_path / "m"), v["raw"], v["seed"], norm_std=v["norm_std"], dtype="bfloat16")
    prompts = [tokens(509, n, 30 + n) for n in (5, 9)]
    params = [SamplingParams(max_tokens=6, temperature=0.0, ignore_eos=True)] * 2
    common = dict(dtype="bfloat16", page_size=v["page_size"], max_total_tokens=512, max_running_req=2)
    want = [r.tokens for r in engine(folder, cuda_graph_bs=0, **common).generate(prompts, params)]
    gc.collect()
    gc.disable()
    try:
        first = engine(folder, cuda_graph_bs=2, **common)
        assert [r.tokens for r in first.generate(prompts, params)] == want       # (its decode graphs exist now)
        ring = [first]
        ring.append(ring)
        del first, ring                                       # unreachable; only the cycle collector can free it
        # (decode graphs are captured when an engine is built: the collector is made to run inside those captures)
        from llm_infer_rust_b200.parts import DecoderModel
        forward, collected = DecoderModel.forward, []

        def collecting_forward(self, *args, **kwargs):
            if torch.cuda.is_current_stream_capturing():
                collected.append(gc.collect())
            return forward(self, *args, **kwargs)

        DecoderModel.forward = collecting_forward
        try:
            second = engine(folder, cuda_graph_bs=2, **common)
        finally:
            DecoderModel.forward = forward
        assert [r.tokens for r in second.generate(prompts, params)] == want
        assert collected, "no decode graph was captured"
    finally:
        gc.enable()
