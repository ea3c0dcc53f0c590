"""The flat index arrays of one step, against hand-checked vectors.

The vectors restate the reference's batch tests with this engine's page ids
(src/engine/batch_context.rs:375-406, :487-576; src/scheduler/decode.rs:484-520):
positions, write slots = page * P + offset, cumulative query lengths, prefix
lengths, the last-token (or any wanted) logit rows and the block table.
"""
import numpy as np
import pytest

from llm_infer_rust_b200.kernels.build import load_host_runtime

rt = load_host_runtime()


def build(mgr, rows, pad_to=0, fixed=None):
    """rows: (id, tokens, want) -> (layout, dict of named arrays)."""
    req = rt.BatchRequest()
    req.ids = [r[0] for r in rows]
    req.counts = [len(r[1]) for r in rows]
    req.tokens = [t for r in rows for t in r[1]]
    req.want_counts = [len(r[2]) for r in rows]
    req.want_index = [i for r in rows for i in r[2]]
    req.pad_rows_to = pad_to
    if fixed is not None:
        req.fixed_table_width = fixed
    plan = rt.plan_batch(mgr, req)
    buf = np.full(plan.total_ints + 8, -7, dtype=np.int32)
    lay = rt.build_batch(mgr, req, buf)
    assert lay.total_ints == plan.total_ints and (buf[lay.total_ints:] == -7).all()
    T, R = lay.num_tokens, lay.num_rows
    arr = {
        "tokens": buf[lay.off_tokens:lay.off_tokens + T], "positions": buf[lay.off_positions:lay.off_positions + T],
        "row_of_token": buf[lay.off_row_of_token:lay.off_row_of_token + T],
        "cu_q": buf[lay.off_cu_q:lay.off_cu_q + R + 1], "kv_len": buf[lay.off_kv_len:lay.off_kv_len + R],
        "prefix_len": buf[lay.off_prefix_len:lay.off_prefix_len + R],
        "state_slot": buf[lay.off_state_slot:lay.off_state_slot + R],
        "decode_rows": buf[lay.off_decode_rows:lay.off_decode_rows + lay.num_decode],
        "prefill_rows": buf[lay.off_prefill_rows:lay.off_prefill_rows + lay.num_prefill],
        "logit_rows": buf[lay.off_logit_rows:lay.off_logit_rows + lay.num_logits],
        "slots": [buf[o:o + T] for o in lay.off_slots],
        "tables": [buf[o:o + R * w].reshape(R, w) for o, w in zip(lay.off_table, lay.table_width)],
    }
    return lay, {k: (v.tolist() if not isinstance(v, list) else [x.tolist() for x in v]) for k, v in arr.items()}


def grown(mgr, rid, cached, total):
    mgr.open(rid)
    assert mgr.grow(rid, total)
    mgr.advance(rid, cached)


def test_prompt_portion_beside_a_whole_prompt():
    m = rt.CacheManager([rt.GroupSpec(2, 10, 0)], 4)
    grown(m, 1, 2, 3)          # pages [10, 9]: two tokens cached, the third comes now
    grown(m, 2, 0, 2)          # page [8]
    lay, a = build(m, [(1, [12], [0]), (2, [20, 21], [1])])
    assert a["tokens"] == [12, 20, 21] and a["positions"] == [2, 0, 1]
    assert a["slots"][0] == [9 * 2 + 0, 8 * 2 + 0, 8 * 2 + 1]
    assert a["cu_q"] == [0, 1, 3] and a["prefix_len"] == [2, 0] and a["kv_len"] == [3, 2]
    assert a["logit_rows"] == [0, 2] and a["row_of_token"] == [0, 1, 1]
    assert a["tables"][0] == [[10, 9], [8, 0]]
    assert (lay.num_decode, lay.num_prefill, lay.max_q_len, lay.max_kv_len) == (1, 1, 2, 3)
    assert a["decode_rows"] == [0] and a["prefill_rows"] == [1] and a["state_slot"] == [1, 2]


def test_middle_portion_of_a_prompt():
    m = rt.CacheManager([rt.GroupSpec(2, 7, 0)], 4)
    grown(m, 5, 2, 4)
    lay, a = build(m, [(5, [12, 13], [])])
    assert a["positions"] == [2, 3] and a["slots"][0] == [6 * 2, 6 * 2 + 1] and a["cu_q"] == [0, 2]
    assert lay.num_logits == 0 and a["logit_rows"] == []


def test_decode_rows_and_wanting_every_position():
    m = rt.CacheManager([rt.GroupSpec(2, 9, 0)], 4)
    grown(m, 1, 2, 3)          # pages [9, 8]
    grown(m, 2, 1, 2)          # page [7]
    lay, a = build(m, [(1, [13], [0]), (2, [22], [0])])
    assert a["tokens"] == [13, 22] and a["positions"] == [2, 1] and a["kv_len"] == [3, 2]
    assert a["slots"][0] == [8 * 2, 7 * 2 + 1] and lay.max_kv_len == 3 and lay.max_q_len == 1
    assert a["tables"][0] == [[9, 8], [7, 0]] and a["decode_rows"] == [0, 1]
    m2 = rt.CacheManager([rt.GroupSpec(4, 9, 0)], 4)
    grown(m2, 1, 0, 5)
    lay, a = build(m2, [(1, [1, 2, 3, 4, 5], [4, 0, 2])])
    assert a["logit_rows"] == [4, 0, 2]


def test_padding_rows_point_at_the_sink():
    m = rt.CacheManager([rt.GroupSpec(2, 9, 0)], 4)
    grown(m, 1, 2, 3)
    lay, a = build(m, [(1, [13], [0])], pad_to=4, fixed=[5])
    assert (lay.num_rows, lay.num_real_rows, lay.num_tokens, lay.num_decode, lay.num_logits) == (4, 1, 4, 4, 4)
    assert a["tokens"] == [13, 0, 0, 0] and a["slots"][0] == [16, 0, 0, 0]
    assert a["kv_len"] == [3, 1, 1, 1] and a["state_slot"] == [1, 0, 0, 0]
    assert a["tables"][0] == [[9, 8, 0, 0, 0]] + [[0] * 5] * 3
    assert a["logit_rows"] == [0, 1, 2, 3] and lay.table_width == [5]


def test_every_group_has_its_own_slots_and_table():
    m = rt.CacheManager([rt.GroupSpec(4, 9, 0), rt.GroupSpec(4, 5, 6)], 4)
    m.open(1)
    m.grow(1, 10)
    m.advance(1, 10)           # the window (6) has passed logical page 0 of group 1
    m.grow(1, 12)
    lay, a = build(m, [(1, [50, 51], [1])])
    t0, t1 = a["tables"]
    assert t0 == [[9, 8, 7]] and t1[0][0] == 0 and t1[0][1] > 0 and t1[0][2] > 0
    assert a["slots"][0] == [7 * 4 + 2, 7 * 4 + 3]
    assert a["slots"][1] == [t1[0][2] * 4 + 2, t1[0][2] * 4 + 3]


def test_refusals():
    m = rt.CacheManager([rt.GroupSpec(2, 4, 0)], 4)
    grown(m, 1, 0, 2)
    with pytest.raises(Exception, match="at least one token"):
        build(m, [(1, [], [])])
    with pytest.raises(Exception, match="holds no cache"):
        build(m, [(9, [1], [])])
    with pytest.raises(Exception, match="once in a step"):
        build(m, [(1, [1], []), (1, [2], [])])
    with pytest.raises(Exception, match="outside its row"):
        build(m, [(1, [1, 2], [2])])
    with pytest.raises(Exception, match="no page"):
        build(m, [(1, [1, 2, 3], [])])          # pages cover two tokens only


@pytest.mark.parametrize("seed", range(12))
def test_random_steps_against_a_recount(seed):
    """Random requests, portions and groups (one keeps all keys, one a window; pages of different sizes): every
    array of every step is counted again here from the requests' lengths and block tables."""
    import random
    rng = random.Random(seed)
    specs = [rt.GroupSpec(rng.choice([1, 2, 4, 16]), 200, 0)]
    if rng.random() < 0.6:
        specs.append(rt.GroupSpec(rng.choice([1, 2, 4, 8]), 200, rng.randrange(3, 20)))
    m = rt.CacheManager(specs, 6)
    live, next_id = [], 1
    for _ in range(60):
        while len(live) < 4 and (not live or rng.random() < 0.5):
            m.open(next_id)
            live.append(next_id)
            next_id += 1
        rows = []
        for rid in rng.sample(live, rng.randrange(1, len(live) + 1)):
            n = rng.choice([1, 1, 2, 3, 5, 9])
            want = [rng.randrange(n) for _ in range(rng.choice([0, 1, 1, n]))]
            rows.append((rid, [rng.randrange(1000) for _ in range(n)], want))
            assert m.grow(rid, m.length(rid) + n)
        pad = rng.choice([0, 0, len(rows) + 2]) if all(len(r[1]) == 1 for r in rows) else 0
        widest = max(m.length(r[0]) + len(r[1]) for r in rows)
        fixed = [-(-(widest + 7) // s.page_size) for s in specs] if pad else None
        lay, a = build(m, rows, pad_to=pad, fixed=fixed)
        R = max(len(rows), pad)
        counts = [len(r[1]) for r in rows] + [1] * (R - len(rows))
        prefix = [m.length(r[0]) for r in rows] + [0] * (R - len(rows))
        cu = [0]
        for c in counts:
            cu.append(cu[-1] + c)
        assert (lay.num_rows, lay.num_real_rows, lay.num_tokens) == (R, len(rows), cu[-1])
        assert a["tokens"] == [t for r in rows for t in r[1]] + [0] * (R - len(rows))
        assert a["positions"] == [p + i for p, c in zip(prefix, counts) for i in range(c)]
        assert a["row_of_token"] == [r for r, c in enumerate(counts) for _ in range(c)]
        assert a["cu_q"] == cu and a["prefix_len"] == prefix and a["kv_len"] == [p + c for p, c in zip(prefix, counts)]
        assert a["state_slot"] == [m.state_slot(r[0]) for r in rows] + [0] * (R - len(rows))
        assert a["decode_rows"] == [r for r, c in enumerate(counts) if c == 1]
        assert a["prefill_rows"] == [r for r, c in enumerate(counts) if c > 1]
        assert a["logit_rows"] == [cu[r] + i for r, row in enumerate(rows) for i in row[2]] + cu[len(rows):R]
        assert lay.max_q_len == max(counts) and lay.max_kv_len == max(p + c for p, c in zip(prefix, counts))
        for g, spec in enumerate(specs):
            P = spec.page_size
            width = fixed[g] if fixed else -(-lay.max_kv_len // P)
            assert lay.table_width[g] == width
            slots, table = [], []
            for r, row in enumerate(rows):
                held = list(m.block_table(row[0], g))
                used = -(-(prefix[r] + counts[r]) // P)
                assert all(page == 0 for page in held[:m.first_live_page(row[0], g)])
                assert all(page > 0 for page in held[m.first_live_page(row[0], g):used])
                table.append((held[:used] + [0] * width)[:width])
                slots += [held[(prefix[r] + i) // P] * P + (prefix[r] + i) % P for i in range(counts[r])]
            assert a["slots"][g] == slots + [0] * (R - len(rows))
            assert a["tables"][g] == table + [[0] * width] * (R - len(rows))
        for rid, tokens, _ in rows:
            m.advance(rid, m.length(rid) + len(tokens))
        assert m.check() == ""
        for rid in [r for r in live if rng.random() < 0.08 or m.length(r) > 150]:
            assert m.release(rid)
            live.remove(rid)
    for rid in live:
        m.release(rid)
    assert m.check() == "" and all(m.free_pages(g) == 200 for g in range(len(specs)))
