"""Parts that the framework does not ship, defined here and plugged in through the
registries alone: a mixer with per-request state of its own (a linear recurrence),
an architecture that alternates it with attention, runs one layer twice and lets
the second run read the first run's keys and values.  Nothing under
``llm_infer_rust_b200/`` knows these parts; the test registers, builds, loads and
steps them, cut in different ways, and compares with a plain whole-sequence
implementation written here.
"""
import dataclasses
import math

import numpy as np
import pytest
import torch

import plain_qwen3 as P

pytestmark = pytest.mark.gpu


# ----------------------------------------------------------------------------- the toy parts
def register_toys():
    from llm_infer_rust_b200 import (Architecture, LayerSpec, ModelSpec, PartSpec, RunEntry,
                                     register_architecture)
    from llm_infer_rust_b200.kernels import ops
    from llm_infer_rust_b200.parts import ParamDecl, Part, StateSpec, register_part
    from llm_infer_rust_b200.weights import SourceTensor, WeightBinding

    class DecayMixer(Part):
        """s_t = decay * s_{t-1} + W_in x_t;  y_t = W_out s_t.  The state s lives in the request's slot;
        a row that starts at position 0 starts from zeros."""
        category = "mixer"

        def __init__(self, spec, env):
            super().__init__(spec, env)
            self.hidden, self.n, self.decay = int(spec["hidden_size"]), int(spec["state_size"]), float(spec["decay"])

        def param_decls(self):
            return {"w_in": ParamDecl((self.n, self.hidden)), "w_out": ParamDecl((self.hidden, self.n))}

        def cache_spec(self):
            return None

        def state_spec(self):
            return StateSpec((self.n,), torch.float32)

        def forward(self, x, ctx, cache):
            u = ops.linear(x, self.params["w_in"]).float()
            lay, host = ctx.layout, ctx.host
            cu = host[lay.off_cu_q: lay.off_cu_q + ctx.num_rows + 1]
            prefix = host[lay.off_prefix_len: lay.off_prefix_len + ctx.num_rows]
            slots = host[lay.off_state_slot: lay.off_state_slot + ctx.num_rows]
            states = torch.empty_like(u)
            for r in range(ctx.num_rows):
                s = cache.state[int(slots[r])]
                if prefix[r] == 0:
                    s = torch.zeros_like(s)
                for t in range(int(cu[r]), int(cu[r + 1])):
                    s = self.decay * s + u[t]
                    states[t] = s
                cache.state[int(slots[r])] = s
            return ops.linear(states.to(x.dtype), self.params["w_out"])

    register_part("mixer", "toy_decay", DecayMixer, replace=True)

    @dataclasses.dataclass(frozen=True)
    class ToyConfig:
        hidden: int
        heads: int
        kv_heads: int
        head_dim: int
        inter: int
        vocab: int
        state: int
        decay: float
        eps: float
        theta: float
        max_pos: int

        @staticmethod
        def parse(raw):
            return ToyConfig(raw["hidden_size"], raw["num_attention_heads"], raw["num_key_value_heads"],
                             raw["head_dim"], raw["intermediate_size"], raw["vocab_size"], raw["state_size"],
                             raw["decay"], raw["rms_norm_eps"], raw["rope_theta"], raw["max_position_embeddings"])

    def model_spec(c):
        norm = PartSpec("rms_norm", {"width": c.hidden, "eps": c.eps})
        ffn = PartSpec("swiglu", {"hidden_size": c.hidden, "intermediate_size": c.inter})
        attn = PartSpec("gqa_attention", {"hidden_size": c.hidden, "num_heads": c.heads, "num_kv_heads": c.kv_heads,
                                          "head_dim": c.head_dim, "qk_norm_eps": c.eps, "window": None,
                                          "softmax_scale": 1.0 / math.sqrt(c.head_dim), "position_encoding": "rope"})
        toy = PartSpec("toy_decay", {"hidden_size": c.hidden, "state_size": c.state, "decay": c.decay})
        block = PartSpec("pre_norm_deferred_add")
        return ModelSpec(
            architecture="ToyHybridForCausalLM", vocab_size=c.vocab, hidden_size=c.hidden, max_positions=c.max_pos,
            embedding=PartSpec("token_embedding", {"vocab_size": c.vocab, "hidden_size": c.hidden}),
            layers=(LayerSpec(block, attn, ffn, norm), LayerSpec(block, toy, ffn, norm)),
            run_list=(RunEntry(0), RunEntry(1), RunEntry(0, reads=0), RunEntry(1)),
            final_norm=norm, lm_head=PartSpec("linear_head", {"vocab_size": c.vocab, "hidden_size": c.hidden,
                                                              "tied": True}),
            position_encodings={"rope": PartSpec("half_split_rope", {"rotary_dim": c.head_dim, "theta": c.theta,
                                                                     "max_positions": c.max_pos})})

    def weight_plan(c):
        h, d = c.hidden, c.head_dim

        def common(i):
            return [WeightBinding(f"layers.{i}.input_norm.weight", (SourceTensor(f"l{i}.norm_in", (h,), "norm"),)),
                    WeightBinding(f"layers.{i}.post_mixer_norm.weight", (SourceTensor(f"l{i}.norm_post", (h,), "norm"),)),
                    WeightBinding(f"layers.{i}.feed_forward.gate_up_proj",
                                  (SourceTensor(f"l{i}.gate", (c.inter, h)), SourceTensor(f"l{i}.up", (c.inter, h)))),
                    WeightBinding(f"layers.{i}.feed_forward.down_proj", (SourceTensor(f"l{i}.down", (h, c.inter)),))]

        plan = [WeightBinding("embedding.weight", (SourceTensor("embed", (c.vocab, h)),))] + common(0) + common(1)
        plan += [WeightBinding("layers.0.mixer.qkv_proj", (SourceTensor("l0.q", (c.heads * d, h)),
                                                          SourceTensor("l0.k", (c.kv_heads * d, h)),
                                                          SourceTensor("l0.v", (c.kv_heads * d, h)))),
                 WeightBinding("layers.0.mixer.q_norm", (SourceTensor("l0.q_norm", (d,), "norm"),)),
                 WeightBinding("layers.0.mixer.k_norm", (SourceTensor("l0.k_norm", (d,), "norm"),)),
                 WeightBinding("layers.0.mixer.o_proj", (SourceTensor("l0.o", (h, c.heads * d)),)),
                 WeightBinding("layers.1.mixer.w_in", (SourceTensor("l1.w_in", (c.state, h)),)),
                 WeightBinding("layers.1.mixer.w_out", (SourceTensor("l1.w_out", (h, c.state)),)),
                 WeightBinding("final_norm.weight", (SourceTensor("norm", (h,), "norm"),)),
                 WeightBinding("lm_head.weight", (SourceTensor("head", (c.vocab, h)),), optional=True,
                               alias_of="embedding.weight")]
        return plan

    register_architecture(Architecture("ToyHybridForCausalLM", "toy_hybrid", ToyConfig.parse, model_spec, weight_plan),
                          replace=True)


RAW = {"model_type": "toy_hybrid", "architectures": ["ToyHybridForCausalLM"], "hidden_size": 72,
       "num_attention_heads": 3, "num_key_value_heads": 1, "head_dim": 32, "intermediate_size": 100,
       "vocab_size": 211, "state_size": 24, "decay": 0.9, "rms_norm_eps": 1e-5, "rope_theta": 1000.0,
       "max_position_embeddings": 96}


# ----------------------------------------------------------------------------- its plain twin
def plain_toy_forward(w, ids):
    w = {n: t.double() for n, t in w.items()}
    T = len(ids)
    pos = torch.arange(T)
    eps, theta = RAW["rms_norm_eps"], RAW["rope_theta"]
    h = P.plain_embedding(torch.tensor(ids), w["embed"])
    residual, kv_first = None, None
    for entry, (layer, reads) in enumerate([(0, None), (1, None), (0, 0), (1, None)]):
        pre = f"l{layer}."
        if residual is None:
            residual, x = h, P.plain_rms_norm(h, w[pre + "norm_in"], eps)
        else:
            x, residual = P.plain_add_rms_norm(h, residual, w[pre + "norm_in"], eps)
        if layer == 0:
            q, k, v = P.plain_qkv(x, w["l0.q"], w["l0.k"], w["l0.v"], 3, 1, 32)
            q, k = P.plain_qk_norm(q, k, w["l0.q_norm"], w["l0.k_norm"], eps)
            q, k = P.plain_rope(q, pos, theta), P.plain_rope(k, pos, theta)
            if reads is None:
                kv_first = (k, v)
            else:
                k, v = kv_first
            a = P.plain_attention(q, k, v) @ w["l0.o"].T
        else:
            u = x @ w["l1.w_in"].T
            s = torch.zeros(RAW["state_size"], dtype=torch.float64)
            states = []
            for t in range(T):
                s = RAW["decay"] * s + u[t]
                states.append(s)
            a = torch.stack(states) @ w["l1.w_out"].T
        x, residual = P.plain_add_rms_norm(a, residual, w[pre + "norm_post"], eps)
        h = P.plain_swiglu(x, w[pre + "gate"], w[pre + "up"], w[pre + "down"])
    x, _ = P.plain_add_rms_norm(h, residual, w["norm"], eps)
    return P.plain_lm_head(x, w["embed"])


def test_a_toy_mixer_with_state_is_registered_built_and_stepped(tmp_path):
    register_toys()
    from llm_infer_rust_b200 import random_tensors, write_random_model
    from llm_infer_rust_b200.engine import Engine, StepEntry
    d = write_random_model(str(tmp_path), RAW, seed=4, norm_std=0.1)
    w = random_tensors(RAW, 4, norm_std=0.1)
    eng = Engine(d, dtype="float32", max_running_req=3, page_size=8, max_total_tokens=256, cuda_graph_bs=0)
    # what the framework derived from the parts: one paged group (two entries share one cache), state for entries 1 and 3
    assert len(eng.cache_plan.groups) == 1 and eng.cache_plan.groups[0].entries == [0]
    assert sorted(eng.cache_plan.state_entries) == [1, 3]
    assert eng.cache.layer_caches[2].k.data_ptr() == eng.cache.layer_caches[0].k.data_ptr()
    assert not eng.cache.layer_caches[2].writes and eng.cache.layer_caches[1].k is None
    assert tuple(eng.cache.layer_caches[1].state.shape) == (4, 24)

    g = torch.Generator().manual_seed(9)
    seqs = {r: torch.randint(0, 211, (n,), generator=g).tolist() for r, n in ((1, 80), (2, 37), (3, 64))}
    want = {r: plain_toy_forward(w, ids).numpy() for r, ids in seqs.items()}

    def feed(plan):
        """plan: list of steps, each a list of (request, count)."""
        fed = {r: 0 for r in seqs}
        got = {r: [] for r in seqs}
        for step in plan:
            entries = []
            for r, n in step:
                if fed[r] == 0:
                    eng.open_request(r)
                entries.append(StepEntry(r, seqs[r][fed[r]: fed[r] + n], list(range(n))))
                fed[r] += n
            logits = eng.step(entries).cpu().numpy()
            at = 0
            for r, n in step:
                got[r].append(logits[at: at + n])
                at += n
        eng.check_kernel_errors()
        for r in seqs:
            if fed[r]:
                eng.close_request(r)
        return {r: np.concatenate(v) for r, v in got.items() if v}

    whole = feed([[(1, 80)], [(2, 37)], [(3, 64)]])
    # the same slots are used again here: the state must start from zeros
    mixed = feed([[(1, 50), (2, 2)], [(1, 1), (2, 30), (3, 3)], [(1, 1), (2, 1), (3, 59)]] +
                 [[(1, 1), (2, 1), (3, 1)]] * 2 + [[(1, 1), (2, 1)]] * 2 + [[(1, 1)]] * 24)
    for name, got in (("whole", whole), ("mixed", mixed)):
        for r in seqs:
            scale = max(1.0, np.abs(want[r]).max())
            err = np.abs(got[r] - want[r]).max()
            assert err <= 1e-5 * scale, (name, r, err)


def test_an_unknown_part_is_refused_by_name():
    from llm_infer_rust_b200 import PartSpec
    from llm_infer_rust_b200.parts import BuildEnv, build_part
    with pytest.raises(KeyError, match="no mixer named 'nonesuch'"):
        build_part("mixer", PartSpec("nonesuch"), BuildEnv(torch.float32, torch.device("cuda"), {}))
