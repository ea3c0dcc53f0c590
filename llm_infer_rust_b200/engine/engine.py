"""The engine: model, cache, step function, scheduler and sampler in one object.

Start-up order follows the reference (src/engine/engine.rs:212-248): validate
what the configuration alone can refuse, build the model, load the weights,
size and allocate the cache from the memory that is left, then (optionally)
capture decode graphs.

``step`` is the one step function: a batch of (request, its next tokens),
portions of prompts beside single decoded tokens, cut anywhere.  It runs only
the tokens it is given, from the cache that earlier steps left, and returns the
logits at the wanted places.  Trace replay, ``generate`` and the scheduler loop
all go through it.
"""
from __future__ import annotations

import logging
from collections import OrderedDict
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Tuple

import torch

from .. import architectures  # noqa: F401  (registers the shipped architectures)
from ..cache import PagedCache, cache_budget_bytes, plan_cache, size_groups
from ..config.registry import resolve_architecture
from ..config.spec import ConfigError
from ..kernels import ops
from ..kernels.build import load_host_runtime
from ..parts import DecoderModel
from ..sampling import Sampler, SamplingParams
from ..weights.loader import load_weights, read_config_json
from ..weights.random_init import bind_random_weights
from .context import StepContext, context_from_layout

_DTYPES = {"bfloat16": torch.bfloat16, "float32": torch.float32}
log = logging.getLogger("llm_infer_rust_b200")


@dataclass
class StepEntry:
    """One row of a step: a live request, its next tokens, and the places (indices
    into ``tokens``) whose logits are wanted."""
    request: int
    tokens: Sequence[int]
    want: Sequence[int] = ()


@dataclass
class GenerationResult:
    tokens: List[int]
    finish_reason: str


def auto_chunked_prefill_size(memory_mib: int) -> int:
    """Chunk budget by GPU memory (reference: src/engine/engine.rs:600-610)."""
    if memory_mib < 20 * 1024:
        return 2048
    if memory_mib < 60 * 1024:
        return 4096
    if memory_mib < 160 * 1024:
        return 8192
    return 16384


def graph_batch_sizes(limit: int) -> List[int]:
    """Decode graph buckets: powers of two up to 256 that fit, and the limit itself
    (reference: src/engine/graph.rs:93-97)."""
    sizes = [s for s in (1, 2, 4, 8, 16, 32, 64, 128, 256) if s <= limit]
    if limit > 0 and limit not in sizes:
        sizes.append(limit)
    return sorted(sizes)


class _MetaBuffers:
    """Pinned staging buffers (a small ring) and the device copy of a step's index arrays."""

    def __init__(self, device: torch.device, ring: int = 4):
        self.device = device
        self.ring = ring
        self.capacity = 0
        self.pinned: List[torch.Tensor] = []
        self.events: List[Optional[torch.cuda.Event]] = []
        self.dev: Optional[torch.Tensor] = None
        self.turn = 0
        self.last_bytes = 0

    def reserve(self, ints: int) -> None:
        if ints <= self.capacity:
            return
        torch.cuda.synchronize(self.device)
        self.capacity = max(ints, 2 * self.capacity, 4096)
        self.pinned = [torch.empty(self.capacity, dtype=torch.int32).pin_memory() for _ in range(self.ring)]
        self.events = [None] * self.ring
        self.dev = torch.empty(self.capacity, dtype=torch.int32, device=self.device)

    def next_host(self) -> Tuple[int, torch.Tensor]:
        self.turn = (self.turn + 1) % self.ring
        ev = self.events[self.turn]
        if ev is not None:
            ev.synchronize()
        return self.turn, self.pinned[self.turn]

    def upload(self, turn: int, ints: int, dst: Optional[torch.Tensor] = None) -> torch.Tensor:
        dst = self.dev if dst is None else dst
        self.last_bytes = 4 * ints
        dst[:ints].copy_(self.pinned[turn][:ints], non_blocking=True)
        ev = torch.cuda.Event()
        ev.record()
        self.events[turn] = ev
        return dst


class _DecodeGraph:
    def __init__(self, bucket: int):
        self.bucket = bucket
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.meta: Optional[torch.Tensor] = None
        self.ctx: Optional[StepContext] = None
        self.logits: Optional[torch.Tensor] = None
        self.layout_key = None
        self.launches = 0          # kernels of this package inside the graph


@dataclass
class _Flight:
    """A step that is on the GPU: its plan, its sampled ids on the device, their read-back."""
    plan: object
    ids: Optional[torch.Tensor]
    read: Optional[object]


class Engine:
    def __init__(self, model_path: Optional[str], *, dtype: str = "auto", device: str = "cuda",
                 max_running_req: int = 256, max_seq_len: Optional[int] = None, page_size: int = 16,
                 memory_ratio: float = 0.9, max_total_tokens: Optional[int] = None,
                 max_prefill_tokens_per_batch: int = 8192, chunked_prefill_size: Optional[int] = None,
                 cuda_graph_bs: Optional[int] = 0, prefill_cuda_graph_max_tokens: int = 0,
                 eos_token_ids: Optional[Sequence[int]] = None, cpu_gpu_overlap: bool = True,
                 seed: int = 0, log_level: str = "info", random_weights_config: Optional[dict] = None,
                 random_weights_seed: int = 0, keep_float32_tensors: Optional[bool] = None):
        """``model_path``: a folder with config.json and model.safetensors.  With ``model_path`` None and
        ``random_weights_config`` (the keys of a config.json) the weights are drawn on the device from
        ``random_weights_seed`` and no file is read: for sizes whose checkpoint would take long to write.
        ``keep_float32_tensors``: what a bfloat16 engine does with tensors stored in 32-bit (None: they stay float32
        in a checkpoint that declares itself 16-bit and are converted otherwise; see weights/loader.py).
        ``log_level``: error, warn(ing), info, debug or trace, for the package's logger."""
        self.model_path = model_path
        self.log_level = log_level
        level = {"error": logging.ERROR, "warn": logging.WARNING, "warning": logging.WARNING, "info": logging.INFO,
                 "debug": logging.DEBUG, "trace": logging.DEBUG}.get(str(log_level).lower())
        if level is None:
            raise ConfigError(f"log level {log_level!r} is refused: error, warn, info, debug and trace are known")
        log.setLevel(level)
        if not log.handlers and not logging.getLogger().handlers:          # (an application's own handlers win)
            handler = logging.StreamHandler()
            handler.setFormatter(logging.Formatter("[llm_infer_rust_b200] %(levelname)s %(message)s"))
            log.addHandler(handler)
        if model_path is None and random_weights_config is None:
            raise ConfigError("a model folder (or random_weights_config) is needed")
        raw = dict(random_weights_config) if model_path is None else read_config_json(model_path)
        self.arch = resolve_architecture(raw)
        self.config = self.arch.parse_config(raw)
        self.raw_config = raw
        spec = self.arch.model_spec(self.config)

        self._setup_device(device)
        if dtype == "auto":
            dtype = self.arch.checkpoint_dtype(self.config)
            dtype = "bfloat16" if dtype == "float16" else dtype
        if dtype not in _DTYPES:
            raise ConfigError(f"dtype {dtype!r} is refused: bfloat16 and float32 are supported")
        self.dtype = _DTYPES[dtype]
        if page_size <= 0:
            raise ConfigError("page_size must be positive")
        if max_running_req <= 0:
            raise ConfigError("max_running_req must be positive")
        if max_seq_len is None:
            max_seq_len = min(8192, spec.max_positions)
        if max_seq_len <= 0 or max_seq_len > spec.max_positions:
            raise ConfigError(f"--max-seq-len {max_seq_len} exceeds the model's max_position_embeddings="
                              f"{spec.max_positions}; lower --max-seq-len")
        self.max_seq_len = max_seq_len
        self.max_running_req = max_running_req
        self.page_size = page_size
        self.seed = seed

        if chunked_prefill_size is None:
            chunked_prefill_size = auto_chunked_prefill_size(self._total_memory_mib)
        budgets = [b for b in (max_prefill_tokens_per_batch, chunked_prefill_size) if b and b > 0]
        self.max_batch_tokens = min(budgets) if budgets else 0

        # The true 32-bit path must not be served by a reduced-precision matrix mode.
        torch.backends.cuda.matmul.allow_tf32 = False
        torch.backends.cudnn.allow_tf32 = False

        self.model = DecoderModel(spec, self.dtype, self.device)
        if model_path is None:
            self.loaded_tensors = bind_random_weights(self.model, self.arch.weight_plan(self.config),
                                                      random_weights_seed, self.dtype, self.device)
        else:
            self.loaded_tensors = load_weights(self.model, self.arch.weight_plan(self.config), model_path,
                                               self.dtype, self.device, keep_float32=keep_float32_tensors)
        unbound = self.model.unbound_parameters()
        if unbound:
            raise RuntimeError(f"the weight plan of {self.arch.name} left parameters unbound: {unbound}")

        itemsize = torch.empty(0, dtype=self.dtype).element_size()
        self.cache_plan = plan_cache(self.model, page_size, itemsize)
        free, total = self._free_and_total_memory()
        budget = cache_budget_bytes(free, total, memory_ratio)
        step_bound = self.max_batch_tokens if self.max_batch_tokens > 0 else max_seq_len
        size_groups(self.cache_plan, budget, max_total_tokens, max_running_req, max_seq_len, step_bound)
        self.cache = PagedCache(self.model, self.cache_plan, max_running_req, self.dtype, self.device)
        self.table_width = [-(-max_seq_len // g.page_size) for g in self.cache_plan.groups]

        rt = load_host_runtime()
        self._rt = rt
        if eos_token_ids is None:
            eos_token_ids = self.arch.stop_ids(self.config)
        self.eos_token_ids = tuple(eos_token_ids)
        self.scheduler = rt.Scheduler(self.cache.manager,
                                      rt.SchedulerOptions(max_running_req, max_seq_len, self.max_batch_tokens),
                                      list(self.eos_token_ids))
        self.sampler = Sampler(self.device)
        self._meta = self._new_meta_buffers()
        self._scratch: Optional[torch.Tensor] = None
        self._outgrown_scratch: List[torch.Tensor] = []
        self._params: Dict[int, SamplingParams] = {}
        self._seeds: Dict[int, int] = {}
        self.cpu_gpu_overlap = bool(cpu_gpu_overlap)
        self._flight: Optional[_Flight] = None          # the step that is already on the GPU (scheduler loop)
        self._launched = False                          # whether the step being built has put work on the GPU
        self.last_step_error = False

        self._graphs: Dict[int, _DecodeGraph] = {}
        if cuda_graph_bs is None:
            cuda_graph_bs = max_running_req
        self.cuda_graph_bs = min(int(cuda_graph_bs), max_running_req) if self.dtype == torch.bfloat16 else 0
        for bucket in graph_batch_sizes(self.cuda_graph_bs):
            self._graphs[bucket] = _DecodeGraph(bucket)
        # Graphs of steps that hold prompt portions, keyed by the exact shape of the batch (the rows'
        # token counts and the number of wanted logits).  A shape is captured when it comes a second
        # time (a long prompt cut into equal portions, a server's usual chunk) and replayed from then
        # on; the least recently used graph goes when there are more than a handful.
        self.prefill_graph_max_tokens = int(prefill_cuda_graph_max_tokens) if self.dtype == torch.bfloat16 else 0
        self._shape_graphs: "OrderedDict[tuple, _DecodeGraph]" = OrderedDict()
        self._shape_seen: Dict[tuple, int] = {}
        self._shape_graph_limit = 6
        # Decode graphs are captured now, while every page and state slot is free: a capture runs on throw-away
        # requests (see _capture), and a full engine has no room for those.  A bucket for which even the empty
        # pool is too small is tried again at its first use.
        for bucket, g in sorted(self._graphs.items()):
            if not self._capture(g, [1] * bucket, [1] * bucket, [0] * bucket):
                log.debug("the decode graph of %d rows waits for free pages and state slots", bucket)

    # ------------------------------------------------------------------ the device
    def _setup_device(self, device: str) -> None:
        if device not in ("cuda", "auto") and not str(device).startswith("cuda"):
            raise ConfigError(f"device {device!r} is refused: this engine runs on CUDA only")
        if not torch.cuda.is_available():
            raise RuntimeError("no CUDA device is visible; this engine has no CPU path")
        self.device = torch.device("cuda:0" if device in ("cuda", "auto") else device)
        torch.cuda.set_device(self.device)
        props = torch.cuda.get_device_properties(self.device)
        self.sm_count = props.multi_processor_count
        self._total_memory_mib = props.total_memory // (1 << 20)

    def _free_and_total_memory(self) -> Tuple[int, int]:
        torch.cuda.synchronize(self.device)
        return torch.cuda.mem_get_info(self.device)

    def _new_meta_buffers(self) -> "_MetaBuffers":
        return _MetaBuffers(self.device)

    # ------------------------------------------------------------------ requests of the step function
    def open_request(self, request: int) -> None:
        """Make ``request`` live without a promise of pages (pages are taken as it grows)."""
        got = self.cache.manager.open(request)
        if got != self._rt.Acquire.Ready:
            raise RuntimeError(f"request {request} cannot be opened: {got.name}")

    def close_request(self, request: int) -> None:
        """Give back everything ``request`` holds."""
        self.cache.manager.release(request)

    def request_length(self, request: int) -> int:
        return self.cache.manager.length(request)

    # ------------------------------------------------------------------ the step function
    def _get_scratch(self, floats: int) -> torch.Tensor:
        if self._scratch is None or self._scratch.numel() < floats:
            if torch.cuda.is_current_stream_capturing():
                raise RuntimeError("scratch memory must be sized before a graph is captured")
            if self._scratch is not None:
                # Graphs captured so far hold the address of the smaller buffer: it stays alive beside the new one.
                self._outgrown_scratch.append(self._scratch)
            self._scratch = torch.empty(max(floats, 1 << 16), dtype=torch.float32, device=self.device)
        return self._scratch

    def _context(self, layout, dev: torch.Tensor, host: Optional[torch.Tensor], kv_len_bound: int) -> StepContext:
        return context_from_layout(layout, dev, host, self.cache.page_sizes, self.device, self.dtype,
                                   kv_len_bound, self._get_scratch, self.sm_count)

    def _batch_request(self, entries: Sequence[StepEntry]):
        req = self._rt.BatchRequest()
        req.ids = [int(e.request) for e in entries]
        req.counts = [len(e.tokens) for e in entries]
        req.tokens = [int(t) for e in entries for t in e.tokens]
        req.want_counts = [len(e.want) for e in entries]
        req.want_index = [int(i) for e in entries for i in e.want]
        return req

    def step(self, entries: Sequence[StepEntry], device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        """Run one batch; float32 logits [wanted, vocab] in the order of the entries and their ``want``.

        The tensor may be overwritten by the next step; copy it if it must outlive that.
        ``device_tokens`` (int32, one per entry, on the device) replaces the entries' token ids when every
        entry brings exactly one token: a token sampled by the step before can go straight into this one
        without a trip to the host.
        """
        if not entries:
            return torch.empty((0, self.model.spec.vocab_size), dtype=torch.float32, device=self.device)
        mgr = self.cache.manager
        self._launched = False                       # nothing of this step is on the GPU yet
        new_lengths = []
        for e in entries:
            if len(e.tokens) == 0:
                raise ValueError("a step entry must bring at least one token")
            new_len = mgr.length(e.request) + len(e.tokens)
            if new_len > self.model.spec.max_positions:
                raise ValueError(f"request {e.request} would reach {new_len} tokens, beyond the model's "
                                 f"{self.model.spec.max_positions} positions")
            new_lengths.append(new_len)
        # pages for all entries or for none: a step that does not fit leaves every request as it was
        short = mgr.grow_all([int(e.request) for e in entries], new_lengths)
        if short >= 0:
            raise MemoryError(f"the cache has no pages left for request {entries[short].request} "
                              f"({new_lengths[short]} tokens) in this step of {len(entries)} entries; nothing was "
                              f"taken; free pages per group: {[mgr.free_pages(g) for g in range(mgr.num_groups())]}")
        req = self._batch_request(entries)
        decode_only = all(c == 1 for c in req.counts)
        if device_tokens is not None and (not decode_only or device_tokens.numel() != len(entries)
                                          or device_tokens.dtype != torch.int32 or not device_tokens.is_cuda):
            raise ValueError("device_tokens needs one int32 token on the device for each one-token entry")
        graph = None
        if decode_only and self._graphs and all(len(e.want) == 1 for e in entries):
            bucket = next((b for b in sorted(self._graphs) if b >= len(entries)), None)
            if bucket is not None and max(mgr.length(e.request) for e in entries) < self.max_seq_len:
                graph = self._graphs[bucket]
        if graph is None and not decode_only and 0 < len(req.tokens) <= self.prefill_graph_max_tokens \
                and max(mgr.length(e.request) + len(e.tokens) for e in entries) <= self.max_seq_len:
            graph = self._shape_graph(tuple(req.counts) + (-1, len(req.want_index)))
        if graph is not None:
            logits = self._step_graph(graph, req, len(entries), device_tokens)
        else:
            logits = self._step_eager(req, device_tokens)
        for e in entries:
            mgr.advance(e.request, mgr.length(e.request) + len(e.tokens))
        return logits

    def _step_eager(self, req, device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        layout = self._rt.plan_batch(self.cache.manager, req)
        self._meta.reserve(layout.total_ints)
        turn, host = self._meta.next_host()
        layout = self._rt.build_batch(self.cache.manager, req, host.numpy())
        dev = self._meta.upload(turn, layout.total_ints)
        if device_tokens is not None:
            dev[layout.off_tokens:layout.off_tokens + layout.num_tokens].copy_(device_tokens, non_blocking=True)
        ctx = self._context(layout, dev, host, layout.max_kv_len)
        self._launched = True
        return self.model.forward(ctx, self.cache.layer_caches)

    def _shape_graph(self, key: tuple) -> Optional[_DecodeGraph]:
        g = self._shape_graphs.get(key)
        if g is not None:
            self._shape_graphs.move_to_end(key)
            return g
        seen = self._shape_seen.get(key, 0) + 1
        if len(self._shape_seen) > 4096:
            self._shape_seen.clear()
        self._shape_seen[key] = seen
        if seen < 2:
            return None                      # a shape that comes once is not worth a capture
        g = _DecodeGraph(0)
        self._shape_graphs[key] = g
        while len(self._shape_graphs) > self._shape_graph_limit:
            self._shape_graphs.popitem(last=False)
        return g

    def _graph_request(self, req, g: _DecodeGraph):
        req.pad_rows_to = g.bucket
        req.fixed_table_width = list(self.table_width)
        return req

    def _capture(self, g: _DecodeGraph, counts: Sequence[int], want_counts: Sequence[int],
                 want_index: Sequence[int]) -> bool:
        """Capture ``g`` for a batch of this shape, on throw-away requests: the step that is captured (and the
        run before it that sizes scratch memory and loads kernels) must not touch a live request, whose cache
        rows and per-request state would else be written twice for one step.  False (and nothing captured) when
        the pages or state slots for the throw-away requests are not free right now."""
        mgr, rt = self.cache.manager, self._rt
        ids = [-(i + 1) for i in range(len(counts))]
        opened = []
        try:
            for rid in ids:
                if mgr.has(rid) or mgr.open(rid) != rt.Acquire.Ready:
                    return False
                opened.append(rid)
            if mgr.grow_all(ids, [int(c) for c in counts]) >= 0:
                return False
            req = rt.BatchRequest()
            req.ids, req.counts, req.tokens = ids, [int(c) for c in counts], [0] * int(sum(counts))
            req.want_counts, req.want_index = [int(c) for c in want_counts], [int(i) for i in want_index]
            self._graph_request(req, g)
            layout = rt.plan_batch(mgr, req)
            self._meta.reserve(layout.total_ints)
            turn, host = self._meta.next_host()
            layout = rt.build_batch(mgr, req, host.numpy())
            g.meta = torch.empty(layout.total_ints, dtype=torch.int32, device=self.device)
            self._meta.upload(turn, layout.total_ints, g.meta)
            g.ctx = self._context(layout, g.meta, None, self.max_seq_len)
            # Warm up outside the capture (sizes scratch, loads kernels), then capture.
            side = torch.cuda.Stream(self.device)
            side.wait_stream(torch.cuda.current_stream())
            before = ops.launch_count()
            with torch.cuda.stream(side):
                self.model.forward(g.ctx, self.cache.layer_caches)
            torch.cuda.current_stream().wait_stream(side)
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            with ops.graph_capture(graph):
                g.logits = self.model.forward(g.ctx, self.cache.layer_caches)
            g.launches = (ops.launch_count() - before) // 2
            ops.add_launches(-2 * g.launches)    # a warm-up on throw-away rows and a capture: not the model's work
            g.graph = graph
            g.layout_key = layout.total_ints
            return True
        finally:
            for rid in opened:
                mgr.release(rid)

    def _step_graph(self, g: _DecodeGraph, req, real_rows: int,
                    device_tokens: Optional[torch.Tensor] = None) -> torch.Tensor:
        if g.graph is None and not self._capture(g, req.counts, req.want_counts, req.want_index):
            return self._step_eager(req, device_tokens)       # no room for the capture now: this step runs as it is
        self._graph_request(req, g)
        layout = self._rt.plan_batch(self.cache.manager, req)
        if layout.total_ints != g.layout_key:
            raise RuntimeError("a graph was given a batch of another shape than it was captured for")
        self._meta.reserve(layout.total_ints)
        turn, host = self._meta.next_host()
        layout = self._rt.build_batch(self.cache.manager, req, host.numpy())
        self._meta.upload(turn, layout.total_ints, g.meta)
        if device_tokens is not None:
            g.meta[layout.off_tokens:layout.off_tokens + real_rows].copy_(device_tokens, non_blocking=True)
        self._launched = True
        g.graph.replay()
        ops.add_launches(g.launches)
        return g.logits[:real_rows] if g.bucket else g.logits

    def capture_graphs(self) -> None:
        """Capture every decode graph bucket now (else each is captured at its first use)."""
        for bucket, g in sorted(self._graphs.items()):
            if g.graph is None and not self._capture(g, [1] * bucket, [1] * bucket, [0] * bucket):
                raise MemoryError(f"not enough free pages or state slots to capture the decode graph of {bucket} rows")

    @property
    def last_upload_bytes(self) -> int:
        """Bytes of index arrays that the last step copied from pinned host memory to the device."""
        return self._meta.last_bytes

    def check_kernel_errors(self) -> None:
        ops.check_errors(self.device)

    # ------------------------------------------------------------------ scheduler loop
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        params = (params or SamplingParams()).normalized()
        rt = self._rt
        uid = self.scheduler.add_request([int(t) for t in prompt],
                                         rt.SamplingParams(params.temperature, params.top_k, params.top_p,
                                                           params.ignore_eos, params.max_tokens,
                                                           (params.seed or 0) & ((1 << 64) - 1)))
        self._params[uid] = params
        self._seeds[uid] = params.seed if params.seed is not None else \
            (self.seed * 0x9E3779B97F4A7C15 + uid * 0xD1B54A32D192ED03) & ((1 << 64) - 1)
        return uid

    def abort_request(self, uid: int) -> bool:
        return self.scheduler.abort_request(uid)

    def is_idle(self) -> bool:
        return self.scheduler.is_idle()

    def _launch(self, plan, relay: Optional[torch.Tensor]) -> "_Flight":
        """Enqueue the forward pass and the sampling of ``plan`` and start the read-back of its tokens.
        ``relay``: the token ids (on the device) that the step before sampled, in the order of ``plan``'s
        entries, when those have not reached the host yet."""
        sched = self.scheduler
        entries, rows = [], []
        for e in plan.entries:
            tokens = [0] * e.count if relay is not None else sched.tokens_of(e)
            entries.append(StepEntry(e.uid, tokens, [e.count - 1] if e.sample else []))
            if e.sample:
                rows.append((self._params[e.uid], self._seeds[e.uid], e.output_index))
        logits = self.step(entries, device_tokens=relay)
        if not rows:
            return _Flight(plan, None, None)
        ids = self.sampler.sample_device(logits, rows)
        return _Flight(plan, ids, ops.begin_read(ids))

    def _forget_finished(self, out) -> None:
        for o in out:
            if o.finished:
                self._params.pop(o.uid, None)
                self._seeds.pop(o.uid, None)

    def schedule_step(self):
        """One scheduler step: plan, run, sample, commit.  Returns the output tokens of one step.

        With ``cpu_gpu_overlap`` the step after this one is put on the GPU before this one's tokens are
        read, whenever the scheduler can name it without them (``Scheduler.successor``: one decoded token
        for every running request, their inputs passed on the device); the host's work between two steps
        then runs beside the GPU's.  A request that ends meanwhile stays in that step as a dead row."""
        sched = self.scheduler
        out = list(sched.drain_outbox())
        flight, self._flight = self._flight, None
        try:
            if flight is None:
                plan = sched.plan_step()
                out += sched.drain_outbox()
                if not plan.entries:
                    if not out and sched.num_pending() and not sched.num_running():
                        # the head of the queue waits for pages or a slot that no running request will ever free
                        # (they are held through open_request / step): waiting again would never end
                        mgr = self.cache.manager
                        raise MemoryError(f"{sched.num_pending()} requests wait and nothing runs: free pages per group "
                                          f"{[mgr.free_pages(g) for g in range(mgr.num_groups())]}, free state slots "
                                          f"{mgr.free_state_slots()}, live requests outside the scheduler {mgr.live_requests()}")
                    self._forget_finished(out)
                    return out
                flight = _Flight(plan, None, None)            # (so that a failing launch fails this plan)
                flight = self._launch(plan, None)
            if self.cpu_gpu_overlap and flight.ids is not None:
                following = sched.successor(flight.plan)
                if following.entries:
                    self._flight = self._launch(following, flight.ids)
            if flight.read is not None:
                sampled = flight.read.finish()
                if any(i < 0 for i in sampled):
                    raise RuntimeError("sampling produced no valid token for a row (were the logits finite?)")
            else:
                sampled = []
                self.check_kernel_errors()
        except Exception:
            self._flight = None
            if flight is not None and flight.read is None and flight.ids is None and not self._launched:
                # the step could not be built and nothing of it ran: what it admitted goes back to the queue's head
                sched.rollback_step(flight.plan)
            elif flight is not None:
                out += sched.fail_step(flight.plan)           # its requests are those of this step: they end here
            self.last_step_error = True
            self._forget_finished(out)
            raise
        out += sched.commit_step(flight.plan, sampled)
        self._forget_finished(out)
        return out

    def generate(self, prompts: Sequence[Sequence[int]],
                 sampling_params=None) -> List[GenerationResult]:
        """Generate for every prompt (host token ids in, host token ids out)."""
        if sampling_params is None or isinstance(sampling_params, SamplingParams):
            sampling_params = [sampling_params or SamplingParams()] * len(prompts)
        if len(sampling_params) != len(prompts):
            raise ValueError("one SamplingParams per prompt, or one for all")
        uids = [self.add_request(p, sp) for p, sp in zip(prompts, sampling_params)]
        results = {uid: GenerationResult([], "") for uid in uids}
        while not self.is_idle():
            for o in self.schedule_step():
                if o.uid not in results:
                    continue
                if o.token >= 0:
                    results[o.uid].tokens.append(o.token)
                if o.finished:
                    results[o.uid].finish_reason = o.reason.name.lower()
        return [results[uid] for uid in uids]
