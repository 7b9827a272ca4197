"""The Python entry point: a model folder (or a configuration and a seed) in, generated token ids out.

    engine = Engine.from_folder("model_dir", dtype="bfloat16", max_len=8192)
    outputs = engine.generate([[5, 17, 3], [9, 9]], SamplingParams(temperature=0.0, max_tokens=16))

`generate` is the reference's plain loop (`generate_greedy`, engine/spec.py:150-199: prefill, pick, one
token per pass until a stop id, the token limit or the window's end), run for many requests at once through
the scheduler and the one step function. `step` exposes the step function itself, as the replay program
uses it. Option names follow the reference's where it has them: `max_len` (--max-len, the window;
server/app.py:12893+, tools/lfm_check.py:374-418), `parallel` (--parallel, requests served at once),
temperature / top_p / top_k / min_p / seed on the request.
"""

from __future__ import annotations

import json
import time
from collections import deque
from dataclasses import dataclass

import numpy as np
import torch

from ..cache.manager import CacheManager
from ..config.registry import read_model_config, resolve_model_folder, spec_of
from ..parts.base import Runtime
from ..parts.model import DecoderModel
from ..sampling.defaults import card_sampling, resolve as resolve_filters
from ..sampling.sampler import NoRepeatIndex, Sampler, SampleRow, SamplingParams
from ..settings import SETTINGS
from ..weights.loader import DictWeights, FolderWeights
from ..weights.random_init import random_weights
from .scheduler import Request, Scheduler
from .step import StepEntry, StepFunction

DTYPES = {"float32": torch.float32, "fp32": torch.float32, "bfloat16": torch.bfloat16, "bf16": torch.bfloat16}


@dataclass
class EngineArgs:
    dtype: str = "bfloat16"
    max_len: int = 8192                 # the window: prompt plus generated tokens of one request
    parallel: int = 8                   # requests running at once (state slots)
    block_size: int = 16                # tokens per cache page
    kv_blocks: int | None = None        # pages per group; None: enough for `parallel` requests of `max_len`
    max_batched_tokens: int = 4096      # token budget of one step
    chunk_size: int = 2048              # longest prompt portion in one step (the reference feeds prompts 4096 rows at a
                                        # time, engine/models/lfm2_moe/engine.py:52; a step of 2048 rows takes 10 ms at the
                                        # 8B sizes and runs 2.5 times the tokens a second of one of 512)
    device: str = "cuda:0"
    graph: bool = True                  # capture decode-only steps in CUDA graphs (bfloat16)
    tensorcore: bool = True             # use the tcgen05 kernels in bfloat16
    overlap: bool = True                # launch the next decode step before this one's tokens are read
    log: str | None = None              # a file that gets one JSON line a scheduler step (default: $TANDEMLLM_STEP_LOG)
    record_routing: bool = False        # count, step by step, the pairs routed to every expert of every routed layer


@dataclass
class _Flight:
    """A step that is launched and not yet accounted."""
    batch: list                         # the scheduler's entries
    host: torch.Tensor                  # pinned int32: the sampled tokens, then the kernels' status word
    n: int                              # sampled tokens
    event: torch.cuda.Event             # recorded behind the copies into `host`
    tokens: torch.Tensor | None         # the sampled tokens on the device
    index: dict                         # request id -> its place among them
    record: dict                        # the step's record, completed when the step is accounted
    started: float                      # host clock at launch
    routed: torch.Tensor | None = None  # pinned: the routing counters as they stood after this step


def require_cuda(device: str) -> torch.device:
    dev = torch.device(device)
    if dev.type != "cuda" or not torch.cuda.is_available():
        raise RuntimeError("this engine runs on a CUDA device only (sm_100a kernels, no CPU path); "
                           f"asked for {device!r}, torch.cuda.is_available() = {torch.cuda.is_available()}")
    return dev


class Engine:
    def __init__(self, model: DecoderModel, args: EngineArgs):
        self.model, self.args = model, args
        self.device = model.runtime.device
        pages = args.kv_blocks
        if pages is None:
            pages = args.parallel * (-(-args.max_len // args.block_size))
        self.cache = CacheManager(model.cache_needs(), num_pages=pages, max_requests=args.parallel,
                                  page_size=args.block_size, dtype=model.runtime.dtype, device=self.device)
        self._results = [None, None]    # pinned host memory for a step's tokens and status, for two steps in the air
        self._turn = 0
        self._flight = None             # a step that is launched and not yet accounted
        self.step_function = StepFunction(model, self.cache, use_graphs=args.graph and model.graph_safe,
                                          max_graph_batch=args.parallel)
        self.sampler = Sampler(self.device, slots=args.parallel)
        self.scheduler = Scheduler(self.cache, max_num_seqs=args.parallel, max_num_batched_tokens=args.max_batched_tokens,
                                   chunk_size=args.chunk_size, max_model_len=args.max_len,
                                   stop_token_ids=model.spec.stop_token_ids)
        self._next_id = 0
        self.card_sampling: dict | None = None      # what the model folder's generation_config.json recommends (top_p, top_k)
        # ---- records: one dict a scheduler step (the reference keeps `route_trace` and `host_ms` per step,
        # engine/models/lfm2_moe/engine.py:125, :236-240, :457) ----
        self.records: deque[dict] = deque(maxlen=4096)
        self._log_path = args.log or SETTINGS.get("STEP_LOG")
        self._log_file = None
        self._routed_parts: list = []
        self._routing = self._routing_seen = None
        self._routed_host = [None, None]
        if args.record_routing:
            self.set_routing_record(True)

    # ---- construction ----
    @classmethod
    def from_folder(cls, folder: str, args: EngineArgs | None = None, **kw) -> "Engine":
        """A model folder: config.json chooses the architecture, model.safetensors holds the weights."""
        args = args or EngineArgs(**kw)
        folder = resolve_model_folder(folder)
        arch, config = read_model_config(folder)
        spec = spec_of(config)
        engine = cls._build(arch, spec, FolderWeights(folder, spec.name_prefixes), args)
        engine.card_sampling = card_sampling(folder)
        return engine

    @classmethod
    def from_config(cls, config, seed: int, args: EngineArgs | None = None, std: float = 0.02, bias_std: float = 0.1,
                    norm_std: float = 0.0, **kw) -> "Engine":
        """Random weights made on the device from a typed configuration and a seed (nothing touches the disk)."""
        args = args or EngineArgs(**kw)
        dev = require_cuda(args.device)
        spec = spec_of(config)
        probe = DecoderModel(spec)
        tensors = random_weights(probe.weight_specs(None), seed, std, bias_std, norm_std, dtype=DTYPES[args.dtype],
                                 device=dev)
        return cls._build(None, spec, DictWeights(tensors), args)

    @classmethod
    def _build(cls, arch, spec, weights, args: EngineArgs) -> "Engine":
        dev = require_cuda(args.device)
        if args.dtype not in DTYPES:
            raise ValueError(f"dtype {args.dtype!r}: one of {', '.join(DTYPES)}")
        runtime = Runtime(dev, DTYPES[args.dtype])
        from ..kernels import ops
        ops.core()                                  # built and loaded now; a missing library fails here, loudly
        if runtime.dtype == torch.bfloat16 and args.tensorcore:
            from ..kernels import tensorcore
            tensorcore.enable(runtime)
        build = arch.build_model if arch is not None and arch.build_model else DecoderModel
        with torch.cuda.device(dev):
            model = build(spec).load(weights, runtime)
            return cls(model, args)

    # ---- the step function, as it is ----
    def admit(self, request_id) -> None:
        self.cache.admit(request_id)

    def release(self, request_id) -> None:
        self.cache.free(request_id)

    def step(self, entries: list[StepEntry]) -> torch.Tensor:
        with torch.cuda.device(self.device):
            return self.step_function.run(entries)

    # ---- generation ----
    def sampling_params(self, flags: dict | None = None, **fields) -> SamplingParams:
        """`SamplingParams(**fields)` with the filters a sampled request runs with when it names none: its own top_p /
        top_k / min_p if it gives any (the rest from `flags`), else `flags`, else the model card's, else none
        (`sampling.defaults`). A greedy request is left as it is."""
        if float(fields.get("temperature") or 0.0) > 0.0:
            chosen = resolve_filters(fields, flags, self.card_sampling)
            fields = dict(fields, top_p=chosen["top_p"], top_k=chosen["top_k"], min_p=chosen["min_p"])
        return SamplingParams(**{k: v for k, v in fields.items() if v is not None})

    def add_request(self, prompt: list[int], params: SamplingParams | None = None, request_id=None) -> Request:
        params = params or SamplingParams()
        if request_id is None:
            request_id = f"r{self._next_id}"
            self._next_id += 1
        vocab = self.model.vocab_size
        bad = [t for t in prompt if not 0 <= int(t) < vocab]
        if bad:
            raise ValueError(f"request {request_id!r}: token id {bad[0]} is outside the vocabulary of {vocab}")
        bad = [t for t in (params.logit_bias or ()) if t >= vocab]
        if bad:
            raise ValueError(f"request {request_id!r}: logit_bias names token {bad[0]}; the vocabulary has {vocab}")
        req = Request(request_id, [int(t) for t in prompt], params)
        self.scheduler.add(req)
        return req

    def abort(self, request: Request) -> None:
        """Take a request out wherever it is (waiting, between two portions of its prompt, decoding, with a step in the
        air): its pages and its slot go back at once. A row that a launched step still computes for it counts for nothing,
        and what that step still writes lands in pages whose next owner overwrites them before reading them (its own
        steps come later on the stream)."""
        if request.state != "finished":
            self.scheduler.abort(request)
            while request.output and request.output[-1] < 0:        # places kept for tokens of steps still in the air
                request.output.pop()

    # ---- records ----
    def set_routing_record(self, on: bool) -> None:
        """Count (or stop counting) the pairs every step routes to each expert of each routed feed-forward; a step's
        record then holds `experts_touched` (per routed layer, in run order) and `pairs_routed`. The counting is a
        kernel of the pass, so it works in steps replayed from graphs; graphs captured before the switch are dropped."""
        parts = []
        for layer in self.model.layers:
            ff = layer.feed_forward
            if hasattr(ff, "count_into") and hasattr(ff, "num_experts"):
                parts.append(ff)
        if self._flight is not None:            # a step launched ahead belongs to the old setting: account it first
            flight, self._flight = self._flight, None
            self._account(flight)
        self.step_function.drop_graphs()
        self._routed_parts = parts if on else []
        self._routing = self._routing_seen = None
        if on and parts:
            sizes = [p.num_experts for p in parts]
            self._routing = torch.zeros(sum(sizes), dtype=torch.int64, device=self.device)
            self._routing_seen = np.zeros(sum(sizes), dtype=np.int64)
            at = 0
            for p, n in zip(parts, sizes):
                p.count_into(self._routing[at:at + n])
                at += n
        else:
            for p in parts:
                p.count_into(None)

    def _finish_record(self, flight: "_Flight", finished: int) -> None:
        rec = flight.record
        rec["ms"] = round((time.perf_counter() - flight.started) * 1e3, 3)
        rec["finished"] = finished
        if flight.routed is not None and self._routing_seen is not None and flight.routed.numel() == self._routing_seen.size:
            now = flight.routed.numpy().copy()
            delta, at, touched = now - self._routing_seen, 0, []
            self._routing_seen = now
            for p in self._routed_parts:
                touched.append(int((delta[at:at + p.num_experts] > 0).sum()))
                at += p.num_experts
            rec["experts_touched"] = touched
            rec["pairs_routed"] = int(delta.sum())
            rec["routed"] = delta          # numpy int64, per routed layer its experts in a row (not written to the log)
        self.records.append(rec)
        if self._log_path:
            if self._log_file is None:
                self._log_file = open(self._log_path, "a")
            self._log_file.write(json.dumps({k: v for k, v in rec.items() if k != "routed"}) + "\n")
            self._log_file.flush()

    @property
    def last_record(self) -> dict | None:
        return self.records[-1] if self.records else None

    def run_step(self) -> list[Request]:
        """One scheduler step: schedule, run, sample, account. Returns the requests that finished.

        With `overlap` (the default) and nothing but decoding to do, the step after this one is scheduled and launched
        before this one's tokens are read: its token ids are the sampler's output, fed on the device, and its
        integers are staged while the GPU works. A request that ends on a stop id has then run one row for nothing,
        which is dropped; requests that end by their token limit are known beforehand and run no such row."""
        sch = self.scheduler
        while True:
            if self._flight is None:
                batch = sch.schedule()
                if not batch:
                    return []
                self._flight = self._launch(batch, None)
                sch.advance(batch)
            cur, self._flight = self._flight, None
            if self.args.overlap and self._runs_ahead(cur):
                batch = sch.schedule()
                if batch:
                    self._flight = self._launch(batch, cur)
                    sch.advance(batch)
            # rows of requests that ended (or were aborted) after the step was launched count for nothing
            live = any(s.request.last_slot is None or s.slot <= s.request.last_slot for s in cur.batch if s.samples) \
                or not any(s.samples for s in cur.batch)
            done = self._account(cur)
            if self._flight is not None and not sch.has_unfinished():
                # nothing is left to schedule: the step launched ahead holds the last tokens of requests that end by
                # their token limit, or nothing but rows of requests that ended on a stop id
                last, self._flight = self._flight, None
                if any(s.finishes for s in last.batch):
                    done += self._account(last)
            if live or not sch.has_unfinished():
                return done

    def _account(self, flight: "_Flight") -> list[Request]:
        """Wait for a launched step and hand its tokens to the scheduler; returns the requests that finished."""
        flight.event.synchronize()
        if self.step_function.check_status and int(flight.host[flight.n]):
            self._flight = None
            self.step_function.raise_on_fault()
        done = self.scheduler.resolve(flight.batch, flight.host[:flight.n].tolist())
        self._finish_record(flight, len(done))
        return done

    def _runs_ahead(self, cur: "_Flight") -> bool:
        """Whether the next step is known before this one's tokens are: every running request has just the token
        pending that `cur` is computing, nobody waits to be admitted, and the rows and their pages fit."""
        sch = self.scheduler
        if sch.waiting or not sch.running or len(sch.running) > sch.budget:
            return False
        if any(r.params.no_repeat_ngram_size for r in sch.running):
            return False            # the rule's next verdict needs this step's token on the host
        if any(r.pending != 1 or r.request_id not in cur.index for r in sch.running):
            return False
        return not sch._pages_short([(r, 1) for r in sch.running])

    def _sample_row(self, r: Request) -> SampleRow:
        """What the sampler needs of a request whose next token is drawn now. A request with penalties also names its
        row of counts (its slot in the cache) and how to read its history; (id, arrival, preemptions) tells the sampler
        when that row holds another request's counts, or this one's from before it lost its place."""
        position = len(r.prompt) + len(r.output)
        blocked = None
        if r.params.no_repeat_ngram_size:
            # the rule's memory lives with the request and follows its text (a request that was preempted kept its text)
            if r.no_repeat is None:
                r.no_repeat = NoRepeatIndex(r.params.no_repeat_ngram_size)
            if r.no_repeat.seen < position:
                r.no_repeat.add(r.span(r.no_repeat.seen, position - r.no_repeat.seen))
            blocked = r.no_repeat.blocked()
        if not r.params.penalizes:
            return SampleRow(r.params, position, blocked=blocked)
        return SampleRow(r.params, position, self.cache.slot_of(r.request_id), (r.request_id, r.order, r.preemptions),
                         lambda: r.span(0, position), blocked)

    def _launch(self, batch, before: "_Flight | None") -> "_Flight":
        """Run `batch` and its sampling without waiting for them. `before`: the step whose tokens this one's rows
        take from the device."""
        fn = self.step_function
        started = time.perf_counter()
        entries = [StepEntry(s.request.request_id, s.request.span(s.start, s.count),
                             [s.count - 1] if s.samples else []) for s in batch]
        feedback = None
        if before is not None:
            feedback = (before.tokens, [before.index[e.request] for e in entries])
        with torch.cuda.device(self.device):
            # one wait a step: the chosen tokens and the kernels' status word come back together
            checks, fn.check_status = fn.check_status, False
            try:
                logits = fn.run(entries, feedback)
            finally:
                fn.check_status = checks
            rows = [self._sample_row(s.request) for s in batch if s.samples]
            n = len(rows)
            self._turn ^= 1
            host = self._results[self._turn]
            if host is None or host.numel() < n + 1:
                host = self._results[self._turn] = torch.empty(max(64, 2 * (n + 1)), dtype=torch.int32).pin_memory()
            tokens = self.sampler(logits, rows) if n else None
            if n:
                host[:n].copy_(tokens, non_blocking=True)
            host[n:n + 1].copy_(self.model.runtime.status, non_blocking=True)
            routed = None
            if self._routing is not None:
                routed = self._routed_host[self._turn]
                if routed is None or routed.numel() != self._routing.numel():
                    routed = self._routed_host[self._turn] = torch.empty(self._routing.numel(), dtype=torch.int64).pin_memory()
                routed.copy_(self._routing, non_blocking=True)
            event = torch.cuda.Event()
            event.record()
        index = {s.request.request_id: i for i, s in enumerate(x for x in batch if x.samples)}
        sch, rows = self.scheduler, sum(s.count for s in batch)
        decode_rows = sum(1 for s in batch if s.count == 1 and s.samples and s.request.output)
        record = {"step": fn.steps, "requests": len(batch), "rows": rows, "prompt_rows": rows - decode_rows,
                  "decode_rows": decode_rows, "sampled": n, "from_graph": fn.last_from_graph,
                  "pages_used": [g.pool.used for g in self.cache.groups],
                  "pages_free": [g.pool.free for g in self.cache.groups],
                  "running": len(sch.running), "waiting": len(sch.waiting), "preemptions": sch.stats.preemptions}
        return _Flight(batch, host, n, event, tokens, index, record, started, routed)

    def generate(self, prompts: list[list[int]], params: SamplingParams | list[SamplingParams] | None = None
                 ) -> list[list[int]]:
        """Generated token ids for each prompt (token ids in, token ids out)."""
        if params is None or isinstance(params, SamplingParams):
            base = params or SamplingParams()
            plist = [SamplingParams(**vars(base)) for _ in prompts]
        else:
            plist = list(params)
            if len(plist) != len(prompts):
                raise ValueError(f"{len(prompts)} prompts with {len(plist)} sampling parameter sets")
        reqs = [self.add_request(p, sp) for p, sp in zip(prompts, plist)]
        while self.scheduler.has_unfinished():
            self.run_step()
        return [r.output for r in reqs]

    def warm_up(self, batch_sizes: list[int] | None = None, prompt_tokens: int | None = None) -> dict:
        """Throwaway requests through the step function, so that the first real request finds every kernel library
        of a prompt step and of a decode step loaded, and the decode graphs of `batch_sizes` (default: 1, 2, 4, ... up
        to `parallel`) captured for short contexts. Nothing of it stays: pages and slots are given back, no record is
        written. Only with no request waiting or running."""
        if self.scheduler.has_unfinished() or self._flight is not None:
            raise RuntimeError("warm_up() while requests are waiting or running")
        args, started = self.args, time.perf_counter()
        if batch_sizes is None:
            batch_sizes, b = [], 1
            while b < args.parallel:
                batch_sizes.append(b)
                b *= 2
            batch_sizes.append(args.parallel)
        bad = [b for b in batch_sizes if not 1 <= b <= args.parallel]
        if bad:
            raise ValueError(f"warm_up: batch size {bad[0]} with {args.parallel} requests running at once at most")
        portion = min(prompt_tokens or args.chunk_size, args.max_batched_tokens, args.max_len - 3)
        most, before = max(batch_sizes), len(self.step_function._graphs)
        ids = [("warm-up", i) for i in range(most)]
        with torch.cuda.device(self.device):
            try:
                for rid in ids:
                    self.admit(rid)
                # a prompt's portion beside nothing, then two tokens of each of the others (a step of portions, which is
                # not captured): every request holds keys
                self.step([StepEntry(ids[0], [0] * max(1, portion), [max(1, portion) - 1])])
                if most > 1:
                    self.step([StepEntry(rid, [0, 0], [1]) for rid in ids[1:]])
                for b in sorted(set(batch_sizes)):
                    for _ in range(2):                 # the first is eager and captured behind it, the second a replay
                        self.step([StepEntry(rid, [0], [0]) for rid in ids[:b]])
                torch.cuda.synchronize(self.device)
            finally:
                for rid in ids:
                    if self.cache.has(rid):
                        self.release(rid)
        return {"seconds": round(time.perf_counter() - started, 3), "batch_sizes": sorted(set(batch_sizes)),
                "graphs_captured": len(self.step_function._graphs) - before}

    def stats(self) -> dict:
        fn = self.step_function
        return {"scheduler": vars(self.scheduler.stats), "cache": self.cache.stats(),
                "steps": fn.steps, "rows": fn.rows_run, "graph_replays": fn.graph_replays, "graphs_kept": len(fn._graphs),
                "graphs_dropped": fn.graphs_dropped}

    def decode_bytes(self, batch: int, context: int, experts_read: list[int] | None = None) -> dict:
        """Bytes one decode step of `batch` requests at `context` tokens has to read: see `DecoderModel.decode_bytes`,
        plus the keys and values of the live requests in every page group (a windowed group holds its window)."""
        out = self.model.decode_bytes(batch, experts_read)
        elem = self.cache.site_cache[self.cache.groups[0].sites[0]].k.element_size() if self.cache.groups else 0
        kv = 0
        for g in self.cache.groups:
            span = context if g.need.window is None else min(context, g.need.window)
            kv += len(g.sites) * 2 * g.need.kv_heads * g.need.head_dim * elem * span * batch
        out["kv"] = kv
        out["total"] += kv
        return out
