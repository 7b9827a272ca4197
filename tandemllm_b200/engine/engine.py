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

from dataclasses import dataclass

import torch

from ..cache.manager import CacheManager
from ..config.registry import read_model_config, resolve_model_folder, spec_of
from ..parts.base import Runtime
from ..parts.model import DecoderModel
from ..sampling.sampler import Sampler, SamplingParams
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
    max_batched_tokens: int = 2048      # token budget of one step
    chunk_size: int = 512               # longest prompt portion in one step
    device: str = "cuda:0"
    graph: bool = True                  # capture decode-only steps in CUDA graphs (bfloat16)
    tensorcore: bool = True             # use the tcgen05 kernels in bfloat16


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
        self.step_function = StepFunction(model, self.cache, use_graphs=args.graph and model.graph_safe,
                                          max_graph_batch=args.parallel)
        self.sampler = Sampler(self.device)
        self.scheduler = Scheduler(self.cache, max_num_seqs=args.parallel, max_num_batched_tokens=args.max_batched_tokens,
                                   chunk_size=args.chunk_size, max_model_len=args.max_len,
                                   stop_token_ids=model.spec.stop_token_ids)
        self._next_id = 0

    # ---- construction ----
    @classmethod
    def from_folder(cls, folder: str, args: EngineArgs | None = None, **kw) -> "Engine":
        """A model folder: config.json chooses the architecture, model.safetensors holds the weights."""
        args = args or EngineArgs(**kw)
        folder = resolve_model_folder(folder)
        arch, config = read_model_config(folder)
        spec = spec_of(config)
        return cls._build(arch, spec, FolderWeights(folder, spec.name_prefixes), args)

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
    def add_request(self, prompt: list[int], params: SamplingParams | None = None, request_id=None) -> Request:
        params = params or SamplingParams()
        if request_id is None:
            request_id = f"r{self._next_id}"
            self._next_id += 1
        vocab = self.model.vocab_size
        bad = [t for t in prompt if not 0 <= int(t) < vocab]
        if bad:
            raise ValueError(f"request {request_id!r}: token id {bad[0]} is outside the vocabulary of {vocab}")
        req = Request(request_id, [int(t) for t in prompt], params)
        self.scheduler.add(req)
        return req

    def add_request_with_context(self, prompt: list[int], params: SamplingParams | None = None, request_id=None) -> Request:
        """For measurement: a running request whose prompt, except its last token, counts as already computed. Its
        pages are reserved and hold whatever they held (fill the cache tensors first for realistic values), so a
        decode step at a long context can be timed without running the prompt. The text it generates is not meaningful."""
        req = self.add_request(prompt, params, request_id)
        self.scheduler.waiting.remove(req)
        self.cache.admit(req.request_id)
        n = len(req.prompt) - 1
        self.cache.reserve(req.request_id, n)
        self.cache.advance(req.request_id, n)
        req.num_computed = n
        req.state = "running"
        self.scheduler.running.append(req)
        return req

    def run_step(self) -> list[Request]:
        """One scheduler step: schedule, run, sample, account. Returns the requests that finished."""
        batch = self.scheduler.schedule()
        if not batch:
            return []
        entries = [StepEntry(s.request.request_id, s.request.tokens[s.start:s.start + s.count],
                             [s.count - 1] if s.samples else []) for s in batch]
        with torch.cuda.device(self.device):
            logits = self.step_function.run(entries)
            rows = [(s.request.params, len(s.request.prompt) + len(s.request.output)) for s in batch if s.samples]
            tokens = self.sampler(logits, rows).tolist() if rows else []
        return self.scheduler.update(batch, tokens)

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

    def stats(self) -> dict:
        return {"scheduler": vars(self.scheduler.stats), "cache": self.cache.stats(),
                "steps": self.step_function.steps, "rows": self.step_function.rows_run}
