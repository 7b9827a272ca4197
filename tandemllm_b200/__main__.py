"""Command line: `python -m tandemllm_b200 <command> ...`

  generate        token ids in, token ids out, through the scheduler and the step function
  random-weights  write a model folder (config.json, model.safetensors) from a config.json and a seed
  audit           a model folder checked from its headers alone, on the CPU: names, shapes, bytes
  compare         two replays of one trace held against each other, row by row
  replay          the trace replay program (the same as bin/trace_run)
  bench           the measurement program (the same as bench.py at the repository's root)

Option names follow the reference's command lines where it has them: `--model`, `--max-len`, `--tokens`,
`--graph on|off`, `--json` (tools/lfm_check.py:374-418), `--temperature`, `--top-p`, `--top-k`, `--parallel`,
`--rep-penalty`, `--presence-penalty`, `--frequency-penalty` (server/app.py:12893-12940). No tokenizer is involved: prompts are token ids.
"""

from __future__ import annotations

import argparse
import json
import sys
import time


def _engine_options(p: argparse.ArgumentParser) -> None:
    p.add_argument("--model", help="a folder with config.json and model.safetensors")
    p.add_argument("--config", help="a config.json to build a random-weights model from (with --random-weights)")
    p.add_argument("--random-weights", type=int, metavar="SEED", help="random weights from this seed instead of --model")
    p.add_argument("--std", type=float, default=0.02, help="standard deviation of random matrices")
    p.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    p.add_argument("--max-len", type=int, default=8192, help="the window: prompt plus generated tokens of a request")
    p.add_argument("--parallel", type=int, default=8, help="requests running at once")
    p.add_argument("--block-size", type=int, default=16, help="tokens per cache page")
    p.add_argument("--kv-blocks", type=int, help="cache pages (default: enough for --parallel requests of --max-len)")
    p.add_argument("--max-batched-tokens", type=int, default=4096, help="token budget of one step")
    p.add_argument("--chunk-size", type=int, default=2048, help="longest prompt portion in one step")
    p.add_argument("--graph", default="on", choices=("on", "off"), help="CUDA graphs for decode-only steps")
    p.add_argument("--device", default="cuda:0")
    p.add_argument("--warm-up", action="store_true",
                   help="run throwaway requests first: kernel libraries loaded and decode graphs captured before the clock starts")
    p.add_argument("--log", help="append one JSON line a scheduler step here (rows, pages, milliseconds)")
    p.add_argument("--log-routing", action="store_true",
                   help="count the experts every step touches in every routed layer (into the step records and --log)")


def _build_engine(a):
    from .config import Lfm2MoeConfig, architecture_of
    from .engine import Engine, EngineArgs
    args = EngineArgs(dtype=a.dtype, max_len=a.max_len, parallel=a.parallel, block_size=a.block_size,
                      kv_blocks=a.kv_blocks, max_batched_tokens=a.max_batched_tokens, chunk_size=a.chunk_size,
                      device=a.device, graph=a.graph == "on", log=a.log, record_routing=a.log_routing)
    if a.random_weights is not None:
        if not a.config:
            raise SystemExit("--random-weights needs --config FILE (a config.json)")
        with open(a.config) as f:
            raw = json.load(f)
        config = architecture_of(raw).read_config(raw, "", None)
        return Engine.from_config(config, a.random_weights, args, std=a.std)
    if not a.model:
        raise SystemExit("give --model DIR, or --config FILE with --random-weights SEED")
    return Engine.from_folder(a.model, args)


def cmd_generate(a) -> int:
    import torch

    from .sampling import SamplingParams
    engine = _build_engine(a)
    vocab = engine.model.vocab_size
    if a.prompt_ids:
        prompts = [[int(t) for t in p.replace(",", " ").split()] for p in a.prompt_ids]
    else:
        g = torch.Generator().manual_seed(a.prompt_seed)
        prompts = [torch.randint(0, vocab, (a.prompt_len,), generator=g).tolist() for _ in range(a.prompts)]
    params = engine.sampling_params(temperature=a.temperature, top_p=a.top_p, top_k=a.top_k, min_p=a.min_p, seed=a.seed,
                            max_tokens=a.tokens, ignore_eos=a.ignore_eos, repetition_penalty=a.rep_penalty,
                            presence_penalty=a.presence_penalty, frequency_penalty=a.frequency_penalty,
                            logit_bias=_logit_bias(a.logit_bias), no_repeat_ngram_size=a.no_repeat_ngram_size,
                            max_pattern_size=a.max_pattern_size, min_pattern_size=a.min_pattern_size, min_count=a.min_count)
    warm = engine.warm_up() if a.warm_up else None
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    outs = engine.generate(prompts, params)
    torch.cuda.synchronize()
    dt = time.perf_counter() - t0
    result = {"outputs": outs, "seconds": round(dt, 4), "generated": sum(len(o) for o in outs),
              "tok_s": round(sum(len(o) for o in outs) / dt, 2), "stats": engine.stats()}
    if warm is not None:
        result["warm_up"] = warm
    for i, o in enumerate(outs):
        print(f"[{i}] " + " ".join(str(t) for t in o))
    print(json.dumps({k: v for k, v in result.items() if k != "outputs"}), file=sys.stderr)
    if a.json:
        with open(a.json, "w") as f:
            json.dump({"prompts": prompts, **result}, f)
    return 0


def cmd_random_weights(a) -> int:
    import torch

    from .config import architecture_of
    from .weights.random_init import write_model_folder
    with open(a.config) as f:
        raw = json.load(f)
    config = architecture_of(raw).read_config(raw, "", None)
    dtype = {"bfloat16": torch.bfloat16, "float32": torch.float32}[a.dtype]
    print(write_model_folder(config, a.out, a.seed, std=a.std, bias_std=a.bias_std, norm_std=a.norm_std, dtype=dtype))
    return 0


def cmd_audit(a) -> int:
    """A model folder's audit record from its headers alone (no tensor is read, no GPU is needed; the reference's
    tools/lfm_check.py:331-347 `audit`): the architecture and its sizes, the stored tensors against what the parts
    would read (`refused`: the loader's one error, or null), the bytes on disk by stored type, and the bytes of weights
    one decode step reads at the batch sizes asked for."""
    import os

    from .config.registry import read_model_config, resolve_model_folder, spec_of
    from .parts.model import DecoderModel
    from .weights.loader import FolderWeights
    from .weights.safetensors_io import CheckpointError
    folder = resolve_model_folder(a.model)
    arch, config = read_model_config(folder)
    spec = spec_of(config)
    build = arch.build_model if arch is not None and arch.build_model else DecoderModel
    model = build(spec)
    weights = FolderWeights(folder, spec.name_prefixes)
    expected = model.weight_specs(weights.present())
    ignored = set(spec.ignored_names)
    try:
        weights.check(expected, ignore=(lambda n: n in ignored) if ignored else None)
        refused = None
    except CheckpointError as e:
        refused = str(e)
    by_type: dict[str, dict] = {}
    for st in weights.stored.values():
        row = by_type.setdefault(st.dtype, {"tensors": 0, "bytes": 0})
        row["tensors"] += 1
        row["bytes"] += st.nbytes
    files = sorted(f for f in os.listdir(folder) if f.endswith(".safetensors"))
    out = {"folder": folder, "architecture": arch.name if arch is not None else None, "layers": len(spec.layers),
           "run_order": len(spec.schedule), "hidden_size": spec.hidden_size, "vocab_size": spec.vocab_size,
           "tensors_expected": len(expected), "tensors_stored": len(weights.stored), "refused": refused,
           "stored": by_type, "files": len(files),
           "safetensors_gb": round(sum(os.path.getsize(os.path.join(folder, f)) for f in files) / 1e9, 3),
           "decode_bytes": {str(b): model.decode_bytes(b) for b in a.batch}}
    print(json.dumps(out, indent=1))
    return 0 if refused is None else 1


def compare_logits(a_dir: str, b_dir: str, vocab: int) -> dict:
    """Two replays of one trace (`bin/trace_run --out`), row by row: `b_dir` is the reference (say, the 32-bit run), `a_dir`
    the run held against it. The record of the reference's teacher-forced comparison (tools/lfm_check.py:100-127):
    positions, how often the largest logit agrees, disagreements split into near ties (the reference's own margin below
    8 * 2^-7 of its row's largest logit, what bfloat16 cannot tell apart) and others, and the largest and mean difference
    relative to a row's largest logit."""
    import os

    import numpy as np
    steps = sorted((f for f in os.listdir(b_dir) if f.endswith(".f32")), key=lambda f: int(f[:-4]))
    agree = total = near = other = 0
    max_rel, means, bad, missing = 0.0, [], [], []
    for f in steps:
        if not os.path.isfile(os.path.join(a_dir, f)):
            missing.append(f)
            continue
        ref = np.fromfile(os.path.join(b_dir, f), dtype="<f4").reshape(-1, vocab).astype(np.float64)
        got = np.fromfile(os.path.join(a_dir, f), dtype="<f4").reshape(-1, vocab).astype(np.float64)
        if got.shape != ref.shape:
            raise SystemExit(f"step {f[:-4]}: {got.shape[0]} rows against {ref.shape[0]}")
        scale = np.abs(ref).max(-1)
        d = np.abs(got - ref)
        max_rel = max(max_rel, float((d.max(-1) / scale).max()))
        means.append(float((d.mean(-1) / scale).mean()))
        ga, ra = got.argmax(-1), ref.argmax(-1)
        for i in range(ref.shape[0]):
            total += 1
            if ga[i] == ra[i]:
                agree += 1
                continue
            margin = float(ref[i, ra[i]] - ref[i, ga[i]])
            tie = margin < 8 * 2 ** -7 * float(scale[i])
            near += tie
            other += not tie
            if len(bad) < 12:
                bad.append({"step": int(f[:-4]), "row": i, "margin": round(margin, 4), "near_tie": bool(tie)})
    return {"steps": len(steps) - len(missing), "missing_steps": [int(f[:-4]) for f in missing], "positions": total,
            "argmax_agree": agree, "agree_pct": round(100 * agree / max(total, 1), 2), "near_tie": near, "other": other,
            "max_rel_diff": round(max_rel, 6), "mean_rel_diff": round(sum(means) / max(len(means), 1), 7),
            "disagreements": bad}


def cmd_compare(a) -> int:
    vocab = a.vocab
    if vocab is None:
        if not a.model:
            raise SystemExit("give --vocab N, or --model DIR to read it from")
        from .config.registry import read_model_config, spec_of
        vocab = spec_of(read_model_config(a.model)[1]).vocab_size
    rec = compare_logits(a.run, a.reference, vocab)
    print(json.dumps(rec, indent=1))
    return 0 if rec["other"] == 0 and not rec["missing_steps"] else 1


def cmd_replay(a) -> int:
    import os
    import runpy
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bin", "trace_run")
    sys.argv = [path] + a.rest
    runpy.run_path(path, run_name="__main__")
    return 0


def cmd_bench(a) -> int:
    import os
    import runpy
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py")
    if not os.path.isfile(path):
        raise SystemExit(f"bench.py is not beside the package ({path})")
    sys.argv = [path] + a.rest
    runpy.run_path(path, run_name="__main__")
    return 0


def _logit_bias(items) -> dict | None:
    """{token: added logit} from TOKEN:VALUE arguments."""
    bias = {}
    for item in items or ():
        token, sep, value = item.partition(":")
        try:
            if not sep:
                raise ValueError
            bias[int(token)] = float(value)
        except ValueError:
            raise SystemExit(f"--logit-bias takes TOKEN:VALUE, as in 17:-4.5; got {item!r}")
    return bias or None


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="python -m tandemllm_b200", description=__doc__,
                                 formatter_class=argparse.RawDescriptionHelpFormatter)
    sub = ap.add_subparsers(dest="cmd", required=True)
    g = sub.add_parser("generate", help="generate token ids")
    _engine_options(g)
    g.add_argument("--prompt-ids", action="append", help="a prompt as token ids separated by spaces or commas (repeatable)")
    g.add_argument("--prompts", type=int, default=1, help="number of random prompts when no --prompt-ids is given")
    g.add_argument("--prompt-len", type=int, default=32)
    g.add_argument("--prompt-seed", type=int, default=0)
    g.add_argument("--tokens", type=int, default=128, help="new tokens per request at most")
    g.add_argument("--temperature", type=float, default=0.0)
    g.add_argument("--top-p", type=float, help="default with a temperature: the model card's (generation_config.json), else 1")
    g.add_argument("--top-k", type=int, help="default with a temperature: the model card's, else 0 (off)")
    g.add_argument("--min-p", type=float, help="default 0")
    g.add_argument("--rep-penalty", type=float, default=1.0,
                   help="repetition penalty: a logit of a token seen in the prompt or the output is divided by this if "
                        "positive, multiplied if negative (1.0: off)")
    g.add_argument("--presence-penalty", type=float, default=0.0, help="subtracted once from the logit of a seen token")
    g.add_argument("--frequency-penalty", type=float, default=0.0,
                   help="subtracted from the logit of a seen token, times the number of times it was seen")
    g.add_argument("--logit-bias", action="append", metavar="TOKEN:VALUE", help="added to this token's logit (repeatable)")
    g.add_argument("--no-repeat-ngram-size", type=int, default=0,
                   help="n >= 2: a token that would repeat an n-gram of the text so far loses 4 from its logit")
    g.add_argument("--max-pattern-size", type=int, default=0,
                   help="with --min-count: end a request whose last tokens are one block of up to this many tokens, repeated")
    g.add_argument("--min-pattern-size", type=int, default=1)
    g.add_argument("--min-count", type=int, default=0, help="repetitions of the block that end the request (>= 2)")
    g.add_argument("--seed", type=int, help="sampling seed (default: from the operating system)")
    g.add_argument("--ignore-eos", action="store_true")
    g.add_argument("--json", help="write prompts, outputs and timing here")
    g.set_defaults(fn=cmd_generate)
    r = sub.add_parser("random-weights", help="write a random model folder")
    r.add_argument("--config", required=True)
    r.add_argument("--out", required=True)
    r.add_argument("--seed", type=int, default=0)
    r.add_argument("--std", type=float, default=0.02)
    r.add_argument("--bias-std", type=float, default=0.1)
    r.add_argument("--norm-std", type=float, default=0.0)
    r.add_argument("--dtype", default="bfloat16", choices=("bfloat16", "float32"))
    r.set_defaults(fn=cmd_random_weights)
    u = sub.add_parser("audit", help="a model folder checked from its headers alone (CPU): names, shapes, bytes")
    u.add_argument("--model", required=True)
    u.add_argument("--batch", type=int, nargs="*", default=[1, 8, 64], help="decode batch sizes to account bytes for")
    u.set_defaults(fn=cmd_audit)
    c = sub.add_parser("compare", help="two replays of one trace, row by row (say bfloat16 against float32)")
    c.add_argument("--run", required=True, help="the --out folder of the replay that is checked")
    c.add_argument("--reference", required=True, help="the --out folder of the replay it is held against")
    c.add_argument("--model", help="the model folder (for the vocabulary size)")
    c.add_argument("--vocab", type=int)
    c.set_defaults(fn=cmd_compare)
    p = sub.add_parser("replay", help="the trace replay program; options as for bin/trace_run")
    p.add_argument("rest", nargs=argparse.REMAINDER)
    p.set_defaults(fn=cmd_replay)
    b = sub.add_parser("bench", help="the measurement program; options as for bench.py")
    b.add_argument("rest", nargs=argparse.REMAINDER)
    b.set_defaults(fn=cmd_bench)
    a = ap.parse_args(argv)
    return a.fn(a)


if __name__ == "__main__":
    sys.exit(main())
