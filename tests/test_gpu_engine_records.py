"""The engine's per-step records and routing counts, the bound on captured decode graphs, and the command line run as a
user runs it (random-weights, then generate), on the GPU."""

import json
import os
import subprocess
import sys

import pytest
import torch

from tests import plain_lfm2 as P
from tests import tiny_configs as T
from tests.helpers import random_model_weights, write_folder

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def folder_of(name, tmp_path, dtype=torch.float32):
    cfg = T.CONFIGS[name]
    W = random_model_weights(cfg, T.SEEDS[name], T.STD[name], bf16_exact=True)
    return write_folder(str(tmp_path / name), cfg, W, dtype), cfg, W


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_every_step_leaves_a_record_and_a_log_line(tmp_path, dtype):
    from tandemllm_b200.engine import Engine, EngineArgs
    from tandemllm_b200.sampling import SamplingParams
    folder, cfg, W = folder_of("c", tmp_path, torch.bfloat16 if dtype == "bfloat16" else torch.float32)
    log = tmp_path / "steps.jsonl"
    eng = Engine.from_folder(folder, EngineArgs(dtype=dtype, max_len=256, parallel=3, chunk_size=16, max_batched_tokens=24,
                                                log=str(log), record_routing=True))
    prompts = [T.long_tokens("c", n, seed=3 + n) for n in (40, 9, 21)]
    outs = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=12, ignore_eos=True))
    records = list(eng.records)
    lines = [json.loads(ln) for ln in log.read_text().splitlines()]
    assert len(lines) == len(records) and len(records) >= 12
    assert [r["step"] for r in records] == sorted(r["step"] for r in records)
    # rows: every prompt token and every generated token but each request's last went through a step exactly once
    assert sum(r["rows"] for r in records) == sum(len(p) for p in prompts) + sum(len(o) - 1 for o in outs)
    assert sum(r["sampled"] for r in records) == sum(len(o) for o in outs)
    assert sum(r["finished"] for r in records) == 3
    moe_layers = sum(1 for i in range(cfg["num_hidden_layers"]) if i >= cfg["num_dense_layers"])
    k, E = cfg["num_experts_per_tok"], cfg["num_experts"]
    for r, line in zip(records, lines):
        assert r["rows"] == r["prompt_rows"] + r["decode_rows"] and r["rows"] <= 24 and r["ms"] > 0
        assert len(r["experts_touched"]) == moe_layers and r["pairs_routed"] == r["rows"] * k * moe_layers
        assert all(1 <= n <= min(E, r["rows"] * k) for n in r["experts_touched"])
        assert r["routed"].shape == (moe_layers * E,) and "routed" not in line
        assert line["experts_touched"] == r["experts_touched"] and line["pages_used"] == r["pages_used"]
        assert r["pages_used"][0] + r["pages_free"][0] == eng.cache.groups[0].pool.num_pages
    assert any(r["from_graph"] for r in records) and not records[0]["from_graph"]
    # one step's count against the plain implementation's routing of the same rows: the first step holds the first
    # portion (16 tokens) of the first prompt and, with what is left of the budget of 24, 8 tokens of the second
    first = records[0]
    assert first["rows"] == 24 and first["requests"] == 2
    if dtype == "float32":
        routes = {}
        orig = P.route

        def spy(n, Wd, p, c, forced=None):
            ids, w = orig(n, Wd, p, c, forced)
            routes.setdefault(p, []).append(ids)
            return ids, w
        P.route = spy
        try:
            P.forward(cfg, W, prompts[0][:16])
            P.forward(cfg, W, prompts[1][:8])
        finally:
            P.route = orig
        want = [int(torch.unique(torch.cat(ids)).numel()) for _, ids in sorted(routes.items())]
        assert first["experts_touched"] == want
    # switching the record off stops the counting and drops nothing else
    eng.set_routing_record(False)
    eng.generate([prompts[1]], SamplingParams(temperature=0.0, max_tokens=3, ignore_eos=True))
    assert "experts_touched" not in eng.last_record


def test_captured_decode_graphs_stay_bounded_while_batch_and_context_grow(tmp_path):
    """Batches of 1 to 6 requests decode, one of them from the third round on at a context in another bucket, with room
    for 4 graphs only: the step function never keeps more, drops the least recently used, keeps giving the eager
    engine's logits bit for bit, and the device memory it holds stops growing."""
    from tandemllm_b200.engine import Engine, EngineArgs, StepEntry
    folder, cfg, W = folder_of("c", tmp_path, torch.bfloat16)
    engines = [Engine.from_folder(folder, EngineArgs(dtype="bfloat16", max_len=8192, parallel=6, graph=g)) for g in (True, False)]
    engines[0].step_function.max_graphs = 4
    toks = {i: T.long_tokens("c", 40, seed=50 + i) for i in range(6)}
    reserved = []
    for eng in engines:
        for i in toks:
            eng.admit(i)
    out = [[], []]
    for j, eng in enumerate(engines):
        fn = eng.step_function
        for i, t in toks.items():
            # contexts that differ by whole buckets without running thousands of tokens: the cache counts positions only
            eng.step([StepEntry(i, t[:8], [])])
        for round_ in range(6):
            if round_ == 2:
                eng.step([StepEntry(0, T.long_tokens("c", 1100, seed=99), [])])
            for B in (1, 2, 3, 6, 4, 5):
                for _ in range(3):
                    entries = [StepEntry(i, [toks[i][8 + len(out[j]) % 30]], [0]) for i in range(B)]
                    out[j].append(eng.step(entries).clone())
                if j == 0:
                    assert len(fn._graphs) <= 4
            if j == 0:
                torch.cuda.synchronize()
                reserved.append(torch.cuda.memory_reserved())
    fn = engines[0].step_function
    assert fn.graphs_dropped >= 6 and fn.graph_replays > 20 and len(fn._graphs) == 4
    assert len({k[2] for k in fn._graphs}) == 1 and fn._graphs and next(iter(fn._graphs))[2] == 2048
    assert reserved[5] <= reserved[3] + (8 << 20), reserved        # no growth once every shape has been seen once
    assert len(out[0]) == len(out[1])
    for a, b in zip(*out):
        assert torch.equal(a, b)


def test_random_weights_then_generate_as_subprocesses(tmp_path):
    """`python -m tandemllm_b200 random-weights` writes a folder, `generate --model` reads it: the printed tokens are
    the plain implementation's greedy text from the same stored weights."""
    from tandemllm_b200.weights.safetensors_io import index_folder, read_tensor
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(T.TINY_A))
    model = tmp_path / "model"
    run = lambda *args: subprocess.run([sys.executable, "-m", "tandemllm_b200", *args], cwd=ROOT, capture_output=True,
                                       text=True, timeout=600)
    r = run("random-weights", "--config", str(cfg), "--out", str(model), "--seed", "9", "--dtype", "float32", "--norm-std", "0.1")
    assert r.returncode == 0, r.stderr[-2000:]
    prompts = ["5 17 3 200 41 8", "9,9,250"]
    log = tmp_path / "log.jsonl"
    r = run("generate", "--model", str(model), "--dtype", "float32", "--tokens", "8", "--ignore-eos", "--max-len", "128",
            "--parallel", "2", "--prompt-ids", prompts[0], "--prompt-ids", prompts[1], "--json", str(tmp_path / "out.json"),
            "--log", str(log), "--log-routing")
    assert r.returncode == 0, r.stderr[-2000:]
    printed = [[int(t) for t in ln.split("] ")[1].split()] for ln in r.stdout.splitlines() if ln.startswith("[")]
    stored = index_folder(str(model))
    W = {name[len("model."):] if name.startswith("model.") else name: read_tensor(st).float() for name, st in stored.items()}
    for text, got in zip(prompts, printed):
        prompt = [int(t) for t in text.replace(",", " ").split()]
        assert got == P.greedy(T.TINY_A, W, prompt, 8)
    saved = json.loads((tmp_path / "out.json").read_text())
    assert saved["outputs"] == printed and saved["generated"] == 16
    lines = [json.loads(ln) for ln in log.read_text().splitlines()]
    assert lines and all("experts_touched" in ln and "ms" in ln for ln in lines)


def test_named_ranges_for_profilers_change_nothing(tmp_path, monkeypatch):
    """With TANDEMLLM_NVTX set every step and layer is an NVTX range (eager steps and the capture of decode graphs alike);
    the tokens are the same bits as without."""
    from tandemllm_b200.engine import Engine, EngineArgs
    from tandemllm_b200.sampling import SamplingParams
    folder, cfg, W = folder_of("a", tmp_path)
    prompts = [T.long_tokens("a", n, seed=5 + n) for n in (19, 6)]

    def run():
        eng = Engine.from_folder(folder, EngineArgs(dtype="float32", max_len=128, parallel=2, chunk_size=8))
        return eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True))
    plain = run()
    monkeypatch.setenv("TANDEMLLM_NVTX", "1")
    assert run() == plain


def test_warm_up_leaves_nothing_behind_and_the_first_decode_steps_replay_graphs(tmp_path):
    """`Engine.warm_up`: the throwaway requests give every page and slot back, the decode graphs of its batch sizes are
    captured, the tokens generated afterwards are those of an engine that was not warmed, and the first decode steps of
    the real requests are replays (an engine that was not warmed runs each new shape eagerly once)."""
    from tandemllm_b200.engine import Engine, EngineArgs
    from tandemllm_b200.sampling import SamplingParams
    folder, cfg, W = folder_of("c", tmp_path, torch.bfloat16)
    args = dict(dtype="bfloat16", max_len=256, parallel=3, chunk_size=16, max_batched_tokens=24)
    prompts = [T.long_tokens("c", n, seed=5 + n) for n in (23, 9, 14)]
    params = SamplingParams(temperature=0.0, max_tokens=10, ignore_eos=True)

    cold = Engine.from_folder(folder, EngineArgs(**args))
    want = cold.generate(prompts, params)
    cold_replays = cold.stats()["graph_replays"]

    eng = Engine.from_folder(folder, EngineArgs(**args))
    def free_now():
        st = eng.cache.stats()
        return st["requests"], st["free_slots"], [g["free"] for g in st["groups"]]
    free_before = free_now()
    info = eng.warm_up()
    assert info["batch_sizes"] == [1, 2, 3] and info["graphs_captured"] == 3
    eng.cache.check()
    assert free_now() == free_before and not eng.records
    replays = eng.stats()["graph_replays"]
    assert eng.generate(prompts, params) == want
    assert eng.stats()["graph_replays"] - replays > cold_replays
    with pytest.raises(ValueError, match="batch size 4"):
        eng.warm_up([4])
    eng.add_request([1, 2, 3], params)
    with pytest.raises(RuntimeError, match="waiting or running"):
        eng.warm_up()


def test_a_sampled_request_without_filters_takes_the_model_cards(tmp_path):
    """`Engine.sampling_params`: generation_config.json's top_k / top_p stand in where a request with a temperature names
    no filter; a filter of the request's own, flags, and greedy requests go before or past them."""
    import json

    from tandemllm_b200.engine import Engine, EngineArgs
    folder, cfg, W = folder_of("a", tmp_path, torch.float32)
    with open(os.path.join(folder, "generation_config.json"), "w") as f:
        json.dump({"eos_token_id": 3, "top_k": 5, "top_p": 0.9}, f)
    eng = Engine.from_folder(folder, EngineArgs(dtype="float32", max_len=64, parallel=2))
    assert eng.card_sampling == {"top_k": 5, "top_p": 0.9}
    sp = eng.sampling_params(temperature=0.8, seed=4, max_tokens=6)
    assert (sp.top_k, sp.top_p, sp.min_p, sp.max_tokens) == (5, 0.9, 0.0, 6)
    sp_own = eng.sampling_params(temperature=0.8, top_k=3, top_p=None)
    assert (sp_own.top_k, sp_own.top_p) == (3, 1.0)
    sp_flags = eng.sampling_params({"top_p": 0.5}, temperature=0.8)
    assert (sp_flags.top_k, sp_flags.top_p) == (0, 0.5)
    greedy = eng.sampling_params(temperature=0.0, top_k=None, max_tokens=4)
    assert (greedy.top_k, greedy.top_p) == (0, 1.0)
    prompt = T.long_tokens("a", 9, seed=2)
    out = eng.generate([prompt], sp)[0]
    # every drawn token is among the card's five most likely at its position
    seq = list(prompt)
    for tok in out:
        logits = P.forward(cfg, W, seq)[-1]
        assert tok in torch.topk(logits, 5).indices.tolist()
        seq.append(tok)


def test_a_bfloat16_replay_held_against_the_32_bit_one_by_the_compare_command(tmp_path):
    """`bin/trace_run` twice over one trace (float32, bfloat16), then `python -m tandemllm_b200 compare`: every wanted row is
    there, the two precisions differ by bfloat16's rounding, and where their largest logits differ the record says whether
    the 32-bit row could tell the two tokens apart."""
    from tests import traces
    folder, cfg, W = folder_of("c", tmp_path, torch.bfloat16)
    reqs = {f"q{i}": T.long_tokens("c", n, seed=40 + i) for i, n in enumerate((50, 23, 37))}
    trace = traces.mixed(reqs, live=2, seed=3)
    lines = "\n".join(json.dumps(s) for s in trace) + "\n"
    held = traces.tokens_held(trace, 64)
    wanted = sum(len(e["want"]) for s in trace for e in s["entries"])
    for dtype in ("float32", "bfloat16"):
        r = subprocess.run([os.path.join(ROOT, "bin", "trace_run"), "--model", folder, "--dtype", dtype, "--out",
                            str(tmp_path / dtype), "--max-tokens", str(held)], input=lines, capture_output=True, text=True,
                           timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
    r = subprocess.run([sys.executable, "-m", "tandemllm_b200", "compare", "--run", str(tmp_path / "bfloat16"), "--reference",
                        str(tmp_path / "float32"), "--model", folder], cwd=ROOT, capture_output=True, text=True, timeout=120)
    rec = json.loads(r.stdout)
    assert rec["positions"] == wanted > 20 and not rec["missing_steps"]
    assert 0 < rec["max_rel_diff"] < 3e-2 and rec["agree_pct"] > 80
    assert rec["argmax_agree"] + rec["near_tie"] + rec["other"] == wanted
    assert r.returncode == (0 if rec["other"] == 0 else 1)


def test_aborting_requests_between_portions_and_with_a_step_in_the_air_leaves_the_others_alone(tmp_path):
    """`Engine.abort`: one request is taken out between two portions of its prompt, one while it decodes and a step launched
    ahead still computes a row for it, one while it waits. Pages and slots are back at once, the aborted texts hold no
    place-holders, and the requests that stay generate what they generate alone."""
    from tandemllm_b200.engine import Engine, EngineArgs
    from tandemllm_b200.sampling import SamplingParams
    folder, cfg, W = folder_of("c", tmp_path, torch.float32)
    args = dict(dtype="float32", max_len=200, parallel=3, chunk_size=16, max_batched_tokens=40)
    prompts = [T.long_tokens("c", n, seed=60 + i) for i, n in enumerate((70, 12, 25, 9, 30))]
    params = lambda: SamplingParams(temperature=0.0, max_tokens=14, ignore_eos=True)
    eng = Engine.from_folder(folder, EngineArgs(**args))
    reqs = [eng.add_request(p, params()) for p in prompts]
    eng.run_step(); eng.run_step()
    assert 0 < reqs[0].num_computed < len(prompts[0]) and reqs[4].state == "waiting"
    eng.abort(reqs[0])                                  # between two portions of its prompt
    eng.abort(reqs[4])                                  # still waiting
    eng.cache.check()
    while not (reqs[1].output and eng._flight is not None):     # decoding, with the next step already launched
        eng.run_step()
    assert reqs[1].state == "running"
    eng.abort(reqs[1])
    eng.abort(reqs[1])                                  # once more: nothing happens
    while eng.scheduler.has_unfinished():
        eng.run_step()
    eng.cache.check()
    st = eng.cache.stats()
    assert st["requests"] == 0 and st["free_slots"] == 3 and all(g["free"] == g["pages"] for g in st["groups"])
    assert [r.finish_reason for r in reqs] == ["aborted", "aborted", "length", "length", "aborted"]
    assert all(t >= 0 for r in reqs for t in r.output) and reqs[4].output == [] and len(reqs[1].output) < 14
    alone = Engine.from_folder(folder, EngineArgs(**dict(args, parallel=1)))
    for i in (2, 3):
        assert alone.generate([prompts[i]], params())[0] == reqs[i].output, i
    assert alone.generate([prompts[1]], params())[0][:len(reqs[1].output)] == reqs[1].output
