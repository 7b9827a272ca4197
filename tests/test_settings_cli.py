"""The knob table, the command line's help and argument errors, the decode-graph context buckets, a slot's initial
value, and the model's byte account: everything here runs without a GPU."""

import os
import re
import subprocess
import sys

import pytest
import torch

from tests import tiny_configs as T

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PACKAGE = os.path.join(ROOT, "tandemllm_b200")


def test_every_knob_is_read_through_the_table():
    """No module of the package looks at the environment except `settings.py` (the reference holds its engine to the
    same rule, tests/test_settings.py there)."""
    offenders = []
    for folder, _, files in os.walk(PACKAGE):
        for name in files:
            if not name.endswith(".py") or os.path.join(folder, name) == os.path.join(PACKAGE, "settings.py"):
                continue
            text = open(os.path.join(folder, name)).read()
            for m in re.finditer(r"os\.environ|os\.getenv|getenv\(|environ\[", text):
                offenders.append(f"{os.path.relpath(os.path.join(folder, name), ROOT)}:{text[:m.start()].count(chr(10)) + 1}")
    assert not offenders, offenders
    for script in ("bin/trace_run", "bench.py", "microbench.py", "__graft_entry__.py"):
        assert "os.environ" not in open(os.path.join(ROOT, script)).read(), script


def test_knobs_have_defaults_readers_and_live_values():
    from tandemllm_b200.settings import KNOBS, Settings
    for name, (default, meaning, reader) in KNOBS.items():
        assert meaning and os.path.isfile(os.path.join(PACKAGE, reader)), name
        text = open(os.path.join(PACKAGE, reader)).read()
        assert f'"{name}"' in text, f"{reader} does not read {name}"
    s = Settings(env={"TANDEMLLM_GRAPHS": "5", "TANDEMLLM_NVCC": ""})
    assert s.get_int("GRAPHS") == 5 and s.is_set("GRAPHS") and s.get("NVCC") is None and not s.is_set("NVCC")
    assert Settings(env={}).get_int("GRAPHS") == int(KNOBS["GRAPHS"][0])
    with pytest.raises(KeyError, match="not a registered knob"):
        s.get("NO_SUCH_KNOB")
    with pytest.raises(ValueError, match="integer"):
        Settings(env={"TANDEMLLM_GRAPHS": "many"}).get_int("GRAPHS")
    d = s.describe()
    assert d["GRAPHS"]["value"] == "5" and d["GRAPHS"]["set"] and d["BUILD_DIR"]["read_in"] == "kernels/build.py"


def test_build_reads_its_knobs_from_the_live_environment(monkeypatch, tmp_path):
    from tandemllm_b200.kernels import build
    monkeypatch.setenv("TANDEMLLM_BUILD_DIR", str(tmp_path / "b"))
    assert build.build_dir() == str(tmp_path / "b")
    fake = tmp_path / "nvcc"
    fake.write_text("#!/bin/sh\n")
    fake.chmod(0o755)
    monkeypatch.setenv("TANDEMLLM_NVCC", str(fake))
    assert build.find_nvcc() == str(fake)


def run_cli(*args):
    return subprocess.run([sys.executable, "-m", "tandemllm_b200", *args], cwd=ROOT, capture_output=True, text=True, timeout=120)


def test_command_line_help_and_argument_errors(tmp_path):
    r = run_cli("--help")
    assert r.returncode == 0 and "generate" in r.stdout and "random-weights" in r.stdout and "replay" in r.stdout
    r = run_cli("generate", "--help")
    for option in ("--model", "--max-len", "--temperature", "--top-p", "--top-k", "--parallel", "--tokens", "--graph", "--json", "--log"):
        assert option in r.stdout, option
    assert run_cli().returncode == 2
    assert run_cli("generate", "--dtype", "float16").returncode == 2
    r = run_cli("generate")
    assert r.returncode != 0 and "--model" in r.stderr
    r = run_cli("generate", "--random-weights", "3")
    assert r.returncode != 0 and "--config" in r.stderr
    r = run_cli("random-weights", "--out", str(tmp_path / "m"))
    assert r.returncode == 2 and "--config" in r.stderr


def test_random_weights_command_writes_a_folder_the_loader_takes(tmp_path):
    import json

    from tandemllm_b200.config import read_model_config, spec_of
    from tandemllm_b200.parts.model import DecoderModel
    from tandemllm_b200.weights.loader import FolderWeights
    cfg = tmp_path / "config.json"
    cfg.write_text(json.dumps(T.TINY_A))
    r = run_cli("random-weights", "--config", str(cfg), "--out", str(tmp_path / "m"), "--seed", "4", "--dtype", "float32")
    assert r.returncode == 0, r.stderr
    arch, config = read_model_config(str(tmp_path / "m"))
    spec = spec_of(config)
    weights = FolderWeights(str(tmp_path / "m"), spec.name_prefixes)
    weights.check(DecoderModel(spec).weight_specs(weights.present()))


def test_context_buckets_of_decode_graphs_are_few_and_close():
    from tandemllm_b200.engine.step import context_bucket
    seen = set()
    for n in list(range(1, 20000)) + list(range(20000, 131073, 7)):
        b = context_bucket(n)
        assert n <= b and (b <= 1024 or b - n < max(1024, n // 7)), (n, b)
        seen.add(b)
    assert len(seen) <= 48


def test_a_slot_starts_from_what_its_need_says():
    from tandemllm_b200.cache.manager import CacheManager
    from tandemllm_b200.parts.base import SlotNeed
    needs = [SlotNeed((2, 3)), SlotNeed((3,), torch.float32, init=1.5), SlotNeed((2, 3), torch.float32, init=torch.arange(3.0))]
    cache = CacheManager(needs, num_pages=4, max_requests=2, device="cpu")
    for sc in cache.site_cache:
        sc.state.fill_(7.0)
    slot = cache.admit("r")
    assert torch.equal(cache.site_cache[0].state[slot], torch.zeros(2, 3))
    assert torch.equal(cache.site_cache[1].state[slot], torch.full((3,), 1.5))
    assert torch.equal(cache.site_cache[2].state[slot], torch.arange(3.0).expand(2, 3))
    assert float(cache.site_cache[0].state[1 - slot].min()) == 7.0           # the other slot is left alone


def test_the_model_accounts_the_bytes_of_a_decode_step_from_its_parts():
    from tandemllm_b200.config import Lfm2MoeConfig
    from tandemllm_b200.parts.model import DecoderModel
    c = Lfm2MoeConfig.from_dict(T.TINY_A)
    model = DecoderModel(c.to_spec())
    H, V, I, Im, E, k = 64, 256, 128, 32, 4, 2
    got = model.decode_bytes(batch=3, experts_read=[2, 3, 4])
    conv = (3 * H * H + H * H) * 2 + H * 3 * 4 + 2 * H * 4               # in/out matrices (bf16), taps and two norms (32-bit)
    attn = (4 * 16 + 2 * 2 * 16) * H * 2 + H * 4 * 16 * 2 + 2 * 16 * 4 + 2 * H * 4
    router = E * H * 4 + E * 4
    want_dense = 2 * conv + 2 * attn + 3 * H * I * 2 + 3 * router + H * 4
    assert got["dense"] == want_dense
    assert got["experts"] == (2 + 3 + 4) * 3 * H * Im * 2
    assert got["head"] == V * H * 2 and got["embedding_rows"] == 3 * H * 2
    assert got["total"] == got["dense"] + got["experts"] + got["head"] + got["embedding_rows"]
    # without a count: what uniform routing would read
    uniform = model.decode_bytes(batch=3)["experts"]
    assert uniform == 3 * int(E * (1 - (1 - k / E) ** 3) * 3 * H * Im * 2)


def test_penalty_options_are_checked_when_the_parameters_are_made():
    from tandemllm_b200.sampling import SamplingParams
    p = SamplingParams()
    assert not p.penalizes and not p.changes_logits and p.logit_bias is None
    assert SamplingParams(repetition_penalty=1.1).penalizes and SamplingParams(frequency_penalty=-0.5).penalizes
    q = SamplingParams(logit_bias={"7": 1.5, 9: 0.0})
    assert q.logit_bias == {7: 1.5} and q.changes_logits and not q.penalizes       # a zero entry is no entry
    assert SamplingParams(logit_bias={3: 0.0}).logit_bias is None
    for bad in (dict(repetition_penalty=0.0), dict(repetition_penalty=float("nan")), dict(presence_penalty=2.5),
                dict(frequency_penalty=-2.5), dict(logit_bias={-1: 1.0}), dict(logit_bias={2.5: 1.0}),
                dict(logit_bias={2: float("nan")})):
        with pytest.raises(ValueError):
            SamplingParams(**bad)


def test_the_command_line_reads_penalties_and_added_logits():
    from tandemllm_b200.__main__ import _logit_bias
    assert _logit_bias(["17:-4.5", "3:2"]) == {17: -4.5, 3: 2.0} and _logit_bias(None) is None
    with pytest.raises(SystemExit, match="TOKEN:VALUE"):
        _logit_bias(["17"])
    out = subprocess.run([sys.executable, "-m", "tandemllm_b200", "generate", "--help"], capture_output=True, text=True,
                         cwd=ROOT).stdout
    for name in ("--rep-penalty", "--presence-penalty", "--frequency-penalty", "--logit-bias"):
        assert name in out


def test_the_audit_command_checks_a_folder_from_its_headers_alone(tmp_path):
    """`python -m tandemllm_b200 audit --model DIR` (no GPU): the stored tensors against what the parts would read, bytes
    by stored type, bytes of a decode step; a folder that lacks a tensor and has a stray one is refused by name, exit 1."""
    import json

    from tests.helpers import random_model_weights, write_folder
    W = random_model_weights(T.TINY_B, 1, 0.02, bf16_exact=True)
    good = write_folder(str(tmp_path / "good"), T.TINY_B, W, torch.bfloat16)
    r = run_cli("audit", "--model", good, "--batch", "1", "8")
    assert r.returncode == 0, r.stderr
    rec = json.loads(r.stdout)
    assert rec["architecture"] == "lfm2_moe" and rec["refused"] is None and rec["layers"] == T.TINY_B["num_hidden_layers"]
    assert rec["tensors_expected"] == rec["tensors_stored"] == len(W) and rec["files"] == 1
    assert sum(v["tensors"] for v in rec["stored"].values()) == len(W)
    assert rec["decode_bytes"]["8"]["experts"] > rec["decode_bytes"]["1"]["experts"] > 0
    assert rec["decode_bytes"]["1"]["dense"] == rec["decode_bytes"]["8"]["dense"]
    lacking = dict(W)
    gone = next(n for n in lacking if n.endswith("operator_norm.weight"))
    del lacking[gone]
    lacking["stray.weight"] = torch.zeros(3)
    bad = write_folder(str(tmp_path / "bad"), T.TINY_B, lacking, torch.bfloat16)
    r = run_cli("audit", "--model", bad)
    assert r.returncode == 1
    refused = json.loads(r.stdout)["refused"]
    assert gone in refused and "stray.weight" in refused and "missing (1)" in refused and "unexpected (1)" in refused


def test_the_compare_command_holds_one_replay_against_another(tmp_path):
    """`python -m tandemllm_b200 compare --run A --reference B --vocab V`: the record of a teacher-forced comparison (rows,
    agreement of the largest logit, near ties and other disagreements, relative differences); exit 1 on a disagreement that
    is no near tie or on a step that is missing."""
    import json

    import numpy as np
    V = 50
    rng = np.random.default_rng(0)
    ref = {0: rng.normal(size=(3, V)).astype("<f4"), 2: rng.normal(size=(1, V)).astype("<f4"), 5: rng.normal(size=(2, V)).astype("<f4")}
    a, b = tmp_path / "a", tmp_path / "b"
    a.mkdir(); b.mkdir()
    order = np.argsort(ref[5][0])
    ref[5][0, order[-2]] = ref[5][0, order[-1]] - 1e-3           # the reference itself can hardly tell these two apart
    for step, rows in ref.items():
        rows.tofile(b / f"{step}.f32")
        (rows + rng.normal(scale=1e-3, size=rows.shape).astype("<f4")).tofile(a / f"{step}.f32")
    r = run_cli("compare", "--run", str(a), "--reference", str(b), "--vocab", str(V))
    rec = json.loads(r.stdout)
    assert r.returncode == 0 and rec["positions"] == 6 and rec["argmax_agree"] == 6 and rec["steps"] == 3
    assert 0 < rec["max_rel_diff"] < 5e-3 and rec["mean_rel_diff"] < rec["max_rel_diff"]
    # a near tie (the runner-up lifted just above the best) and a plain disagreement
    rows = ref[5].copy()
    rows[0, order[-2]] = rows[0, order[-1]] + 1e-4
    rows[1, int(np.argmin(rows[1]))] = 100.0
    rows.tofile(a / "5.f32")
    (a / "2.f32").unlink()
    r = run_cli("compare", "--run", str(a), "--reference", str(b), "--vocab", str(V))
    rec = json.loads(r.stdout)
    assert r.returncode == 1 and rec["missing_steps"] == [2] and rec["positions"] == 5
    assert rec["near_tie"] == 1 and rec["other"] == 1 and rec["argmax_agree"] == 3
    assert [d["near_tie"] for d in rec["disagreements"]] == [True, False]
    assert run_cli("compare", "--run", str(a), "--reference", str(b)).returncode != 0       # neither --vocab nor --model
