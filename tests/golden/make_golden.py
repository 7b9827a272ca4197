"""Writes the golden logits of the reference's own model code for the tiny test models.

    python tests/golden/make_golden.py --reference <checkout of the reference project>

It imports the reference's `Lfm2MoeRef` (engine/models/lfm2_moe/ref.py) and `config_from_dict`
(engine/models/lfm2_moe/config.py) on the CPU, runs each prompt whole in 32-bit, and stores the logits of
every position in `tiny_a_reference.npz` and `tiny_b_reference.npz` beside this file, with a checksum of
the weights they were computed from. The weights come from the test helpers' seeded generator, so the
files hold numbers only. Model A is run exactly as configured; model B is run without the three options
the reference refuses (conv bias, un-normalised top-k weights; the untied head is passed as
`lm_head.weight`, which the reference's `head_weight` reads).
"""

from __future__ import annotations

import argparse
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from tests import tiny_configs as T  # noqa: E402
from tests.helpers import random_model_weights  # noqa: E402


def checksum(W: dict) -> float:
    return float(sum(float(t.double().abs().sum()) for _, t in sorted(W.items())))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="a checkout of the reference project")
    a = ap.parse_args()
    sys.path.insert(0, a.reference)
    from engine.models.lfm2_moe.config import config_from_dict
    from engine.models.lfm2_moe.ref import Lfm2MoeRef

    for name, cfg, ref_cfg in (("a", T.TINY_A, T.TINY_A), ("b", T.TINY_B_REFERENCE, T.TINY_B_REFERENCE)):
        W = random_model_weights(cfg, T.SEEDS[name], T.STD[name])
        # the reference's config reader wants tie_word_embeddings True; an untied head is simply a W entry
        rc = config_from_dict({**ref_cfg, "tie_word_embeddings": True})
        ref = Lfm2MoeRef(rc, W, dtype=torch.float32)
        out = {"weights_checksum": np.float64(checksum(W))}
        for i, prompt in enumerate(T.prompts(name)):
            st = ref.new_state(len(prompt) + 8)
            out[f"prompt_{i}"] = np.asarray(prompt, dtype=np.int64)
            out[f"logits_{i}"] = ref.prefill(torch.tensor(prompt), st).numpy()
        path = os.path.join(HERE, f"tiny_{name}_reference.npz")
        np.savez_compressed(path, **out)
        print(path, {k: getattr(v, "shape", v) for k, v in out.items()})


if __name__ == "__main__":
    main()
