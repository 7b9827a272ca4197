"""Every environment knob the package reads, in one table, read through one object.

The reference keeps its environment variables in one registry and reads them only through
`SETTINGS.get(name)` (engine/settings.py:35, :527-553), so that a knob's default is written once and a test
can hold every module to that rule. The same here, in small: `KNOBS` maps a name (without the prefix
`TANDEMLLM_`) to its default, what it means and the module that reads it, and `SETTINGS.get` is the only
call in the package that looks at `os.environ` (a test greps the package for any other read).

A knob is read when the code that needs it runs, from the live environment, so a test can set one and see it.
"""

from __future__ import annotations

import os
from typing import Mapping

PREFIX = "TANDEMLLM_"

# name -> (default, meaning, the module that reads it)
KNOBS: dict[str, tuple] = {
    "NVCC": (None, "the nvcc to build the CUDA libraries with (default: the one on PATH, then /usr/local/cuda/bin/nvcc)",
             "kernels/build.py"),
    "BUILD_DIR": (None, "where the built libraries go (default: csrc/_build in the tree, else a per-user folder under "
                        "the temp dir)", "kernels/build.py"),
    "GRAPHS": ("32", "decode graphs kept at a time by a step function; the least recently replayed is dropped beyond it",
               "engine/step.py"),
    "NVTX": (None, "when set, every step and every layer of it is an NVTX range (for `ncu --nvtx --nvtx-include` and other "
                   "tools that read them); off by default: a range costs a host call", "parts/model.py"),
    "PROMPT_PRODUCT": ("pair", "prompt-sized bfloat16 products: `pair` (two SMs a tile, tcgen05 cta_group::2) or `single` "
                               "(one CTA a tile)", "kernels/tensorcore.py"),
    "STEP_LOG": (None, "a file to which every engine appends one JSON line a scheduler step (rows, pages, milliseconds)",
                 "engine/engine.py"),
}


class Settings:
    """The knobs over an environment mapping (the live `os.environ` by default)."""

    def __init__(self, env: Mapping[str, str] | None = None, prefix: str = PREFIX):
        self._env = env
        self.prefix = prefix

    @property
    def env(self) -> Mapping[str, str]:
        return os.environ if self._env is None else self._env

    def get(self, name: str):
        """The string the environment holds for `name`, else the table's default. A name the table does not
        hold is an error: a knob exists by being listed."""
        if name not in KNOBS:
            raise KeyError(f"{self.prefix}{name} is not a registered knob (tandemllm_b200/settings.py KNOBS: "
                           f"{', '.join(sorted(KNOBS))})")
        value = self.env.get(self.prefix + name)
        return KNOBS[name][0] if value in (None, "") else value

    def get_int(self, name: str) -> int:
        raw = self.get(name)
        try:
            return int(raw)
        except (TypeError, ValueError):
            raise ValueError(f"{self.prefix}{name}={raw!r}: an integer is wanted") from None

    def is_set(self, name: str) -> bool:
        return bool(self.env.get(self.prefix + name))

    def describe(self) -> dict[str, dict]:
        """Every knob with its effective value, its default, whether the environment set it, and its reader."""
        return {k: {"value": self.get(k), "default": d, "set": self.is_set(k), "meaning": what, "read_in": where}
                for k, (d, what, where) in sorted(KNOBS.items())}


SETTINGS = Settings()
