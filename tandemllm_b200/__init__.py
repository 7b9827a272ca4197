"""tandemllm_b200: a small, whole inference engine for one B200 and the LFM2 / LFM2.5 MoE architecture."""

from .config import Lfm2MoeConfig, ModelSpec, read_model_config, register  # noqa: F401

__version__ = "0.1.0"


def __getattr__(name):
    # the engine and sampling need torch with CUDA kernels; import them on first use
    if name in ("Engine", "EngineArgs", "StepEntry"):
        from . import engine
        return getattr(engine, name)
    if name in ("SamplingParams", "Sampler"):
        from . import sampling
        return getattr(sampling, name)
    raise AttributeError(name)
