"""Configuration: the typed per-architecture readers, the neutral `ModelSpec`, and the registry."""

from .lfm2_moe import ARCHITECTURES as _LFM2_ARCHS
from .lfm2_moe import MODEL_TYPES as _LFM2_TYPES
from .lfm2_moe import Lfm2MoeConfig
from .registry import (REGISTRY, Architecture, architecture_of, read_model_config, register, resolve_model_folder,
                       spec_of, unregister)
from .spec import LayerSpec, ModelSpec, PartSpec, Site, plain_schedule

register(Architecture(name="lfm2_moe", architectures=_LFM2_ARCHS, model_types=_LFM2_TYPES,
                      read_config=Lfm2MoeConfig.from_dict))

__all__ = ["REGISTRY", "Architecture", "architecture_of", "read_model_config", "register", "unregister",
           "resolve_model_folder", "spec_of", "LayerSpec", "ModelSpec", "PartSpec", "Site", "plain_schedule",
           "Lfm2MoeConfig"]
