from .registry import ARCHITECTURES, config_from_dict, load_config, model_spec_for, register_architecture
from .spec import LayerSpec, ModelSpec, RunEntry

__all__ = ["ARCHITECTURES", "config_from_dict", "load_config", "model_spec_for", "register_architecture",
           "LayerSpec", "ModelSpec", "RunEntry"]
