"""Model specifications and the generic model that runs them."""
from ..config.model_config import YiConfig
from ..config.registry import register_architecture
from .model import Model
from .spec import LayerSpec, ModelSpec, RunEntry
from .yi import yi_spec

for _name in ("LlamaForCausalLM", "YiForCausalLM"):
    register_architecture(_name, YiConfig.from_dict, yi_spec)
