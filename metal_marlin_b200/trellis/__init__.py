from .generate import GenerationConfig, TrellisGenerator
from .lm import TrellisForCausalLM, TrellisModelConfig

__all__ = ["GenerationConfig", "TrellisGenerator", "TrellisForCausalLM", "TrellisModelConfig"]
