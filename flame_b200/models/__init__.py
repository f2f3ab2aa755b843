from .config import ModelConfig
from .modeling import CausalLM, CausalLMOutput, build_model, get_blocks

__all__ = ["ModelConfig", "CausalLM", "CausalLMOutput", "build_model", "get_blocks"]
