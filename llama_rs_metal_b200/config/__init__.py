from .base import read_config_json, read_generation_eos, read_int, read_real, read_bool, normalize_token_ids
from .llama import LlamaConfig, RopeScaling

__all__ = ["LlamaConfig", "RopeScaling", "read_config_json", "read_generation_eos",
           "read_int", "read_real", "read_bool", "normalize_token_ids"]
