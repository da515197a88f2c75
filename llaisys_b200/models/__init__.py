from .causal_lm import CausalLM, DeviceType, Qwen2

__all__ = ["CausalLM", "DeviceType", "Qwen2"]
