from .causal import CausalTransformerModel, GPT2Model, LlamaModel, QwenModel
from .layered import LayeredCausalModel

__all__ = ["CausalTransformerModel", "GPT2Model", "LlamaModel", "QwenModel", "LayeredCausalModel"]
