"""Model definitions used by the benchmarks and tests (random initialisation, no checkpoints)."""
from .bert import BertConfig, BertMLM, mask_tokens
from .gpt2 import GPT2, GPT2Config
from .llama import Llama, LlamaConfig
from .resnet import ResNet, resnet50, resnet_tiny

__all__ = ["GPT2", "GPT2Config", "BertMLM", "BertConfig", "mask_tokens", "Llama", "LlamaConfig", "ResNet", "resnet50",
           "resnet_tiny"]
