from .serving import ContinuousBatcher, Request
from .qwen3 import DecodeSession, Qwen3Config, Qwen3Decoder, Qwen3Weights, reference_forward, reference_forward_tp

__all__ = ["ContinuousBatcher", "Request", "DecodeSession", "Qwen3Config", "Qwen3Decoder", "Qwen3Weights", "reference_forward", "reference_forward_tp"]
