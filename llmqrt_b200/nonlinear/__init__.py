from .attn import QuantAttentionFused, RoPE
from .block import LlamaLikeBlock, LlamaLikeModel
from .cache import WindowedCache
from .norm import RMSNorm

__all__ = ["QuantAttentionFused", "RoPE", "LlamaLikeBlock", "LlamaLikeModel", "WindowedCache", "RMSNorm"]
